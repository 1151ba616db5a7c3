#include "host_utils.h"

#include <cudaTypedefs.h>
#include <stdarg.h>

namespace cpb {

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return CPB_OK;
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

int encode_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, int swizzle128) {
  auto fn = get_encode();
  if (fn == nullptr) return set_error(CPB_ERR_DRIVER, "cuTensorMapEncodeTiled entry point unavailable");
  // The driver call needs a current context; a thread that has made no runtime call yet (an autograd
  // worker thread, for instance) has none until the runtime binds the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if (((uintptr_t)base & 15) != 0) return set_error(CPB_ERR_ARG, "tensor map base %p not 16-byte aligned", base);
  cuuint64_t gdim[5], gstride[5];
  cuuint32_t bdim[5], estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i > 0) {
      gstride[i - 1] = strides_bytes[i];
      if (strides_bytes[i] % 16) return set_error(CPB_ERR_ARG, "tensor map stride %llu not a multiple of 16", (unsigned long long)strides_bytes[i]);
    }
  }
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(CPB_ERR_DRIVER, "cuTensorMapEncodeTiled failed with %d (rank %d, dim0 %llu, box0 %u)", (int)r, rank, (unsigned long long)dims[0], box[0]);
  return CPB_OK;
}

}  // namespace cpb

extern "C" const char* cpb_last_error() { return cpb::last_error_buf(); }
