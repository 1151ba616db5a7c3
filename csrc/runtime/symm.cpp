// Symmetric peer-memory heap for one node: every rank allocates an arena of the same size with
// cudaMalloc, exports a CUDA IPC handle, and maps every peer's arena; kernels then address remote
// memory as (peer_base[rank] + offset) with plain loads/stores over NVLink.  The arenas live outside
// the PyTorch caching allocator, so a buffer a peer may still be reading is never recycled behind its
// back (the reference needed recordStream() on cross-stream buffers to avoid exactly that,
// context_parallel/RingRotator.h:146-149,260-270).
//
// Takes the place of the NCCL-only communicator layer of the reference
// (process_group/processGroupNCCL.cpp:36-126) for the fused kernels; NCCL (through torch.distributed)
// remains the transport of the baseline paths.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../kernels/host_utils.h"

using namespace cpb;

extern "C" int cpb_symm_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "symm_alloc(%zu): %s", bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "symm_alloc memset: %s", cudaGetErrorString(e));
  *out = p;
  return CPB_OK;
}

extern "C" int cpb_symm_free(void* p) {
  cudaError_t e = cudaFree(p);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "symm_free: %s", cudaGetErrorString(e));
  return CPB_OK;
}

// handle_out: 64 bytes
extern "C" int cpb_symm_export(void* p, unsigned char* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  static_assert(sizeof(h) == 64, "ipc handle size");
  memcpy(handle_out, &h, 64);
  return CPB_OK;
}

extern "C" int cpb_symm_import(const unsigned char* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *out = p;
  return CPB_OK;
}

extern "C" int cpb_symm_close(void* p) {
  cudaError_t e = cudaIpcCloseMemHandle(p);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  return CPB_OK;
}

// Same-process peers (several GPUs driven by one process, used by single-process tests): enable
// direct access instead of IPC.
extern "C" int cpb_enable_peer_access(int peer_device) {
  int can = 0, dev = 0;
  cudaGetDevice(&dev);
  if (peer_device == dev) return CPB_OK;
  cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (!can) return set_error(CPB_ERR_CUDA, "device %d cannot access peer %d", dev, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return set_error(CPB_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
  cudaGetLastError();
  return CPB_OK;
}
