// Native NCCL process group: communicators, streams and asynchronous work handles behind a C ABI.
//
// One group owns TWO communicators over the same ranks: `comm` for collectives (gradient reduction, loss, all-to-all)
// and a dedicated `ring_comm` with its own non-blocking stream for the ring's neighbour exchange, so that ring traffic
// never queues behind, or deadlocks with, a collective on the same communicator
// (the reference does the same, process_group/processGroupNCCL.cpp:53-63,562-577).  Sub-groups for the mesh axes are
// made with ncclCommSplit (process_group/device_mesh.cpp:143-176).  Every operation
//   1. makes the communication stream wait for an event recorded on the caller's stream (inputs are ready),
//   2. enqueues the NCCL call on the communication stream,
//   3. returns a work handle (csrc/runtime/work.cpp) whose event follows the call: the caller waits on the device
//      (`cpb_work_stream_wait`) or on the host with a deadline (`cpb_work_wait`); on a time-out the owner calls
//      `cpb_pg_abort`, which tears the communicators down instead of leaving the process hung inside NCCL
//      (the reference left this watcher commented out, process_group/processGroupNCCL.cpp:719-744).
// The unique ids are created here and distributed by the caller's bootstrap (torch.distributed's store; the
// reference used MPI_Bcast, processGroupNCCL.cpp:62,118).
//
// This is the transport of the NCCL baseline paths; the product paths use the peer-memory kernels.
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "../kernels/host_utils.h"

using namespace cpb;

extern "C" int cpb_work_create(cudaStream_t stream, int with_event, double timeout_s, void** out);

namespace {

struct Group {
  ncclComm_t comm = nullptr, ring_comm = nullptr;
  cudaStream_t stream = nullptr, ring_stream = nullptr;
  cudaEvent_t ready = nullptr;      // records "inputs ready" on the caller's stream
  int world = 0, rank = 0, device = 0;
  double timeout_s = 0;
  std::mutex mu;
};

int nccl_fail(const char* what, ncclResult_t r) { return set_error(CPB_ERR_CUDA, "%s: %s", what, ncclGetErrorString(r)); }
#define NCCL_OK(expr)                                  \
  do {                                                 \
    ncclResult_t _r = (expr);                          \
    if (_r != ncclSuccess) return nccl_fail(#expr, _r); \
  } while (0)

bool to_dtype(int code, ncclDataType_t* out) {
  switch (code) {          // 0 f32, 1 bf16, 2 f16, 3 i32, 4 i64, 5 u8, 6 f64
    case 0: *out = ncclFloat32; return true;
    case 1: *out = ncclBfloat16; return true;
    case 2: *out = ncclFloat16; return true;
    case 3: *out = ncclInt32; return true;
    case 4: *out = ncclInt64; return true;
    case 5: *out = ncclUint8; return true;
    case 6: *out = ncclFloat64; return true;
  }
  return false;
}
bool to_op(int code, ncclRedOp_t* out) {
  switch (code) {          // 0 sum, 1 avg, 2 max, 3 min, 4 prod
    case 0: *out = ncclSum; return true;
    case 1: *out = ncclAvg; return true;
    case 2: *out = ncclMax; return true;
    case 3: *out = ncclMin; return true;
    case 4: *out = ncclProd; return true;
  }
  return false;
}
size_t dtype_bytes(int code) { static const size_t b[7] = {4, 2, 2, 4, 8, 1, 8}; return code >= 0 && code < 7 ? b[code] : 0; }

// inputs on `user` are ready -> the communication stream may start
int begin(Group* g, cudaStream_t user, cudaStream_t comm_stream) {
  CPB_CUDA_OK(cudaEventRecord(g->ready, user));
  CPB_CUDA_OK(cudaStreamWaitEvent(comm_stream, g->ready, 0));
  return CPB_OK;
}
int finish(Group* g, cudaStream_t comm_stream, void** work) {
  if (work == nullptr) return CPB_OK;
  return cpb_work_create(comm_stream, 1, g->timeout_s, work);
}

}  // namespace

extern "C" int cpb_pg_unique_id(unsigned char* out128) {
  ncclUniqueId id;
  NCCL_OK(ncclGetUniqueId(&id));
  static_assert(sizeof(id) == 128, "nccl unique id size");
  memcpy(out128, &id, 128);
  return CPB_OK;
}

// id / ring_id: unique ids made on rank 0 and handed to every rank by the caller.  ring_id may be null (no dedicated
// ring communicator).  timeout_s is the deadline given to every work handle (0 = none).
extern "C" int cpb_pg_create(const unsigned char* id128, const unsigned char* ring_id128, int world, int rank,
                             double timeout_s, void** out) {
  auto* g = new Group();
  g->world = world; g->rank = rank; g->timeout_s = timeout_s;
  cudaGetDevice(&g->device);
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  ncclResult_t r = ncclCommInitRank(&g->comm, world, id, rank);
  if (r != ncclSuccess) { delete g; return nccl_fail("ncclCommInitRank", r); }
  if (ring_id128 != nullptr) {
    ncclUniqueId rid;
    memcpy(&rid, ring_id128, 128);
    r = ncclCommInitRank(&g->ring_comm, world, rid, rank);
    if (r != ncclSuccess) { ncclCommDestroy(g->comm); delete g; return nccl_fail("ncclCommInitRank (ring)", r); }
  }
  CPB_CUDA_OK(cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking));
  CPB_CUDA_OK(cudaStreamCreateWithFlags(&g->ring_stream, cudaStreamNonBlocking));
  CPB_CUDA_OK(cudaEventCreateWithFlags(&g->ready, cudaEventDisableTiming));
  *out = g;
  return CPB_OK;
}

// Sub-group: ranks with the same colour, ordered by key (ncclCommSplit on both communicators).
extern "C" int cpb_pg_split(void* h, int color, int key, int new_world, int new_rank, void** out) {
  auto* p = (Group*)h;
  auto* g = new Group();
  g->world = new_world; g->rank = new_rank; g->timeout_s = p->timeout_s; g->device = p->device;
  ncclResult_t r = ncclCommSplit(p->comm, color, key, &g->comm, nullptr);
  if (r != ncclSuccess) { delete g; return nccl_fail("ncclCommSplit", r); }
  if (p->ring_comm) {
    r = ncclCommSplit(p->ring_comm, color, key, &g->ring_comm, nullptr);
    if (r != ncclSuccess) { ncclCommDestroy(g->comm); delete g; return nccl_fail("ncclCommSplit (ring)", r); }
  }
  CPB_CUDA_OK(cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking));
  CPB_CUDA_OK(cudaStreamCreateWithFlags(&g->ring_stream, cudaStreamNonBlocking));
  CPB_CUDA_OK(cudaEventCreateWithFlags(&g->ready, cudaEventDisableTiming));
  *out = g;
  return CPB_OK;
}

extern "C" int cpb_pg_world(void* h) { return ((Group*)h)->world; }
extern "C" int cpb_pg_rank(void* h) { return ((Group*)h)->rank; }

extern "C" int cpb_pg_all_reduce(void* h, void* buf, long count, int dtype, int op, cudaStream_t user, void** work) {
  auto* g = (Group*)h;
  ncclDataType_t dt; ncclRedOp_t ro;
  if (!to_dtype(dtype, &dt) || !to_op(op, &ro)) return set_error(CPB_ERR_ARG, "all_reduce: bad dtype/op");
  std::lock_guard<std::mutex> lk(g->mu);
  int rc = begin(g, user, g->stream);
  if (rc) return rc;
  NCCL_OK(ncclAllReduce(buf, buf, (size_t)count, dt, ro, g->comm, g->stream));
  return finish(g, g->stream, work);
}

extern "C" int cpb_pg_broadcast(void* h, void* buf, long count, int dtype, int root, cudaStream_t user, void** work) {
  auto* g = (Group*)h;
  ncclDataType_t dt;
  if (!to_dtype(dtype, &dt)) return set_error(CPB_ERR_ARG, "broadcast: bad dtype");
  std::lock_guard<std::mutex> lk(g->mu);
  int rc = begin(g, user, g->stream);
  if (rc) return rc;
  NCCL_OK(ncclBroadcast(buf, buf, (size_t)count, dt, root, g->comm, g->stream));
  return finish(g, g->stream, work);
}

// recv holds world * count elements
extern "C" int cpb_pg_all_gather(void* h, const void* send, void* recv, long count, int dtype, cudaStream_t user, void** work) {
  auto* g = (Group*)h;
  ncclDataType_t dt;
  if (!to_dtype(dtype, &dt)) return set_error(CPB_ERR_ARG, "all_gather: bad dtype");
  std::lock_guard<std::mutex> lk(g->mu);
  int rc = begin(g, user, g->stream);
  if (rc) return rc;
  NCCL_OK(ncclAllGather(send, recv, (size_t)count, dt, g->comm, g->stream));
  return finish(g, g->stream, work);
}

// send holds world * count elements, recv count
extern "C" int cpb_pg_reduce_scatter(void* h, const void* send, void* recv, long count, int dtype, int op, cudaStream_t user,
                                     void** work) {
  auto* g = (Group*)h;
  ncclDataType_t dt; ncclRedOp_t ro;
  if (!to_dtype(dtype, &dt) || !to_op(op, &ro)) return set_error(CPB_ERR_ARG, "reduce_scatter: bad dtype/op");
  std::lock_guard<std::mutex> lk(g->mu);
  int rc = begin(g, user, g->stream);
  if (rc) return rc;
  NCCL_OK(ncclReduceScatter(send, recv, (size_t)count, dt, ro, g->comm, g->stream));
  return finish(g, g->stream, work);
}

// Equal-split all-to-all: chunk r of `send` (count elements) goes to rank r; a group of send/recv pairs
// (the reference's alltoallv, process_group/processGroupNCCL.cpp:477-505).
extern "C" int cpb_pg_all_to_all(void* h, const void* send, void* recv, long count, int dtype, cudaStream_t user, void** work) {
  auto* g = (Group*)h;
  ncclDataType_t dt;
  if (!to_dtype(dtype, &dt)) return set_error(CPB_ERR_ARG, "all_to_all: bad dtype");
  const size_t stride = (size_t)count * dtype_bytes(dtype);
  std::lock_guard<std::mutex> lk(g->mu);
  int rc = begin(g, user, g->stream);
  if (rc) return rc;
  NCCL_OK(ncclGroupStart());
  for (int r = 0; r < g->world; ++r) {
    NCCL_OK(ncclSend((const char*)send + r * stride, (size_t)count, dt, r, g->comm, g->stream));
    NCCL_OK(ncclRecv((char*)recv + r * stride, (size_t)count, dt, r, g->comm, g->stream));
  }
  NCCL_OK(ncclGroupEnd());
  return finish(g, g->stream, work);
}

// Ring hop on the dedicated ring communicator and stream: send `count` elements to `dst`, receive from `src`.
extern "C" int cpb_pg_sendrecv(void* h, const void* send, void* recv, long count, int dtype, int dst, int src,
                               cudaStream_t user, void** work) {
  auto* g = (Group*)h;
  ncclDataType_t dt;
  if (!to_dtype(dtype, &dt)) return set_error(CPB_ERR_ARG, "sendrecv: bad dtype");
  ncclComm_t c = g->ring_comm ? g->ring_comm : g->comm;
  cudaStream_t s = g->ring_comm ? g->ring_stream : g->stream;
  std::lock_guard<std::mutex> lk(g->mu);
  int rc = begin(g, user, s);
  if (rc) return rc;
  NCCL_OK(ncclGroupStart());
  NCCL_OK(ncclSend(send, (size_t)count, dt, dst, c, s));
  NCCL_OK(ncclRecv(recv, (size_t)count, dt, src, c, s));
  NCCL_OK(ncclGroupEnd());
  return finish(g, s, work);
}

// 0 = no error; otherwise the NCCL result code of the first asynchronous failure on either communicator.
extern "C" int cpb_pg_async_error(void* h) {
  auto* g = (Group*)h;
  ncclResult_t e = ncclSuccess;
  if (g->comm && ncclCommGetAsyncError(g->comm, &e) == ncclSuccess && e != ncclSuccess) return (int)e;
  if (g->ring_comm && ncclCommGetAsyncError(g->ring_comm, &e) == ncclSuccess && e != ncclSuccess) return (int)e;
  return 0;
}

// Tear the communicators down without waiting for outstanding operations (after a work handle timed out).
extern "C" int cpb_pg_abort(void* h) {
  auto* g = (Group*)h;
  if (g->ring_comm) { ncclCommAbort(g->ring_comm); g->ring_comm = nullptr; }
  if (g->comm) { ncclCommAbort(g->comm); g->comm = nullptr; }
  return CPB_OK;
}

extern "C" void cpb_pg_destroy(void* h) {
  auto* g = (Group*)h;
  if (!g) return;
  if (g->stream) cudaStreamSynchronize(g->stream);
  if (g->ring_stream) cudaStreamSynchronize(g->ring_stream);
  if (g->ring_comm) ncclCommDestroy(g->ring_comm);
  if (g->comm) ncclCommDestroy(g->comm);
  if (g->ready) cudaEventDestroy(g->ready);
  if (g->stream) cudaStreamDestroy(g->stream);
  if (g->ring_stream) cudaStreamDestroy(g->ring_stream);
  delete g;
}
