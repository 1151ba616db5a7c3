// Asynchronous work handle with a watchdog: a CUDA event recorded after a piece of stream work, plus
// a wall-clock deadline.  query()/wait() mirror the reference `Work` (process_group/CpuSync_fixed.hpp:
// 89-187: lazily created event, stream-side wait, host-side poll); what the reference left commented
// out -- the timeout watcher (process_group/processGroupNCCL.cpp:719-744) -- is implemented here: a
// background thread polls registered handles and marks a handle TIMED_OUT when its deadline passes,
// so the owner can tear down (abort the communicator, raise) instead of hanging forever.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

#include "../kernels/host_utils.h"

using namespace cpb;

namespace {
using Clock = std::chrono::steady_clock;
enum : int { W_PENDING = 0, W_DONE = 1, W_TIMED_OUT = 2, W_ERROR = 3 };

struct Work {
  cudaEvent_t ev = nullptr;
  std::atomic<int> state{W_PENDING};
  Clock::time_point deadline;
  bool has_deadline = false;
};

struct Watchdog {
  std::mutex mu;
  std::condition_variable cv;
  std::vector<Work*> live;
  std::thread th;
  bool stop = false;
  std::atomic<long> timeouts{0};

  void run() {
    std::unique_lock<std::mutex> lk(mu);
    while (!stop) {
      cv.wait_for(lk, std::chrono::milliseconds(20));
      const auto now = Clock::now();
      for (Work* w : live) {
        if (w->state.load() != W_PENDING) continue;
        // a handle without an event is completed explicitly by its owner (cpb_work_complete)
        cudaError_t e = w->ev ? cudaEventQuery(w->ev) : cudaErrorNotReady;
        if (e == cudaSuccess) w->state.store(W_DONE);
        else if (e != cudaErrorNotReady) { cudaGetLastError(); w->state.store(W_ERROR); }
        else if (w->has_deadline && now > w->deadline) { w->state.store(W_TIMED_OUT); timeouts++; }
      }
    }
  }
  void add(Work* w) {
    std::lock_guard<std::mutex> g(mu);
    if (!th.joinable()) th = std::thread([this] { run(); });
    live.push_back(w);
  }
  void remove(Work* w) {
    std::lock_guard<std::mutex> g(mu);
    for (size_t i = 0; i < live.size(); ++i) if (live[i] == w) { live[i] = live.back(); live.pop_back(); break; }
  }
  ~Watchdog() {
    { std::lock_guard<std::mutex> g(mu); stop = true; }
    cv.notify_all();
    if (th.joinable()) th.join();
  }
};
Watchdog& dog() { static Watchdog d; return d; }
}  // namespace

// Record an event on `stream` (may be null for a host-only handle) and register it with the watchdog.
extern "C" int cpb_work_create(cudaStream_t stream, int with_event, double timeout_s, void** out) {
  auto* w = new Work();
  if (with_event) {
    cudaError_t e = cudaEventCreateWithFlags(&w->ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(w->ev, stream);
    if (e != cudaSuccess) { delete w; return set_error(CPB_ERR_CUDA, "work_create: %s", cudaGetErrorString(e)); }
  }
  if (timeout_s > 0) { w->has_deadline = true; w->deadline = Clock::now() + std::chrono::microseconds((long)(timeout_s * 1e6)); }
  dog().add(w);
  *out = w;
  return CPB_OK;
}
// 0 pending, 1 done, 2 timed out, 3 error
extern "C" int cpb_work_query(void* h) { return ((Work*)h)->state.load(); }
// Host-only handles are completed explicitly.
extern "C" void cpb_work_complete(void* h) { int exp = W_PENDING; ((Work*)h)->state.compare_exchange_strong(exp, W_DONE); }
// Make `stream` wait for the work (device-side, no host block).
extern "C" int cpb_work_stream_wait(void* h, cudaStream_t stream) {
  auto* w = (Work*)h;
  if (!w->ev) return CPB_OK;
  cudaError_t e = cudaStreamWaitEvent(stream, w->ev, 0);
  if (e != cudaSuccess) return set_error(CPB_ERR_CUDA, "work_stream_wait: %s", cudaGetErrorString(e));
  return CPB_OK;
}
// Block the host until done / timed out / error; returns the final state.
extern "C" int cpb_work_wait(void* h, double poll_s) {
  auto* w = (Work*)h;
  for (;;) {
    int s = w->state.load();
    if (s != W_PENDING) return s;
    std::this_thread::sleep_for(std::chrono::microseconds((long)((poll_s > 0 ? poll_s : 0.001) * 1e6)));
  }
}
extern "C" void cpb_work_destroy(void* h) {
  auto* w = (Work*)h;
  dog().remove(w);
  if (w->ev) cudaEventDestroy(w->ev);
  delete w;
}
extern "C" long cpb_watchdog_timeouts() { return dog().timeouts.load(); }
