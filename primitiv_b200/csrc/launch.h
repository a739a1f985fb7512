// How every kernel of this library is launched.
//
// Two things hang on the one helper below.
//
// 1. Programmatic dependent launch.  Each kernel begins with pdl_enter(): it lets the grid
//    queued behind it on the stream be scheduled at once (its CTAs take whatever room is free,
//    run their prologue and then block), and itself blocks until the grid in front of it has
//    finished and its writes are visible.  Launched with the programmatic-serialization
//    attribute, a chain of small kernels then overlaps each launch latency with its
//    predecessor's execution instead of paying it in between.  A kernel launched without the
//    attribute sees both instructions as no-ops.
//
// 2. The launch queue.  A graph-level step is thousands of 3 us kernels, and the host spends
//    about as long in the driver's launch call as the GPU spends on the kernel, on top of the
//    caller's own bookkeeping per operation.  With b200_set_async_launch(ctx, 1) the launch
//    call itself moves to a worker thread: the entry point does everything else on the caller's
//    thread as before (argument checks, pool and cache bookkeeping, tensor maps), copies the
//    kernel arguments into a ring slot and returns.  The worker issues the launches in order.
//    Everything that is not a kernel launch but is ordered on the stream (copies, memsets,
//    events, synchronisation) first waits for the worker to catch up (queue_drain) and then
//    runs on the caller's thread, so stream order is program order, exactly as without the queue.
#ifndef PRIMITIV_B200_CSRC_LAUNCH_H_
#define PRIMITIV_B200_CSRC_LAUNCH_H_

#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>
#include <chrono>
#include <thread>
#include <tuple>
#include <type_traits>
#include <utility>

namespace b200 {

#ifdef __CUDACC__
// First statement of every kernel (see above).  Must precede any access to global memory.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// The two halves, for a kernel whose set-up (barriers, tensor memory) needs no global data and
// can run while the grid in front is still working.
__device__ __forceinline__ void pdl_release_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_previous() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// Single-producer single-consumer ring of small closures, executed in order by one worker thread.
class LaunchQueue {
 public:
  static constexpr std::size_t kPayload = 4096 - 2 * sizeof(void *);  // the largest kernel argument block is ~2.5 KB
  static constexpr std::uint64_t kSlots = 1024;

  explicit LaunchQueue(int device);
  ~LaunchQueue();
  LaunchQueue(const LaunchQueue &) = delete;
  LaunchQueue &operator=(const LaunchQueue &) = delete;

  // Copies f into the ring (blocks while the ring is full); the worker calls it later.
  template <class F>
  void push(const F &f) {
    static_assert(sizeof(F) <= kPayload, "closure too large for a ring slot");
    static_assert(std::is_trivially_copyable<F>::value || std::is_copy_constructible<F>::value, "closure must be copyable");
    const std::uint64_t at = head_.load(std::memory_order_relaxed);
    while (at - tail_.load(std::memory_order_acquire) >= kSlots) cpu_relax();
    Slot &sl = slots_[at % kSlots];
    new (sl.payload) F(f);
    sl.run = [](void *p) {
      F *g = static_cast<F *>(p);
      (*g)();
      g->~F();
    };
    head_.store(at + 1, std::memory_order_release);
    if (sleeping_.load(std::memory_order_acquire)) wake();
  }

  // Returns when the worker has executed everything pushed so far.
  void drain() {
    const std::uint64_t want = head_.load(std::memory_order_relaxed);
    while (tail_.load(std::memory_order_acquire) < want) cpu_relax();
  }
  bool idle() const { return tail_.load(std::memory_order_acquire) == head_.load(std::memory_order_relaxed); }

  // First CUDA error a queued launch returned (0 if none); cleared by the read.
  int take_error() { return error_.exchange(0, std::memory_order_acq_rel); }
  void note_error(int code) {
    int none = 0;
    if (code != 0) error_.compare_exchange_strong(none, code, std::memory_order_acq_rel);
  }

 private:
  struct Slot {
    void (*run)(void *);
    void *pad;
    alignas(16) unsigned char payload[kPayload];
  };
  static void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#else
    std::this_thread::yield();
#endif
  }
  void loop(int device);
  void wake();

  Slot *slots_;
  std::atomic<std::uint64_t> head_{0}, tail_{0};
  std::atomic<bool> sleeping_{false}, stop_{false};
  std::atomic<int> error_{0};
  std::mutex mu_;
  std::condition_variable cv_;
  std::thread worker_;
};

}  // namespace b200

struct b200_ctx;

namespace b200 {

// The queue of a context if launches are being deferred right now, else null.
LaunchQueue *active_queue(b200_ctx *ctx);
// Before anything that is ordered on a stream but is not a kernel launch: let the worker catch up.
void queue_drain(b200_ctx *ctx);
bool ctx_pdl(const b200_ctx *ctx);
void count_launch_error(b200_ctx *ctx, cudaError_t e);

namespace detail {

template <typename Tuple, std::size_t... I>
inline cudaError_t launch_tuple(const void *kernel, const cudaLaunchConfig_t &cfg, Tuple &args, std::index_sequence<I...>) {
  void *ptrs[sizeof...(I) + 1] = {static_cast<void *>(&std::get<I>(args))..., nullptr};
  return cudaLaunchKernelExC(&cfg, kernel, ptrs);
}

}  // namespace detail

// kernel<<<grid, block, smem, stream>>>(args...) with the library's launch policy.  cluster_x > 1
// launches thread-block clusters of that many CTAs along x.
template <typename... KArgs, typename... Args>
inline void launch(b200_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, std::size_t smem, cudaStream_t stream,
                   unsigned cluster_x, Args &&...args) {
  static_assert(sizeof...(KArgs) == sizeof...(Args), "argument count does not match the kernel");
  std::tuple<typename std::decay<KArgs>::type...> pack{static_cast<typename std::decay<KArgs>::type>(args)...};
  const bool pdl = ctx_pdl(ctx);
  const void *fn = reinterpret_cast<const void *>(kernel);
  auto issue = [=]() mutable -> cudaError_t {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_x > 1) {
      attr[n].id = cudaLaunchAttributeClusterDimension;
      attr[n].val.clusterDim.x = cluster_x;
      attr[n].val.clusterDim.y = 1;
      attr[n].val.clusterDim.z = 1;
      ++n;
    }
    if (pdl) {
      attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return detail::launch_tuple(fn, cfg, pack, std::index_sequence_for<KArgs...>{});
  };
  if (LaunchQueue *q = active_queue(ctx)) {
    q->push([=]() mutable { q->note_error(static_cast<int>(issue())); });
  } else {
    count_launch_error(ctx, issue());
  }
}

}  // namespace b200

#endif  // PRIMITIV_B200_CSRC_LAUNCH_H_
