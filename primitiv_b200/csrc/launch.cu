// Worker thread of the launch queue and the context-level switches of the launch policy (launch.h).
#include "ctx.h"

namespace b200 {

LaunchQueue::LaunchQueue(int device) : slots_(new Slot[kSlots]) {
  worker_ = std::thread([this, device] { loop(device); });
}

LaunchQueue::~LaunchQueue() {
  drain();
  stop_.store(true, std::memory_order_release);
  wake();
  if (worker_.joinable()) worker_.join();
  delete[] slots_;
}

void LaunchQueue::wake() {
  std::lock_guard<std::mutex> lock(mu_);
  cv_.notify_one();
}

void LaunchQueue::loop(int device) {
  cudaSetDevice(device);
  unsigned idle = 0;
  for (;;) {
    const std::uint64_t at = tail_.load(std::memory_order_relaxed);
    if (at != head_.load(std::memory_order_acquire)) {
      Slot &sl = slots_[at % kSlots];
      sl.run(sl.payload);
      tail_.store(at + 1, std::memory_order_release);
      idle = 0;
      continue;
    }
    if (stop_.load(std::memory_order_acquire)) return;
    if (++idle < 20000u) {   // a few tens of microseconds of polling, then sleep until the next push
      cpu_relax();
      continue;
    }
    std::unique_lock<std::mutex> lock(mu_);
    sleeping_.store(true, std::memory_order_release);
    cv_.wait_for(lock, std::chrono::milliseconds(50), [this] {
      return stop_.load(std::memory_order_acquire) ||
             tail_.load(std::memory_order_relaxed) != head_.load(std::memory_order_acquire);
    });
    sleeping_.store(false, std::memory_order_release);
    idle = 0;
  }
}

LaunchQueue *active_queue(b200_ctx *ctx) {
  return (ctx->async && ctx->queue && !ctx->profiling && ctx->inline_depth == 0) ? ctx->queue : nullptr;
}

void queue_drain(b200_ctx *ctx) {
  if (ctx->queue) ctx->queue->drain();
}

bool ctx_pdl(const b200_ctx *ctx) { return ctx->pdl; }

void count_launch_error(b200_ctx *ctx, cudaError_t e) {
  if (e != cudaSuccess && ctx->launch_error == 0) ctx->launch_error = static_cast<int>(e);
}

}  // namespace b200
