// Caching device-memory pool of the B200 backend.
//
// Plays the part of primitiv::MemoryPool (primitiv/core/memory_pool.cc:35-94) for
// this backend, with two deliberate differences: size classes are finer than
// powers of two (a 205 MB tensor takes a 224 MiB block, not 256 MiB), and the
// free lists are keyed by exact class size in an ordered map rather than by 64
// fixed bins.  The behaviour the reference's tests pin is kept: a freed block is
// handed back for the next request of the same class (same pointer), and when the
// device allocator fails every cached block is released and the request retried
// once before giving up.
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>

#include "ctx.h"

namespace b200 {

std::size_t Pool::size_class(std::size_t bytes) {
  if (bytes <= 256) return 256;
  if (bytes <= 1024) return (bytes + 255) & ~std::size_t(255);
  // smallest  q * 2^(e-2), q in {4,5,6,7}, that is >= bytes
  int e = 63 - __builtin_clzll((unsigned long long)bytes);
  std::size_t step = std::size_t(1) << (e - 2);
  std::size_t c = (bytes + step - 1) & ~(step - 1);
  return c;
}

int Pool::raw_alloc(std::size_t bytes, void **ptr) {
  if (limit_ && bytes_in_use_ + bytes_cached_ + bytes > limit_) return B200_ERR_OUT_OF_MEMORY;
  char *base = nullptr;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&base), bytes + 2 * guard_);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();  // clear the sticky-less error so later calls start clean
    return B200_ERR_OUT_OF_MEMORY;
  }
  if (e != cudaSuccess) return (int)e;
  if (guard_) {
    // nothing legitimate ever touches these bytes, so the order against the streams is free;
    // the wait only makes sure the pattern is there before the first check looks for it
    cudaMemset(base, kGuardByte, guard_);
    cudaMemset(base + guard_ + bytes, kGuardByte, guard_);
    cudaStreamSynchronize(nullptr);
  }
  *ptr = base + guard_;
  ++n_malloc_;
  return B200_OK;
}

int Pool::set_guard(std::size_t bytes) {
  if (!in_use_.empty()) return B200_ERR_INVALID_ARG;
  release_cached();
  guard_ = (bytes + 255) & ~std::size_t(255);
  return B200_OK;
}

void Pool::blocks(std::vector<std::pair<void *, std::size_t>> *out) const {
  out->clear();
  for (const auto &kv : in_use_) out->emplace_back(kv.first, kv.second);
  for (const auto &kv : cached_)
    for (void *p : kv.second) out->emplace_back(p, kv.first);
}

int Pool::alloc(std::size_t bytes, void **ptr, std::size_t *allocated) {
  if (!ptr) return B200_ERR_INVALID_ARG;
  const std::size_t cls = size_class(bytes ? bytes : 1);
  auto it = cached_.find(cls);
  if (it != cached_.end() && !it->second.empty()) {
    *ptr = it->second.back();
    it->second.pop_back();
    bytes_cached_ -= cls;
    ++n_hit_;
  } else {
    int rc = raw_alloc(cls, ptr);
    if (rc == B200_ERR_OUT_OF_MEMORY) {
      release_cached();
      rc = raw_alloc(cls, ptr);
    }
    if (rc != B200_OK) return rc;
  }
  in_use_[*ptr] = cls;
  bytes_in_use_ += cls;
  if (allocated) *allocated = cls;
  return B200_OK;
}

int Pool::free(void *ptr) {
  if (!ptr) return B200_OK;
  auto it = in_use_.find(ptr);
  if (it == in_use_.end()) return B200_ERR_INVALID_ARG;
  const std::size_t cls = it->second;
  in_use_.erase(it);
  bytes_in_use_ -= cls;
  if (on_free) on_free(ptr, cls);   // may free further blocks (planes derived from this one)
  cached_[cls].push_back(ptr);
  bytes_cached_ += cls;
  return B200_OK;
}

void Pool::release_cached() {
  bool any = false;
  for (auto &kv : cached_) any = any || !kv.second.empty();
  if (!any) return;
  if (before_release) before_release();   // launches a worker thread has not issued yet
  cudaDeviceSynchronize();  // cached blocks may still be read by queued kernels
  for (auto &kv : cached_) {
    for (void *p : kv.second) cudaFree(static_cast<char *>(p) - guard_);
    kv.second.clear();
  }
  bytes_cached_ = 0;
}

void Pool::stats(std::uint64_t out[4]) const {
  out[0] = bytes_in_use_;
  out[1] = bytes_cached_;
  out[2] = n_malloc_;
  out[3] = n_hit_;
}

Pool::~Pool() {
  // Everything goes back to the driver, blocks still handed out included: a tensor may
  // outlive its device (garbage-collected bindings), and its handle then only needs to be
  // safe to drop, not to use (primitiv/core/memory_pool.cc:18-33 does the same).
  for (auto &kv : cached_)
    for (void *p : kv.second) cudaFree(static_cast<char *>(p) - guard_);
  for (auto &kv : in_use_) cudaFree(static_cast<char *>(kv.first) - guard_);
}

}  // namespace b200

// ---------------------------------------------------------------------------------
// StagingRing

namespace b200 {

int StagingRing::prepare() {
  if (base_) return B200_OK;
  void *p = nullptr;
  cudaError_t e = cudaHostAlloc(&p, kSlotBytes * kSlots, cudaHostAllocDefault);
  if (e != cudaSuccess) return static_cast<int>(e);
  for (int i = 0; i < kSlots; ++i) {
    e = cudaEventCreateWithFlags(&events_[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(events_[j]);
      cudaFreeHost(p);
      return static_cast<int>(e);
    }
  }
  base_ = static_cast<char *>(p);
  return B200_OK;
}

// A few threads that run a list of memcpy jobs side by side with the calling thread.
class CopyGang {
 public:
  struct Job {
    void *dst;
    const void *src;
    std::size_t bytes;
  };
  explicit CopyGang(int helpers) {
    for (int i = 0; i < helpers; ++i) threads_.emplace_back([this] { loop(); });
  }
  ~CopyGang() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      stop_ = true;
    }
    wake_.notify_all();
    for (std::thread &t : threads_) t.join();
  }
  // Returns when every job has been copied.
  void run(const Job *jobs, int n) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      jobs_ = jobs;
      n_jobs_ = n;
      next_.store(0, std::memory_order_relaxed);
      busy_ = static_cast<int>(threads_.size());
      ++epoch_;
    }
    wake_.notify_all();
    work();
    std::unique_lock<std::mutex> lock(mu_);
    done_.wait(lock, [this] { return busy_ == 0; });
  }

 private:
  void work() {
    for (;;) {
      const int i = next_.fetch_add(1, std::memory_order_relaxed);
      if (i >= n_jobs_) return;
      std::memcpy(jobs_[i].dst, jobs_[i].src, jobs_[i].bytes);
    }
  }
  void loop() {
    std::uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lock(mu_);
        wake_.wait(lock, [&] { return stop_ || epoch_ != seen; });
        if (stop_) return;
        seen = epoch_;
      }
      work();
      std::lock_guard<std::mutex> lock(mu_);
      if (--busy_ == 0) done_.notify_one();
    }
  }
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable wake_, done_;
  const Job *jobs_ = nullptr;
  int n_jobs_ = 0, busy_ = 0;
  std::atomic<int> next_{0};
  std::uint64_t epoch_ = 0;
  bool stop_ = false;
};

// Half a ring at a time: wait for those slots' previous DMAs, fill them in parallel, queue their DMAs.
int StagingRing::upload_wave(char *to, const char *from, std::size_t bytes, cudaStream_t stream) {
  constexpr int kWave = kSlots / 2;
  if (!gang_) {
    const unsigned cores = std::thread::hardware_concurrency();
    gang_ = new CopyGang(cores >= 8 ? 3 : (cores >= 4 ? 1 : 0));
  }
  while (bytes > 0) {
    const int first = next_ < kWave ? 0 : kWave;   // a wave never straddles the two halves
    CopyGang::Job jobs[kWave];
    int n_jobs = 0;
    std::size_t taken = 0;
    for (int s = first; s < first + kWave && taken < bytes; ++s) {
      if (pending_[s]) {
        const cudaError_t e = cudaEventSynchronize(events_[s]);
        if (e != cudaSuccess) return static_cast<int>(e);
        pending_[s] = false;
      }
      const std::size_t n = bytes - taken < kSlotBytes ? bytes - taken : kSlotBytes;
      jobs[n_jobs++] = CopyGang::Job{base_ + static_cast<std::size_t>(s) * kSlotBytes, from + taken, n};
      taken += n;
    }
    gang_->run(jobs, n_jobs);
    if (before_copy) before_copy();
    std::size_t done = 0;
    for (int j = 0; j < n_jobs; ++j) {
      const int s = first + j;
      cudaError_t e = cudaMemcpyAsync(to + done, jobs[j].dst, jobs[j].bytes, cudaMemcpyHostToDevice, stream);
      if (e == cudaSuccess) e = cudaEventRecord(events_[s], stream);
      if (e != cudaSuccess) return static_cast<int>(e);
      pending_[s] = true;
      done += jobs[j].bytes;
    }
    next_ = first == 0 ? kWave : 0;
    from += taken;
    to += taken;
    bytes -= taken;
  }
  return B200_OK;
}

int StagingRing::upload(void *dst, const void *src, std::size_t bytes, cudaStream_t stream) {
  int rc = prepare();
  if (rc != B200_OK) return rc;
  const char *from = static_cast<const char *>(src);
  char *to = static_cast<char *>(dst);
  if (bytes >= kGangBytes) return upload_wave(to, from, bytes, stream);
  while (bytes > 0) {
    const std::size_t n = bytes < kSlotBytes ? bytes : kSlotBytes;
    const int slot = next_;
    next_ = (next_ + 1) % kSlots;
    if (pending_[slot]) {
      const cudaError_t e = cudaEventSynchronize(events_[slot]);
      if (e != cudaSuccess) return static_cast<int>(e);
      pending_[slot] = false;
    }
    char *stage = base_ + static_cast<std::size_t>(slot) * kSlotBytes;
    std::memcpy(stage, from, n);
    if (before_copy) before_copy();   // stream order is program order: queued launches are issued first
    cudaError_t e = cudaMemcpyAsync(to, stage, n, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(events_[slot], stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    pending_[slot] = true;
    from += n;
    to += n;
    bytes -= n;
  }
  return B200_OK;
}

void StagingRing::drain() {
  if (!base_) return;
  for (int i = 0; i < kSlots; ++i) {
    if (pending_[i]) cudaEventSynchronize(events_[i]);
    pending_[i] = false;
  }
}

StagingRing::~StagingRing() {
  delete gang_;
  if (!base_) return;
  drain();
  for (int i = 0; i < kSlots; ++i) cudaEventDestroy(events_[i]);
  cudaFreeHost(base_);
}

}  // namespace b200
