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
#include <cstring>

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
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();  // clear the sticky-less error so later calls start clean
    return B200_ERR_OUT_OF_MEMORY;
  }
  if (e != cudaSuccess) return (int)e;
  ++n_malloc_;
  return B200_OK;
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
    for (void *p : kv.second) cudaFree(p);
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
    for (void *p : kv.second) cudaFree(p);
  for (auto &kv : in_use_) cudaFree(kv.first);
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

int StagingRing::upload(void *dst, const void *src, std::size_t bytes, cudaStream_t stream) {
  int rc = prepare();
  if (rc != B200_OK) return rc;
  const char *from = static_cast<const char *>(src);
  char *to = static_cast<char *>(dst);
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
  if (!base_) return;
  drain();
  for (int i = 0; i < kSlots; ++i) cudaEventDestroy(events_[i]);
  cudaFreeHost(base_);
}

}  // namespace b200
