// Internal context shared by the translation units of libprimitiv_b200.so.
#ifndef PRIMITIV_B200_CSRC_CTX_H_
#define PRIMITIV_B200_CSRC_CTX_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <unordered_map>
#include <vector>

#include "../../include/primitiv_b200.h"
#include "launch.h"

namespace b200 {

// Caching device-memory pool.  Size classes are geometric with four steps per
// octave (1, 1.25, 1.5, 1.75 x 2^e), 256-byte granularity below 1 KiB.  All
// blocks are handed out and reused in stream order on the caller's single
// stream, so no event tracking is needed (the contract of primitiv::Device is
// one host thread and one stream per device).
class Pool {
 public:
  Pool() = default;
  ~Pool();
  int alloc(std::size_t bytes, void **ptr, std::size_t *allocated);
  int free(void *ptr);
  void release_cached();
  void stats(std::uint64_t out[4]) const;
  // Test hook: a soft capacity (0 = none).  Requests that would push
  // in-use + cached bytes past it behave exactly like a failed cudaMalloc.
  void set_limit(std::size_t bytes) { limit_ = bytes; }
  static std::size_t size_class(std::size_t bytes);
  // Debug aid: `bytes` (rounded up to 256) of a known pattern in front of and behind every block,
  // checked by pool_check_guards().  Only while the pool holds no block at all.
  int set_guard(std::size_t bytes);
  std::size_t guard() const { return guard_; }
  // Every block the pool owns, handed out or cached: (pointer the caller sees, class size).
  void blocks(std::vector<std::pair<void *, std::size_t>> *out) const;
  static constexpr unsigned char kGuardByte = 0xA5;
  // Called with (block, bytes) whenever a block goes back to the pool: whatever was derived from
  // its contents (cached operand planes) is stale from then on.
  std::function<void(const void *, std::size_t)> on_free;
  // Called before cached blocks are handed back to the driver: the context uses it to issue
  // launches that are still waiting in its launch queue and may read those blocks.
  std::function<void()> before_release;

 private:
  std::map<std::size_t, std::vector<void *>> cached_;
  std::unordered_map<void *, std::size_t> in_use_;
  std::size_t bytes_in_use_ = 0, bytes_cached_ = 0, limit_ = 0, guard_ = 0;
  std::uint64_t n_malloc_ = 0, n_hit_ = 0;
  int raw_alloc(std::size_t bytes, void **ptr);
};

typedef CUresult (*EncodeTiledFn)(
    CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace b200

namespace b200 {

// Pinned staging ring for host-to-device copies of caller memory that may be pageable.
// A copy from pageable memory makes the CUDA runtime wait for the stream first; staging
// through pinned slots keeps uploads asynchronous: the host copies into a slot, queues the
// DMA and an event, and only waits when it comes round to a slot whose DMA is still pending.
//
// One core copies into pinned memory at 8-9 GB/s, a sixth of what the bus then moves.  An upload
// of kGangBytes or more is therefore staged half a ring at a time with a few helper threads
// copying side by side (started on first use, asleep otherwise), while the DMA of the other half
// is in flight.
class CopyGang;
class StagingRing {
 public:
  static constexpr std::size_t kSlotBytes = 1u << 20;
  static constexpr int kSlots = 16;
  static constexpr std::size_t kGangBytes = 8u << 20;
  ~StagingRing();
  // dst (device) <- src (host, any kind), bytes; ordered on `stream`.  The source may be
  // reused as soon as this returns.
  int upload(void *dst, const void *src, std::size_t bytes, cudaStream_t stream);
  // waits for every pending DMA out of the ring
  void drain();
  // Called before each copy is queued on the stream (the context lets its launch queue catch up).
  std::function<void()> before_copy;

 private:
  char *base_ = nullptr;
  cudaEvent_t events_[kSlots] = {};
  bool pending_[kSlots] = {};
  int next_ = 0;
  CopyGang *gang_ = nullptr;
  int prepare();
  int upload_wave(char *to, const char *from, std::size_t bytes, cudaStream_t stream);
};

}  // namespace b200

namespace b200 {

// Cache of packed operand planes (fp32 mode).  An entry maps a dense source range of the caller's
// memory to the block that holds its three planes in the source's own layout.  Entries live
// while the cache is enabled (b200_operand_cache_enable) or while an entry point that uses an
// operand more than once is running (scope > 0), and die when their source range is written
// (b200_operand_cache_invalidate), returned to the pool, or evicted to stay under the byte cap.
struct PlaneCache {
  struct Entry {
    const void *src;
    std::size_t src_bytes;
    void *block;
    std::size_t block_bytes;
    std::uint64_t stamp;
  };
  std::vector<Entry> entries;
  std::size_t bytes = 0, cap = 0;   // cap == 0: not enabled by the caller
  int scope = 0;                    // > 0 inside an entry point that shares planes between its products
  std::uint64_t clock = 0, hits = 0, misses = 0;
  bool active() const { return cap != 0 || scope > 0; }
};

}  // namespace b200

struct b200_ctx {
  int device = 0;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  std::size_t smem_optin = 0;
  b200::Pool pool;
  // Status word of the bounded device-side waits.  It lives in pinned host memory that the
  // GPU writes through a mapped alias (d_status): a kernel whose wait ran out stores its code
  // there, and the host reads it after any synchronisation without another copy.
  int *h_status = nullptr;       // host address
  int *d_status = nullptr;       // the same word as the kernels address it
  b200::EncodeTiledFn encode_tiled = nullptr;
  std::uint64_t launches = 0;
  bool tc_smem_configured = false;
  int path_policy = 0;           // 0 = choose per problem, 1 = CUDA-core kernel, 2 = tensor-core kernel when eligible
  int debug_stage_cap = 0;       // development: cap on pipeline stages (0 = none)
  int pair_policy = 0;           // see b200_set_pair_policy
  int split_policy = 0;          // 0 = split k over idle CTAs when there are few output tiles, 1 = never
  int correction_policy = 0;     // fp32 mode: 0 = correction passes on the bf16 pipe, flat planes where possible;
                                 // 1 = TF32 planes throughout; 2 = bf16 correction passes, operands always repacked K-major
  std::uint64_t rng_seed = 0, rng_calls = 0;  // Philox key and fill counter (b200_seed / b200_random)
  // optional per-launch timing (b200_profile_*): event pairs, summed when read
  bool profiling = false;
  struct ProfRec { cudaEvent_t start, stop; int kind; };
  std::vector<ProfRec> prof;
  // host-buffer entry points (b200_matmul_*_host): upload, compute and download streams
  // and the events that chain them, created on first use
  b200::StagingRing staging;     // uploads of host arrays (tensor contents, index lists)
  cudaStream_t pipe_streams[3] = {nullptr, nullptr, nullptr};
  std::vector<cudaEvent_t> pipe_events;
  cudaEvent_t barrier_event = nullptr;  // b200_stream_barrier: marks this GPU's default stream
  b200::PlaneCache planes;
  // launch policy (launch.h): programmatic dependent launch on every kernel; kernel launches issued
  // by a worker thread when the caller has asked for it
  bool pdl = true;
  bool async = false;
  int inline_depth = 0;            // > 0 inside an entry point that interleaves launches with other stream work
  b200::LaunchQueue *queue = nullptr;
  int launch_error = 0;            // first error of a launch issued on the caller's thread
};

namespace b200 {

// RAII device guard: every entry point makes its context's device current, as
// the reference does with cudaSetDevice at the top of every op
// (primitiv/devices/cuda/ops/matmul.cu:33), and restores the previous one.
struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

// Kernel kinds for b200_profile_read.
enum { kProfGemmTc = 0, kProfPack = 1, kProfGemmSimt = 2, kProfElementwise = 3, kProfKinds = 4 };

// Brackets one kernel launch with CUDA events on its stream when profiling is on.
struct ProfScope {
  b200_ctx *ctx;
  cudaStream_t stream;
  cudaEvent_t stop = nullptr;
  ProfScope(b200_ctx *c, int kind, cudaStream_t s) : ctx(c), stream(s) {
    if (!c->profiling) return;
    queue_drain(c);  // (launches are not deferred while profiling; this covers the moment it is switched on)
    cudaEvent_t start;
    if (cudaEventCreate(&start) != cudaSuccess) return;
    if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start); stop = nullptr; return; }
    cudaEventRecord(start, s);
    c->prof.push_back({start, stop, kind});
  }
  ~ProfScope() { if (stop) cudaEventRecord(stop, stream); }
};

struct GemmArgs {
  int mode;
  int trans_a, trans_b;
  const void *A, *B;
  void *C;
  std::uint32_t m, n, k, groups, red;
  std::uint64_t a_gs, a_rs, b_gs, b_rs, c_gs;
  int accumulate;
};

// CUDA-core path: any shape, any alignment.
int gemm_simt(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream);
// CUDA-core kernels for products with one tiny extent against large ones (gemm_skinny.cu).
bool gemm_skinny_eligible(const GemmArgs &g);
int gemm_skinny(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream);
// tcgen05 path.  tc_eligible() says whether the operands meet TMA's alignment rules.
bool gemm_tc_eligible(const b200_ctx *ctx, const GemmArgs &g);
int gemm_tc(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream);
// Checks (and re-arms) the guard bands of every pool block; see b200_pool_check_guards.
int pool_check_guards(b200_ctx *ctx, cudaStream_t stream, std::uint64_t *damaged, void **first, int *side);
// Streams L2-resident data into every SM's shared memory and reports the rate; see b200_measure_l2_ingest.
int measure_l2_ingest(b200_ctx *ctx, cudaStream_t stream, double *bytes_per_clock_per_sm, double *gb_per_s_per_sm);
// Launches a kernel whose only wait runs out (see b200_selftest_wait_timeout).
int selftest_wait_timeout(b200_ctx *ctx, cudaStream_t stream);
// 3xTF32 product whose packing planes live in a fixed device array: allocates nothing.
int gemm_3xtf32_noalloc(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream);

// Operand-plane cache (see PlaneCache).  drop_range forgets every entry whose source overlaps
// [ptr, ptr + bytes) (everything when ptr is null) and returns its block to the pool.
void plane_cache_drop_range(b200_ctx *ctx, const void *ptr, std::size_t bytes);
// Brackets an entry point that hands the same operand to several products.
struct PlaneScope {
  b200_ctx *ctx;
  explicit PlaneScope(b200_ctx *c) : ctx(c) { ++ctx->planes.scope; }
  ~PlaneScope() {
    if (--ctx->planes.scope == 0 && ctx->planes.cap == 0) plane_cache_drop_range(ctx, nullptr, 0);
  }
};

inline int elem_bytes(int mode) { return mode == B200_MODE_FP16 ? 2 : 4; }

// Reads and clears the status word.  Meaningful once the work that may have written it has
// been waited for; every entry point that synchronises calls this and returns the code, which is
// how a wait that ran out becomes an error of the next host-visible result.
// First error of a kernel launch since the last call (launches return nothing to their entry
// point once a worker thread issues them); cleared by the read.  Call after queue_drain.
inline int take_launch_error(b200_ctx *ctx) {
  int e = ctx->launch_error;
  ctx->launch_error = 0;
  if (ctx->queue) {
    const int q = ctx->queue->take_error();
    if (e == 0) e = q;
  }
  return e;
}

inline int take_status(b200_ctx *ctx) {
  volatile int *w = ctx->h_status;
  const int code = *w;
  if (code != 0) *w = 0;
  return code;
}

#ifdef __CUDACC__
// Device side of the same word: a plain store through the mapped alias (every writer stores the
// same kind of code, so no atomic is needed), made visible to the host before the kernel ends.
__device__ __forceinline__ void report_status(int *status, int code) {
  *reinterpret_cast<volatile int *>(status) = code;
  __threadfence_system();
}
#endif

}  // namespace b200

namespace b200 {
// Marks an entry point that mixes kernel launches with copies, events or several streams: launches
// inside it are issued on the caller's thread, after the worker has caught up.
struct InlineLaunches {
  b200_ctx *ctx;
  explicit InlineLaunches(b200_ctx *c) : ctx(c) {
    queue_drain(c);
    ++c->inline_depth;
  }
  ~InlineLaunches() { --ctx->inline_depth; }
};
}  // namespace b200

#define B200_CUDA_TRY(expr)                     \
  do {                                          \
    cudaError_t e__ = (expr);                   \
    if (e__ != cudaSuccess) return (int)e__;    \
  } while (0)

#endif  // PRIMITIV_B200_CSRC_CTX_H_
