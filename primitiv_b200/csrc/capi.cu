// extern "C" entry points of libprimitiv_b200.so: context, pool, and the mapping of
// primitiv's matmul_fw / matmul_bw onto the general contraction.
#include <cstdio>
#include <cstring>
#include <new>

#include <nvtx3/nvToolsExt.h>

#include "ctx.h"

using b200::DeviceGuard;
using b200::GemmArgs;

namespace {

// NVTX range round one product (packing, the kernel, a split-k reduction), named by its shape,
// so that a timeline shows which launches belong to which matmul_fw / matmul_bw call.  The
// header-only NVTX does nothing but test a pointer unless a profiler has attached itself.
struct GemmRange {
  GemmRange(int mode, int ta, int tb, uint32_t m, uint32_t n, uint32_t k, uint32_t groups, uint32_t red, int acc) {
    char name[96];
    std::snprintf(name, sizeof(name), "b200_gemm %s%s %ux%ux%u g%u r%u mode%d%s", ta ? "T" : "N", tb ? "T" : "N", m, n, k,
                  groups, red, mode, acc ? " +=" : "");
    nvtxRangePushA(name);
  }
  ~GemmRange() { nvtxRangePop(); }
};

}  // namespace

extern "C" {

const char *b200_error_string(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_ERR_INVALID_ARG: return "primitiv_b200: invalid argument";
    case B200_ERR_NO_DEVICE: return "primitiv_b200: no CUDA device of compute capability 10.x (there is no CPU fallback)";
    case B200_ERR_OUT_OF_MEMORY: return "primitiv_b200: device memory exhausted (after releasing the pool's cached blocks)";
    case B200_ERR_KERNEL_TIMEOUT: return "primitiv_b200: a bounded device-side wait ran out";
    case B200_ERR_DRIVER: return "primitiv_b200: tensor-map encoding failed or driver entry point missing";
    case B200_ERR_TOO_LARGE: return "primitiv_b200: size beyond a documented maximum";
    default: break;
  }
  if (code > 0 && code < 1000) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "primitiv_b200: unknown error";
}

int b200_ctx_create(int device_id, b200_ctx **out) {
  if (!out) return B200_ERR_INVALID_ARG;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return B200_ERR_NO_DEVICE;
  }
  if (device_id < 0 || device_id >= n) return B200_ERR_INVALID_ARG;
  cudaDeviceProp prop;
  B200_CUDA_TRY(cudaGetDeviceProperties(&prop, device_id));
  if (prop.major != 10) return B200_ERR_NO_DEVICE;
  b200_ctx *ctx = new (std::nothrow) b200_ctx();
  if (!ctx) return B200_ERR_OUT_OF_MEMORY;
  ctx->device = device_id;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->cc_major = prop.major;
  ctx->cc_minor = prop.minor;
  ctx->smem_optin = prop.sharedMemPerBlockOptin;
  DeviceGuard guard(device_id);
  void *word = nullptr, *alias = nullptr;
  cudaError_t e = cudaHostAlloc(&word, 256, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) {
    memset(word, 0, 256);
    e = cudaHostGetDevicePointer(&alias, word, 0);
    if (e != cudaSuccess) cudaFreeHost(word);
  }
  if (e != cudaSuccess) {
    delete ctx;
    return static_cast<int>(e);
  }
  ctx->h_status = static_cast<int *>(word);
  ctx->d_status = static_cast<int *>(alias);
  // a block that returns to the pool takes the planes packed from its contents with it
  ctx->pool.on_free = [ctx](const void *p, std::size_t bytes) { b200::plane_cache_drop_range(ctx, p, bytes); };
  ctx->pool.before_release = [ctx]() { b200::queue_drain(ctx); };
  ctx->staging.before_copy = [ctx]() { b200::queue_drain(ctx); };
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess) {
    ctx->encode_tiled = reinterpret_cast<b200::EncodeTiledFn>(fn);
  } else {
    cudaGetLastError();
    cudaFreeHost(ctx->h_status);
    delete ctx;
    return B200_ERR_DRIVER;
  }
  *out = ctx;
  return B200_OK;
}

int b200_ctx_destroy(b200_ctx *ctx) {
  if (!ctx) return B200_OK;
  DeviceGuard guard(ctx->device);
  delete ctx->queue;   // issues what is still queued, then stops the worker
  ctx->queue = nullptr;
  cudaDeviceSynchronize();
  b200::plane_cache_drop_range(ctx, nullptr, 0);
  ctx->pool.on_free = nullptr;
  for (cudaStream_t st : ctx->pipe_streams) if (st) cudaStreamDestroy(st);
  for (cudaEvent_t ev : ctx->pipe_events) cudaEventDestroy(ev);
  if (ctx->barrier_event) cudaEventDestroy(ctx->barrier_event);
  cudaFreeHost(ctx->h_status);
  delete ctx;  // the pool's destructor returns cached blocks
  return B200_OK;
}

int b200_ctx_device(const b200_ctx *ctx, int *device_id, int *sm_count) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  if (device_id) *device_id = ctx->device;
  if (sm_count) *sm_count = ctx->sm_count;
  return B200_OK;
}

int b200_status_poll(b200_ctx *ctx, void *stream, int *code) {
  if (!ctx || !code) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  b200::queue_drain(ctx);
  B200_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  *code = b200::take_status(ctx);
  return b200::take_launch_error(ctx);
}

int b200_status_peek(b200_ctx *ctx, int *code) {
  if (!ctx || !code) return B200_ERR_INVALID_ARG;
  *code = b200::take_status(ctx);
  return B200_OK;
}

int b200_selftest_wait_timeout(b200_ctx *ctx, void *stream) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  return b200::selftest_wait_timeout(ctx, static_cast<cudaStream_t>(stream));
}

int b200_measure_l2_ingest(b200_ctx *ctx, void *stream, double *bytes_per_clock_per_sm, double *gb_per_s_per_sm) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  return b200::measure_l2_ingest(ctx, static_cast<cudaStream_t>(stream), bytes_per_clock_per_sm, gb_per_s_per_sm);
}

int b200_pool_alloc(b200_ctx *ctx, size_t bytes, void **ptr, size_t *allocated) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  return ctx->pool.alloc(bytes, ptr, allocated);
}

int b200_pool_free(b200_ctx *ctx, void *ptr) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  return ctx->pool.free(ptr);
}

int b200_pool_release_cached(b200_ctx *ctx) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  ctx->pool.release_cached();
  return B200_OK;
}

int b200_pool_stats(const b200_ctx *ctx, uint64_t stats[4]) {
  if (!ctx || !stats) return B200_ERR_INVALID_ARG;
  ctx->pool.stats(stats);
  return B200_OK;
}

size_t b200_pool_size_class(size_t bytes) { return b200::Pool::size_class(bytes ? bytes : 1); }

int b200_pool_set_limit(b200_ctx *ctx, size_t bytes) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  ctx->pool.set_limit(bytes);
  return B200_OK;
}

int b200_pool_set_guard(b200_ctx *ctx, size_t bytes) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  b200::plane_cache_drop_range(ctx, nullptr, 0);   // cached planes are pool blocks too
  return ctx->pool.set_guard(bytes);
}

int b200_pool_check_guards(b200_ctx *ctx, void *stream, uint64_t *damaged_blocks, void **first_block, int *side) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  return b200::pool_check_guards(ctx, static_cast<cudaStream_t>(stream), damaged_blocks, first_block, side);
}

int b200_set_path_policy(b200_ctx *ctx, int policy) {
  if (!ctx || policy < 0 || policy > 2) return B200_ERR_INVALID_ARG;
  ctx->path_policy = policy;
  return B200_OK;
}

int b200_set_pair_policy(b200_ctx *ctx, int policy) {
  if (!ctx || policy < 0 || policy > 3) return B200_ERR_INVALID_ARG;
  ctx->pair_policy = policy;
  return B200_OK;
}

int b200_set_async_launch(b200_ctx *ctx, int on) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  if (on && !ctx->queue) {
    ctx->queue = new (std::nothrow) b200::LaunchQueue(ctx->device);
    if (!ctx->queue) return B200_ERR_OUT_OF_MEMORY;
  }
  if (!on) b200::queue_drain(ctx);
  ctx->async = on != 0;
  return B200_OK;
}

int b200_launch_flush(b200_ctx *ctx) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  b200::queue_drain(ctx);
  return B200_OK;
}

int b200_set_dependent_launch(b200_ctx *ctx, int on) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  ctx->pdl = on != 0;
  return B200_OK;
}

int b200_operand_cache_enable(b200_ctx *ctx, size_t max_bytes) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  ctx->planes.cap = max_bytes;
  if (max_bytes == 0 && ctx->planes.scope == 0) b200::plane_cache_drop_range(ctx, nullptr, 0);
  return B200_OK;
}

int b200_operand_cache_invalidate(b200_ctx *ctx, const void *ptr, size_t bytes) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  b200::plane_cache_drop_range(ctx, ptr, ptr ? bytes : 0);
  return B200_OK;
}

int b200_operand_cache_stats(const b200_ctx *ctx, uint64_t stats[4]) {
  if (!ctx || !stats) return B200_ERR_INVALID_ARG;
  stats[0] = ctx->planes.hits;
  stats[1] = ctx->planes.misses;
  stats[2] = ctx->planes.bytes;
  stats[3] = ctx->planes.entries.size();
  return B200_OK;
}

int b200_set_correction_policy(b200_ctx *ctx, int policy) {
  if (!ctx || policy < 0 || policy > 2) return B200_ERR_INVALID_ARG;
  ctx->correction_policy = policy;
  return B200_OK;
}

int b200_profile_enable(b200_ctx *ctx, int on) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  ctx->profiling = on != 0;
  return B200_OK;
}

int b200_profile_read(b200_ctx *ctx, double ms[4], uint64_t launches[4]) {
  if (!ctx || !ms || !launches) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  for (int i = 0; i < b200::kProfKinds; ++i) { ms[i] = 0.0; launches[i] = 0; }
  b200::queue_drain(ctx);
  B200_CUDA_TRY(cudaDeviceSynchronize());
  for (auto &r : ctx->prof) {
    float t = 0.f;
    if (cudaEventElapsedTime(&t, r.start, r.stop) == cudaSuccess && r.kind >= 0 && r.kind < b200::kProfKinds) {
      ms[r.kind] += t;
      launches[r.kind] += 1;
    }
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  ctx->prof.clear();
  return B200_OK;
}

int b200_launch_count(const b200_ctx *ctx, uint64_t *launches) {
  if (!ctx || !launches) return B200_ERR_INVALID_ARG;
  *launches = ctx->launches;
  return B200_OK;
}

int b200_gemm(b200_ctx *ctx, int mode, int trans_a, int trans_b, const void *A, const void *B,
              void *C, uint32_t m, uint32_t n, uint32_t k, uint32_t groups, uint32_t red,
              uint64_t a_gs, uint64_t a_rs, uint64_t b_gs, uint64_t b_rs, uint64_t c_gs,
              int accumulate, int force_path, void *stream) {
  if (!ctx || !A || !B || !C) return B200_ERR_INVALID_ARG;
  if (mode < B200_MODE_FP32_3XTF32 || mode > B200_MODE_FP32_3XFP16) return B200_ERR_INVALID_ARG;
  if (m == 0 || n == 0 || groups == 0) return B200_OK;
  if (k == 0 || red == 0) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  GemmRange range(mode, trans_a, trans_b, m, n, k, groups, red, accumulate);
  GemmArgs g{mode, trans_a ? 1 : 0, trans_b ? 1 : 0, A, B, C, m, n, k, groups, red,
             a_gs, a_rs, b_gs, b_rs, c_gs, accumulate ? 1 : 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!ctx->planes.entries.empty()) {
    // planes packed from the array this product writes are stale from here on
    const size_t span = ((size_t)(groups - 1) * c_gs + (size_t)m * n) * b200::elem_bytes(mode);
    b200::plane_cache_drop_range(ctx, C, span);
  }
  const bool eligible = b200::gemm_tc_eligible(ctx, g);
  if (force_path == 2) return eligible ? b200::gemm_tc(ctx, g, s) : B200_ERR_INVALID_ARG;
  if (force_path == 1) return b200::gemm_simt(ctx, g, s);
  if (force_path == 3) return b200::gemm_skinny_eligible(g) ? b200::gemm_skinny(ctx, g, s) : B200_ERR_INVALID_ARG;
  if (ctx->path_policy == 2 && eligible) return b200::gemm_tc(ctx, g, s);
  if (ctx->path_policy == 1) return b200::gemm_simt(ctx, g, s);
  // A 128-row MMA tile on a problem this small is mostly padding; the CUDA-core
  // kernel wins below roughly a tile's worth of work.
  // One tiny extent against large ones is HBM-bound.  In the fp32-grade modes the tensor-core
  // path would first pack the large operand into planes (three more passes over it): there the
  // CUDA-core kernels that stream it once win (255-335 us against 675 us for the three products of
  // a 10 x 1024 layer over 65536 items) and are exact fp32.  The single-pass modes need no
  // packing and stay on the tensor-core path where TMA's alignment rules admit the operands; where
  // they do not (ten rows of halves are 20 bytes) the alternative is the general CUDA-core kernel,
  // which takes 5.8 ms for the reduce shape against 0.12 ms here.
  if ((mode == B200_MODE_FP32_3XTF32 || mode == B200_MODE_FP32_3XFP16 || !eligible) && b200::gemm_skinny_eligible(g))
    return b200::gemm_skinny(ctx, g, s);
  const double macs = static_cast<double>(m) * n * k * groups * red;
  // (a few rows against a long contraction are still worth it: the tensor-core path splits k
  // over all SMs and streams the big operand once, the CUDA-core kernel would run on a few CTAs)
  if (eligible && n >= 16 && macs >= 2097152.0 && (m >= 32 || macs >= 67108864.0)) return b200::gemm_tc(ctx, g, s);
  return b200::gemm_simt(ctx, g, s);
}

int b200_gemm_3xtf32_noalloc(b200_ctx *ctx, int trans_a, int trans_b, const void *A, const void *B,
                             void *C, uint32_t m, uint32_t n, uint32_t k, int accumulate,
                             void *stream) {
  if (!ctx || !A || !B || !C) return B200_ERR_INVALID_ARG;
  if (m == 0 || n == 0 || k == 0) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  GemmArgs g{B200_MODE_FP32_3XTF32, trans_a ? 1 : 0, trans_b ? 1 : 0, A, B, C, m, n, k, 1, 1,
             0, 0, 0, 0, 0, accumulate ? 1 : 0};
  return b200::gemm_3xtf32_noalloc(ctx, g, static_cast<cudaStream_t>(stream));
}

static int check_matmul(const b200_ctx *ctx, int mode, uint32_t ba, uint32_t bb) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  if (mode < B200_MODE_FP32_3XTF32 || mode > B200_MODE_FP32_3XFP16) return B200_ERR_INVALID_ARG;
  if (ba == 0 || bb == 0) return B200_ERR_INVALID_ARG;
  if (ba != bb && ba != 1 && bb != 1) return B200_ERR_INVALID_ARG;  // Shape::has_compatible_batch
  return B200_OK;
}

int b200_matmul_fw(b200_ctx *ctx, int mode, const void *a, const void *b, void *y, uint32_t di,
                   uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb, void *stream) {
  int rc = check_matmul(ctx, mode, ba, bb);
  if (rc) return rc;
  if (!a || !b || !y) return B200_ERR_INVALID_ARG;
  const uint64_t na = (uint64_t)di * dj, nb = (uint64_t)dj * dk, ny = (uint64_t)di * dk;
  if (ny == 0) return B200_OK;  // an empty result (primitiv's Shape never has a zero extent)
  if (dj == 0) {                // an empty contraction: y = 0
    DeviceGuard guard(ctx->device);
    b200::queue_drain(ctx);
    B200_CUDA_TRY(cudaMemsetAsync(y, 0, ny * (ba > bb ? ba : bb) * b200::elem_bytes(mode),
                                  static_cast<cudaStream_t>(stream)));
    return B200_OK;
  }
  if (ba == 1) {
    // one product over the combined {dj, dk*bb} matrix: b's batches are adjacent columns
    const uint64_t dkb = (uint64_t)dk * bb;
    if (dkb > 0xffffffffull) return B200_ERR_TOO_LARGE;  // extents are 32-bit, as primitiv's Shape is
    return b200_gemm(ctx, mode, 0, 0, a, b, y, di, (uint32_t)dkb, dj, 1, 1, 0, 0, 0, 0, 0, 0, 0, stream);
  }
  return b200_gemm(ctx, mode, 0, 0, a, b, y, di, dk, dj, ba, 1, na, 0, bb > 1 ? nb : 0, 0, ny, 0, 0,
                   stream);
}

int b200_matmul_bw(b200_ctx *ctx, int mode, const void *a, const void *b, const void *gy, void *ga,
                   void *gb, uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb,
                   void *stream) {
  return b200_matmul_bw_ex(ctx, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb, 1, 1, stream);
}

int b200_matmul_bw_ex(b200_ctx *ctx, int mode, const void *a, const void *b, const void *gy, void *ga,
                      void *gb, uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb,
                      int accumulate_a, int accumulate_b, void *stream) {
  const int acc_a = accumulate_a ? 1 : 0, acc_b = accumulate_b ? 1 : 0;
  int rc = check_matmul(ctx, mode, ba, bb);
  if (rc) return rc;
  if (!a || !b || !gy) return B200_ERR_INVALID_ARG;
  // gy is an operand of both products (and a, b may already have planes from the forward call):
  // operand planes are shared for the duration of the call
  b200::PlaneScope share(ctx);
  const uint64_t na = (uint64_t)di * dj, nb = (uint64_t)dj * dk, ny = (uint64_t)di * dk;
  if (di == 0 || dj == 0 || dk == 0) {
    // some extent is empty: nothing to add; a gradient that was to be written becomes zeros
    DeviceGuard guard(ctx->device);
    b200::queue_drain(ctx);
    const size_t eb = b200::elem_bytes(mode);
    if (ga && !acc_a && na) B200_CUDA_TRY(cudaMemsetAsync(ga, 0, na * ba * eb, static_cast<cudaStream_t>(stream)));
    if (gb && !acc_b && nb) B200_CUDA_TRY(cudaMemsetAsync(gb, 0, nb * bb * eb, static_cast<cudaStream_t>(stream)));
    return B200_OK;
  }
  if (ba == 1) {
    if ((uint64_t)dk * bb > 0xffffffffull) return B200_ERR_TOO_LARGE;
    const uint32_t dkb = dk * bb;
    // ga += gy_all . b_all^T : the batch sum is the tail of one long contraction
    if (ga) {
      rc = b200_gemm(ctx, mode, 0, 1, gy, b, ga, di, dj, dkb, 1, 1, 0, 0, 0, 0, 0, acc_a, 0, stream);
      if (rc) return rc;
    }
    // gb_all += a^T . gy_all
    if (gb) rc = b200_gemm(ctx, mode, 1, 0, a, gy, gb, dj, dkb, di, 1, 1, 0, 0, 0, 0, 0, acc_b, 0, stream);
    return rc;
  }
  // ga[n] += gy[n] . b[n or 0]^T
  if (ga) {
    rc = b200_gemm(ctx, mode, 0, 1, gy, b, ga, di, dj, dk, ba, 1, ny, 0, bb > 1 ? nb : 0, 0, na, acc_a, 0,
                   stream);
    if (rc) return rc;
  }
  if (gb) {
    if (bb > 1) {
      // gb[n] += a[n]^T . gy[n]
      rc = b200_gemm(ctx, mode, 1, 0, a, gy, gb, dj, dk, di, ba, 1, na, 0, ny, 0, nb, acc_b, 0, stream);
    } else {
      // gb += sum_n a[n]^T . gy[n] : one launch, the batch is a second contraction axis
      rc = b200_gemm(ctx, mode, 1, 0, a, gy, gb, dj, dk, di, 1, ba, 0, na, 0, ny, 0, acc_b, 0, stream);
    }
  }
  return rc;
}

namespace {

struct Scratch {
  b200_ctx *ctx;
  void *p = nullptr;
  explicit Scratch(b200_ctx *c) : ctx(c) {}
  ~Scratch() { if (p) ctx->pool.free(p); }
  int get(size_t bytes) { return ctx->pool.alloc(bytes, &p, nullptr); }
};

}  // namespace

// The host-buffer entry points run as a three-stream pipeline over chunks of the batch:
// while chunk c is multiplied, chunk c+1 is on its way up and chunk c-1 on its way down,
// so the call costs about max(upload, download, compute) instead of their sum.  Tensors
// with batch 1 (and their gradients) travel once, before the first / after the last chunk.
// The streams are ordinary blocking streams: their first work waits for whatever the caller
// queued on the legacy default stream, and the call returns only when all three are idle.
namespace {

constexpr int kPipeUp = 0, kPipeRun = 1, kPipeDown = 2;
// In fp16 mode every chunk rounds a batch-summed gradient to half once more, hence fewer chunks.
constexpr uint32_t kPipeMaxChunks = 16, kPipeMaxChunksHalf = 8;
constexpr size_t kPipeMinChunkBytes = 4u << 20;

int pipe_prepare(b200_ctx *ctx, uint32_t events) {
  for (cudaStream_t &st : ctx->pipe_streams)
    if (!st) B200_CUDA_TRY(cudaStreamCreate(&st));
  while (ctx->pipe_events.size() < events) {
    cudaEvent_t ev;
    B200_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    ctx->pipe_events.push_back(ev);
  }
  return B200_OK;
}

// Number of batch chunks: enough for overlap, each still a worthwhile transfer.
uint32_t pipe_chunks(int mode, uint32_t bs, size_t batched_bytes) {
  const uint32_t cap = mode == B200_MODE_FP16 ? kPipeMaxChunksHalf : kPipeMaxChunks;
  uint32_t c = bs < cap ? bs : cap;
  while (c > 1 && batched_bytes / c < kPipeMinChunkBytes) --c;
  return c;
}

int pipe_finish(b200_ctx *ctx, int rc) {
  // drain all three streams whatever happened, so that the scratch blocks can go back to the pool
  for (cudaStream_t st : ctx->pipe_streams) {
    const cudaError_t e = cudaStreamSynchronize(st);
    if (!rc && e != cudaSuccess) rc = static_cast<int>(e);
  }
  const int status = b200::take_status(ctx);  // the results are on the host now: a wait that ran out is an error
  return rc ? rc : status;
}

inline const char *cbytes(const void *p, size_t off) { return static_cast<const char *>(p) + off; }
inline char *mbytes(void *p, size_t off) { return static_cast<char *>(p) + off; }

}  // namespace

int b200_matmul_fw_host(b200_ctx *ctx, int mode, const void *a_host, const void *b_host,
                        void *y_host, uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba,
                        uint32_t bb) {
  int rc = check_matmul(ctx, mode, ba, bb);
  if (rc) return rc;
  if (!a_host || !b_host || !y_host) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  b200::InlineLaunches inline_launches(ctx);  // three streams and events: everything on this thread
  const size_t eb = b200::elem_bytes(mode);
  const uint32_t bs = ba > bb ? ba : bb;
  const size_t ia = (size_t)di * dj * eb, ib = (size_t)dj * dk * eb, iy = (size_t)di * dk * eb;  // one item
  const size_t sa = ia * ba, sb = ib * bb, sy = iy * bs;
  if (sa == 0 || sb == 0 || sy == 0) return sy == 0 ? B200_OK : B200_ERR_INVALID_ARG;
  Scratch da(ctx), db(ctx), dy(ctx);
  if ((rc = da.get(sa)) || (rc = db.get(sb)) || (rc = dy.get(sy))) return rc;
  const uint32_t chunks = pipe_chunks(mode, bs, (ba > 1 ? sa : 0) + (bb > 1 ? sb : 0) + sy);
  if ((rc = pipe_prepare(ctx, 2 * chunks))) return rc;
  cudaStream_t up = ctx->pipe_streams[kPipeUp], run = ctx->pipe_streams[kPipeRun],
               down = ctx->pipe_streams[kPipeDown];
  auto body = [&]() -> int {
    if (ba == 1) B200_CUDA_TRY(cudaMemcpyAsync(da.p, a_host, sa, cudaMemcpyHostToDevice, up));
    if (bb == 1) B200_CUDA_TRY(cudaMemcpyAsync(db.p, b_host, sb, cudaMemcpyHostToDevice, up));
    for (uint32_t c = 0; c < chunks; ++c) {
      const uint32_t n0 = (uint32_t)((uint64_t)bs * c / chunks), n1 = (uint32_t)((uint64_t)bs * (c + 1) / chunks);
      const uint32_t cnt = n1 - n0;
      const size_t oa = ba > 1 ? ia * n0 : 0, ob = bb > 1 ? ib * n0 : 0, oy = iy * n0;
      if (ba > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(da.p, oa), cbytes(a_host, oa), ia * cnt, cudaMemcpyHostToDevice, up));
      if (bb > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(db.p, ob), cbytes(b_host, ob), ib * cnt, cudaMemcpyHostToDevice, up));
      cudaEvent_t uploaded = ctx->pipe_events[2 * c], computed = ctx->pipe_events[2 * c + 1];
      B200_CUDA_TRY(cudaEventRecord(uploaded, up));
      B200_CUDA_TRY(cudaStreamWaitEvent(run, uploaded, 0));
      const int r = b200_matmul_fw(ctx, mode, cbytes(da.p, oa), cbytes(db.p, ob), mbytes(dy.p, oy), di, dj, dk,
                                   ba > 1 ? cnt : 1, bb > 1 ? cnt : 1, run);
      if (r) return r;
      B200_CUDA_TRY(cudaEventRecord(computed, run));
      B200_CUDA_TRY(cudaStreamWaitEvent(down, computed, 0));
      B200_CUDA_TRY(cudaMemcpyAsync(mbytes(y_host, oy), cbytes(dy.p, oy), iy * cnt, cudaMemcpyDeviceToHost, down));
    }
    return B200_OK;
  };
  return pipe_finish(ctx, body());
}

int b200_matmul_bw_host(b200_ctx *ctx, int mode, const void *a_host, const void *b_host,
                        const void *gy_host, void *ga_host, void *gb_host, uint32_t di, uint32_t dj,
                        uint32_t dk, uint32_t ba, uint32_t bb) {
  int rc = check_matmul(ctx, mode, ba, bb);
  if (rc) return rc;
  if (!a_host || !b_host || !gy_host || !ga_host || !gb_host) return B200_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  b200::InlineLaunches inline_launches(ctx);  // three streams and events: everything on this thread
  const size_t eb = b200::elem_bytes(mode);
  const uint32_t bs = ba > bb ? ba : bb;
  const size_t ia = (size_t)di * dj * eb, ib = (size_t)dj * dk * eb, iy = (size_t)di * dk * eb;
  const size_t sa = ia * ba, sb = ib * bb, sy = iy * bs;
  if (sa == 0 || sb == 0 || sy == 0) return B200_OK;  // an empty extent: nothing to add
  Scratch da(ctx), db(ctx), dgy(ctx), dga(ctx), dgb(ctx);
  if ((rc = da.get(sa)) || (rc = db.get(sb)) || (rc = dgy.get(sy)) || (rc = dga.get(sa)) ||
      (rc = dgb.get(sb)))
    return rc;
  const uint32_t chunks = pipe_chunks(mode, bs, (ba > 1 ? 2 * sa : 0) + (bb > 1 ? 2 * sb : 0) + sy);
  if ((rc = pipe_prepare(ctx, 2 * chunks))) return rc;
  cudaStream_t up = ctx->pipe_streams[kPipeUp], run = ctx->pipe_streams[kPipeRun],
               down = ctx->pipe_streams[kPipeDown];
  auto body = [&]() -> int {
    // batch-1 operands and the gradients that every chunk adds into go up first
    if (ba == 1) {
      B200_CUDA_TRY(cudaMemcpyAsync(da.p, a_host, sa, cudaMemcpyHostToDevice, up));
      B200_CUDA_TRY(cudaMemcpyAsync(dga.p, ga_host, sa, cudaMemcpyHostToDevice, up));
    }
    if (bb == 1) {
      B200_CUDA_TRY(cudaMemcpyAsync(db.p, b_host, sb, cudaMemcpyHostToDevice, up));
      B200_CUDA_TRY(cudaMemcpyAsync(dgb.p, gb_host, sb, cudaMemcpyHostToDevice, up));
    }
    for (uint32_t c = 0; c < chunks; ++c) {
      const uint32_t n0 = (uint32_t)((uint64_t)bs * c / chunks), n1 = (uint32_t)((uint64_t)bs * (c + 1) / chunks);
      const uint32_t cnt = n1 - n0;
      const size_t oa = ba > 1 ? ia * n0 : 0, ob = bb > 1 ? ib * n0 : 0, oy = iy * n0;
      if (ba > 1) {
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(da.p, oa), cbytes(a_host, oa), ia * cnt, cudaMemcpyHostToDevice, up));
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(dga.p, oa), cbytes(ga_host, oa), ia * cnt, cudaMemcpyHostToDevice, up));
      }
      if (bb > 1) {
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(db.p, ob), cbytes(b_host, ob), ib * cnt, cudaMemcpyHostToDevice, up));
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(dgb.p, ob), cbytes(gb_host, ob), ib * cnt, cudaMemcpyHostToDevice, up));
      }
      B200_CUDA_TRY(cudaMemcpyAsync(mbytes(dgy.p, oy), cbytes(gy_host, oy), iy * cnt, cudaMemcpyHostToDevice, up));
      cudaEvent_t uploaded = ctx->pipe_events[2 * c], computed = ctx->pipe_events[2 * c + 1];
      B200_CUDA_TRY(cudaEventRecord(uploaded, up));
      B200_CUDA_TRY(cudaStreamWaitEvent(run, uploaded, 0));
      const int r = b200_matmul_bw(ctx, mode, cbytes(da.p, oa), cbytes(db.p, ob), cbytes(dgy.p, oy),
                                   mbytes(dga.p, oa), mbytes(dgb.p, ob), di, dj, dk,
                                   ba > 1 ? cnt : 1, bb > 1 ? cnt : 1, run);
      if (r) return r;
      B200_CUDA_TRY(cudaEventRecord(computed, run));
      B200_CUDA_TRY(cudaStreamWaitEvent(down, computed, 0));
      if (ba > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(ga_host, oa), cbytes(dga.p, oa), ia * cnt, cudaMemcpyDeviceToHost, down));
      if (bb > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(gb_host, ob), cbytes(dgb.p, ob), ib * cnt, cudaMemcpyDeviceToHost, down));
    }
    // `down` already waits for the last chunk's products: the batch-summed gradients are complete
    if (ba == 1) B200_CUDA_TRY(cudaMemcpyAsync(ga_host, dga.p, sa, cudaMemcpyDeviceToHost, down));
    if (bb == 1) B200_CUDA_TRY(cudaMemcpyAsync(gb_host, dgb.p, sb, cudaMemcpyDeviceToHost, down));
    return B200_OK;
  };
  return pipe_finish(ctx, body());
}

// Forward and backward of one product from host buffers in ONE pipelined pass: every operand
// crosses the bus once (a and b serve the forward product and both gradients), a gradient that
// the caller declares to start from zeros is neither uploaded nor read, and y travels down while
// the gradients are still being computed.  Per chunk of the batch: a, b up -> forward -> y down;
// gy (and any gradient to be added to) up -> backward -> batched gradients down.
int b200_matmul_fw_bw_host(b200_ctx *ctx, int mode, const void *a_host, const void *b_host,
                           const void *gy_host, void *y_host, void *ga_host, void *gb_host,
                           uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb,
                           int accumulate_a, int accumulate_b) {
  int rc = check_matmul(ctx, mode, ba, bb);
  if (rc) return rc;
  if (!a_host || !b_host) return B200_ERR_INVALID_ARG;
  const bool want_bw = ga_host || gb_host;
  if (want_bw && !gy_host) return B200_ERR_INVALID_ARG;
  if (!y_host && !want_bw) return B200_OK;
  DeviceGuard guard(ctx->device);
  b200::InlineLaunches inline_launches(ctx);  // three streams and events: everything on this thread
  const size_t eb = b200::elem_bytes(mode);
  const uint32_t bs = ba > bb ? ba : bb;
  const size_t ia = (size_t)di * dj * eb, ib = (size_t)dj * dk * eb, iy = (size_t)di * dk * eb;  // one item
  const size_t sa = ia * ba, sb = ib * bb, sy = iy * bs;
  if (sa == 0 || sb == 0 || sy == 0) {
    // an empty extent: y (if any) is empty or zero, and nothing is added to the gradients
    if (y_host && sy && dj == 0) memset(y_host, 0, sy);
    if (ga_host && !accumulate_a && sa) memset(ga_host, 0, sa);
    if (gb_host && !accumulate_b && sb) memset(gb_host, 0, sb);
    return B200_OK;
  }
  // a and b serve the forward product and a gradient each, gy both gradients: their planes are shared
  // for the duration of the call (declared before the buffers, so it outlives them)
  b200::PlaneScope share(ctx);
  Scratch da(ctx), db(ctx), dgy(ctx), dy(ctx), dga(ctx), dgb(ctx);
  if ((rc = da.get(sa)) || (rc = db.get(sb))) return rc;
  if (y_host && (rc = dy.get(sy))) return rc;
  if (want_bw && (rc = dgy.get(sy))) return rc;
  if (ga_host && (rc = dga.get(sa))) return rc;
  if (gb_host && (rc = dgb.get(sb))) return rc;
  const size_t per_step = (ba > 1 ? sa : 0) + (bb > 1 ? sb : 0) + (want_bw ? sy : 0);
  const uint32_t chunks = pipe_chunks(mode, bs, per_step);
  if ((rc = pipe_prepare(ctx, 4 * chunks))) return rc;
  cudaStream_t up = ctx->pipe_streams[kPipeUp], run = ctx->pipe_streams[kPipeRun],
               down = ctx->pipe_streams[kPipeDown];
  const int acc_a = accumulate_a ? 1 : 0, acc_b = accumulate_b ? 1 : 0;
  auto body = [&]() -> int {
    // batch-1 operands, and the batch-1 gradients every chunk adds into, go up first
    if (ba == 1) {
      B200_CUDA_TRY(cudaMemcpyAsync(da.p, a_host, sa, cudaMemcpyHostToDevice, up));
      if (ga_host && acc_a) B200_CUDA_TRY(cudaMemcpyAsync(dga.p, ga_host, sa, cudaMemcpyHostToDevice, up));
    }
    if (bb == 1) {
      B200_CUDA_TRY(cudaMemcpyAsync(db.p, b_host, sb, cudaMemcpyHostToDevice, up));
      if (gb_host && acc_b) B200_CUDA_TRY(cudaMemcpyAsync(dgb.p, gb_host, sb, cudaMemcpyHostToDevice, up));
    }
    for (uint32_t c = 0; c < chunks; ++c) {
      const uint32_t n0 = (uint32_t)((uint64_t)bs * c / chunks), n1 = (uint32_t)((uint64_t)bs * (c + 1) / chunks);
      const uint32_t cnt = n1 - n0;
      const size_t oa = ba > 1 ? ia * n0 : 0, ob = bb > 1 ? ib * n0 : 0, oy = iy * n0;
      const uint32_t ca = ba > 1 ? cnt : 1, cb = bb > 1 ? cnt : 1;
      cudaEvent_t operands_up = ctx->pipe_events[4 * c], grads_up = ctx->pipe_events[4 * c + 1],
                  fw_done = ctx->pipe_events[4 * c + 2], bw_done = ctx->pipe_events[4 * c + 3];
      if (ba > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(da.p, oa), cbytes(a_host, oa), ia * cnt, cudaMemcpyHostToDevice, up));
      if (bb > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(db.p, ob), cbytes(b_host, ob), ib * cnt, cudaMemcpyHostToDevice, up));
      B200_CUDA_TRY(cudaEventRecord(operands_up, up));
      B200_CUDA_TRY(cudaStreamWaitEvent(run, operands_up, 0));
      if (y_host) {
        const int r = b200_matmul_fw(ctx, mode, cbytes(da.p, oa), cbytes(db.p, ob), mbytes(dy.p, oy), di, dj, dk, ca, cb, run);
        if (r) return r;
        B200_CUDA_TRY(cudaEventRecord(fw_done, run));
        B200_CUDA_TRY(cudaStreamWaitEvent(down, fw_done, 0));
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(y_host, oy), cbytes(dy.p, oy), iy * cnt, cudaMemcpyDeviceToHost, down));
      }
      if (!want_bw) continue;
      B200_CUDA_TRY(cudaMemcpyAsync(mbytes(dgy.p, oy), cbytes(gy_host, oy), iy * cnt, cudaMemcpyHostToDevice, up));
      if (ga_host && acc_a && ba > 1)
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(dga.p, oa), cbytes(ga_host, oa), ia * cnt, cudaMemcpyHostToDevice, up));
      if (gb_host && acc_b && bb > 1)
        B200_CUDA_TRY(cudaMemcpyAsync(mbytes(dgb.p, ob), cbytes(gb_host, ob), ib * cnt, cudaMemcpyHostToDevice, up));
      B200_CUDA_TRY(cudaEventRecord(grads_up, up));
      B200_CUDA_TRY(cudaStreamWaitEvent(run, grads_up, 0));
      // a batch-1 gradient is one array for all chunks: only the first chunk may store into it
      const int r = b200_matmul_bw_ex(ctx, mode, cbytes(da.p, oa), cbytes(db.p, ob), cbytes(dgy.p, oy),
                                      ga_host ? mbytes(dga.p, oa) : nullptr, gb_host ? mbytes(dgb.p, ob) : nullptr,
                                      di, dj, dk, ca, cb, (ba == 1 && c > 0) ? 1 : acc_a,
                                      (bb == 1 && c > 0) ? 1 : acc_b, run);
      if (r) return r;
      B200_CUDA_TRY(cudaEventRecord(bw_done, run));
      B200_CUDA_TRY(cudaStreamWaitEvent(down, bw_done, 0));
      if (ga_host && ba > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(ga_host, oa), cbytes(dga.p, oa), ia * cnt, cudaMemcpyDeviceToHost, down));
      if (gb_host && bb > 1) B200_CUDA_TRY(cudaMemcpyAsync(mbytes(gb_host, ob), cbytes(dgb.p, ob), ib * cnt, cudaMemcpyDeviceToHost, down));
    }
    // `down` already waits for the last chunk's products: the batch-summed gradients are complete
    if (ga_host && ba == 1) B200_CUDA_TRY(cudaMemcpyAsync(ga_host, dga.p, sa, cudaMemcpyDeviceToHost, down));
    if (gb_host && bb == 1) B200_CUDA_TRY(cudaMemcpyAsync(gb_host, dgb.p, sb, cudaMemcpyDeviceToHost, down));
    return B200_OK;
  };
  return pipe_finish(ctx, body());
}

}  // extern "C"
