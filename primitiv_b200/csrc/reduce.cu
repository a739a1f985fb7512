// Reductions along one dimension (sum, logsumexp, max, min, argmax, argmin, max/min
// backward) and over the batch.
//
// A tensor is seen as [hi][n][skip1]; output element o = (hi, lo) reduces the n values
// at hi*n*skip1 + j*skip1 + lo.  Two launch shapes:
//   * skip1 == 1 (reduction along the leading dimension, the softmax / argmax case): one
//     warp per output, lanes read consecutive addresses, warp-shuffle tree at the end;
//   * skip1 > 1: one thread per output, consecutive threads read consecutive addresses.
// The reference uses one CTA per output with a shared-memory tree
// (primitiv/devices/cuda/ops/sum.cu:9-48).
#include <cfloat>

#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr unsigned kBlock = 256;

struct SumOp {
  __device__ static float merge(float a, float b) { return a + b; }
};
struct MaxOp {
  __device__ static float merge(float a, float b) { return fmaxf(a, b); }
};
struct MinOp {
  __device__ static float merge(float a, float b) { return fminf(a, b); }
};

template <typename Op>
__device__ __forceinline__ float warp_all(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = Op::merge(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

// ---- generic reduce: RED 0 sum, 1 logsumexp, 2 max, 3 min ----
template <typename T, int RED>
__device__ __forceinline__ float reduce_serial(const T *x, u64 first, u64 step, uint32_t n) {
  if constexpr (RED == B200_RED_SUM) {
    float a = 0.f;
    for (uint32_t j = 0; j < n; ++j) a += ld(x, first + j * step);
    return a;
  } else if constexpr (RED == B200_RED_MAX) {
    float a = -INFINITY;
    for (uint32_t j = 0; j < n; ++j) a = fmaxf(a, ld(x, first + j * step));
    return a;
  } else if constexpr (RED == B200_RED_MIN) {
    float a = INFINITY;
    for (uint32_t j = 0; j < n; ++j) a = fminf(a, ld(x, first + j * step));
    return a;
  } else {
    float m = -INFINITY;
    for (uint32_t j = 0; j < n; ++j) m = fmaxf(m, ld(x, first + j * step));
    if (m == -INFINITY || m == INFINITY) return m;
    float a = 0.f;
    for (uint32_t j = 0; j < n; ++j) a += expf(ld(x, first + j * step) - m);
    return m + logf(a);
  }
}

template <typename T, int RED>
__global__ void __launch_bounds__(kBlock) reduce_thread_kernel(const T *__restrict__ x, T *__restrict__ y,
                                                               uint32_t n, u64 skip1, u64 outputs) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 o = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; o < outputs; o += stride) {
    const u64 first = (o / skip1) * skip1 * n + o % skip1;
    st(y, o, reduce_serial<T, RED>(x, first, skip1, n));
  }
}

template <typename T, int RED>
__global__ void __launch_bounds__(kBlock) reduce_warp_kernel(const T *__restrict__ x, T *__restrict__ y, uint32_t n,
                                                             u64 outputs) {
  pdl_enter();
  const uint32_t lane = threadIdx.x & 31u;
  const u64 warp = (static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const u64 nwarps = (static_cast<u64>(gridDim.x) * blockDim.x) >> 5;
  for (u64 o = warp; o < outputs; o += nwarps) {
    const u64 first = o * n;
    float r;
    if constexpr (RED == B200_RED_SUM) {
      float a = 0.f;
      for (uint32_t j = lane; j < n; j += 32u) a += ld(x, first + j);
      r = warp_all<SumOp>(a);
    } else if constexpr (RED == B200_RED_MAX) {
      float a = -INFINITY;
      for (uint32_t j = lane; j < n; j += 32u) a = fmaxf(a, ld(x, first + j));
      r = warp_all<MaxOp>(a);
    } else if constexpr (RED == B200_RED_MIN) {
      float a = INFINITY;
      for (uint32_t j = lane; j < n; j += 32u) a = fminf(a, ld(x, first + j));
      r = warp_all<MinOp>(a);
    } else {
      float m = -INFINITY;
      for (uint32_t j = lane; j < n; j += 32u) m = fmaxf(m, ld(x, first + j));
      m = warp_all<MaxOp>(m);
      if (m == -INFINITY || m == INFINITY) {
        r = m;
      } else {
        float a = 0.f;
        for (uint32_t j = lane; j < n; j += 32u) a += expf(ld(x, first + j) - m);
        r = m + logf(warp_all<SumOp>(a));
      }
    }
    if (lane == 0) st(y, o, r);
  }
}

// index of the first extreme value along the dimension (ties: lowest index, as the reference)
template <typename T>
__device__ __forceinline__ uint32_t first_extreme(const T *x, u64 first, u64 step, uint32_t n, bool want_max) {
  float best = ld(x, first);
  uint32_t arg = 0;
  for (uint32_t j = 1; j < n; ++j) {
    const float v = ld(x, first + j * step);
    if (want_max ? v > best : v < best) {
      best = v;
      arg = j;
    }
  }
  return arg;
}

template <typename T>
__global__ void __launch_bounds__(kBlock) argminmax_kernel(const T *__restrict__ x, uint32_t *__restrict__ ids,
                                                           uint32_t n, u64 skip1, u64 outputs, int want_max) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 o = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; o < outputs; o += stride) {
    const u64 first = (o / skip1) * skip1 * n + o % skip1;
    ids[o] = first_extreme(x, first, skip1, n, want_max != 0);
  }
}

// gx[first position whose value equals y[o]] += gy[o]   (max.cc / min.cc backward)
template <typename T>
__global__ void __launch_bounds__(kBlock) minmax_bw_kernel(const T *__restrict__ x, const T *__restrict__ y,
                                                           const T *__restrict__ gy, T *gx, uint32_t n, u64 skip1,
                                                           u64 outputs) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 o = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; o < outputs; o += stride) {
    const u64 first = (o / skip1) * skip1 * n + o % skip1;
    const float target = ld(y, o);
    for (uint32_t j = 0; j < n; ++j) {
      const u64 e = first + j * skip1;
      if (ld(x, e) == target) {
        st(gx, e, ld(gx, e) + ld(gy, o));
        break;
      }
    }
  }
}

template <typename T, int RED>
void launch_reduce(b200_ctx *ctx, cudaStream_t s, const void *x, void *y, uint32_t n, u64 skip1, u64 outputs) {
  if (skip1 == 1 && n >= 64) {
    const unsigned grid = grid_for(ctx, outputs * 32ull, kBlock);
    b200::launch(ctx, reduce_warp_kernel<T, RED>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), n, outputs);
  } else {
    b200::launch(ctx, reduce_thread_kernel<T, RED>, dim3(grid_for(ctx, outputs, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), n, skip1, outputs);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_reduce_fw(b200_ctx *ctx, int mode, int red, const void *x, void *y, uint32_t n, uint64_t skip1,
                   uint64_t outputs, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (outputs == 0) return B200_OK;
  if (!x || !y || n == 0 || skip1 == 0 || red < 0 || red > B200_RED_MIN) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    switch (red) {
      case B200_RED_SUM: launch_reduce<T, B200_RED_SUM>(ctx, s, x, y, n, skip1, outputs); break;
      case B200_RED_LOGSUMEXP: launch_reduce<T, B200_RED_LOGSUMEXP>(ctx, s, x, y, n, skip1, outputs); break;
      case B200_RED_MAX: launch_reduce<T, B200_RED_MAX>(ctx, s, x, y, n, skip1, outputs); break;
      default: launch_reduce<T, B200_RED_MIN>(ctx, s, x, y, n, skip1, outputs); break;
    }
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_minmax_bw(b200_ctx *ctx, int mode, const void *x, const void *y, const void *gy, void *gx, uint32_t n,
                   uint64_t skip1, uint64_t outputs, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (outputs == 0) return B200_OK;
  if (!x || !y || !gy || !gx || n == 0 || skip1 == 0) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, minmax_bw_kernel<T>, dim3(grid_for(ctx, outputs, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<const T *>(y), static_cast<const T *>(gy), static_cast<T *>(gx), n,
        skip1, outputs);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_argminmax(b200_ctx *ctx, int mode, int want_max, const void *x, uint32_t *ids_host, uint32_t n,
                   uint64_t skip1, uint64_t outputs, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (outputs == 0) return B200_OK;
  if (!x || !ids_host || n == 0 || skip1 == 0) return B200_ERR_INVALID_ARG;
  void *d_ids = nullptr;
  int rc = ctx->pool.alloc(outputs * sizeof(uint32_t), &d_ids, nullptr);
  if (rc) return rc;
  {
    ProfScope prof(ctx, kProfElementwise, s);
    if (mode == B200_MODE_FP16)
      b200::launch(ctx, argminmax_kernel<__half>, dim3(grid_for(ctx, outputs, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const __half *>(x), static_cast<uint32_t *>(d_ids), n, skip1, outputs, want_max);
    else
      b200::launch(ctx, argminmax_kernel<float>, dim3(grid_for(ctx, outputs, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const float *>(x), static_cast<uint32_t *>(d_ids), n, skip1, outputs, want_max);
  }
  ++ctx->launches;
  b200::queue_drain(ctx);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(ids_host, d_ids, outputs * sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  ctx->pool.free(d_ids);
  return e == cudaSuccess ? b200::take_status(ctx) : static_cast<int>(e);
}

int b200_batch_sum_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t volume, uint32_t batch,
                      void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (volume == 0) return B200_OK;
  if (!x || !y) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    const int rc = launch_batch_sum<T>(ctx, s, x, y, volume, batch, 1.f, 0);
    if (rc != B200_OK) return rc;
  });
  B200_OPS_EPILOGUE(ctx);
}

}  // extern "C"
