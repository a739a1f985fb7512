// Shared pieces of the elementwise / movement / reduction kernels.
#ifndef PRIMITIV_B200_CSRC_OPS_COMMON_CUH_
#define PRIMITIV_B200_CSRC_OPS_COMMON_CUH_

#include <cuda_fp16.h>

#include "../../include/primitiv_b200_ops.h"
#include "ctx.h"

namespace b200 {

typedef unsigned long long u64;

__device__ __forceinline__ float ld(const float *p, u64 i) { return p[i]; }
__device__ __forceinline__ float ld(const __half *p, u64 i) { return __half2float(p[i]); }
__device__ __forceinline__ void st(float *p, u64 i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__half *p, u64 i, float v) { p[i] = __float2half_rn(v); }

// 128-bit vectors: 4 floats or 8 halves.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float *p) { raw = *reinterpret_cast<const float4 *>(p); }
  __device__ __forceinline__ void store(float *p) const { *reinterpret_cast<float4 *>(p) = raw; }
  __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float *>(&raw)[i]; }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<float *>(&raw)[i] = v; }
};
template <> struct Vec<__half> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const __half *p) { raw = *reinterpret_cast<const uint4 *>(p); }
  __device__ __forceinline__ void store(__half *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
  __device__ __forceinline__ float get(int i) const {
    return __half2float(reinterpret_cast<const __half *>(&raw)[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    reinterpret_cast<__half *>(&raw)[i] = __float2half_rn(v);
  }
};

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a grid-stride loop over `work` items: enough CTAs to fill the machine a few
// times over, a multiple of the SM count, never more than the work needs.
inline unsigned grid_for(const b200_ctx *ctx, u64 work, unsigned block) {
  const u64 need = (work + block - 1) / block;
  const u64 cap = static_cast<u64>(ctx->sm_count) * 8ull;
  const u64 g = need < cap ? need : cap;
  return static_cast<unsigned>(g ? g : 1);
}

// ---- sums over the batch axis, deterministic and parallel in both directions ----
//
// A CTA is 32 x 8 threads: 32 consecutive elements i of the volume (coalesced) by 8 batch
// lanes.  grid.x walks the volume, grid.y cuts the batch into slices so that a small volume
// with a large batch (a bias gradient over 65536 samples) still fills the machine.  Inside a
// slice, batch lane t adds items t, t + 8, ... in order and the 8 lanes are combined in lane
// order; slices are combined in slice order by batch_final_kernel.  No atomics: the result is
// the same bits on every run.
constexpr unsigned kSumLanes = 8;

struct BatchSlices {
  unsigned tiles;      // grid.x: volume / 32, rounded up
  unsigned slices;     // grid.y
  uint32_t slice_len;  // batch items per slice
};

// tile_elems: consecutive elements of the volume per CTA (32, or 32 vectors of 4 / 8 in the vector forms)
inline BatchSlices batch_slices(const b200_ctx *ctx, u64 volume, uint32_t batch, unsigned tile_elems = 32u) {
  BatchSlices r;
  const u64 tiles = (volume + tile_elems - 1ull) / tile_elems;
  r.tiles = static_cast<unsigned>(tiles < 0x7fffffffull ? tiles : 0x7fffffffull);
  u64 want = (2ull * static_cast<u64>(ctx->sm_count) + tiles - 1) / tiles;  // about two CTAs per SM
  // at least 128 items per slice: a short batch (a recurrent step's 64 items) is one slice and one launch
  const u64 most = batch / (16u * kSumLanes) ? batch / (16u * kSumLanes) : 1;
  if (want > most) want = most;
  if (want > 65535ull) want = 65535ull;
  if (want < 1) want = 1;
  r.slice_len = static_cast<uint32_t>((batch + want - 1) / want);
  r.slices = static_cast<unsigned>((batch + r.slice_len - 1) / r.slice_len);
  return r;
}

// Combines the 8 batch lanes of a CTA (lane order) and returns the total in batch lane 0.
__device__ __forceinline__ float combine_batch_lanes(float v, float (*buf)[32]) {
  buf[threadIdx.y][threadIdx.x] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.y == 0) {
#pragma unroll
    for (unsigned l = 0; l < kSumLanes; ++l) t += buf[l][threadIdx.x];
  }
  __syncthreads();
  return t;
}

// y[i] = (accumulate ? y[i] : 0) + scale * sum over slices of partial[slice][i]
template <typename T>
__global__ void __launch_bounds__(256) batch_final_kernel(const float *__restrict__ partial, T *y, u64 volume,
                                                          unsigned slices, float scale, int accumulate) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 i = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; i < volume; i += stride) {
    float t = 0.f;
    for (unsigned sl = 0; sl < slices; ++sl) t += partial[static_cast<u64>(sl) * volume + i];
    st(y, i, (accumulate ? ld(y, i) : 0.f) + scale * t);
  }
}

// The same for a few outputs with many slices (a scalar loss over 65536 items: one output, 300
// slices): a warp per output, lane l adds slices l, l + 32, ... in order, and the lanes are
// combined by a fixed shuffle tree.  One thread per output would walk the slices as a chain of
// dependent loads.
template <typename T>
__global__ void __launch_bounds__(256) batch_final_warp_kernel(const float *__restrict__ partial, T *y, u64 volume,
                                                               unsigned slices, float scale, int accumulate) {
  pdl_enter();
  const unsigned lane = threadIdx.x & 31u;
  const u64 warps = (static_cast<u64>(gridDim.x) * blockDim.x) >> 5;
  for (u64 i = (static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < volume; i += warps) {
    float t = 0.f;
    for (unsigned sl = lane; sl < slices; sl += 32u) t += partial[static_cast<u64>(sl) * volume + i];
#pragma unroll
    for (unsigned d = 16u; d > 0u; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
    if (lane == 0) st(y, i, (accumulate ? ld(y, i) : 0.f) + scale * t);
  }
}

// Picks the form of the final pass: many slices of few outputs go to the warp form.
template <typename T>
inline void launch_batch_final(b200_ctx *ctx, cudaStream_t s, const float *partial, T *y, u64 volume, unsigned slices,
                               float scale, int accumulate) {
  if (slices >= 64u && volume <= 4096ull)
    b200::launch(ctx, batch_final_warp_kernel<T>, dim3(grid_for(ctx, volume * 32ull, 256)), dim3(256), 0, s, 1u, partial, y,
                 volume, slices, scale, accumulate);
  else
    b200::launch(ctx, batch_final_kernel<T>, dim3(grid_for(ctx, volume, 256)), dim3(256), 0, s, 1u, partial, y, volume,
                 slices, scale, accumulate);
  ++ctx->launches;
}

// y[i] = (accumulate ? y[i] : 0) + scale * sum_n x[n][i]; with more than one slice the CTA's
// sum goes to partial[slice][i] instead.
template <typename T>
__global__ void __launch_bounds__(256) batch_sum_tile_kernel(const T *__restrict__ x, T *y, float *partial,
                                                             u64 volume, uint32_t batch, uint32_t slice_len,
                                                             float scale, int accumulate) {
  pdl_enter();
  __shared__ float buf[kSumLanes][32];
  for (u64 tile = blockIdx.x; tile * 32ull < volume; tile += gridDim.x) {
    const u64 i = tile * 32ull + threadIdx.x;
    const uint32_t lo = blockIdx.y * slice_len;
    const uint32_t hi = lo + slice_len < batch ? lo + slice_len : batch;
    float v = 0.f;
    if (i < volume)
      for (uint32_t n = lo + threadIdx.y; n < hi; n += kSumLanes) v += ld(x, static_cast<u64>(n) * volume + i);
    const float t = combine_batch_lanes(v, buf);
    if (threadIdx.y == 0 && i < volume) {
      if (gridDim.y == 1) st(y, i, (accumulate ? ld(y, i) : 0.f) + scale * t);
      else partial[static_cast<u64>(blockIdx.y) * volume + i] = t;
    }
  }
}

// Combines the 8 batch lanes of a CTA for the N values each thread holds (vector forms).
template <int N>
__device__ __forceinline__ void combine_batch_lanes_vec(float (&v)[N], float (*buf)[32 * N]) {
#pragma unroll
  for (int j = 0; j < N; ++j) buf[threadIdx.y][threadIdx.x * N + j] = v[j];
  __syncthreads();
  if (threadIdx.y == 0) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float t = 0.f;
#pragma unroll
      for (unsigned l = 0; l < kSumLanes; ++l) t += buf[l][threadIdx.x * N + j];
      v[j] = t;
    }
  }
  __syncthreads();
}

// Vector form of batch_sum_tile_kernel (volume a multiple of the vector width, 16-byte aligned
// arrays): a thread owns one 128-bit vector of the volume and keeps four items in flight.
template <typename T>
__global__ void __launch_bounds__(256) batch_sum_tile_vec_kernel(const T *__restrict__ x, T *y, float *partial,
                                                                 u64 volume, uint32_t batch, uint32_t slice_len,
                                                                 float scale, int accumulate) {
  pdl_enter();
  constexpr int N = Vec<T>::N;
  constexpr unsigned U = 4;
  __shared__ float buf[kSumLanes][32 * N];
  for (u64 tile = blockIdx.x; tile * (32ull * N) < volume; tile += gridDim.x) {
    const u64 i = (tile * 32ull + threadIdx.x) * N;
    const uint32_t lo = blockIdx.y * slice_len;
    const uint32_t hi = lo + slice_len < batch ? lo + slice_len : batch;
    float v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = 0.f;
    if (i < volume) {
      for (uint32_t n = lo + threadIdx.y; n < hi; n += kSumLanes * U) {
        Vec<T> vx[U];
#pragma unroll
        for (unsigned u = 0; u < U; ++u)
          if (n + u * kSumLanes < hi) vx[u].load(x + static_cast<u64>(n + u * kSumLanes) * volume + i);
#pragma unroll
        for (unsigned u = 0; u < U; ++u)
          if (n + u * kSumLanes < hi) {
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] += vx[u].get(j);
          }
      }
    }
    combine_batch_lanes_vec<N>(v, buf);
    if (threadIdx.y == 0 && i < volume) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        if (gridDim.y == 1) st(y, i + j, (accumulate ? ld(y, i + j) : 0.f) + scale * v[j]);
        else partial[static_cast<u64>(blockIdx.y) * volume + i + j] = v[j];
      }
    }
  }
}

// Host side of the kernels above.  Returns a CUDA / library status.
template <typename T>
int launch_batch_sum(b200_ctx *ctx, cudaStream_t s, const void *x, void *y, u64 volume, uint32_t batch,
                     float scale, int accumulate) {
  constexpr unsigned N = Vec<T>::N;
  const bool vec = volume % N == 0 && volume >= 32ull * N && aligned16(x);
  const BatchSlices bs = batch_slices(ctx, volume, batch, vec ? 32u * N : 32u);
  void *partial = nullptr;
  if (bs.slices > 1) {
    const int rc = ctx->pool.alloc(static_cast<size_t>(bs.slices) * volume * sizeof(float), &partial, nullptr);
    if (rc != B200_OK) return rc;
  }
  if (vec)
    b200::launch(ctx, batch_sum_tile_vec_kernel<T>, dim3(bs.tiles, bs.slices), dim3(32, kSumLanes), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), static_cast<float *>(partial), volume, batch, bs.slice_len,
        scale, accumulate);
  else
    b200::launch(ctx, batch_sum_tile_kernel<T>, dim3(bs.tiles, bs.slices), dim3(32, kSumLanes), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), static_cast<float *>(partial), volume, batch, bs.slice_len,
        scale, accumulate);
  if (bs.slices > 1) {
    launch_batch_final<T>(ctx, s, static_cast<const float *>(partial), static_cast<T *>(y), volume, bs.slices, scale, accumulate);
    ctx->pool.free(partial);  // stream-ordered reuse
  }
  return B200_OK;
}

#define B200_OPS_PROLOGUE(ctx)                         \
  if (!(ctx)) return B200_ERR_INVALID_ARG;             \
  b200::DeviceGuard guard__((ctx)->device);            \
  cudaStream_t s = static_cast<cudaStream_t>(stream)

#define B200_OPS_EPILOGUE(ctx)   \
  ++(ctx)->launches;             \
  return static_cast<int>(cudaGetLastError())

// Dispatch on storage type: BODY sees `T` as float or __half.
#define B200_DISPATCH_MODE(mode, ...)                          \
  do {                                                         \
    if ((mode) == B200_MODE_FP16) {                            \
      typedef __half T;                                        \
      __VA_ARGS__                                              \
    } else if ((mode) == B200_MODE_FP32_3XTF32 ||              \
               (mode) == B200_MODE_TF32 ||                     \
               (mode) == B200_MODE_FP32_3XFP16) {              \
      typedef float T;                                         \
      __VA_ARGS__                                              \
    } else {                                                   \
      return B200_ERR_INVALID_ARG;                             \
    }                                                          \
  } while (0)

}  // namespace b200

#endif  // PRIMITIV_B200_CSRC_OPS_COMMON_CUH_
