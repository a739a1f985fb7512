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
               (mode) == B200_MODE_TF32) {                     \
      typedef float T;                                         \
      __VA_ARGS__                                              \
    } else {                                                   \
      return B200_ERR_INVALID_ARG;                             \
    }                                                          \
  } while (0)

}  // namespace b200

#endif  // PRIMITIV_B200_CSRC_OPS_COMMON_CUH_
