// Random fills: Bernoulli, uniform, normal, log-normal.
//
// Counter-based Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as
// 1, 2, 3", SC'11): the 128-bit counter is (element block, call number), the 64-bit key
// is the device seed, so the value of element i of the c-th fill depends only on
// (seed, c, i) and never on the launch geometry.  The reference's CUDA device uses
// cuRAND's XORWOW (primitiv/internal/cuda/utils.h:114-118); its streams are a property
// of that generator and are not reproduced here.
//   uniform   : (lower, upper], as primitiv/core/random.h documents
//   bernoulli : 1 with probability p
//   normal    : Box-Muller on two uniforms
#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr unsigned kBlock = 256;

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

__device__ __forceinline__ float u01_open_low(uint32_t x) { return ((x >> 8) + 1u) * 5.9604644775390625e-8f; }  // (0, 1]
__device__ __forceinline__ float u01_open_high(uint32_t x) { return (x >> 8) * 5.9604644775390625e-8f; }        // [0, 1)

template <typename T>
__global__ void __launch_bounds__(kBlock) random_kernel(T *__restrict__ y, u64 n, int kind, float p0, float p1,
                                                        uint2 key, u64 call) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 blocks = (n + 3) / 4;
  for (u64 b = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; b < blocks; b += stride) {
    const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(b), static_cast<uint32_t>(b >> 32),
                                             static_cast<uint32_t>(call), static_cast<uint32_t>(call >> 32)),
                                  key);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    float v[4];
    if (kind == B200_RAND_BERNOULLI) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = u01_open_high(w[j]) < p0 ? 1.f : 0.f;
    } else if (kind == B200_RAND_UNIFORM) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = p0 + (p1 - p0) * u01_open_low(w[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const float rad = sqrtf(-2.f * logf(u01_open_low(w[j])));
        float sn, cs;
        sincospif(2.f * u01_open_high(w[j + 1]), &sn, &cs);
        v[j] = p0 + p1 * rad * cs;
        v[j + 1] = p0 + p1 * rad * sn;
      }
      if (kind == B200_RAND_LOG_NORMAL) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = expf(v[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const u64 i = b * 4 + j;
      if (i < n) st(y, i, v[j]);
    }
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_seed(b200_ctx *ctx, uint64_t seed) {
  if (!ctx) return B200_ERR_INVALID_ARG;
  ctx->rng_seed = seed;
  ctx->rng_calls = 0;
  return B200_OK;
}

int b200_random(b200_ctx *ctx, int mode, int kind, float p0, float p1, void *y, uint64_t n, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!y || kind < B200_RAND_BERNOULLI || kind > B200_RAND_LOG_NORMAL) return B200_ERR_INVALID_ARG;
  const uint2 key = make_uint2(static_cast<uint32_t>(ctx->rng_seed), static_cast<uint32_t>(ctx->rng_seed >> 32));
  const u64 call = ctx->rng_calls++;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, random_kernel<T>, dim3(grid_for(ctx, (n + 3) / 4, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<T *>(y), n, kind, p0, p1, key,
                                                                           call);
  });
  B200_OPS_EPILOGUE(ctx);
}

}  // extern "C"
