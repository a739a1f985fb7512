// CUDA-core matrix product: the path for operands the tensor-core kernel cannot
// take (leading dimensions or pointers not 16-byte aligned, e.g. 123x123 or
// {10,1024}) and for problems too small to fill a 128-row MMA tile.
//
//   C[g] = (acc ? C[g] : 0) + sum_{r<red} opA(A[g*a_gs + r*a_rs]) . opB(B[g*b_gs + r*b_rs])
//
// 64x64 output tile per CTA, 16-deep k slices staged in shared memory, 4x4
// outputs per thread, fp32 FMA accumulation for both float and half storage;
// half results are rounded once on store.  The reduction over `red` runs inside
// the k loop, so a broadcast operand's gradient is summed without atomics and
// without the serial per-batch GEMM loop of the reference
// (primitiv/devices/cuda/ops/matmul.cu:113-123).
#include <cuda_fp16.h>

#include "ctx.h"

namespace b200 {
namespace {

constexpr int TM = 64, TN = 64, TK = 16, NT = 256;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ void from_f32(float &d, float v) { d = v; }
__device__ __forceinline__ void from_f32(__half &d, float v) { d = __float2half_rn(v); }

template <typename T, bool kTA, bool kTB>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(
    const T *__restrict__ A, const T *__restrict__ B, T *__restrict__ C,
    uint32_t m, uint32_t n, uint32_t k, uint32_t red,
    uint64_t a_gs, uint64_t a_rs, uint64_t b_gs, uint64_t b_rs, uint64_t c_gs,
    int accumulate, uint32_t tiles_m, uint32_t tiles_n) {
  pdl_enter();
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];

  const uint32_t tile = blockIdx.x;
  const uint32_t g = tile / (tiles_m * tiles_n);
  const uint32_t rem = tile - g * tiles_m * tiles_n;
  const uint32_t m0 = (rem % tiles_m) * TM;
  const uint32_t n0 = (rem / tiles_m) * TN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (uint32_t r = 0; r < red; ++r) {
    const T *Ag = A + g * a_gs + r * a_rs;
    const T *Bg = B + g * b_gs + r * b_rs;
    for (uint32_t k0 = 0; k0 < k; k0 += TK) {
#pragma unroll
      for (int i = 0; i < (TM * TK) / NT; ++i) {
        const int e = tid + i * NT;
        int mm, kk;
        if (kTA) { kk = e % TK; mm = e / TK; } else { mm = e % TM; kk = e / TM; }
        const uint32_t gm = m0 + mm, gk = k0 + kk;
        float v = 0.f;
        if (gm < m && gk < k)
          v = to_f32(kTA ? Ag[(uint64_t)gk + (uint64_t)gm * k] : Ag[(uint64_t)gm + (uint64_t)gk * m]);
        As[kk][mm] = v;
      }
#pragma unroll
      for (int i = 0; i < (TN * TK) / NT; ++i) {
        const int e = tid + i * NT;
        int nn, kk;
        if (kTB) { nn = e % TN; kk = e / TN; } else { kk = e % TK; nn = e / TK; }
        const uint32_t gn = n0 + nn, gk = k0 + kk;
        float v = 0.f;
        if (gn < n && gk < k)
          v = to_f32(kTB ? Bg[(uint64_t)gn + (uint64_t)gk * n] : Bg[(uint64_t)gk + (uint64_t)gn * k]);
        Bs[kk][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        float av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = As[kk][tx + 16 * i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][ty + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

  T *Cg = C + g * c_gs;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t gn = n0 + ty + 16 * j;
    if (gn >= n) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t gm = m0 + tx + 16 * i;
      if (gm >= m) continue;
      T *p = Cg + (uint64_t)gm + (uint64_t)gn * m;
      float v = acc[i][j];
      if (accumulate) v += to_f32(*p);
      from_f32(*p, v);
    }
  }
}

template <typename T>
int launch(b200_ctx *ctx, const GemmArgs &a, cudaStream_t s) {
  const uint32_t tiles_m = (a.m + TM - 1) / TM, tiles_n = (a.n + TN - 1) / TN;
  const uint64_t tiles = (uint64_t)tiles_m * tiles_n * a.groups;
  if (tiles == 0) return B200_OK;
  if (tiles > 0x7fffffffull) return B200_ERR_TOO_LARGE;
  const dim3 grid((unsigned)tiles), block(NT);
  const T *A = static_cast<const T *>(a.A);
  const T *B = static_cast<const T *>(a.B);
  T *C = static_cast<T *>(a.C);
  ProfScope prof(ctx, kProfGemmSimt, s);
#define B200_SIMT_LAUNCH(TA, TB)                                                              \
  b200::launch(ctx, gemm_simt_kernel<T, TA, TB>, dim3(grid), dim3(block), 0, s, 1u, A, B, C, a.m, a.n, a.k, a.red, a.a_gs, \
                                                     a.a_rs, a.b_gs, a.b_rs, a.c_gs,        \
                                                     a.accumulate, tiles_m, tiles_n)
  if (a.trans_a) {
    if (a.trans_b) B200_SIMT_LAUNCH(true, true); else B200_SIMT_LAUNCH(true, false);
  } else {
    if (a.trans_b) B200_SIMT_LAUNCH(false, true); else B200_SIMT_LAUNCH(false, false);
  }
#undef B200_SIMT_LAUNCH
  ++ctx->launches;
  return (int)cudaGetLastError();
}

}  // namespace

int gemm_simt(b200_ctx *ctx, const GemmArgs &a, cudaStream_t s) {
  if (a.mode == B200_MODE_FP16) return launch<__half>(ctx, a, s);
  return launch<float>(ctx, a, s);
}

}  // namespace b200
