// Products with one tiny extent against large ones, on CUDA cores in fp32: the 10-row output
// layer of a perceptron over a 65536-item minibatch and its two gradients
// (primitiv/examples/mnist/mnist.cc:105-117 at a large batch).  They are HBM-bound: the large
// operand (or the large result) should cross HBM once.  The tensor-core path would pack that
// operand into planes first (three passes over it) and run 128-row tiles that are 92 % padding.
//
// Three shapes, each with the operand layout that primitiv's matmul_fw / matmul_bw produce for it
// (C is m x n column-major; A(i,kk), B(kk,j)):
//   rows    m <= 16, B stored k x n (a column's k values contiguous):   y = W . X
//   reduce  m <= 16, A stored m x k, B stored n x k, k long:            gW += gy . X^T
//   outer   k <= 16, A stored k x m, B stored k x n:                    gX += W^T . gy
// Arithmetic is fp32 FMA in a fixed order (no atomics): results do not depend on the launch.
#include <cstdint>

#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr uint32_t kSkinnyMax = 16;          // the tiny extent
constexpr uint32_t kSmemFloats = 12288;      // 48 KB of staging, no opt-in needed

// Padded length of a staged tiny vector: a multiple of 4 floats (128-bit shared loads) and
// congruent to 4 mod 8, so that eight consecutive vectors start in eight different bank groups.
__host__ __device__ inline uint32_t padded(uint32_t t) { return t <= 4 ? 4u : (t <= 12 ? 12u : 20u); }

// ---- rows: each warp owns kCols columns of B and C; lanes stride over k ----
template <typename T, uint32_t MP, uint32_t kCols>
__global__ void __launch_bounds__(256, MP <= 12 ? 4 : 2) skinny_rows_kernel(const T *__restrict__ A, const T *__restrict__ B, T *C,
                                                          uint32_t m, uint32_t n, uint32_t k, u64 a_si, u64 a_sk,
                                                          int accumulate) {
  pdl_enter();
  constexpr uint32_t kDepth = 4;  // k-steps whose loads are in flight together (8 measured slower)
  extern __shared__ __align__(16) float As[];  // [k][MP], rows past m are zero
  for (uint32_t e = threadIdx.x; e < k * MP; e += blockDim.x) {
    const uint32_t kk = e / MP, i = e % MP;
    As[e] = i < m ? ld(A, i * a_si + kk * a_sk) : 0.f;
  }
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (u64 j0 = (static_cast<u64>(blockIdx.x) * warps + warp) * kCols; j0 < n;
       j0 += static_cast<u64>(gridDim.x) * warps * kCols) {
    float acc[kCols][MP];
#pragma unroll
    for (uint32_t c = 0; c < kCols; ++c)
#pragma unroll
      for (uint32_t i = 0; i < MP; ++i) acc[c][i] = 0.f;
    // kDepth k-steps per pass: their loads are issued together (kDepth x kCols requests of 128 B in flight per warp)
    for (uint32_t kk0 = lane; kk0 < k; kk0 += 32u * kDepth) {
      float b[kDepth][kCols];
#pragma unroll
      for (uint32_t u = 0; u < kDepth; ++u)
#pragma unroll
        for (uint32_t c = 0; c < kCols; ++c)
          b[u][c] = (kk0 + 32u * u < k && j0 + c < n) ? ld(B, (j0 + c) * k + kk0 + 32u * u) : 0.f;
#pragma unroll
      for (uint32_t u = 0; u < kDepth; ++u) {
        const uint32_t kk = kk0 + 32u * u < k ? kk0 + 32u * u : 0u;  // b is zero there
        const float4 *arow = reinterpret_cast<const float4 *>(As + kk * MP);
#pragma unroll
        for (uint32_t q = 0; q < MP / 4; ++q) {
          const float4 a = arow[q];
#pragma unroll
          for (uint32_t c = 0; c < kCols; ++c) {
            acc[c][4 * q + 0] += a.x * b[u][c];
            acc[c][4 * q + 1] += a.y * b[u][c];
            acc[c][4 * q + 2] += a.z * b[u][c];
            acc[c][4 * q + 3] += a.w * b[u][c];
          }
        }
      }
    }
    // Lanes hold partial sums over their k values.  Three halving steps (lane bits 4, 3, 2): a
    // lane passes the half of its values that its partner keeps and adds what it receives, so
    // V values cost V/2 + V/4 + V/8 shuffles instead of 3 V; the V/8 values left are summed over
    // lane bits 1 and 0 the plain way.  The order of additions is fixed.
    constexpr uint32_t V = kCols * MP;  // 16, 24 or 40: a multiple of 8
    float *v = &acc[0][0];
#pragma unroll
    for (uint32_t step = 0; step < 3u; ++step) {
      const uint32_t off = 16u >> step, half = V >> (step + 1u);
      const bool upper = (lane & off) != 0u;
#pragma unroll
      for (uint32_t i = 0; i < half; ++i) {
        const float send = upper ? v[i] : v[i + half];
        const float keep = upper ? v[i + half] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
    constexpr uint32_t R = V / 8u;
#pragma unroll
    for (uint32_t i = 0; i < R; ++i) {
      v[i] += __shfl_xor_sync(0xffffffffu, v[i], 2u);
      v[i] += __shfl_xor_sync(0xffffffffu, v[i], 1u);
    }
    // which values this lane ended up with follows from the halves it kept
    const uint32_t first = ((lane >> 4) & 1u) * (V / 2u) + ((lane >> 3) & 1u) * (V / 4u) + ((lane >> 2) & 1u) * R;
    if ((lane & 3u) == 0u) {
#pragma unroll
      for (uint32_t t = 0; t < R; ++t) {
        const uint32_t e = first + t, c = e / MP, i = e % MP;
        if (i < m && j0 + c < n) {
          const u64 at = (j0 + c) * m + i;
          st(C, at, (accumulate ? ld(C, at) : 0.f) + v[t]);
        }
      }
    }
  }
}

// ---- reduce: thread owns kCols columns j (coalesced along j), the CTA owns a slice of k ----
// Writes the slice's partial C to partial[slice][j * m + i]; reduce_final_kernel adds the slices in order.
template <typename T, uint32_t MP, uint32_t kCols>
__global__ void __launch_bounds__(256, MP <= 12 ? 4 : 2) skinny_reduce_kernel(const T *__restrict__ A, const T *__restrict__ B,
                                                            float *__restrict__ partial, uint32_t m, uint32_t n,
                                                            uint32_t k, uint32_t slice_len) {
  pdl_enter();
  constexpr uint32_t kDepth = 4;  // k-steps whose loads are in flight together (8 measured slower)
  extern __shared__ __align__(16) float As[];  // [chunk][MP]
  const uint32_t chunk_cap = kSmemFloats / MP;
  const uint32_t k_lo = blockIdx.y * slice_len;
  const uint32_t k_hi = k_lo + slice_len < k ? k_lo + slice_len : k;
  const u64 jbase = static_cast<u64>(blockIdx.x) * blockDim.x * kCols + threadIdx.x;
  float acc[kCols][MP];
#pragma unroll
  for (uint32_t c = 0; c < kCols; ++c)
#pragma unroll
    for (uint32_t i = 0; i < MP; ++i) acc[c][i] = 0.f;
  for (uint32_t c0 = k_lo; c0 < k_hi; c0 += chunk_cap) {
    const uint32_t len = k_hi - c0 < chunk_cap ? k_hi - c0 : chunk_cap;
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < len * MP; e += blockDim.x) {
      const uint32_t kk = e / MP, i = e % MP;
      As[e] = i < m ? ld(A, static_cast<u64>(c0 + kk) * m + i) : 0.f;  // A stored m x k
    }
    __syncthreads();
    for (uint32_t kk0 = 0; kk0 < len; kk0 += kDepth) {
      float b[kDepth][kCols];
#pragma unroll
      for (uint32_t u = 0; u < kDepth; ++u)
#pragma unroll
        for (uint32_t c = 0; c < kCols; ++c) {
          const u64 j = jbase + static_cast<u64>(c) * blockDim.x;
          b[u][c] = (kk0 + u < len && j < n) ? ld(B, static_cast<u64>(c0 + kk0 + u) * n + j) : 0.f;  // B stored n x k
        }
#pragma unroll
      for (uint32_t u = 0; u < kDepth; ++u) {
        const uint32_t kk = kk0 + u < len ? kk0 + u : 0u;  // b is zero there
        const float4 *arow = reinterpret_cast<const float4 *>(As + kk * MP);  // one address per warp: broadcast
#pragma unroll
        for (uint32_t q = 0; q < MP / 4; ++q) {
          const float4 a = arow[q];
#pragma unroll
          for (uint32_t c = 0; c < kCols; ++c) {
            acc[c][4 * q + 0] += a.x * b[u][c];
            acc[c][4 * q + 1] += a.y * b[u][c];
            acc[c][4 * q + 2] += a.z * b[u][c];
            acc[c][4 * q + 3] += a.w * b[u][c];
          }
        }
      }
    }
  }
  float *out = partial + static_cast<u64>(blockIdx.y) * m * n;
#pragma unroll
  for (uint32_t c = 0; c < kCols; ++c) {
    const u64 j = jbase + static_cast<u64>(c) * blockDim.x;
    if (j < n) {
#pragma unroll
      for (uint32_t i = 0; i < MP; ++i)
        if (i < m) out[j * m + i] = acc[c][i];
    }
  }
}

// C[e] = (accumulate ? C[e] : 0) + sum over slices, in slice order within a lane and lane order
// across the 8 lanes that share an element: 32 consecutive elements (coalesced) by 8 slice lanes.
template <typename T>
__global__ void __launch_bounds__(256) reduce_final_kernel(const float *__restrict__ partial, T *C, u64 count,
                                                           uint32_t slices, int accumulate) {
  pdl_enter();
  __shared__ float buf[8][32];
  const u64 e = static_cast<u64>(blockIdx.x) * 32u + threadIdx.x;
  float t = 0.f;
  if (e < count)
    for (uint32_t s = threadIdx.y; s < slices; s += 8u) t += partial[static_cast<u64>(s) * count + e];
  buf[threadIdx.y][threadIdx.x] = t;
  __syncthreads();
  if (threadIdx.y == 0 && e < count) {
    float total = 0.f;
#pragma unroll
    for (uint32_t l = 0; l < 8u; ++l) total += buf[l][threadIdx.x];
    st(C, e, (accumulate ? ld(C, e) : 0.f) + total);
  }
}

// ---- outer: thread owns two rows, the CTA a strip of columns; A's k values sit in registers ----
template <typename T, uint32_t KP, bool accumulate>
__global__ void __launch_bounds__(256, 4) skinny_outer_kernel(const T *__restrict__ A, const T *__restrict__ B, T *C,
                                                              uint32_t m, uint32_t n, uint32_t k, uint32_t strip) {
  pdl_enter();
  extern __shared__ __align__(16) float Bs[];  // [strip][KP], entries past k are zero
  const u64 j_lo = static_cast<u64>(blockIdx.y) * strip;
  const uint32_t cols = n - j_lo < strip ? static_cast<uint32_t>(n - j_lo) : strip;
  for (uint32_t e = threadIdx.x; e < cols * KP; e += blockDim.x) {
    const uint32_t c = e / KP, kk = e % KP;
    Bs[e] = kk < k ? ld(B, (j_lo + c) * k + kk) : 0.f;  // B stored k x n
  }
  // two rows per thread, a block apart (each store of a warp stays one 128-byte line)
  const u64 i0 = static_cast<u64>(blockIdx.x) * blockDim.x * 2u + threadIdx.x, i1 = i0 + blockDim.x;
  float a0[KP], a1[KP];
#pragma unroll
  for (uint32_t kk = 0; kk < KP; ++kk) {
    a0[kk] = (i0 < m && kk < k) ? ld(A, i0 * k + kk) : 0.f;  // A stored k x m
    a1[kk] = (i1 < m && kk < k) ? ld(A, i1 * k + kk) : 0.f;
  }
  __syncthreads();
  if (i0 >= m) return;
  const bool two = i1 < m;
  // four columns at a time: for += the old values are fetched before the first store
  // (a load-add-store per column would pay one memory latency per column)
  for (uint32_t c0 = 0; c0 < cols; c0 += 4u) {
    float old0[4], old1[4];
#pragma unroll
    for (uint32_t u = 0; u < 4u; ++u) {
      const bool live = accumulate && c0 + u < cols;
      old0[u] = live ? ld(C, (j_lo + c0 + u) * m + i0) : 0.f;
      old1[u] = (live && two) ? ld(C, (j_lo + c0 + u) * m + i1) : 0.f;
    }
#pragma unroll
    for (uint32_t u = 0; u < 4u; ++u) {
      if (c0 + u < cols) {
        const float4 *bcol = reinterpret_cast<const float4 *>(Bs + (c0 + u) * KP);  // broadcast
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (uint32_t q = 0; q < KP / 4; ++q) {
          const float4 b = bcol[q];
          t0 += a0[4 * q + 0] * b.x; t1 += a1[4 * q + 0] * b.x;
          t0 += a0[4 * q + 1] * b.y; t1 += a1[4 * q + 1] * b.y;
          t0 += a0[4 * q + 2] * b.z; t1 += a1[4 * q + 2] * b.z;
          t0 += a0[4 * q + 3] * b.w; t1 += a1[4 * q + 3] * b.w;
        }
        st(C, (j_lo + c0 + u) * m + i0, old0[u] + t0);
        if (two) st(C, (j_lo + c0 + u) * m + i1, old1[u] + t1);
      }
    }
  }
}

}  // namespace

// Which of the three kernels takes this product, if any.
enum SkinnyKind { kNotSkinny = 0, kRows, kReduce, kOuter };

static SkinnyKind skinny_kind(const GemmArgs &g) {
  if (g.groups != 1 || g.red != 1) return kNotSkinny;
  const u64 m = g.m, n = g.n, k = g.k;
  if (m <= kSkinnyMax && !g.trans_b && n >= 2048 && k >= 64 && padded(g.m) * k <= kSmemFloats) return kRows;
  if (m <= kSkinnyMax && !g.trans_a && g.trans_b && k >= 8192 && n >= 256) return kReduce;
  if (k <= kSkinnyMax && g.trans_a && !g.trans_b && m >= 256 && n >= 1024) return kOuter;
  return kNotSkinny;
}

bool gemm_skinny_eligible(const GemmArgs &g) { return skinny_kind(g) != kNotSkinny; }

template <typename T>
static int skinny_run(b200_ctx *ctx, const GemmArgs &g, cudaStream_t s) {
  const T *A = static_cast<const T *>(g.A), *B = static_cast<const T *>(g.B);
  T *C = static_cast<T *>(g.C);
  const SkinnyKind kind = skinny_kind(g);
  ProfScope prof(ctx, kProfGemmSimt, s);
  if (kind == kRows) {
    const uint32_t mp = padded(g.m);
    const u64 a_si = g.trans_a ? g.k : 1, a_sk = g.trans_a ? 1 : g.m;
    const size_t smem = static_cast<size_t>(mp) * g.k * sizeof(float);
    const u64 col_groups = (static_cast<u64>(g.n) + 1) / 2;  // two columns per warp pass (four with mp == 4)
    const u64 want = (col_groups + 7) / 8, cap = static_cast<u64>(ctx->sm_count) * 4;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    if (mp == 4) b200::launch(ctx, skinny_rows_kernel<T, 4, 4>, dim3(grid), dim3(256), smem, s, 1u, A, B, C, g.m, g.n, g.k, a_si, a_sk, g.accumulate);
    else if (mp == 12) b200::launch(ctx, skinny_rows_kernel<T, 12, 2>, dim3(grid), dim3(256), smem, s, 1u, A, B, C, g.m, g.n, g.k, a_si, a_sk, g.accumulate);
    else b200::launch(ctx, skinny_rows_kernel<T, 20, 2>, dim3(grid), dim3(256), smem, s, 1u, A, B, C, g.m, g.n, g.k, a_si, a_sk, g.accumulate);
    ++ctx->launches;
    return static_cast<int>(cudaGetLastError());
  }
  if (kind == kReduce) {
    const uint32_t mp = padded(g.m);
    const uint32_t cols = mp == 4 ? 4u : 2u;
    const unsigned gx = static_cast<unsigned>((static_cast<u64>(g.n) + 256ull * cols - 1) / (256ull * cols));
    // about four CTAs per SM, slices of at least 64 k values
    u64 slices = (4ull * ctx->sm_count + gx - 1) / gx;
    if (slices > g.k / 64) slices = g.k / 64;
    if (slices < 1) slices = 1;
    const uint32_t slice_len = static_cast<uint32_t>((g.k + slices - 1) / slices);
    const unsigned gy = (g.k + slice_len - 1) / slice_len;
    const u64 count = static_cast<u64>(g.m) * g.n;
    void *partial = nullptr;
    const int rc = ctx->pool.alloc(static_cast<size_t>(gy) * count * sizeof(float), &partial, nullptr);
    if (rc != B200_OK) return rc;
    const uint32_t chunk = slice_len < kSmemFloats / mp ? slice_len : kSmemFloats / mp;
    const size_t smem = static_cast<size_t>(chunk) * mp * sizeof(float);
    float *pp = static_cast<float *>(partial);
    if (mp == 4) b200::launch(ctx, skinny_reduce_kernel<T, 4, 4>, dim3(gx, gy), dim3(256), smem, s, 1u, A, B, pp, g.m, g.n, g.k, slice_len);
    else if (mp == 12) b200::launch(ctx, skinny_reduce_kernel<T, 12, 2>, dim3(gx, gy), dim3(256), smem, s, 1u, A, B, pp, g.m, g.n, g.k, slice_len);
    else b200::launch(ctx, skinny_reduce_kernel<T, 20, 2>, dim3(gx, gy), dim3(256), smem, s, 1u, A, B, pp, g.m, g.n, g.k, slice_len);
    b200::launch(ctx, reduce_final_kernel<T>, dim3(static_cast<unsigned>((count + 31) / 32)), dim3(32, 8), 0, s, 1u, pp, C, count, gy, g.accumulate);
    ctx->launches += 2;
    ctx->pool.free(partial);  // stream-ordered reuse
    return static_cast<int>(cudaGetLastError());
  }
  if (kind == kOuter) {
    const uint32_t kp = (g.k + 3u) & ~3u;
    const uint32_t strip = 256;  // columns per CTA: the staging of B and of A's rows is paid once per strip
    const dim3 grid((g.m + 511u) / 512u, (g.n + strip - 1) / strip);
    if (grid.y > 65535u) return gemm_simt(ctx, g, s);
    const size_t smem = static_cast<size_t>(strip) * kp * sizeof(float);
#define B200_OUTER(KP)                                                                                   \
  (g.accumulate ? b200::launch(ctx, skinny_outer_kernel<T, KP, true>, dim3(grid), dim3(256), smem, s, 1u, A, B, C, g.m, g.n, g.k, strip) \
                : b200::launch(ctx, skinny_outer_kernel<T, KP, false>, dim3(grid), dim3(256), smem, s, 1u, A, B, C, g.m, g.n, g.k, strip))
    if (kp == 4) B200_OUTER(4);
    else if (kp == 8) B200_OUTER(8);
    else if (kp == 12) B200_OUTER(12);
    else B200_OUTER(16);
#undef B200_OUTER
    ++ctx->launches;
    return static_cast<int>(cudaGetLastError());
  }
  return B200_ERR_INVALID_ARG;
}

int gemm_skinny(b200_ctx *ctx, const GemmArgs &g, cudaStream_t s) {
  if (g.mode == B200_MODE_FP16) return skinny_run<__half>(ctx, g, s);
  return skinny_run<float>(ctx, g, s);
}

}  // namespace b200
