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
#include <cstdlib>

#include "mbar.cuh"
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

// ---------------------------------------------------------------------------------------------
// Fast forms of the three kernels for fp32 storage with 16-byte aligned, 4-divisible extents (the
// shapes a layer of a few rows over a large minibatch produces).  They move 128 bits per access,
// keep the tiny operand in registers where the kernels above re-read it from shared memory for
// every loaded element (24 bytes of shared memory per 4-byte element of the large operand), and
// need no warp reduction per column pair where a different split of the work avoids it.

// Packed fp32 arithmetic (sm_100: two independent fp32 FMAs per instruction, round-to-nearest each,
// the same results as two scalar FMAs).  These kernels are bound by instruction issue, ten FMAs per
// loaded element, so halving the FMA instructions is most of what there is to win.
typedef unsigned long long f32x2;   // {low float, high float}
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ void fma2(f32x2 &acc, f32x2 a, f32x2 b) { asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b)); }

// rows, k <= 1024: the CTA's 8 warps split k, 128 values each, 4 consecutive ones per lane, and
// every lane keeps its 4 x MP values of A in registers for the whole launch.  All warps walk the
// CTA's columns together, four at a time (the next four already in flight): one 128-bit load per
// lane and column, 4 MP FMAs, and a halving reduction across the warp (V/2 + V/4 + V/8 + V/4
// shuffles for V = 4 MP values).  The warps' sums over their k-slices meet in shared memory, one
// tile of 32 columns at a time, and are added in warp order: no atomics, a fixed order.
template <uint32_t MP>
__global__ void __launch_bounds__(256, 2) skinny_rows_reg_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                                 float *C, uint32_t m, uint32_t n, uint32_t k, u64 a_si,
                                                                 u64 a_sk, int accumulate) {
  pdl_enter();
  static_assert(MP % 2 == 0 && MP <= 16, "rows padded to an even count");
  constexpr uint32_t V = 4 * MP, R = V / 8;   // values per four columns; values a lane keeps after three halvings
  __shared__ float part[2][8][32 * MP];       // [buffer][warp][column in tile][row]
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t kk0 = warp * 128u + lane * 4u;
  f32x2 w[4][MP / 2];   // rows (2p, 2p + 1) of A at the lane's four k values
#pragma unroll
  for (uint32_t t = 0; t < 4u; ++t)
#pragma unroll
    for (uint32_t pr = 0; pr < MP / 2; ++pr) {
      const uint32_t i = 2u * pr;
      const float lo = (i < m && kk0 + t < k) ? A[i * a_si + (kk0 + t) * a_sk] : 0.f;
      const float hi = (i + 1u < m && kk0 + t < k) ? A[(i + 1u) * a_si + (kk0 + t) * a_sk] : 0.f;
      w[t][pr] = pack2(lo, hi);
    }
  const bool live = kk0 < k;   // k % 4 == 0: a lane's four values are all inside or all outside
  const uint32_t tiles = (n + 31u) / 32u;
  uint32_t buf = 0;
  for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, buf ^= 1u) {
    const u64 j0 = static_cast<u64>(tile) * 32u;
    float4 nxt[4];
#pragma unroll
    for (uint32_t u = 0; u < 4u; ++u)
      nxt[u] = (live && j0 + u < n) ? *reinterpret_cast<const float4 *>(B + (j0 + u) * k + kk0) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t c0 = 0; c0 < 32u; c0 += 4u) {
      float4 b[4];
#pragma unroll
      for (uint32_t u = 0; u < 4u; ++u) b[u] = nxt[u];
      if (c0 + 4u < 32u) {
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u)
          nxt[u] = (live && j0 + c0 + 4u + u < n) ? *reinterpret_cast<const float4 *>(B + (j0 + c0 + 4u + u) * k + kk0)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float v[V];   // v[u * MP + i]
#pragma unroll
      for (uint32_t u = 0; u < 4u; ++u) {
        const f32x2 bx = pack2(b[u].x, b[u].x), by = pack2(b[u].y, b[u].y), bz = pack2(b[u].z, b[u].z),
                    bw = pack2(b[u].w, b[u].w);
#pragma unroll
        for (uint32_t pr = 0; pr < MP / 2; ++pr) {
          f32x2 t = pack2(0.f, 0.f);
          fma2(t, w[0][pr], bx);
          fma2(t, w[1][pr], by);
          fma2(t, w[2][pr], bz);
          fma2(t, w[3][pr], bw);
          unpack2(t, v[u * MP + 2u * pr], v[u * MP + 2u * pr + 1u]);
        }
      }
      // three halving steps (lane bits 4, 3, 2): a lane sends the half its partner keeps
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
#pragma unroll
      for (uint32_t i = 0; i < R; ++i) {
        v[i] += __shfl_xor_sync(0xffffffffu, v[i], 2u);
        v[i] += __shfl_xor_sync(0xffffffffu, v[i], 1u);
      }
      const uint32_t first = ((lane >> 4) & 1u) * (V / 2u) + ((lane >> 3) & 1u) * (V / 4u) + ((lane >> 2) & 1u) * R;
      if ((lane & 3u) == 0u) {
#pragma unroll
        for (uint32_t t = 0; t < R; ++t) part[buf][warp][c0 * MP + first + t] = v[t];
      }
    }
    __syncthreads();   // (the other buffer is free again once every warp has passed this point)
    // 32 columns x m rows of C are contiguous: warps' sums added in warp order
    for (uint32_t e = threadIdx.x; e < 32u * m; e += blockDim.x) {
      const uint32_t c = e / m, i = e - c * m;
      if (j0 + c < n) {
        float t = 0.f;
#pragma unroll
        for (uint32_t wv = 0; wv < 8u; ++wv) t += part[buf][wv][c * MP + i];
        const u64 at = (j0 + c) * m + i;
        C[at] = (accumulate ? C[at] : 0.f) + t;
      }
    }
  }
}

// reduce, n % 4 == 0: a thread owns four consecutive columns (one 128-bit load per k value), the
// CTA a slice of k; A's slice is staged in shared memory and broadcast.
template <uint32_t MP>
__global__ void __launch_bounds__(256, 2) skinny_reduce4_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                                float *__restrict__ partial, uint32_t m, uint32_t n,
                                                                uint32_t k, uint32_t slice_len) {
  pdl_enter();
  constexpr uint32_t kDepth = 8;   // k values whose 128-bit loads are in flight together: 32 KB per CTA
  constexpr uint32_t AP = (MP + 3u) & ~3u;   // staged row length: whole 128-bit words
  extern __shared__ __align__(16) float As[];  // [chunk][AP]
  const uint32_t chunk_cap = kSmemFloats / AP;
  const uint32_t k_lo = blockIdx.y * slice_len;
  const uint32_t k_hi = k_lo + slice_len < k ? k_lo + slice_len : k;
  const u64 j = (static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x) * 4u;
  const bool col_ok = j < n;   // n % 4 == 0: all four columns or none
  f32x2 acc[4][MP / 2];   // rows (2p, 2p + 1) of the four columns
#pragma unroll
  for (uint32_t c = 0; c < 4u; ++c)
#pragma unroll
    for (uint32_t pr = 0; pr < MP / 2; ++pr) acc[c][pr] = pack2(0.f, 0.f);
  for (uint32_t c0 = k_lo; c0 < k_hi; c0 += chunk_cap) {
    const uint32_t len = k_hi - c0 < chunk_cap ? k_hi - c0 : chunk_cap;
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < len * AP; e += blockDim.x) {
      const uint32_t kk = e / AP, i = e % AP;
      As[e] = i < m ? A[static_cast<u64>(c0 + kk) * m + i] : 0.f;  // A stored m x k
    }
    __syncthreads();
    for (uint32_t kk0 = 0; kk0 < len; kk0 += kDepth) {
      float4 b[kDepth];
#pragma unroll
      for (uint32_t u = 0; u < kDepth; ++u)
        b[u] = (kk0 + u < len && col_ok) ? *reinterpret_cast<const float4 *>(B + static_cast<u64>(c0 + kk0 + u) * n + j)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);   // B stored n x k
#pragma unroll
      for (uint32_t u = 0; u < kDepth; ++u) {
        const uint32_t kk = kk0 + u < len ? kk0 + u : 0u;  // b is zero there
        // one address per warp: broadcast; a 128-bit load is two ready-made pairs of A's rows
        const ulonglong2 *arow = reinterpret_cast<const ulonglong2 *>(As + kk * AP);
        f32x2 a[AP / 2];
#pragma unroll
        for (uint32_t q = 0; q < AP / 4; ++q) {
          const ulonglong2 t = arow[q];
          a[2 * q] = t.x;
          a[2 * q + 1] = t.y;
        }
        const f32x2 bx = pack2(b[u].x, b[u].x), by = pack2(b[u].y, b[u].y), bz = pack2(b[u].z, b[u].z),
                    bw = pack2(b[u].w, b[u].w);
#pragma unroll
        for (uint32_t pr = 0; pr < MP / 2; ++pr) {
          fma2(acc[0][pr], a[pr], bx);
          fma2(acc[1][pr], a[pr], by);
          fma2(acc[2][pr], a[pr], bz);
          fma2(acc[3][pr], a[pr], bw);
        }
      }
    }
  }
  if (col_ok) {
    float *out = partial + static_cast<u64>(blockIdx.y) * m * n;
#pragma unroll
    for (uint32_t c = 0; c < 4u; ++c)
#pragma unroll
      for (uint32_t pr = 0; pr < MP / 2; ++pr) {
        float lo, hi;
        unpack2(acc[c][pr], lo, hi);
        if (2u * pr < m) out[(j + c) * m + 2u * pr] = lo;
        if (2u * pr + 1u < m) out[(j + c) * m + 2u * pr + 1u] = hi;
      }
  }
}

// reduce through a shared-memory ring: the CTA owns a slice of k and up to 1024 columns.  One
// producer thread streams the slice of B (rows of n contiguous floats) into a four-stage ring with
// bulk copies, eight rows = 32 KB per stage, 128 KB in flight per SM, so the consumers never wait on
// a load of their own; the sixteen consumer warps own two columns per thread and read B with one
// 64-bit shared load per k value, A's slice as broadcasts.  One CTA per SM.
constexpr uint32_t kRingStages = 4, kRingRows = 8, kRingCols = 1024;
constexpr size_t kRingBytes = static_cast<size_t>(kRingStages) * kRingRows * kRingCols * sizeof(float);

template <uint32_t MP>
__global__ void __launch_bounds__(544, 1) skinny_reduce_ring_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                                    float *__restrict__ partial, uint32_t m, uint32_t n,
                                                                    uint32_t k, uint32_t slice_len, int *status) {
  pdl_enter();
  constexpr uint32_t AP = (MP + 3u) & ~3u;
  extern __shared__ __align__(128) unsigned char ring_smem[];
  float *stages = reinterpret_cast<float *>(ring_smem);                 // [stage][row][cols]
  float *As = stages + kRingStages * kRingRows * kRingCols;             // [row of the slice][AP]
  __shared__ __align__(8) uint64_t full_bar[kRingStages];
  __shared__ __align__(8) uint64_t empty_bar[kRingStages];
  __shared__ int s_abort;
  volatile int *abort_flag = &s_abort;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t col0 = blockIdx.x * kRingCols;
  const uint32_t cols = n - col0 < kRingCols ? n - col0 : kRingCols;    // a multiple of 4
  const uint32_t k_lo = blockIdx.y * slice_len;
  const uint32_t k_hi = k_lo + slice_len < k ? k_lo + slice_len : k;
  const uint32_t rows_total = k_hi - k_lo;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (uint32_t st = 0; st < kRingStages; ++st) {
      ring::init(ring::smem_addr(&full_bar[st]), 1);
      ring::init(ring::smem_addr(&empty_bar[st]), 16);
    }
    ring::fence_init();
  }
  for (uint32_t e = threadIdx.x; e < rows_total * AP; e += blockDim.x) {
    const uint32_t r = e / AP, i = e % AP;
    As[e] = i < m ? A[static_cast<u64>(k_lo + r) * m + i] : 0.f;  // A stored m x k
  }
  __syncthreads();
  if (warp == 16u) {
    // ---- producer ----
    if (lane == 0u) {
      uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
      for (uint32_t r0 = 0; r0 < rows_total; r0 += kRingRows) {
        if (!ring::wait(ring::smem_addr(&empty_bar[stage]), phase ^ 1u, abort_flag)) break;
        const uint32_t nrows = rows_total - r0 < kRingRows ? rows_total - r0 : kRingRows;
        const uint32_t bar = ring::smem_addr(&full_bar[stage]);
        const uint32_t dst = ring::smem_addr(stages + static_cast<size_t>(stage) * kRingRows * kRingCols);
        const float *src = B + static_cast<u64>(k_lo + r0) * n + col0;  // B stored n x k
        ring::arrive_expect_tx(bar, nrows * cols * 4u);
        armed |= 1u << stage;
        armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
        if (cols == n) {
          ring::bulk_load(dst, src, nrows * cols * 4u, bar);     // the rows are adjacent in memory: one copy
        } else {
          for (uint32_t r = 0; r < nrows; ++r)
            ring::bulk_load(dst + r * cols * 4u, src + static_cast<u64>(r) * n, cols * 4u, bar);
        }
        if (++stage == kRingStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (*abort_flag) {
        // let the copies in flight land before the CTA gives its shared memory up
        for (uint32_t st = 0; st < kRingStages; ++st)
          if (armed & (1u << st)) ring::wait_quiet(ring::smem_addr(&full_bar[st]), (armed_parity >> st) & 1u);
      }
    }
  } else {
    // ---- consumers: sixteen warps, two columns per thread ----
    const uint32_t j = threadIdx.x * 2u;
    const bool col_ok = j < cols;
    f32x2 acc[2][MP / 2];   // rows (2p, 2p + 1) of the two columns
#pragma unroll
    for (uint32_t c = 0; c < 2u; ++c)
#pragma unroll
      for (uint32_t pr = 0; pr < MP / 2; ++pr) acc[c][pr] = pack2(0.f, 0.f);
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t r0 = 0; ok && r0 < rows_total; r0 += kRingRows) {
      uint32_t got = 1u;
      if (lane == 0u) got = ring::wait(ring::smem_addr(&full_bar[stage]), phase, abort_flag) ? 1u : 0u;
      if (!__shfl_sync(0xffffffffu, got, 0)) {
        ok = false;
        break;
      }
      const uint32_t nrows = rows_total - r0 < kRingRows ? rows_total - r0 : kRingRows;
      const float *st_base = stages + static_cast<size_t>(stage) * kRingRows * kRingCols;
#pragma unroll 4
      for (uint32_t r = 0; r < nrows; ++r) {
        const float2 b = col_ok ? *reinterpret_cast<const float2 *>(st_base + r * cols + j) : make_float2(0.f, 0.f);
        // one address per warp: broadcast; a 128-bit load is two ready-made pairs of A's rows
        const ulonglong2 *arow = reinterpret_cast<const ulonglong2 *>(As + (r0 + r) * AP);
        f32x2 a[AP / 2];
#pragma unroll
        for (uint32_t q = 0; q < AP / 4; ++q) {
          const ulonglong2 t = arow[q];
          a[2 * q] = t.x;
          a[2 * q + 1] = t.y;
        }
        const f32x2 bx = pack2(b.x, b.x), by = pack2(b.y, b.y);
#pragma unroll
        for (uint32_t pr = 0; pr < MP / 2; ++pr) {
          fma2(acc[0][pr], a[pr], bx);
          fma2(acc[1][pr], a[pr], by);
        }
      }
      __syncwarp();
      if (lane == 0u) ring::arrive(ring::smem_addr(&empty_bar[stage]));
      if (++stage == kRingStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (ok && col_ok) {
      float *out = partial + static_cast<u64>(blockIdx.y) * m * n;
#pragma unroll
      for (uint32_t c = 0; c < 2u; ++c)
#pragma unroll
        for (uint32_t pr = 0; pr < MP / 2; ++pr) {
          float lo, hi;
          unpack2(acc[c][pr], lo, hi);
          if (2u * pr < m) out[static_cast<u64>(col0 + j + c) * m + 2u * pr] = lo;
          if (2u * pr + 1u < m) out[static_cast<u64>(col0 + j + c) * m + 2u * pr + 1u] = hi;
        }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_abort) report_status(status, B200_ERR_KERNEL_TIMEOUT);
}

// outer, m % 4 == 0: a lane owns four consecutive rows of C (one 128-bit store per column) with
// their K values of A in registers for the whole launch; a warp owns 128 rows, the CTA's eight
// warps 1024 rows and a strip of 64 columns at a time, whose K values of B are staged in shared
// memory once per strip and read as broadcasts.  Per column and lane: K / 4 shared loads, 4 K FMAs,
// one 128-bit store.
template <uint32_t K, bool accumulate>
__global__ void __launch_bounds__(256, 2) skinny_outer4_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                               float *C, uint32_t m, uint32_t n) {
  pdl_enter();
  constexpr uint32_t KP = (K + 3u) & ~3u, kStrip = 64;
  __shared__ __align__(16) float Bs[kStrip * KP];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t i0 = (blockIdx.y * 8u + warp) * 128u + lane * 4u;
  const bool row_ok = i0 < m;   // m % 4 == 0
  f32x2 a[4][KP / 2];   // pairs of consecutive k values of the lane's four rows (zero past K)
#pragma unroll
  for (uint32_t r = 0; r < 4u; ++r)
#pragma unroll
    for (uint32_t q = 0; q < KP / 2; ++q) {
      const float lo = (row_ok && 2u * q < K) ? A[static_cast<u64>(i0 + r) * K + 2u * q] : 0.f;  // A stored k x m
      const float hi = (row_ok && 2u * q + 1u < K) ? A[static_cast<u64>(i0 + r) * K + 2u * q + 1u] : 0.f;
      a[r][q] = pack2(lo, hi);
    }
  constexpr uint32_t KH = (K + 1u) / 2u;   // pairs that hold at least one live k value
  const uint32_t strips = (n + kStrip - 1) / kStrip;
  for (uint32_t strip = blockIdx.x; strip < strips; strip += gridDim.x) {
    const u64 j_lo = static_cast<u64>(strip) * kStrip;
    const uint32_t cols = n - j_lo < kStrip ? static_cast<uint32_t>(n - j_lo) : kStrip;
    __syncthreads();   // the previous strip's readers are done
    for (uint32_t e = threadIdx.x; e < cols * KP; e += blockDim.x) {
      const uint32_t c = e / KP, kk = e % KP;
      Bs[e] = kk < K ? B[(j_lo + c) * K + kk] : 0.f;  // B stored k x n
    }
    __syncthreads();
    if (!row_ok) continue;
    for (uint32_t c0 = 0; c0 < cols; c0 += 4u) {
      float4 old[4];
#pragma unroll
      for (uint32_t u = 0; u < 4u; ++u)
        old[u] = (accumulate && c0 + u < cols) ? *reinterpret_cast<const float4 *>(C + (j_lo + c0 + u) * m + i0)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (uint32_t u = 0; u < 4u; ++u) {
        if (c0 + u < cols) {
          const ulonglong2 *bcol = reinterpret_cast<const ulonglong2 *>(Bs + (c0 + u) * KP);  // broadcast
          f32x2 bv[KP / 2];   // the column's k values in pairs (zero past K)
#pragma unroll
          for (uint32_t q = 0; q < KP / 4; ++q) {
            const ulonglong2 t = bcol[q];
            bv[2 * q] = t.x;
            bv[2 * q + 1] = t.y;
          }
          // even and odd k values accumulate side by side and meet at the end
          float t[4];
#pragma unroll
          for (uint32_t r = 0; r < 4u; ++r) {
            f32x2 s2 = pack2(0.f, 0.f);
#pragma unroll
            for (uint32_t q = 0; q < KH; ++q) fma2(s2, a[r][q], bv[q]);
            float lo, hi;
            unpack2(s2, lo, hi);
            t[r] = lo + hi;
          }
          *reinterpret_cast<float4 *>(C + (j_lo + c0 + u) * m + i0) =
              make_float4(old[u].x + t[0], old[u].y + t[1], old[u].z + t[2], old[u].w + t[3]);
        }
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
#ifdef PRIMITIV_B200_DEV_KNOBS
  static const bool fast_off = std::getenv("PRIMITIV_B200_SKINNY_FAST") && std::atoi(std::getenv("PRIMITIV_B200_SKINNY_FAST")) == 0;
  const bool kFloat = sizeof(T) == 4 && !fast_off;
#else
  constexpr bool kFloat = sizeof(T) == 4;
#endif
  auto aligned = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (kind == kRows && kFloat && g.k % 4u == 0 && g.k <= 1024u && aligned(g.B)) {
    // the small operand in registers, 128-bit loads of the large one (see skinny_rows_reg_kernel)
    const u64 a_si = g.trans_a ? g.k : 1, a_sk = g.trans_a ? 1 : g.m;
    const uint32_t tiles = (g.n + 31u) / 32u;
    const uint32_t cap = static_cast<uint32_t>(ctx->sm_count) * 2u;
    const dim3 grid(tiles < cap ? tiles : cap), block(256);
    const float *Af = reinterpret_cast<const float *>(A), *Bf = reinterpret_cast<const float *>(B);
    float *Cf = reinterpret_cast<float *>(C);
#define B200_ROWS_REG(MPV) b200::launch(ctx, skinny_rows_reg_kernel<MPV>, grid, block, 0, s, 1u, Af, Bf, Cf, g.m, g.n, g.k, a_si, a_sk, g.accumulate)
    switch ((g.m + 1u) & ~1u) {
      case 2: B200_ROWS_REG(2); break;
      case 4: B200_ROWS_REG(4); break;
      case 6: B200_ROWS_REG(6); break;
      case 8: B200_ROWS_REG(8); break;
      case 10: B200_ROWS_REG(10); break;
      case 12: B200_ROWS_REG(12); break;
      case 14: B200_ROWS_REG(14); break;
      default: B200_ROWS_REG(16); break;
    }
#undef B200_ROWS_REG
    ++ctx->launches;
    return static_cast<int>(cudaGetLastError());
  }
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
  if (kind == kReduce && kFloat && g.n % 4u == 0 && aligned(g.B)) {
    // the large operand through a shared-memory ring filled by bulk copies (skinny_reduce_ring_kernel),
    // when a slice of A fits beside the ring; otherwise four columns per thread with direct loads
    const uint32_t mp2r = (g.m + 1u) & ~1u, apr = (mp2r + 3u) & ~3u;
    const unsigned rgx = (g.n + kRingCols - 1) / kRingCols;
    u64 rslices = static_cast<u64>(ctx->sm_count) / rgx;   // one CTA per SM
    if (rslices < 1) rslices = 1;
    if (rslices > g.k / 64) rslices = g.k / 64 ? g.k / 64 : 1;
    // (the kernel needs n % 2 == 0 for its 64-bit loads and 16-byte rows for the bulk copies: n % 4 == 0 gives both)
    const uint32_t rslice_len = static_cast<uint32_t>((g.k + rslices - 1) / rslices);
    const unsigned rgy = (g.k + rslice_len - 1) / rslice_len;
    const size_t a_bytes = static_cast<size_t>(rslice_len) * apr * sizeof(float);
    const size_t ring_smem = kRingBytes + a_bytes;
    if (ring_smem + 1024 <= ctx->smem_optin) {
      const u64 count = static_cast<u64>(g.m) * g.n;
      void *partial = nullptr;
      const int rc = ctx->pool.alloc(static_cast<size_t>(rgy) * count * sizeof(float), &partial, nullptr);
      if (rc != B200_OK) return rc;
      float *pp = static_cast<float *>(partial);
      const float *Af = reinterpret_cast<const float *>(A), *Bf = reinterpret_cast<const float *>(B);
      const dim3 grid(rgx, rgy), block(544);
      cudaError_t attr = cudaSuccess;
#define B200_RING(MPV)                                                                                                   \
  case MPV:                                                                                                              \
    attr = cudaFuncSetAttribute(skinny_reduce_ring_kernel<MPV>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                                static_cast<int>(ctx->smem_optin - 1024));                                               \
    if (attr == cudaSuccess)                                                                                             \
      b200::launch(ctx, skinny_reduce_ring_kernel<MPV>, grid, block, ring_smem, s, 1u, Af, Bf, pp, g.m, g.n, g.k, rslice_len, \
                   ctx->d_status);                                                                                       \
    break;
      switch (mp2r) {
        B200_RING(2) B200_RING(4) B200_RING(6) B200_RING(8) B200_RING(10) B200_RING(12) B200_RING(14) B200_RING(16)
        default: attr = cudaErrorInvalidValue; break;
      }
#undef B200_RING
      if (attr != cudaSuccess) {
        ctx->pool.free(partial);
        return static_cast<int>(attr);
      }
      b200::launch(ctx, reduce_final_kernel<T>, dim3(static_cast<unsigned>((count + 31) / 32)), dim3(32, 8), 0, s, 1u, pp, C, count, rgy, g.accumulate);
      ctx->launches += 2;
      ctx->pool.free(partial);  // stream-ordered reuse
      return static_cast<int>(cudaGetLastError());
    }
  }
  if (kind == kReduce && kFloat && g.n % 4u == 0 && aligned(g.B)) {
    // four consecutive columns per thread, 128-bit loads (see skinny_reduce4_kernel)
    const uint32_t mp2 = (g.m + 1u) & ~1u, ap = (mp2 + 3u) & ~3u;
    const unsigned gx = static_cast<unsigned>((static_cast<u64>(g.n) / 4u + 255u) / 256u);
    u64 slices = (2ull * ctx->sm_count + gx - 1) / gx;   // two CTAs per SM
    if (slices > g.k / 64) slices = g.k / 64;
    if (slices < 1) slices = 1;
    const uint32_t slice_len = static_cast<uint32_t>((g.k + slices - 1) / slices);
    const unsigned gy = (g.k + slice_len - 1) / slice_len;
    const u64 count = static_cast<u64>(g.m) * g.n;
    void *partial = nullptr;
    const int rc = ctx->pool.alloc(static_cast<size_t>(gy) * count * sizeof(float), &partial, nullptr);
    if (rc != B200_OK) return rc;
    const uint32_t chunk = slice_len < kSmemFloats / ap ? slice_len : kSmemFloats / ap;
    const size_t smem = static_cast<size_t>(chunk) * ap * sizeof(float);
    float *pp = static_cast<float *>(partial);
    const float *Af = reinterpret_cast<const float *>(A), *Bf = reinterpret_cast<const float *>(B);
    const dim3 grid(gx, gy), block(256);
#define B200_REDUCE4(MPV) b200::launch(ctx, skinny_reduce4_kernel<MPV>, grid, block, smem, s, 1u, Af, Bf, pp, g.m, g.n, g.k, slice_len)
    switch (mp2) {
      case 2: B200_REDUCE4(2); break;
      case 4: B200_REDUCE4(4); break;
      case 6: B200_REDUCE4(6); break;
      case 8: B200_REDUCE4(8); break;
      case 10: B200_REDUCE4(10); break;
      case 12: B200_REDUCE4(12); break;
      case 14: B200_REDUCE4(14); break;
      default: B200_REDUCE4(16); break;
    }
#undef B200_REDUCE4
    b200::launch(ctx, reduce_final_kernel<T>, dim3(static_cast<unsigned>((count + 31) / 32)), dim3(32, 8), 0, s, 1u, pp, C, count, gy, g.accumulate);
    ctx->launches += 2;
    ctx->pool.free(partial);  // stream-ordered reuse
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
  if (kind == kOuter && kFloat && g.m % 4u == 0 && aligned(g.C)) {
    // four consecutive rows per lane, 128-bit stores, k compiled in (see skinny_outer4_kernel)
    const unsigned row_groups = (g.m + 1023u) / 1024u;
    const unsigned strips = (g.n + 63u) / 64u;
    unsigned gx = static_cast<unsigned>(ctx->sm_count) * 2u / row_groups;
    if (gx < 1) gx = 1;
    if (gx > strips) gx = strips;
    const dim3 grid(gx, row_groups), block(256);
    const float *Af = reinterpret_cast<const float *>(A), *Bf = reinterpret_cast<const float *>(B);
    float *Cf = reinterpret_cast<float *>(C);
#define B200_OUTER4(KV)                                                                                          \
  case KV:                                                                                                       \
    if (g.accumulate) b200::launch(ctx, skinny_outer4_kernel<KV, true>, grid, block, 0, s, 1u, Af, Bf, Cf, g.m, g.n); \
    else b200::launch(ctx, skinny_outer4_kernel<KV, false>, grid, block, 0, s, 1u, Af, Bf, Cf, g.m, g.n);        \
    break;
    switch (g.k) {
      B200_OUTER4(1) B200_OUTER4(2) B200_OUTER4(3) B200_OUTER4(4) B200_OUTER4(5) B200_OUTER4(6) B200_OUTER4(7) B200_OUTER4(8)
      B200_OUTER4(9) B200_OUTER4(10) B200_OUTER4(11) B200_OUTER4(12) B200_OUTER4(13) B200_OUTER4(14) B200_OUTER4(15)
      B200_OUTER4(16)
      default: return B200_ERR_INVALID_ARG;
    }
#undef B200_OUTER4
    ++ctx->launches;
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
