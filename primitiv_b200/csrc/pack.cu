// Packing pre-pass of the tensor-core matrix product (see pack.h): the kernels that split fp32
// operands into TF32 hi / lo planes (3xTF32, and TF32 for operands TMA cannot read where they
// lie) or into row-scaled half planes (3xFP16), and the host code that picks among them.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <vector>

#include "pack.h"

namespace b200 {
namespace {

// ------------------------------ packing pre-pass ------------------------------

// x rounded to TF32 (10 explicit mantissa bits), nearest with ties away from zero.
// The result has its 13 low mantissa bits clear, so the tensor core sees it exactly.
__device__ __forceinline__ float rn_tf32(float x) {
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;  // inf / nan pass through
  u = (u + 0x1000u) & 0xffffe000u;
  return __uint_as_float(u);
}

// Packs one fp32 operand into K-major planes: dst[b][i][p], i < mn, p < k, row
// stride k_pad (a multiple of 4 so TMA strides are 16-byte multiples).
//   hi = rn_tf32(x), lo = rn_tf32(x - hi) (lo written only when lo != nullptr).
// Source element (i, p) of matrix b is at src[b*src_bs + i*s_mn + p*s_k]:
// (s_mn, s_k) = (1, mn) for an MN-major source (the kernel transposes through
// shared memory), (k, 1) for a K-major source.  One 32x32 tile per CTA iteration,
// flat 1-D grid so the batch can exceed 65535.
template <bool kTranspose>
__global__ void __launch_bounds__(256) pack_tf32_kernel(
    const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo, uint32_t mn,
    uint32_t k, uint32_t k_pad, unsigned long long src_bs, uint32_t tiles_mn, uint32_t tiles_k,
    unsigned long long total_tiles) {
  pdl_enter();
  __shared__ float tile[32][33];
  const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;  // 32 x 8
  for (unsigned long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const unsigned long long per_b = static_cast<unsigned long long>(tiles_mn) * tiles_k;
    const unsigned long long b = t / per_b;
    const uint32_t rem = static_cast<uint32_t>(t - b * per_b);
    const uint32_t i0 = (rem % tiles_mn) * 32u, p0 = (rem / tiles_mn) * 32u;
    const float *s = src + b * src_bs;
    const unsigned long long dst_b = b * static_cast<unsigned long long>(mn) * k_pad;
    if (kTranspose) {
      // read coalesced along mn, write coalesced along k
#pragma unroll
      for (uint32_t j = 0; j < 32u; j += 8u) {
        const uint32_t i = i0 + tx, pp = p0 + ty + j;
        tile[ty + j][tx] = (i < mn && pp < k) ? s[static_cast<unsigned long long>(pp) * mn + i] : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (uint32_t j = 0; j < 32u; j += 8u) {
        const uint32_t i = i0 + ty + j, pp = p0 + tx;
        if (i < mn && pp < k) {
          const float x = tile[tx][ty + j];
          const float h = rn_tf32(x);
          const unsigned long long o = dst_b + static_cast<unsigned long long>(i) * k_pad + pp;
          hi[o] = h;
          if (lo) lo[o] = rn_tf32(x - h);
        }
      }
      __syncthreads();
    } else {
#pragma unroll
      for (uint32_t j = 0; j < 32u; j += 8u) {
        const uint32_t i = i0 + ty + j, pp = p0 + tx;
        if (i < mn && pp < k) {
          const float x = s[static_cast<unsigned long long>(i) * k + pp];
          const float h = rn_tf32(x);
          const unsigned long long o = dst_b + static_cast<unsigned long long>(i) * k_pad + pp;
          hi[o] = h;
          if (lo) lo[o] = rn_tf32(x - h);
        }
      }
    }
  }
}

// ---- pre-pass of the 3xFP16 mode ----
//
// Every row of an operand (index mn, all of k) gets a power-of-two scale s that brings its
// largest magnitude into [2^14, 2^15), half's top binades; then x*s = h0 + h1 with
// h0 = rn_half(x*s), h1 = rn_half(x*s - h0): two half planes with 11 + 11 mantissa bits, the
// same as TF32 hi + lo.  The scale arrays hold the row maxima themselves; the split kernels and
// the epilogue both derive 1/s = 2^(floor(log2 max) - 14) from them (inv_scale_for).  When the
// batch is itself a contraction axis (`shared`), one maximum per row covers all batches.
// K-major source (k contiguous): one warp per row.
__global__ void __launch_bounds__(256) row_max_kmajor_kernel(const float *__restrict__ src, float *__restrict__ amax_out,
                                                             uint32_t mn, uint32_t k, unsigned long long ld,
                                                             unsigned long long src_bs, uint32_t nbatch, int shared) {
  pdl_enter();
  const uint32_t lane = threadIdx.x & 31u;
  const unsigned long long rows = static_cast<unsigned long long>(mn) * (shared ? 1u : nbatch);
  for (unsigned long long r = blockIdx.x * 8ull + (threadIdx.x >> 5); r < rows; r += gridDim.x * 8ull) {
    const unsigned long long b0 = shared ? 0 : r / mn, i = r - b0 * mn;
    float amax = 0.f;
    for (uint32_t b = 0; b < (shared ? nbatch : 1u); ++b) {
      const float *row = src + (b0 + b) * src_bs + i * ld;
      for (uint32_t p = lane; p < k; p += 32u) amax = fmaxf(amax, fabsf(row[p]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) amax_out[r] = amax;
  }
}

// MN-major source (mn contiguous): 32 rows x 8 k-lanes per CTA, coalesced along mn; the k range
// is cut into slices over grid.y so that a tall, narrow operand still fills the GPU, and the
// slices meet in an atomic maximum on the (non-negative) float's bit pattern, which orders
// like the value: the result does not depend on the order.  amax_out starts zeroed.
__global__ void __launch_bounds__(256) row_max_mnmajor_kernel(const float *__restrict__ src, float *amax_out,
                                                              uint32_t mn, uint32_t k, unsigned long long ld,
                                                              unsigned long long src_bs, uint32_t nbatch, int shared,
                                                              uint32_t k_slice) {
  pdl_enter();
  __shared__ float buf[8][32];
  const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
  const uint32_t tiles = (mn + 31u) / 32u;
  const unsigned long long total = static_cast<unsigned long long>(tiles) * nbatch;
  const uint32_t p_lo = blockIdx.y * k_slice, p_hi = p_lo + k_slice < k ? p_lo + k_slice : k;
  for (unsigned long long t = blockIdx.x; t < total; t += gridDim.x) {
    const unsigned long long b = t / tiles;
    const uint32_t i = static_cast<uint32_t>(t - b * tiles) * 32u + tx;
    float amax = 0.f;
    if (i < mn) {
      const float *m0 = src + b * src_bs + i;
      for (uint32_t p = p_lo + ty; p < p_hi; p += 8u) amax = fmaxf(amax, fabsf(m0[static_cast<unsigned long long>(p) * ld]));
    }
    buf[ty][tx] = amax;
    __syncthreads();
    if (ty == 0 && i < mn) {
#pragma unroll
      for (uint32_t l = 1; l < 8u; ++l) amax = fmaxf(amax, buf[l][tx]);
      // NaNs: fmaxf drops them and their bit pattern would not order; the products of such a row are NaN anyway
      atomicMax(reinterpret_cast<int *>(amax_out) + (shared ? 0ull : b * mn) + i, __float_as_int(amax));
    }
    __syncthreads();
  }
}

// Writes the two half planes, K-major [b][i][k_pad] (k_pad a multiple of 8: 16-byte rows).
// Same tiling as pack_tf32_kernel; amax holds the row maxima ([b][i], or [i] when shared).
template <bool kTranspose>
__global__ void __launch_bounds__(256) pack_f16_kernel(const float *__restrict__ src, const float *__restrict__ amax,
                                                       __half *__restrict__ h0, __half *__restrict__ h1, uint32_t mn,
                                                       uint32_t k, uint32_t k_pad, unsigned long long ld,
                                                       unsigned long long src_bs, uint32_t tiles_mn, uint32_t tiles_k,
                                                       unsigned long long total_tiles, int shared) {
  pdl_enter();
  __shared__ float tile[32][33];
  const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;  // 32 x 8
  for (unsigned long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const unsigned long long per_b = static_cast<unsigned long long>(tiles_mn) * tiles_k;
    const unsigned long long b = t / per_b;
    const uint32_t rem = static_cast<uint32_t>(t - b * per_b);
    const uint32_t i0 = (rem % tiles_mn) * 32u, p0 = (rem / tiles_mn) * 32u;
    const float *s = src + b * src_bs;
    const float *iv = amax + (shared ? 0ull : b * mn);
    const unsigned long long dst_b = b * static_cast<unsigned long long>(mn) * k_pad;
    if (kTranspose) {
#pragma unroll
      for (uint32_t j = 0; j < 32u; j += 8u) {
        const uint32_t i = i0 + tx, pp = p0 + ty + j;
        tile[ty + j][tx] = (i < mn && pp < k) ? s[static_cast<unsigned long long>(pp) * ld + i] : 0.f;
      }
      __syncthreads();
    }
#pragma unroll
    for (uint32_t j = 0; j < 32u; j += 8u) {
      const uint32_t i = i0 + ty + j, pp = p0 + tx;
      if (i < mn && pp < k) {
        const float x = kTranspose ? tile[tx][ty + j] : s[static_cast<unsigned long long>(i) * ld + pp];
        const float xs = x * (1.f / inv_scale_for(iv[i]));  // the power-of-two scale: exact
        const __half a = __float2half_rn(xs);
        const unsigned long long o = dst_b + static_cast<unsigned long long>(i) * k_pad + pp;
        h0[o] = a;
        h1[o] = __float2half_rn(xs - __half2float(a));
      }
    }
    if (kTranspose) __syncthreads();
  }
}

// Fast paths of the packing pre-pass (both move 128 bits per thread per access).
//
// pack_flat_kernel: a K-major source whose rows need no padding (k % 4 == 0) and whose
// matrices are back to back is one flat array; the planes have the same layout, so the
// split is purely elementwise.
__global__ void __launch_bounds__(256) pack_flat_kernel(const float4 *__restrict__ src, float4 *__restrict__ hi,
                                                        float4 *__restrict__ lo, unsigned long long n4) {
  pdl_enter();
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += stride) {
    const float4 v = src[i];
    float4 h, l;
    h.x = rn_tf32(v.x); l.x = rn_tf32(v.x - h.x);
    h.y = rn_tf32(v.y); l.y = rn_tf32(v.y - h.y);
    h.z = rn_tf32(v.z); l.z = rn_tf32(v.z - h.z);
    h.w = rn_tf32(v.w); l.w = rn_tf32(v.w - h.w);
    hi[i] = h;
    if (lo) lo[i] = l;
  }
}

// pack_transpose64_kernel: an MN-major source with mn % 4 == 0 and k % 4 == 0.  64 x 64
// tiles through shared memory: float4 reads along mn, float4 writes along k.
__global__ void __launch_bounds__(256) pack_transpose64_kernel(const float *__restrict__ src, float *__restrict__ hi,
                                                               float *__restrict__ lo, uint32_t mn, uint32_t k,
                                                               unsigned long long src_bs, uint32_t tiles_mn,
                                                               uint32_t tiles_k, unsigned long long total_tiles) {
  pdl_enter();
  __shared__ float tile[64][65];  // [k][mn]
  const uint32_t t = threadIdx.x;
  for (unsigned long long tl = blockIdx.x; tl < total_tiles; tl += gridDim.x) {
    const unsigned long long per_b = static_cast<unsigned long long>(tiles_mn) * tiles_k;
    const unsigned long long b = tl / per_b;
    const uint32_t rem = static_cast<uint32_t>(tl - b * per_b);
    const uint32_t i0 = (rem % tiles_mn) * 64u, p0 = (rem / tiles_mn) * 64u;
    const float *s = src + b * src_bs;
    const unsigned long long dst_b = b * static_cast<unsigned long long>(mn) * k;
    // 64 k-rows x 16 float4 along mn = 1024 float4, 4 per thread
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
      const uint32_t e = t + r * 256u;
      const uint32_t pk = e >> 4, im = (e & 15u) * 4u;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p0 + pk < k && i0 + im < mn)
        v = *reinterpret_cast<const float4 *>(s + static_cast<unsigned long long>(p0 + pk) * mn + i0 + im);
      tile[pk][im] = v.x; tile[pk][im + 1] = v.y; tile[pk][im + 2] = v.z; tile[pk][im + 3] = v.w;
    }
    __syncthreads();
    // 64 mn-rows x 16 float4 along k
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
      const uint32_t e = t + r * 256u;
      const uint32_t im = e >> 4, pk = (e & 15u) * 4u;
      if (i0 + im < mn && p0 + pk < k) {
        const float x0 = tile[pk][im], x1 = tile[pk + 1][im], x2 = tile[pk + 2][im], x3 = tile[pk + 3][im];
        float4 h, l;
        h.x = rn_tf32(x0); l.x = rn_tf32(x0 - h.x);
        h.y = rn_tf32(x1); l.y = rn_tf32(x1 - h.y);
        h.z = rn_tf32(x2); l.z = rn_tf32(x2 - h.z);
        h.w = rn_tf32(x3); l.w = rn_tf32(x3 - h.w);
        const unsigned long long o = dst_b + static_cast<unsigned long long>(i0 + im) * k + p0 + pk;
        *reinterpret_cast<float4 *>(hi + o) = h;
        if (lo) *reinterpret_cast<float4 *>(lo + o) = l;
      }
    }
    __syncthreads();
  }
}

// Fast paths of the 3xFP16 pre-pass.
//
// pack_f16_rows_kernel: a K-major source with 16-byte aligned rows and k % 8 == 0.  A group of
// kGroup threads (a whole CTA for long rows, a warp for short ones) takes one row at a time: the
// row's largest magnitude (float4 loads, reduction), then the row once more (it is still in
// L1 / L2) split into the two half planes with 16-byte stores.  Maximum and split in one kernel:
// 4 bytes read from HBM and 4 written per element.
template <uint32_t kGroup>
__global__ void __launch_bounds__(256) pack_f16_rows_kernel(const float *__restrict__ src, float *__restrict__ amax_out,
                                                            __half *__restrict__ h0, __half *__restrict__ h1,
                                                            uint32_t mn, uint32_t k, unsigned long long ld,
                                                            unsigned long long src_bs, unsigned long long rows) {
  pdl_enter();
  static_assert(kGroup == 32 || kGroup == 256, "a warp or the CTA");
  __shared__ float red[8];
  const uint32_t t = threadIdx.x % kGroup, lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t k8 = k >> 3;
  constexpr uint32_t kPerCta = 256u / kGroup;
  const unsigned long long first = static_cast<unsigned long long>(blockIdx.x) * kPerCta + threadIdx.x / kGroup;
  const unsigned long long step = static_cast<unsigned long long>(gridDim.x) * kPerCta;
  // (for kGroup == 256 every thread of the CTA walks the same rows, so the barriers below are uniform)
  for (unsigned long long r = first; r < rows; r += step) {
    const unsigned long long b = r / mn, i = r - b * mn;
    const float4 *row = reinterpret_cast<const float4 *>(src + b * src_bs + i * ld);
    float amax = 0.f;
    for (uint32_t c = t; c < 2u * k8; c += kGroup) {
      const float4 v = row[c];
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (kGroup == 256) {
      if (lane == 0) red[warp] = amax;
      __syncthreads();
      amax = red[0];
#pragma unroll
      for (uint32_t w = 1; w < 8u; ++w) amax = fmaxf(amax, red[w]);
    }
    const float sc = 1.f / inv_scale_for(amax);
    if (t == 0) amax_out[r] = amax;
    uint4 *d0 = reinterpret_cast<uint4 *>(h0 + r * static_cast<unsigned long long>(k));
    uint4 *d1 = reinterpret_cast<uint4 *>(h1 + r * static_cast<unsigned long long>(k));
    for (uint32_t c = t; c < k8; c += kGroup) {
      const float4 u = row[2u * c], v = row[2u * c + 1u];
      const float x[8] = {u.x * sc, u.y * sc, u.z * sc, u.w * sc, v.x * sc, v.y * sc, v.z * sc, v.w * sc};
      __align__(16) __half a[8], e[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] = __float2half_rn(x[j]);
        e[j] = __float2half_rn(x[j] - __half2float(a[j]));
      }
      d0[c] = *reinterpret_cast<const uint4 *>(a);
      d1[c] = *reinterpret_cast<const uint4 *>(e);
    }
    if (kGroup == 256) __syncthreads();  // red[] is reused by the next row
  }
}

// pack_f16_transpose64_kernel: an MN-major source with mn % 4 == 0 and k % 8 == 0 whose row
// maxima are already known (row_max_mnmajor_kernel).  64 x 64 tiles through shared memory:
// float4 reads along mn, 16-byte half stores along k.
__global__ void __launch_bounds__(256) pack_f16_transpose64_kernel(const float *__restrict__ src,
                                                                   const float *__restrict__ amax,
                                                                   __half *__restrict__ h0, __half *__restrict__ h1,
                                                                   uint32_t mn, uint32_t k, unsigned long long ld,
                                                                   unsigned long long src_bs, uint32_t tiles_mn,
                                                                   uint32_t tiles_k, unsigned long long total_tiles,
                                                                   int shared) {
  pdl_enter();
  __shared__ float tile[64][65];  // [k][mn]
  const uint32_t t = threadIdx.x;
  for (unsigned long long tl = blockIdx.x; tl < total_tiles; tl += gridDim.x) {
    const unsigned long long per_b = static_cast<unsigned long long>(tiles_mn) * tiles_k;
    const unsigned long long b = tl / per_b;
    const uint32_t rem = static_cast<uint32_t>(tl - b * per_b);
    const uint32_t i0 = (rem % tiles_mn) * 64u, p0 = (rem / tiles_mn) * 64u;
    const float *s = src + b * src_bs;
    const float *iv = amax + (shared ? 0ull : b * mn);
    const unsigned long long dst_b = b * static_cast<unsigned long long>(mn) * k;
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
      const uint32_t e = t + r * 256u;
      const uint32_t pk = e >> 4, im = (e & 15u) * 4u;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p0 + pk < k && i0 + im < mn)
        v = *reinterpret_cast<const float4 *>(s + static_cast<unsigned long long>(p0 + pk) * ld + i0 + im);
      tile[pk][im] = v.x; tile[pk][im + 1] = v.y; tile[pk][im + 2] = v.z; tile[pk][im + 3] = v.w;
    }
    __syncthreads();
    // 64 mn-rows x 8 groups of 8 k = 512 groups, 2 per thread
#pragma unroll
    for (uint32_t r = 0; r < 2u; ++r) {
      const uint32_t e = t + r * 256u;
      const uint32_t im = e >> 3, pk = (e & 7u) * 8u;
      if (i0 + im < mn && p0 + pk < k) {
        const float sc = 1.f / inv_scale_for(iv[i0 + im]);
        __align__(16) __half a[8], d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float x = tile[pk + j][im] * sc;
          a[j] = __float2half_rn(x);
          d[j] = __float2half_rn(x - __half2float(a[j]));
        }
        const unsigned long long o = dst_b + static_cast<unsigned long long>(i0 + im) * k + p0 + pk;
        *reinterpret_cast<uint4 *>(h0 + o) = *reinterpret_cast<const uint4 *>(a);
        *reinterpret_cast<uint4 *>(h1 + o) = *reinterpret_cast<const uint4 *>(d);
      }
    }
    __syncthreads();
  }
}

// ---- pre-pass of the fp32 mode with bf16 correction passes (see MixPlanes in pack.h) ----

struct Mix8 {   // eight consecutive k-elements of one row, split
  float4 h0, h1;          // hi plane
  uint4 h8, l8;           // hi8 and lo8 planes (8 bf16 each)
};

__device__ __forceinline__ uint32_t bf16_pair(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);   // a in the low half: lower address
  return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ __forceinline__ Mix8 mix_split8(const float (&x)[8]) {
  float h[8], l[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    h[j] = rn_tf32(x[j]);
    l[j] = x[j] - h[j];      // exact in fp32
  }
  Mix8 m;
  m.h0 = make_float4(h[0], h[1], h[2], h[3]);
  m.h1 = make_float4(h[4], h[5], h[6], h[7]);
  m.h8 = make_uint4(bf16_pair(x[0], x[1]), bf16_pair(x[2], x[3]), bf16_pair(x[4], x[5]), bf16_pair(x[6], x[7]));
  m.l8 = make_uint4(bf16_pair(l[0], l[1]), bf16_pair(l[2], l[3]), bf16_pair(l[4], l[5]), bf16_pair(l[6], l[7]));
  return m;
}

// A K-major source whose rows need no padding (k % 8 == 0) and whose matrices are back to back is
// one flat array with the planes' own layout: the split is elementwise.  Four elements per thread
// and access (one 128-bit load, one 128-bit and two 64-bit stores, all fully coalesced), four such
// accesses in flight per thread; the source is read once and marked so in the cache.
__global__ void __launch_bounds__(256) pack_mix_flat_kernel(const float4 *__restrict__ src, float4 *__restrict__ hi,
                                                            uint2 *__restrict__ h8, uint2 *__restrict__ l8,
                                                            unsigned long long n4) {
  pdl_enter();
  constexpr unsigned kUnroll = 4;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x * kUnroll;
  for (unsigned long long base = static_cast<unsigned long long>(blockIdx.x) * blockDim.x * kUnroll + threadIdx.x;
       base < n4; base += stride) {
    float4 x[kUnroll];
#pragma unroll
    for (unsigned u = 0; u < kUnroll; ++u) {
      const unsigned long long i = base + static_cast<unsigned long long>(u) * blockDim.x;
      x[u] = i < n4 ? __ldcs(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (unsigned u = 0; u < kUnroll; ++u) {
      const unsigned long long i = base + static_cast<unsigned long long>(u) * blockDim.x;
      if (i < n4) {
        const float4 v = x[u];
        const float4 h = make_float4(rn_tf32(v.x), rn_tf32(v.y), rn_tf32(v.z), rn_tf32(v.w));
        hi[i] = h;
        h8[i] = make_uint2(bf16_pair(v.x, v.y), bf16_pair(v.z, v.w));
        l8[i] = make_uint2(bf16_pair(v.x - h.x, v.y - h.y), bf16_pair(v.z - h.z, v.w - h.w));   // differences exact in fp32
      }
    }
  }
}

// An MN-major source with mn % 4 == 0 and k % 8 == 0: 64 x 64 tiles through shared memory,
// float4 reads along mn, 16- and 32-byte writes along k.
__global__ void __launch_bounds__(256) pack_mix_transpose64_kernel(const float *__restrict__ src, float *__restrict__ hi,
                                                                   __nv_bfloat16 *__restrict__ h8,
                                                                   __nv_bfloat16 *__restrict__ l8, uint32_t mn,
                                                                   uint32_t k, unsigned long long src_bs,
                                                                   uint32_t tiles_mn, uint32_t tiles_k,
                                                                   unsigned long long total_tiles) {
  pdl_enter();
  __shared__ float tile[64][65];  // [k][mn]
  const uint32_t t = threadIdx.x;
  for (unsigned long long tl = blockIdx.x; tl < total_tiles; tl += gridDim.x) {
    const unsigned long long per_b = static_cast<unsigned long long>(tiles_mn) * tiles_k;
    const unsigned long long b = tl / per_b;
    const uint32_t rem = static_cast<uint32_t>(tl - b * per_b);
    const uint32_t i0 = (rem % tiles_mn) * 64u, p0 = (rem / tiles_mn) * 64u;
    const float *s = src + b * src_bs;
    const unsigned long long dst_b = b * static_cast<unsigned long long>(mn) * k;
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
      const uint32_t e = t + r * 256u;
      const uint32_t pk = e >> 4, im = (e & 15u) * 4u;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p0 + pk < k && i0 + im < mn)
        v = *reinterpret_cast<const float4 *>(s + static_cast<unsigned long long>(p0 + pk) * mn + i0 + im);
      tile[pk][im] = v.x; tile[pk][im + 1] = v.y; tile[pk][im + 2] = v.z; tile[pk][im + 3] = v.w;
    }
    __syncthreads();
    // 64 mn-rows x 8 groups of 8 k = 512 groups, 2 per thread
#pragma unroll
    for (uint32_t r = 0; r < 2u; ++r) {
      const uint32_t e = t + r * 256u;
      const uint32_t im = e >> 3, pk = (e & 7u) * 8u;
      if (i0 + im < mn && p0 + pk < k) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = tile[pk + j][im];
        const Mix8 m = mix_split8(x);
        const unsigned long long o = dst_b + static_cast<unsigned long long>(i0 + im) * k + p0 + pk;
        *reinterpret_cast<float4 *>(hi + o) = m.h0;
        *reinterpret_cast<float4 *>(hi + o + 4) = m.h1;
        if (h8) {
          *reinterpret_cast<uint4 *>(h8 + o) = m.h8;
          *reinterpret_cast<uint4 *>(l8 + o) = m.l8;
        }
      }
    }
    __syncthreads();
  }
}

// Any other source (unaligned, ragged k, strided batches): 32 x 32 tiles, one element per thread
// and step, row stride k_pad in the planes.  Same indexing as pack_tf32_kernel.
template <bool kTranspose>
__global__ void __launch_bounds__(256) pack_mix_kernel(const float *__restrict__ src, float *__restrict__ hi,
                                                       __nv_bfloat16 *__restrict__ h8, __nv_bfloat16 *__restrict__ l8,
                                                       uint32_t mn, uint32_t k, uint32_t k_pad, unsigned long long ld,
                                                       unsigned long long src_bs, uint32_t tiles_mn, uint32_t tiles_k,
                                                       unsigned long long total_tiles) {
  pdl_enter();
  __shared__ float tile[32][33];
  const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;  // 32 x 8
  for (unsigned long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const unsigned long long per_b = static_cast<unsigned long long>(tiles_mn) * tiles_k;
    const unsigned long long b = t / per_b;
    const uint32_t rem = static_cast<uint32_t>(t - b * per_b);
    const uint32_t i0 = (rem % tiles_mn) * 32u, p0 = (rem / tiles_mn) * 32u;
    const float *s = src + b * src_bs;
    const unsigned long long dst_b = b * static_cast<unsigned long long>(mn) * k_pad;
    if (kTranspose) {
#pragma unroll
      for (uint32_t j = 0; j < 32u; j += 8u) {
        const uint32_t i = i0 + tx, pp = p0 + ty + j;
        tile[ty + j][tx] = (i < mn && pp < k) ? s[static_cast<unsigned long long>(pp) * ld + i] : 0.f;
      }
      __syncthreads();
    }
#pragma unroll
    for (uint32_t j = 0; j < 32u; j += 8u) {
      const uint32_t i = i0 + ty + j, pp = p0 + tx;
      if (i < mn && pp < k) {
        const float x = kTranspose ? tile[tx][ty + j] : s[static_cast<unsigned long long>(i) * ld + pp];
        const float h = rn_tf32(x);
        const unsigned long long o = dst_b + static_cast<unsigned long long>(i) * k_pad + pp;
        hi[o] = h;
        if (h8) {
          h8[o] = __float2bfloat16_rn(x);
          l8[o] = __float2bfloat16_rn(x - h);
        }
      }
    }
    if (kTranspose) __syncthreads();
  }
}

}  // namespace

Tf32Planes tf32_planes(const OperandView &v) {
  Tf32Planes lay;
  lay.kpad = (v.k + 3u) & ~3u;
  lay.plane_elems = (static_cast<uint64_t>(v.nbatch) * v.mn * lay.kpad + 63ull) & ~63ull;
  return lay;
}

void pack_tf32(b200_ctx *ctx, cudaStream_t stream, OperandView &v, bool two_planes, float *dst,
               const Tf32Planes &lay, const void *planes_out[2]) {
  float *hi = dst;
  float *lo = two_planes ? dst + lay.plane_elems : nullptr;
  const bool src_ok = (reinterpret_cast<uintptr_t>(v.ptr) & 15u) == 0 && v.k % 4u == 0 &&
                      (v.nbatch <= 1 || v.batch_stride % 4u == 0);
  const bool dense = v.nbatch <= 1 || v.batch_stride == static_cast<uint64_t>(v.mn) * v.k;
  {
    ProfScope prof(ctx, kProfPack, stream);
    if (!v.mn_major && src_ok && dense) {
      const unsigned long long n4 = static_cast<unsigned long long>(v.nbatch) * v.mn * v.k / 4ull;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 16ull;
      const unsigned long long need = (n4 + 255ull) / 256ull;
      b200::launch(ctx, pack_flat_kernel, dim3(static_cast<unsigned>(need < cap ? need : cap)), dim3(256), 0, stream, 1u, static_cast<const float4 *>(v.ptr), reinterpret_cast<float4 *>(hi), reinterpret_cast<float4 *>(lo), n4);
    } else if (v.mn_major && src_ok && v.mn % 4u == 0) {
      const uint32_t tiles_mn = (v.mn + 63u) / 64u, tiles_k = (v.k + 63u) / 64u;
      const unsigned long long tt = static_cast<unsigned long long>(tiles_mn) * tiles_k * v.nbatch;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 8ull;
      b200::launch(ctx, pack_transpose64_kernel, dim3(static_cast<unsigned>(tt < cap ? tt : cap)), dim3(256), 0, stream, 1u, static_cast<const float *>(v.ptr), hi, lo, v.mn, v.k, v.batch_stride, tiles_mn, tiles_k, tt);
    } else {
      const uint32_t tiles_mn = (v.mn + 31u) / 32u, tiles_k = (v.k + 31u) / 32u;
      const unsigned long long tt = static_cast<unsigned long long>(tiles_mn) * tiles_k * v.nbatch;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 16ull;
      const unsigned blocks = static_cast<unsigned>(tt < cap ? tt : cap);
      if (v.mn_major)
        b200::launch(ctx, pack_tf32_kernel<true>, dim3(blocks), dim3(256), 0, stream, 1u, static_cast<const float *>(v.ptr), hi, lo, v.mn, v.k,
                                                          lay.kpad, v.batch_stride, tiles_mn, tiles_k, tt);
      else
        b200::launch(ctx, pack_tf32_kernel<false>, dim3(blocks), dim3(256), 0, stream, 1u, static_cast<const float *>(v.ptr), hi, lo, v.mn, v.k,
                                                           lay.kpad, v.batch_stride, tiles_mn, tiles_k, tt);
    }
  }
  ++ctx->launches;
  planes_out[0] = hi;
  planes_out[1] = lo;
  v.ptr = hi;
  v.mn_major = false;
  v.ld = lay.kpad;
  v.batch_stride = static_cast<uint64_t>(v.mn) * lay.kpad;
}

MixPlanes mix_planes(const OperandView &v) {
  MixPlanes lay;
  lay.kpad = (v.k + 7u) & ~7u;
  const uint64_t n = static_cast<uint64_t>(v.nbatch) * v.mn * lay.kpad;
  lay.hi_elems = (n + 63ull) & ~63ull;
  lay.h8_elems = (n + 127ull) & ~127ull;
  return lay;
}

void pack_mix(b200_ctx *ctx, cudaStream_t stream, OperandView &v, float *dst, const MixPlanes &lay,
              const void *planes_out[3], bool hi_only) {
  float *hi = dst;
  // (the kernels below skip the bf16 planes when their pointers are null)
  __nv_bfloat16 *h8 = hi_only ? nullptr : reinterpret_cast<__nv_bfloat16 *>(dst + lay.hi_elems);
  __nv_bfloat16 *l8 = hi_only ? nullptr : h8 + lay.h8_elems;
  const bool src_ok = (reinterpret_cast<uintptr_t>(v.ptr) & 15u) == 0 && v.k % 8u == 0 &&
                      (v.nbatch <= 1 || v.batch_stride % 4u == 0);
  const bool dense = v.nbatch <= 1 || v.batch_stride == static_cast<uint64_t>(v.mn) * v.k;
  const float *src = static_cast<const float *>(v.ptr);
  {
    ProfScope prof(ctx, kProfPack, stream);
    if (!hi_only && !v.mn_major && src_ok && dense && v.ld == v.k) {
      const unsigned long long n4 = static_cast<unsigned long long>(v.nbatch) * v.mn * v.k / 4ull;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 16ull;
      const unsigned long long need = (n4 + 1023ull) / 1024ull;
      b200::launch(ctx, pack_mix_flat_kernel, dim3(static_cast<unsigned>(need < cap ? need : cap)), dim3(256), 0, stream, 1u, reinterpret_cast<const float4 *>(src), reinterpret_cast<float4 *>(hi), reinterpret_cast<uint2 *>(h8),
          reinterpret_cast<uint2 *>(l8), n4);
    } else if (v.mn_major && src_ok && v.mn % 4u == 0 && v.ld == v.mn) {
      const uint32_t tiles_mn = (v.mn + 63u) / 64u, tiles_k = (v.k + 63u) / 64u;
      const unsigned long long tt = static_cast<unsigned long long>(tiles_mn) * tiles_k * v.nbatch;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 8ull;
      b200::launch(ctx, pack_mix_transpose64_kernel, dim3(static_cast<unsigned>(tt < cap ? tt : cap)), dim3(256), 0, stream, 1u, src, hi, h8, l8, v.mn, v.k, v.batch_stride, tiles_mn, tiles_k, tt);
    } else {
      const uint32_t tiles_mn = (v.mn + 31u) / 32u, tiles_k = (v.k + 31u) / 32u;
      const unsigned long long tt = static_cast<unsigned long long>(tiles_mn) * tiles_k * v.nbatch;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 16ull;
      const unsigned blocks = static_cast<unsigned>(tt < cap ? tt : cap);
      if (v.mn_major)
        b200::launch(ctx, pack_mix_kernel<true>, dim3(blocks), dim3(256), 0, stream, 1u, src, hi, h8, l8, v.mn, v.k, lay.kpad, v.ld, v.batch_stride,
                                                         tiles_mn, tiles_k, tt);
      else
        b200::launch(ctx, pack_mix_kernel<false>, dim3(blocks), dim3(256), 0, stream, 1u, src, hi, h8, l8, v.mn, v.k, lay.kpad, v.ld, v.batch_stride,
                                                          tiles_mn, tiles_k, tt);
    }
  }
  ++ctx->launches;
  planes_out[0] = hi;
  planes_out[1] = h8;
  planes_out[2] = l8;
  v.ptr = hi;
  v.mn_major = false;
  v.ld = lay.kpad;
  v.batch_stride = static_cast<uint64_t>(v.mn) * lay.kpad;
}

// ------------------------------ flat planes and their cache ------------------------------

bool mix_flat_ok(const OperandView &v) {
  if (reinterpret_cast<uintptr_t>(v.ptr) & 31u) return false;
  const uint64_t inner = v.mn_major ? v.mn : v.k;
  if (v.ld != inner || inner % 8u) return false;                                        // dense, 32-byte rows
  if (v.nbatch > 1 && v.batch_stride != static_cast<uint64_t>(v.mn) * v.k) return false;  // matrices back to back
  return true;
}

void plane_cache_drop_range(b200_ctx *ctx, const void *ptr, std::size_t bytes) {
  PlaneCache &pc = ctx->planes;
  if (pc.entries.empty()) return;
  // collect first, free afterwards: returning a block to the pool calls back into this function
  std::vector<void *> blocks;
  const char *lo = static_cast<const char *>(ptr), *hi = lo + bytes;
  for (std::size_t i = 0; i < pc.entries.size();) {
    const PlaneCache::Entry &e = pc.entries[i];
    const char *s0 = static_cast<const char *>(e.src), *s1 = s0 + e.src_bytes;
    if (!ptr || (s0 < hi && lo < s1)) {
      blocks.push_back(e.block);
      pc.bytes -= e.block_bytes;
      pc.entries[i] = pc.entries.back();
      pc.entries.pop_back();
    } else {
      ++i;
    }
  }
  for (void *b : blocks) ctx->pool.free(b);   // stream-ordered reuse: queued products that read them run first
}

bool mix_flat_cached(const b200_ctx *ctx, const OperandView &v) {
  const PlaneCache &pc = ctx->planes;
  if (!pc.active()) return false;
  const uint64_t n = static_cast<uint64_t>(v.nbatch > 1 ? v.nbatch : 1u) * v.mn * v.k;
  for (const PlaneCache::Entry &e : pc.entries)
    if (e.src == v.ptr && e.src_bytes == n * sizeof(float)) return true;
  return false;
}

int mix_flat_planes(b200_ctx *ctx, cudaStream_t stream, const OperandView &v, const void *planes_out[3],
                    void **owned_block) {
  PlaneCache &pc = ctx->planes;
  const uint64_t n = static_cast<uint64_t>(v.nbatch > 1 ? v.nbatch : 1u) * v.mn * v.k;
  const uint64_t hi_elems = (n + 63ull) & ~63ull, h8_elems = (n + 127ull) & ~127ull;
  const std::size_t block_bytes = hi_elems * sizeof(float) + 2 * h8_elems * sizeof(__nv_bfloat16);
  auto planes_of = [&](void *block) {
    float *hi = static_cast<float *>(block);
    __nv_bfloat16 *h8 = reinterpret_cast<__nv_bfloat16 *>(hi + hi_elems);
    planes_out[0] = hi;
    planes_out[1] = h8;
    planes_out[2] = h8 + h8_elems;
  };
  *owned_block = nullptr;
  if (pc.active()) {
    for (PlaneCache::Entry &e : pc.entries) {
      if (e.src == v.ptr && e.src_bytes == n * sizeof(float)) {
        e.stamp = ++pc.clock;
        ++pc.hits;
        planes_of(e.block);
        return B200_OK;
      }
    }
    ++pc.misses;
  }
  void *block = nullptr;
  const int rc = ctx->pool.alloc(block_bytes, &block, nullptr);
  if (rc != B200_OK) return rc;
  planes_of(block);
  {
    ProfScope prof(ctx, kProfPack, stream);
    const unsigned long long n4 = n / 4ull;
    const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 16ull;
    const unsigned long long need = (n4 + 1023ull) / 1024ull;
    b200::launch(ctx, pack_mix_flat_kernel, dim3(static_cast<unsigned>(need < cap ? need : cap)), dim3(256), 0, stream, 1u, static_cast<const float4 *>(v.ptr), reinterpret_cast<float4 *>(const_cast<void *>(planes_out[0])),
        reinterpret_cast<uint2 *>(const_cast<void *>(planes_out[1])),
        reinterpret_cast<uint2 *>(const_cast<void *>(planes_out[2])), n4);
  }
  ++ctx->launches;
  // inside an entry point that shares planes (scope) without a caller-set cap, keep at most 4 GiB
  const std::size_t cap = pc.cap ? pc.cap : (std::size_t(4) << 30);
  if (!pc.active() || block_bytes > cap) {
    *owned_block = block;
    return B200_OK;
  }
  while (pc.bytes + block_bytes > cap && !pc.entries.empty()) {   // least recently used first
    std::size_t oldest = 0;
    for (std::size_t i = 1; i < pc.entries.size(); ++i)
      if (pc.entries[i].stamp < pc.entries[oldest].stamp) oldest = i;
    void *old = pc.entries[oldest].block;
    pc.bytes -= pc.entries[oldest].block_bytes;
    pc.entries[oldest] = pc.entries.back();
    pc.entries.pop_back();
    ctx->pool.free(old);
  }
  pc.entries.push_back({v.ptr, static_cast<std::size_t>(n * sizeof(float)), block, block_bytes, ++pc.clock});
  pc.bytes += block_bytes;
  return B200_OK;
}

F16Planes f16_planes(const OperandView &v, bool shared) {
  F16Planes lay;
  lay.kpad = (v.k + 7u) & ~7u;
  lay.plane_halves = (static_cast<uint64_t>(v.nbatch) * v.mn * lay.kpad + 127ull) & ~127ull;
  lay.shared = shared;
  lay.scale_floats = (static_cast<uint64_t>(v.mn) * (shared ? 1u : v.nbatch) + 63ull) & ~63ull;
  return lay;
}

void pack_f16(b200_ctx *ctx, cudaStream_t stream, OperandView &v, const F16Planes &lay, char *dst,
              const void *planes_out[2], const float **amax_out) {
  float *amax = reinterpret_cast<float *>(dst);
  __half *h0 = reinterpret_cast<__half *>(dst + lay.scale_floats * sizeof(float));
  __half *h1 = h0 + lay.plane_halves;
  const float *src = static_cast<const float *>(v.ptr);
  const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 16ull;
  const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && v.ld % 4u == 0 &&
                       (v.nbatch <= 1 || v.batch_stride % 4u == 0) && v.k % 8u == 0;
  const unsigned long long scale_rows = static_cast<unsigned long long>(v.mn) * (lay.shared ? 1u : v.nbatch);
  {
    ProfScope prof(ctx, kProfPack, stream);
    if (!v.mn_major && aligned && !lay.shared) {
      // maximum and split in one kernel: a row per CTA, or per warp when rows are short
      const unsigned long long rows = static_cast<unsigned long long>(v.mn) * v.nbatch;
      if (v.k >= 2048u) {
        b200::launch(ctx, pack_f16_rows_kernel<256>, dim3(static_cast<unsigned>(rows < cap ? rows : cap)), dim3(256), 0, stream, 1u, src, amax, h0, h1, v.mn, v.k, v.ld, v.batch_stride, rows);
      } else {
        const unsigned long long ctas = (rows + 7ull) / 8ull;
        b200::launch(ctx, pack_f16_rows_kernel<32>, dim3(static_cast<unsigned>(ctas < cap ? ctas : cap)), dim3(256), 0, stream, 1u, src, amax, h0, h1, v.mn, v.k, v.ld, v.batch_stride, rows);
      }
      ctx->launches += 1;
    } else {
      if (v.mn_major) {
        // k slices over grid.y so that at least ~2 CTAs per SM work on a tall, narrow operand
        const unsigned long long tiles = static_cast<unsigned long long>((v.mn + 31u) / 32u) * v.nbatch;
        unsigned long long slices = (2ull * ctx->sm_count + tiles - 1) / tiles;
        const unsigned long long most = v.k / 64u ? v.k / 64u : 1;
        if (slices > most) slices = most;
        if (slices > 1024ull) slices = 1024ull;
        const uint32_t k_slice = static_cast<uint32_t>((v.k + slices - 1) / slices);
        const unsigned gy = static_cast<unsigned>((v.k + k_slice - 1) / k_slice);
        queue_drain(ctx);
        cudaMemsetAsync(amax, 0, scale_rows * sizeof(float), stream);
        b200::launch(ctx, row_max_mnmajor_kernel, dim3(static_cast<unsigned>(tiles < cap ? tiles : cap), gy), dim3(256), 0, stream, 1u, src, amax, v.mn, v.k, v.ld, v.batch_stride, v.nbatch, lay.shared, k_slice);
      } else {
        const unsigned long long t = (scale_rows + 7ull) / 8ull;
        b200::launch(ctx, row_max_kmajor_kernel, dim3(static_cast<unsigned>(t < cap ? t : cap)), dim3(256), 0, stream, 1u, src, amax, v.mn, v.k, v.ld, v.batch_stride, v.nbatch, lay.shared);
      }
      if (v.mn_major && aligned && v.mn % 4u == 0) {
        const uint32_t tiles_mn = (v.mn + 63u) / 64u, tiles_k = (v.k + 63u) / 64u;
        const unsigned long long tt = static_cast<unsigned long long>(tiles_mn) * tiles_k * v.nbatch;
        b200::launch(ctx, pack_f16_transpose64_kernel, dim3(static_cast<unsigned>(tt < cap ? tt : cap)), dim3(256), 0, stream, 1u, src, amax, h0, h1, v.mn, v.k, v.ld, v.batch_stride, tiles_mn, tiles_k, tt, lay.shared);
      } else {
        const uint32_t tiles_mn = (v.mn + 31u) / 32u, tiles_k = (v.k + 31u) / 32u;
        const unsigned long long tt = static_cast<unsigned long long>(tiles_mn) * tiles_k * v.nbatch;
        const unsigned blocks = static_cast<unsigned>(tt < cap ? tt : cap);
        if (v.mn_major)
          b200::launch(ctx, pack_f16_kernel<true>, dim3(blocks), dim3(256), 0, stream, 1u, src, amax, h0, h1, v.mn, v.k, lay.kpad, v.ld,
                                                          v.batch_stride, tiles_mn, tiles_k, tt, lay.shared);
        else
          b200::launch(ctx, pack_f16_kernel<false>, dim3(blocks), dim3(256), 0, stream, 1u, src, amax, h0, h1, v.mn, v.k, lay.kpad, v.ld,
                                                           v.batch_stride, tiles_mn, tiles_k, tt, lay.shared);
      }
      ctx->launches += 2;
    }
  }
  planes_out[0] = h0;
  planes_out[1] = h1;
  *amax_out = amax;
  v.ptr = h0;
  v.mn_major = false;
  v.ld = lay.kpad;
  v.batch_stride = static_cast<uint64_t>(v.mn) * lay.kpad;
}

}  // namespace b200
