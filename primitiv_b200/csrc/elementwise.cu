// Elementwise kernels: unary (+ constant), scalar-operand, binary with batch
// broadcasting, in-place add / scale, fill, identity, host I/O and copies.
//
// Flat kernels move 128 bits per thread per access (4 floats / 8 halves) when the
// pointers are 16-byte aligned, with a scalar tail; arithmetic is fp32 for both storage
// types.  A gradient that is not batched receives the sum over the batch: one thread
// per element walks the batch in order, so results are deterministic and no kernel uses
// atomics.
#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr unsigned kBlock = 256;

// ------------------------------- unary ---------------------------------------

template <int OP>
__device__ __forceinline__ float unary_f(float x, float k, int ik) {
  if constexpr (OP == B200_OP_NEGATE) return -x;
  else if constexpr (OP == B200_OP_ABS) return fabsf(x);
  else if constexpr (OP == B200_OP_SQRT) return sqrtf(x);
  else if constexpr (OP == B200_OP_EXP) return expf(x);
  else if constexpr (OP == B200_OP_LOG) return logf(x);
  else if constexpr (OP == B200_OP_TANH) return tanhf(x);
  else if constexpr (OP == B200_OP_SIGMOID) return .5f + .5f * tanhf(.5f * x);
  else if constexpr (OP == B200_OP_SOFTPLUS) return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
  else if constexpr (OP == B200_OP_SIN) return sinf(x);
  else if constexpr (OP == B200_OP_COS) return cosf(x);
  else if constexpr (OP == B200_OP_TAN) return tanf(x);
  else if constexpr (OP == B200_OP_ADD_CONST) return x + k;
  else if constexpr (OP == B200_OP_SUB_CONST_R) return x - k;
  else if constexpr (OP == B200_OP_SUB_CONST_L) return k - x;
  else if constexpr (OP == B200_OP_MUL_CONST) return x * k;
  else if constexpr (OP == B200_OP_DIV_CONST_R) return x / k;
  else if constexpr (OP == B200_OP_DIV_CONST_L) return k / x;
  else if constexpr (OP == B200_OP_POW_CONST_R) return powf(x, k);
  else if constexpr (OP == B200_OP_POW_CONST_L) return powf(k, x);
  else if constexpr (OP == B200_OP_PRELU) return x > 0.f ? x : k * x;
  else if constexpr (OP == B200_OP_ELU) return x > 0.f ? x : k * (expf(x) - 1.f);
  else if constexpr (OP == B200_OP_POWN) {
    // exponentiation by squaring on |ik|, reciprocal for negative exponents
    unsigned r = ik < 0 ? 0u - static_cast<unsigned>(ik) : static_cast<unsigned>(ik);
    float ret = 1.f, f = x;
    while (r) {
      if (r & 1u) ret *= f;
      f *= f;
      r >>= 1;
    }
    return ik >= 0 ? ret : 1.f / ret;
  }
  return 0.f;
}

// the amount added to gx
template <int OP>
__device__ __forceinline__ float unary_d(float x, float y, float gy, float k, int ik) {
  if constexpr (OP == B200_OP_NEGATE) return -gy;
  else if constexpr (OP == B200_OP_ABS) return ((x > 0.f) - (x < 0.f)) * gy;
  else if constexpr (OP == B200_OP_SQRT) return .5f * gy / y;
  else if constexpr (OP == B200_OP_EXP) return y * gy;
  else if constexpr (OP == B200_OP_LOG) return gy / x;
  else if constexpr (OP == B200_OP_TANH) return (1.f - y * y) * gy;
  else if constexpr (OP == B200_OP_SIGMOID) return y * (1.f - y) * gy;
  else if constexpr (OP == B200_OP_SOFTPLUS) return (.5f + .5f * tanhf(.5f * x)) * gy;
  else if constexpr (OP == B200_OP_SIN) return cosf(x) * gy;
  else if constexpr (OP == B200_OP_COS) return -sinf(x) * gy;
  else if constexpr (OP == B200_OP_TAN) return (1.f + y * y) * gy;
  else if constexpr (OP == B200_OP_ADD_CONST) return gy;
  else if constexpr (OP == B200_OP_SUB_CONST_R) return gy;
  else if constexpr (OP == B200_OP_SUB_CONST_L) return -gy;
  else if constexpr (OP == B200_OP_MUL_CONST) return k * gy;
  else if constexpr (OP == B200_OP_DIV_CONST_R) return gy / k;
  else if constexpr (OP == B200_OP_DIV_CONST_L) return -y * gy / x;
  else if constexpr (OP == B200_OP_POW_CONST_R) return k * gy * y / x;
  else if constexpr (OP == B200_OP_POW_CONST_L) return logf(k) * gy * y;
  else if constexpr (OP == B200_OP_PRELU) return x > 0.f ? gy : k * gy;
  else if constexpr (OP == B200_OP_ELU) return x > 0.f ? gy : (y + k) * gy;
  else if constexpr (OP == B200_OP_POWN) return static_cast<float>(ik) * gy * y / x;
  return 0.f;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kBlock) unary_fw_kernel(const T *__restrict__ x, T *__restrict__ y,
                                                          u64 n, float k, int ik, int vec) {
  pdl_enter();
  const u64 tid = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x;
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  constexpr int N = Vec<T>::N;
  const u64 nv = vec ? n / N : 0;
  for (u64 i = tid; i < nv; i += stride) {
    Vec<T> v;
    v.load(x + i * N);
#pragma unroll
    for (int j = 0; j < N; ++j) v.set(j, unary_f<OP>(v.get(j), k, ik));
    v.store(y + i * N);
  }
  for (u64 i = nv * N + tid; i < n; i += stride) st(y, i, unary_f<OP>(ld(x, i), k, ik));
}

template <typename T, int OP>
__global__ void __launch_bounds__(kBlock) unary_bw_kernel(const T *__restrict__ x, const T *__restrict__ y,
                                                          const T *__restrict__ gy, T *__restrict__ gx,
                                                          u64 n, float k, int ik, int vec, int accumulate) {
  pdl_enter();
  const u64 tid = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x;
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  constexpr int N = Vec<T>::N;
  const u64 nv = vec ? n / N : 0;
  for (u64 i = tid; i < nv; i += stride) {
    Vec<T> vx, vy, vg, vo;
    vx.load(x + i * N);
    vy.load(y + i * N);
    vg.load(gy + i * N);
    if (accumulate) vo.load(gx + i * N);
#pragma unroll
    for (int j = 0; j < N; ++j)
      vo.set(j, (accumulate ? vo.get(j) : 0.f) + unary_d<OP>(vx.get(j), vy.get(j), vg.get(j), k, ik));
    vo.store(gx + i * N);
  }
  for (u64 i = nv * N + tid; i < n; i += stride)
    st(gx, i, (accumulate ? ld(gx, i) : 0.f) + unary_d<OP>(ld(x, i), ld(y, i), ld(gy, i), k, ik));
}

// ------------------------------- binary --------------------------------------

template <int OP>
__device__ __forceinline__ float binary_f(float a, float b) {
  if constexpr (OP == B200_OP_ADD) return a + b;
  else if constexpr (OP == B200_OP_SUBTRACT) return a - b;
  else if constexpr (OP == B200_OP_MULTIPLY) return a * b;
  else if constexpr (OP == B200_OP_DIVIDE) return a / b;
  else if constexpr (OP == B200_OP_POW) return powf(a, b);
  else if constexpr (OP == B200_OP_SUBTRACT_L) return b - a;
  else if constexpr (OP == B200_OP_DIVIDE_L) return b / a;
  else if constexpr (OP == B200_OP_POW_L) return powf(b, a);
  return 0.f;
}

template <int OP>
__device__ __forceinline__ void binary_d(float a, float b, float y, float gy, float &da, float &db) {
  if constexpr (OP == B200_OP_ADD) { da = gy; db = gy; }
  else if constexpr (OP == B200_OP_SUBTRACT) { da = gy; db = -gy; }
  else if constexpr (OP == B200_OP_MULTIPLY) { da = gy * b; db = gy * a; }
  else if constexpr (OP == B200_OP_DIVIDE) { const float t = gy / b; da = t; db = -t * y; }
  else if constexpr (OP == B200_OP_POW) { const float t = gy * y; da = t * b / a; db = t * logf(a); }
  else { da = 0.f; db = 0.f; }
}

// y[n][i] = f(a[n or 0][i], b[n or 0][i]); flat over volume * batch
template <typename T, int OP>
__global__ void __launch_bounds__(kBlock) binary_fw_kernel(const T *__restrict__ a, const T *__restrict__ b,
                                                           T *__restrict__ y, u64 volume, u64 total,
                                                           int a_batched, int b_batched, int vec) {
  pdl_enter();
  const u64 tid = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x;
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  constexpr int N = Vec<T>::N;
  const u64 nv = vec ? total / N : 0;  // vec implies volume % N == 0: a vector never straddles a batch
  for (u64 i = tid; i < nv; i += stride) {
    const u64 e = i * N;
    const u64 in_vol = e % volume;
    Vec<T> va, vb, vo;
    va.load(a + (a_batched ? e : in_vol));
    vb.load(b + (b_batched ? e : in_vol));
#pragma unroll
    for (int j = 0; j < N; ++j) vo.set(j, binary_f<OP>(va.get(j), vb.get(j)));
    vo.store(y + e);
  }
  for (u64 e = nv * N + tid; e < total; e += stride) {
    const u64 in_vol = e % volume;
    st(y, e, binary_f<OP>(ld(a, a_batched ? e : in_vol), ld(b, b_batched ? e : in_vol)));
  }
}

// Both operands batched (or no batch at all): every gradient element receives exactly one term.
template <typename T, int OP>
__global__ void __launch_bounds__(kBlock) binary_bw_flat_kernel(const T *__restrict__ a, const T *__restrict__ b,
                                                                const T *__restrict__ y, const T *__restrict__ gy,
                                                                T *ga, T *gb, u64 total, int acc_a, int acc_b) {
  pdl_enter();
  // ga and gb are deliberately not __restrict__: for x + x (or x * x) they are the same array,
  // and the two updates of an element must then happen one after the other.
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 e = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    float da, db;
    binary_d<OP>(ld(a, e), ld(b, e), ld(y, e), ld(gy, e), da, db);
    st(ga, e, (acc_a ? ld(ga, e) : 0.f) + da);
    st(gb, e, (acc_b ? ld(gb, e) : 0.f) + db);
  }
}

// One operand is broadcast over the batch: its gradient is the sum over the batch of the
// per-item terms (32 x 8 CTAs over volume x batch slices, see batch_sum_tile_kernel); the
// batched operand's gradient is updated in place on the way.
template <typename T, int OP>
__global__ void __launch_bounds__(256) binary_bw_mixed_kernel(const T *__restrict__ a, const T *__restrict__ b,
                                                              const T *__restrict__ y, const T *__restrict__ gy,
                                                              T *ga, T *gb, float *partial, u64 volume,
                                                              uint32_t batch, uint32_t slice_len, int a_batched,
                                                              int acc_batched, int acc_summed) {
  pdl_enter();
  __shared__ float buf[kSumLanes][32];
  T *g_batched = a_batched ? ga : gb, *g_summed = a_batched ? gb : ga;
  for (u64 tile = blockIdx.x; tile * 32ull < volume; tile += gridDim.x) {
    const u64 i = tile * 32ull + threadIdx.x;
    const uint32_t lo = blockIdx.y * slice_len;
    const uint32_t hi = lo + slice_len < batch ? lo + slice_len : batch;
    float v = 0.f;
    if (i < volume) {
      for (uint32_t n = lo + threadIdx.y; n < hi; n += kSumLanes) {
        const u64 e = static_cast<u64>(n) * volume + i;
        float da, db;
        binary_d<OP>(ld(a, a_batched ? e : i), ld(b, a_batched ? i : e), ld(y, e), ld(gy, e), da, db);
        st(g_batched, e, (acc_batched ? ld(g_batched, e) : 0.f) + (a_batched ? da : db));
        v += a_batched ? db : da;
      }
    }
    const float t = combine_batch_lanes(v, buf);
    if (threadIdx.y == 0 && i < volume) {
      if (gridDim.y == 1) st(g_summed, i, (acc_summed ? ld(g_summed, i) : 0.f) + t);
      else partial[static_cast<u64>(blockIdx.y) * volume + i] = t;
    }
  }
}

// Vector form of binary_bw_mixed_kernel (volume a multiple of the vector width, every array 16-byte
// aligned): a thread owns one 128-bit vector of the volume, and four batch items are loaded before
// the first of them is stored, so that the stores (which may alias the loads as far as the
// compiler knows) do not put one memory latency between every two items.  Only the operands the
// derivative needs are read at all (none for + and -).
template <typename T, int OP>
__global__ void __launch_bounds__(256) binary_bw_mixed_vec_kernel(const T *__restrict__ a, const T *__restrict__ b,
                                                                  const T *__restrict__ y, const T *__restrict__ gy,
                                                                  T *ga, T *gb, float *partial, u64 volume,
                                                                  uint32_t batch, uint32_t slice_len, int a_batched,
                                                                  int acc_batched, int acc_summed) {
  pdl_enter();
  constexpr int N = Vec<T>::N;
  constexpr unsigned U = 4;
  constexpr bool kNeedA = OP == B200_OP_MULTIPLY || OP == B200_OP_POW;                        // db or da reads a
  constexpr bool kNeedB = OP == B200_OP_MULTIPLY || OP == B200_OP_DIVIDE || OP == B200_OP_POW;
  constexpr bool kNeedY = OP == B200_OP_DIVIDE || OP == B200_OP_POW;
  __shared__ float buf[kSumLanes][32 * N];
  T *g_batched = a_batched ? ga : gb, *g_summed = a_batched ? gb : ga;
  const T *op_batched = a_batched ? a : b, *op_shared = a_batched ? b : a;
  const bool need_batched = a_batched ? kNeedA : kNeedB, need_shared = a_batched ? kNeedB : kNeedA;
  for (u64 tile = blockIdx.x; tile * (32ull * N) < volume; tile += gridDim.x) {
    const u64 i = (tile * 32ull + threadIdx.x) * N;
    const uint32_t lo = blockIdx.y * slice_len;
    const uint32_t hi = lo + slice_len < batch ? lo + slice_len : batch;
    float v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = 0.f;
    if (i < volume) {
      Vec<T> vs;
      vs.raw = {};
      if (need_shared) vs.load(op_shared + i);
      for (uint32_t n = lo + threadIdx.y; n < hi; n += kSumLanes * U) {
        Vec<T> vgy[U], vop[U], vy[U], vold[U];
#pragma unroll
        for (unsigned u = 0; u < U; ++u) {
          vop[u].raw = {};
          vy[u].raw = {};
          vold[u].raw = {};
          if (n + u * kSumLanes < hi) {
            const u64 e = static_cast<u64>(n + u * kSumLanes) * volume + i;
            vgy[u].load(gy + e);
            if (need_batched) vop[u].load(op_batched + e);
            if (kNeedY) vy[u].load(y + e);
            if (acc_batched) vold[u].load(g_batched + e);
          }
        }
#pragma unroll
        for (unsigned u = 0; u < U; ++u) {
          if (n + u * kSumLanes < hi) {
            const u64 e = static_cast<u64>(n + u * kSumLanes) * volume + i;
            Vec<T> out;
#pragma unroll
            for (int j = 0; j < N; ++j) {
              const float av = a_batched ? vop[u].get(j) : vs.get(j), bv = a_batched ? vs.get(j) : vop[u].get(j);
              float da, db;
              binary_d<OP>(av, bv, vy[u].get(j), vgy[u].get(j), da, db);
              out.set(j, (acc_batched ? vold[u].get(j) : 0.f) + (a_batched ? da : db));
              v[j] += a_batched ? db : da;
            }
            out.store(g_batched + e);
          }
        }
      }
    }
    combine_batch_lanes_vec<N>(v, buf);
    if (threadIdx.y == 0 && i < volume) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        if (gridDim.y == 1) st(g_summed, i + j, (acc_summed ? ld(g_summed, i + j) : 0.f) + v[j]);
        else partial[static_cast<u64>(blockIdx.y) * volume + i + j] = v[j];
      }
    }
  }
}

// y[n][i] = x[n or 0][i] op k[n or 0]
template <typename T, int OP>
__global__ void __launch_bounds__(kBlock) scalar_fw_kernel(const T *__restrict__ x, const T *__restrict__ k,
                                                           T *__restrict__ y, u64 volume, u64 total,
                                                           int x_batched, int k_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 e = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const u64 n = e / volume, i = e - n * volume;
    st(y, e, binary_f<OP>(ld(x, x_batched ? e : i), ld(k, k_batched ? n : 0)));
  }
}

// y[n or 0] += sign * x[n or 0]
template <typename T>
__global__ void __launch_bounds__(kBlock) inplace_add_kernel(const T *__restrict__ x, T *__restrict__ y,
                                                             u64 volume, uint32_t bx, uint32_t by, float sign,
                                                             int vec, int accumulate) {
  pdl_enter();
  const u64 tid = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x;
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  constexpr int N = Vec<T>::N;
  {
    // every destination element gets exactly one source element: flat and vectorised
    // (a batch-1 destination of a batched source is a batch sum: launch_batch_sum);
    // accumulate == 0: y holds nothing yet and is stored, not added to
    const u64 total = volume * by;
    const u64 nv = vec ? total / N : 0;
    for (u64 i = tid; i < nv; i += stride) {
      const u64 e = i * N;
      Vec<T> vx, vy;
      vx.load(x + (bx > 1 ? e : e % volume));
      if (accumulate) vy.load(y + e);
#pragma unroll
      for (int j = 0; j < N; ++j) vy.set(j, (accumulate ? vy.get(j) : 0.f) + sign * vx.get(j));
      vy.store(y + e);
    }
    for (u64 e = nv * N + tid; e < total; e += stride)
      st(y, e, (accumulate ? ld(y, e) : 0.f) + sign * ld(x, bx > 1 ? e : e % volume));
  }
}

template <typename T>
__global__ void __launch_bounds__(kBlock) fill_kernel(T *__restrict__ y, u64 n, float value, int vec) {
  pdl_enter();
  const u64 tid = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x;
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  constexpr int N = Vec<T>::N;
  const u64 nv = vec ? n / N : 0;
  Vec<T> v;
#pragma unroll
  for (int j = 0; j < N; ++j) v.set(j, value);
  for (u64 i = tid; i < nv; i += stride) v.store(y + i * N);
  for (u64 i = nv * N + tid; i < n; i += stride) st(y, i, value);
}

// in place, so no __restrict__ / read-only loads here
template <typename T>
__global__ void __launch_bounds__(kBlock) scale_kernel(T *x, u64 n, float k) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 i = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    st(x, i, ld(x, i) * k);
}

template <typename T>
__global__ void __launch_bounds__(kBlock) identity_kernel(T *__restrict__ y, uint32_t size) {
  pdl_enter();
  const u64 total = static_cast<u64>(size) * size;
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 e = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride)
    st(y, e, (e % (static_cast<u64>(size) + 1)) == 0 ? 1.f : 0.f);
}

template <typename S, typename D>
__global__ void __launch_bounds__(kBlock) convert_kernel(const S *__restrict__ x, D *__restrict__ y, u64 n) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 i = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) st(y, i, ld(x, i));
}

#define B200_UNARY_OPS(X) \
  X(0) X(1) X(2) X(3) X(4) X(5) X(6) X(7) X(8) X(9) X(10) X(11) X(12) X(13) X(14) X(15) X(16) X(17) \
  X(18) X(19) X(20) X(21)
#define B200_BINARY_OPS(X) X(0) X(1) X(2) X(3) X(4)
#define B200_SCALAR_OPS(X) X(0) X(1) X(2) X(3) X(4) X(5) X(6) X(7)

template <typename T>
void launch_unary_fw(b200_ctx *ctx, cudaStream_t s, int op, const void *x, void *y, u64 n, float k,
                     int ik, int vec) {
  const unsigned grid = grid_for(ctx, n / (vec ? Vec<T>::N : 1) + 1, kBlock);
  switch (op) {
#define X(OP) case OP: b200::launch(ctx, unary_fw_kernel<T, OP>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), n, k, ik, vec); break;
    B200_UNARY_OPS(X)
#undef X
  }
}

template <typename T>
void launch_unary_bw(b200_ctx *ctx, cudaStream_t s, int op, const void *x, const void *y, const void *gy,
                     void *gx, u64 n, float k, int ik, int vec, int accumulate) {
  const unsigned grid = grid_for(ctx, n / (vec ? Vec<T>::N : 1) + 1, kBlock);
  switch (op) {
#define X(OP) case OP: b200::launch(ctx, unary_bw_kernel<T, OP>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<const T *>(y), static_cast<const T *>(gy), static_cast<T *>(gx), n, k, ik, vec, accumulate); break;
    B200_UNARY_OPS(X)
#undef X
  }
}

template <typename T>
void launch_scalar_fw(b200_ctx *ctx, cudaStream_t s, int op, const void *x, const void *k, void *y,
                      u64 volume, u64 total, int x_batched, int k_batched) {
  const unsigned grid = grid_for(ctx, total, kBlock);
  switch (op) {
#define X(OP) case OP: b200::launch(ctx, scalar_fw_kernel<T, OP>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<const T *>(k), static_cast<T *>(y), volume, total, x_batched, k_batched); break;
    B200_SCALAR_OPS(X)
#undef X
  }
}

template <typename T>
void launch_binary_fw(b200_ctx *ctx, cudaStream_t s, int op, const void *a, const void *b, void *y,
                      u64 volume, u64 total, int a_batched, int b_batched) {
  const int vec = aligned16(a) && aligned16(b) && aligned16(y) && volume % Vec<T>::N == 0;
  const unsigned grid = grid_for(ctx, total / (vec ? Vec<T>::N : 1) + 1, kBlock);
  switch (op) {
#define X(OP) case OP: b200::launch(ctx, binary_fw_kernel<T, OP>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(y), volume, total, a_batched, b_batched, vec); break;
    B200_BINARY_OPS(X)
#undef X
  }
}

template <typename T>
int launch_binary_bw(b200_ctx *ctx, cudaStream_t s, int op, const void *a, const void *b, const void *y,
                     const void *gy, void *ga, void *gb, u64 volume, uint32_t batch, int a_batched,
                     int b_batched, int acc_a, int acc_b) {
  const T *pa = static_cast<const T *>(a), *pb = static_cast<const T *>(b), *py = static_cast<const T *>(y),
          *pgy = static_cast<const T *>(gy);
  T *pga = static_cast<T *>(ga), *pgb = static_cast<T *>(gb);
  if (batch == 1 || (a_batched && b_batched)) {
    const u64 total = volume * batch;
    const unsigned grid = grid_for(ctx, total, kBlock);
    switch (op) {
#define X(OP) case OP: b200::launch(ctx, binary_bw_flat_kernel<T, OP>, dim3(grid), dim3(kBlock), 0, s, 1u, pa, pb, py, pgy, pga, pgb, total, acc_a, acc_b); break;
      B200_BINARY_OPS(X)
#undef X
    }
    return B200_OK;
  }
  constexpr unsigned N = Vec<T>::N;
  const bool vec = volume % N == 0 && volume >= 32ull * N && aligned16(a) && aligned16(b) && aligned16(y) &&
                   aligned16(gy) && aligned16(ga) && aligned16(gb);
  const BatchSlices bs = batch_slices(ctx, volume, batch, vec ? 32u * N : 32u);
  void *partial = nullptr;
  if (bs.slices > 1) {
    const int rc = ctx->pool.alloc(static_cast<size_t>(bs.slices) * volume * sizeof(float), &partial, nullptr);
    if (rc != B200_OK) return rc;
  }
  const dim3 grid(bs.tiles, bs.slices), block(32, kSumLanes);
  if (vec) {
    switch (op) {
#define X(OP) case OP: b200::launch(ctx, binary_bw_mixed_vec_kernel<T, OP>, dim3(grid), dim3(block), 0, s, 1u, pa, pb, py, pgy, pga, pgb, static_cast<float *>(partial), volume, batch, bs.slice_len, a_batched, a_batched ? acc_a : acc_b, a_batched ? acc_b : acc_a); break;
      B200_BINARY_OPS(X)
#undef X
    }
  } else {
    switch (op) {
#define X(OP) case OP: b200::launch(ctx, binary_bw_mixed_kernel<T, OP>, dim3(grid), dim3(block), 0, s, 1u, pa, pb, py, pgy, pga, pgb, static_cast<float *>(partial), volume, batch, bs.slice_len, a_batched, a_batched ? acc_a : acc_b, a_batched ? acc_b : acc_a); break;
      B200_BINARY_OPS(X)
#undef X
    }
  }
  if (bs.slices > 1) {
    launch_batch_final<T>(ctx, s, static_cast<const float *>(partial), a_batched ? pgb : pga, volume, bs.slices, 1.f,
                          a_batched ? acc_b : acc_a);
    ctx->pool.free(partial);  // stream-ordered reuse
  }
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_unary_fw(b200_ctx *ctx, int mode, int op, const void *x, void *y, uint64_t n, float k,
                  int32_t ik, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!x || !y || op < 0 || op >= B200_OP_UNARY_COUNT) return B200_ERR_INVALID_ARG;
  const int vec = aligned16(x) && aligned16(y);
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, { launch_unary_fw<T>(ctx, s, op, x, y, n, k, ik, vec); });
  B200_OPS_EPILOGUE(ctx);
}

int b200_unary_bw(b200_ctx *ctx, int mode, int op, const void *x, const void *y, const void *gy,
                  void *gx, uint64_t n, float k, int32_t ik, int accumulate, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!x || !y || !gy || !gx || op < 0 || op >= B200_OP_UNARY_COUNT) return B200_ERR_INVALID_ARG;
  const int vec = aligned16(x) && aligned16(y) && aligned16(gy) && aligned16(gx);
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, { launch_unary_bw<T>(ctx, s, op, x, y, gy, gx, n, k, ik, vec, accumulate ? 1 : 0); });
  B200_OPS_EPILOGUE(ctx);
}

int b200_scalar_fw(b200_ctx *ctx, int mode, int op, const void *x, const void *k, void *y,
                   uint64_t volume, uint32_t batch, int x_batched, int k_batched, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 total = volume * batch;
  if (total == 0) return B200_OK;
  if (!x || !k || !y || op < 0 || op >= B200_OP_BINARY_COUNT) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, { launch_scalar_fw<T>(ctx, s, op, x, k, y, volume, total, x_batched, k_batched); });
  B200_OPS_EPILOGUE(ctx);
}

int b200_binary_fw(b200_ctx *ctx, int mode, int op, const void *a, const void *b, void *y,
                   uint64_t volume, uint32_t batch, int a_batched, int b_batched, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 total = volume * batch;
  if (total == 0) return B200_OK;
  if (!a || !b || !y || op < 0 || op > B200_OP_POW) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, { launch_binary_fw<T>(ctx, s, op, a, b, y, volume, total, a_batched, b_batched); });
  B200_OPS_EPILOGUE(ctx);
}

int b200_binary_bw(b200_ctx *ctx, int mode, int op, const void *a, const void *b, const void *y,
                   const void *gy, void *ga, void *gb, uint64_t volume, uint32_t batch, int a_batched,
                   int b_batched, int accumulate_a, int accumulate_b, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (volume == 0 || batch == 0) return B200_OK;
  if (!a || !b || !y || !gy || !ga || !gb || op < 0 || op > B200_OP_POW) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    const int rc = launch_binary_bw<T>(ctx, s, op, a, b, y, gy, ga, gb, volume, batch, a_batched, b_batched,
                                       accumulate_a ? 1 : 0, accumulate_b ? 1 : 0);
    if (rc != B200_OK) return rc;
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_inplace_add(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t volume, uint32_t bx,
                     uint32_t by, float sign, void *stream) {
  return b200_inplace_add_ex(ctx, mode, x, y, volume, bx, by, sign, 1, stream);
}

int b200_inplace_add_ex(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t volume, uint32_t bx,
                        uint32_t by, float sign, int accumulate, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (volume == 0 || bx == 0 || by == 0) return B200_OK;
  if (!x || !y || (bx != by && bx != 1 && by != 1)) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    if (by == 1 && bx > 1) {
      // the destination receives the sum over the batch
      const int rc = launch_batch_sum<T>(ctx, s, x, y, volume, bx, sign, accumulate ? 1 : 0);
      if (rc != B200_OK) return rc;
    } else {
      const int vec = aligned16(x) && aligned16(y) && volume % Vec<T>::N == 0;
      const u64 work = volume * by / (vec ? Vec<T>::N : 1) + 1;
      b200::launch(ctx, inplace_add_kernel<T>, dim3(grid_for(ctx, work, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), volume, bx, by, sign, vec, accumulate ? 1 : 0);
    }
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_inplace_multiply_const(b200_ctx *ctx, int mode, void *x, uint64_t n, float k, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!x) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, scale_kernel<T>, dim3(grid_for(ctx, n, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<T *>(x), n, k);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_fill(b200_ctx *ctx, int mode, void *y, uint64_t n, float value, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!y) return B200_ERR_INVALID_ARG;
  const int vec = aligned16(y);
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, fill_kernel<T>, dim3(grid_for(ctx, n / (vec ? Vec<T>::N : 1) + 1, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<T *>(y), n, value, vec);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_identity(b200_ctx *ctx, int mode, void *y, uint32_t size, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (size == 0) return B200_OK;
  if (!y) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, identity_kernel<T>, dim3(grid_for(ctx, static_cast<u64>(size) * size, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<T *>(y), size);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_upload(b200_ctx *ctx, int mode, const float *values_host, void *y, uint64_t n, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!values_host || !y) return B200_ERR_INVALID_ARG;
  // Through the context's pinned staging ring: the caller's array may be reused when this
  // returns, and the stream is not waited for (a copy straight from pageable memory would
  // make the runtime drain the stream first, once per input of every step).
  if (mode != B200_MODE_FP16) return ctx->staging.upload(y, values_host, n * sizeof(float), s);
  void *tmp = nullptr;
  int rc = ctx->pool.alloc(n * sizeof(float), &tmp, nullptr);
  if (rc) return rc;
  rc = ctx->staging.upload(tmp, values_host, n * sizeof(float), s);
  if (rc == B200_OK) {
    b200::launch(ctx, convert_kernel<float, __half>, dim3(grid_for(ctx, n, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const float *>(tmp), static_cast<__half *>(y), n);
    ++ctx->launches;
    rc = static_cast<int>(cudaGetLastError());
  }
  ctx->pool.free(tmp);  // stream-ordered reuse
  return rc;
}

int b200_download(b200_ctx *ctx, int mode, const void *x, float *values_host, uint64_t n, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!values_host || !x) return B200_ERR_INVALID_ARG;
  if (mode != B200_MODE_FP16) {
    b200::queue_drain(ctx);
    B200_CUDA_TRY(cudaMemcpyAsync(values_host, x, n * sizeof(float), cudaMemcpyDeviceToHost, s));
    B200_CUDA_TRY(cudaStreamSynchronize(s));
    const int launch_rc = b200::take_launch_error(ctx);
    const int status = b200::take_status(ctx);
    return launch_rc ? launch_rc : status;  // values computed by a kernel whose wait ran out are not handed over silently
  }
  void *tmp = nullptr;
  int rc = ctx->pool.alloc(n * sizeof(float), &tmp, nullptr);
  if (rc) return rc;
  b200::launch(ctx, convert_kernel<__half, float>, dim3(grid_for(ctx, n, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const __half *>(x), static_cast<float *>(tmp), n);
  ++ctx->launches;
  b200::queue_drain(ctx);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(values_host, tmp, n * sizeof(float), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  ctx->pool.free(tmp);
  return e == cudaSuccess ? b200::take_status(ctx) : static_cast<int>(e);
}

int b200_copy(b200_ctx *ctx, int src_mode, const void *x, int dst_mode, void *y, uint64_t n, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (n == 0) return B200_OK;
  if (!x || !y) return B200_ERR_INVALID_ARG;
  const bool sh = src_mode == B200_MODE_FP16, dh = dst_mode == B200_MODE_FP16;
  if (sh == dh) {
    // cudaMemcpyDefault: also right when x lives on another GPU of this process (unified addressing)
    b200::queue_drain(ctx);
    B200_CUDA_TRY(cudaMemcpyAsync(y, x, n * (sh ? 2 : 4), cudaMemcpyDefault, s));
    return B200_OK;
  }
  const unsigned grid = grid_for(ctx, n, kBlock);
  if (sh)
    b200::launch(ctx, convert_kernel<__half, float>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const __half *>(x), static_cast<float *>(y), n);
  else
    b200::launch(ctx, convert_kernel<float, __half>, dim3(grid), dim3(kBlock), 0, s, 1u, static_cast<const float *>(x), static_cast<__half *>(y), n);
  B200_OPS_EPILOGUE(ctx);
}

}  // extern "C"
