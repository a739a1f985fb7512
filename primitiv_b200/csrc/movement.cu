// Data-movement kernels: slice / concat / pick / broadcast / batch_pick / transpose /
// permute_dims / flip, forward (copy) and backward (accumulate) forms.
//
// Index conventions are the reference's (primitiv/devices/naive/ops/<op>.cc): a tensor
// is seen as [repeat][dim extent][base] with base = Shape::lower_volume(dim).  Backward
// kernels that may receive several sources for one destination element (a gradient that
// is not batched, or repeated pick ids) give each destination-independent index to one
// thread, which walks the batch in order: deterministic, no atomics.
#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr unsigned kBlock = 256;

// y[r][j][i] (j < y_dim) = x[r][offset + j][i]
template <typename T>
__global__ void __launch_bounds__(kBlock) slice_fw_kernel(const T *__restrict__ x, T *__restrict__ y, u64 base,
                                                          u64 span, u64 skip, u64 off, u64 total) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 e = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const u64 r = e / span, j = e - r * span;
    st(y, e, ld(x, off + r * skip + j));
  }
}

// gx[n][r][offset + j][i] += gy[n or 0][r][j][i]: gx has the full batch, every destination
// element receives exactly one term
template <typename T>
__global__ void __launch_bounds__(kBlock) slice_bw_flat_kernel(const T *__restrict__ gy, T *gx, u64 span, u64 skip,
                                                               u64 off, u64 per_batch, u64 x_volume, u64 total,
                                                               int gy_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / per_batch, e = t - n * per_batch;
    const u64 r = e / span, j = e - r * span;
    const u64 d = n * x_volume + off + r * skip + j;
    st(gx, d, ld(gx, d) + ld(gy, gy_batched ? t : e));
  }
}

// The same when gx is known to hold zeros that were never written (a fresh gradient): every element of
// gx is stored, the slice from gy and the rest as zero, in place of a zero-fill followed by an add.
template <typename T>
__global__ void __launch_bounds__(kBlock) slice_bw_store_kernel(const T *__restrict__ gy, T *__restrict__ gx, u64 span,
                                                                u64 skip, u64 off, u64 per_batch, u64 x_volume,
                                                                u64 total_x, int gy_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 d = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; d < total_x; d += stride) {
    const u64 n = d / x_volume, rem = d - n * x_volume;
    const u64 r = rem / skip, jj = rem - r * skip;
    float v = 0.f;
    if (jj >= off && jj < off + span) {
      const u64 e = r * span + (jj - off);
      v = ld(gy, gy_batched ? n * per_batch + e : e);
    }
    st(gx, d, v);
  }
}

// gx[0][r][offset + j][i] += sum_n gy[n][r][j][i]: a batch-1 destination of a batched gradient
// (32 x 8 CTAs over elements x batch lanes, lanes combined in order: deterministic)
template <typename T>
__global__ void __launch_bounds__(256) slice_bw_sum_kernel(const T *__restrict__ gy, T *gx, u64 span, u64 skip,
                                                           u64 off, u64 per_batch, uint32_t batch) {
  pdl_enter();
  __shared__ float buf[kSumLanes][32];
  for (u64 tile = blockIdx.x; tile * 32ull < per_batch; tile += gridDim.x) {
    const u64 e = tile * 32ull + threadIdx.x;
    float v = 0.f;
    if (e < per_batch)
      for (uint32_t n = threadIdx.y; n < batch; n += kSumLanes) v += ld(gy, static_cast<u64>(n) * per_batch + e);
    const float t = combine_batch_lanes(v, buf);
    if (threadIdx.y == 0 && e < per_batch) {
      const u64 r = e / span, j = e - r * span;
      const u64 d = off + r * skip + j;
      st(gx, d, ld(gx, d) + t);
    }
  }
}

// y[n][r][offset + j][i] = x[n or 0][r][j][i]
template <typename T>
__global__ void __launch_bounds__(kBlock) concat_part_kernel(const T *__restrict__ x, T *__restrict__ y, u64 span,
                                                             u64 skip, u64 off, u64 per_batch, u64 y_volume,
                                                             u64 total, int x_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / per_batch, e = t - n * per_batch;
    const u64 r = e / span, j = e - r * span;
    st(y, n * y_volume + off + r * skip + j, ld(x, (x_batched ? n * per_batch : 0) + e));
  }
}

// y[n][r][i] = x[n or 0][r][ids[n or 0]][i]
template <typename T>
__global__ void __launch_bounds__(kBlock) pick_fw_kernel(const T *__restrict__ x, const uint32_t *__restrict__ ids,
                                                         T *__restrict__ y, u64 base, u64 skip, u64 per_batch,
                                                         u64 x_volume, u64 total, int x_batched, int ids_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / per_batch, e = t - n * per_batch;
    const u64 r = e / base, i = e - r * base;
    const u64 id = ids[ids_batched ? n : 0];
    st(y, t, ld(x, (x_batched ? n * x_volume : 0) + base * id + r * skip + i));
  }
}

// gx[n or 0][r][ids[n or 0]][i] += gy[n][r][i]; (r, i) decides the destination uniquely for any id
template <typename T>
__global__ void __launch_bounds__(kBlock) pick_bw_kernel(const T *__restrict__ gy, const uint32_t *__restrict__ ids,
                                                         T *gx, u64 base, u64 skip, u64 per_batch, u64 x_volume,
                                                         uint32_t batch, int gx_batched, int ids_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 e = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; e < per_batch; e += stride) {
    const u64 r = e / base, i = e - r * base;
    for (uint32_t n = 0; n < batch; ++n) {
      const u64 id = ids[ids_batched ? n : 0];
      const u64 d = (gx_batched ? static_cast<u64>(n) * x_volume : 0) + base * id + r * skip + i;
      st(gx, d, ld(gx, d) + ld(gy, static_cast<u64>(n) * per_batch + e));
    }
  }
}

// the same with a batched gx: item n only touches gx[n], so (n, r, i) decides the destination
template <typename T>
__global__ void __launch_bounds__(kBlock) pick_bw_flat_kernel(const T *__restrict__ gy,
                                                              const uint32_t *__restrict__ ids, T *gx, u64 base,
                                                              u64 skip, u64 per_batch, u64 x_volume, u64 total,
                                                              int ids_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / per_batch, e = t - n * per_batch;
    const u64 r = e / base, i = e - r * base;
    const u64 d = n * x_volume + base * ids[ids_batched ? n : 0] + r * skip + i;
    st(gx, d, ld(gx, d) + ld(gy, t));
  }
}

// y[.., j, ..] = x[.., 0, ..], j < size
template <typename T>
__global__ void __launch_bounds__(kBlock) broadcast_fw_kernel(const T *__restrict__ x, T *__restrict__ y, u64 skip1,
                                                              u64 size, u64 total_out) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 skip2 = skip1 * size;
  for (u64 o = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; o < total_out; o += stride) {
    const u64 hi = o / skip2, lo = o % skip1;
    st(y, o, ld(x, hi * skip1 + lo));
  }
}

// y[n][i] = x[ids[n]][i]
template <typename T>
__global__ void __launch_bounds__(kBlock) batch_pick_fw_kernel(const T *__restrict__ x,
                                                               const uint32_t *__restrict__ ids, T *__restrict__ y,
                                                               u64 volume, u64 total) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / volume, i = t - n * volume;
    st(y, t, ld(x, static_cast<u64>(ids[n]) * volume + i));
  }
}

// gx[ids[n]][i] += gy[n][i]; one thread per i, batches in order
template <typename T>
__global__ void __launch_bounds__(kBlock) batch_pick_bw_kernel(const T *__restrict__ gy,
                                                               const uint32_t *__restrict__ ids, T *gx, u64 volume,
                                                               uint32_t n_ids) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 i = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; i < volume; i += stride) {
    for (uint32_t n = 0; n < n_ids; ++n) {
      const u64 d = static_cast<u64>(ids[n]) * volume + i;
      st(gx, d, ld(gx, d) + ld(gy, static_cast<u64>(n) * volume + i));
    }
  }
}

// {d1, d2} x batch -> {d2, d1} x batch through a 32x32 shared-memory tile; flat grid over tiles
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *__restrict__ x, T *y, uint32_t d1, uint32_t d2,
                                                        uint32_t tiles1, uint32_t tiles2, u64 total_tiles,
                                                        int accumulate) {
  pdl_enter();
  __shared__ float tile[32][33];
  const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
  const u64 ms = static_cast<u64>(d1) * d2;
  for (u64 t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const u64 per = static_cast<u64>(tiles1) * tiles2;
    const u64 n = t / per;
    const uint32_t rem = static_cast<uint32_t>(t - n * per);
    const uint32_t i0 = (rem % tiles1) * 32u, j0 = (rem / tiles1) * 32u;
#pragma unroll
    for (uint32_t k = 0; k < 32u; k += 8u) {
      const uint32_t i = i0 + tx, j = j0 + ty + k;
      tile[ty + k][tx] = (i < d1 && j < d2) ? ld(x, n * ms + i + static_cast<u64>(j) * d1) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (uint32_t k = 0; k < 32u; k += 8u) {
      const uint32_t j = j0 + tx, i = i0 + ty + k;
      if (i < d1 && j < d2) {
        const u64 o = n * ms + j + static_cast<u64>(i) * d2;
        const float v = tile[tx][ty + k];
        st(y, o, accumulate ? ld(y, o) + v : v);
      }
    }
    __syncthreads();
  }
}

struct PermuteArgs {
  uint32_t ndims;
  uint32_t x_strides[8];  // most significant dimension first, as the reference walks them
  uint32_t y_strides[8];
};

// forward: y[perm(i)] = x[i];  backward: gx[i] += gy[perm(i)]
template <typename T>
__global__ void __launch_bounds__(kBlock) permute_kernel(const T *__restrict__ src, T *dst, PermuteArgs a, u64 volume,
                                                         u64 total, int backward) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / volume;
    uint32_t tmp = static_cast<uint32_t>(t - n * volume);
    const uint32_t i = tmp;
    uint32_t j = 0;
    for (uint32_t d = 0; d < a.ndims; ++d) {
      const uint32_t p = tmp / a.x_strides[d];
      tmp -= p * a.x_strides[d];
      j += p * a.y_strides[d];
    }
    if (backward)
      st(dst, n * volume + i, ld(dst, n * volume + i) + ld(src, n * volume + j));
    else
      st(dst, n * volume + j, ld(src, n * volume + i));
  }
}

// y[.., j, ..] (+)= x[.., n - 1 - j, ..]
template <typename T>
__global__ void __launch_bounds__(kBlock) flip_kernel(const T *__restrict__ x, T *y, u64 skip, u64 n, u64 total,
                                                      int accumulate) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  for (u64 e = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const u64 lo = e % skip, j = (e / skip) % n, hi = e / (skip * n);
    const u64 s = hi * skip * n + (n - 1 - j) * skip + lo;
    st(y, e, accumulate ? ld(y, e) + ld(x, s) : ld(x, s));
  }
}

// Index lists live on the host in primitiv; they are staged through pool memory.
struct DeviceIds {
  b200_ctx *ctx;
  void *p = nullptr;
  explicit DeviceIds(b200_ctx *c) : ctx(c) {}
  ~DeviceIds() { if (p) ctx->pool.free(p); }
  int put(const uint32_t *host, uint32_t n, cudaStream_t s) {
    int rc = ctx->pool.alloc(static_cast<size_t>(n) * sizeof(uint32_t), &p, nullptr);
    if (rc) return rc;
    return ctx->staging.upload(p, host, static_cast<size_t>(n) * sizeof(uint32_t), s);
  }
  const uint32_t *get() const { return static_cast<const uint32_t *>(p); }
};

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_slice_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t base, uint32_t x_dim,
                  uint32_t y_dim, uint32_t offset, uint64_t repeat, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 span = base * y_dim, skip = base * x_dim, total = span * repeat;
  if (total == 0) return B200_OK;
  if (!x || !y || offset + y_dim > x_dim) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, slice_fw_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), base, span, skip, base * offset, total);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_slice_bw(b200_ctx *ctx, int mode, const void *gy, void *gx, uint64_t base, uint32_t x_dim,
                  uint32_t y_dim, uint32_t offset, uint64_t repeat, uint32_t bx, uint32_t by, void *stream) {
  return b200_slice_bw_ex(ctx, mode, gy, gx, base, x_dim, y_dim, offset, repeat, bx, by, 1, stream);
}

int b200_slice_bw_ex(b200_ctx *ctx, int mode, const void *gy, void *gx, uint64_t base, uint32_t x_dim,
                     uint32_t y_dim, uint32_t offset, uint64_t repeat, uint32_t bx, uint32_t by, int accumulate,
                     void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 span = base * y_dim, skip = base * x_dim, per_batch = span * repeat;
  if (bx == 0 || by == 0 || skip * repeat == 0) return B200_OK;
  if (!gx || (per_batch && !gy) || offset + y_dim > x_dim) return B200_ERR_INVALID_ARG;
  if (!accumulate && !(bx > 1 || by == 1)) {
    // a batch-1 destination of a batched gradient: zeros first, then the summing form
    const int rc = b200_fill(ctx, mode, gx, skip * repeat * bx, 0.f, stream);
    if (rc != B200_OK) return rc;
    accumulate = 1;
  }
  if (per_batch == 0 && accumulate) return B200_OK;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    if (!accumulate) {
      const u64 total_x = skip * repeat * bx;
      b200::launch(ctx, slice_bw_store_kernel<T>, dim3(grid_for(ctx, total_x, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(gy), static_cast<T *>(gx), span, skip, base * offset, per_batch, skip * repeat,
          total_x, by > 1);
    } else if (bx > 1 || by == 1) {
      const u64 total = per_batch * bx;
      b200::launch(ctx, slice_bw_flat_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(gy), static_cast<T *>(gx), span, skip, base * offset, per_batch, skip * repeat,
          total, by > 1);
    } else {
      const u64 tiles = (per_batch + 31ull) / 32ull;
      const u64 cap = static_cast<u64>(ctx->sm_count) * 16ull;
      b200::launch(ctx, slice_bw_sum_kernel<T>, dim3(static_cast<unsigned>(tiles < cap ? tiles : cap)), dim3(32, kSumLanes), 0, s, 1u, static_cast<const T *>(gy), static_cast<T *>(gx), span, skip, base * offset, per_batch, by);
    }
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_concat_part(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t base, uint32_t x_dim,
                     uint32_t y_dim, uint32_t offset, uint64_t repeat, uint32_t batch, int x_batched,
                     void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 span = base * x_dim, skip = base * y_dim, per_batch = span * repeat, total = per_batch * batch;
  if (total == 0) return B200_OK;
  if (!x || !y || offset + x_dim > y_dim) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, concat_part_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), span, skip, base * offset, per_batch, skip * repeat,
        total, x_batched);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_pick_fw(b200_ctx *ctx, int mode, const void *x, const uint32_t *ids_host, uint32_t n_ids, void *y,
                 uint64_t base, uint32_t x_dim, uint64_t repeat, uint32_t batch, int x_batched, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 per_batch = base * repeat, total = per_batch * batch, skip = base * x_dim;
  if (total == 0) return B200_OK;
  if (!x || !y || !ids_host || (n_ids != 1 && n_ids != batch)) return B200_ERR_INVALID_ARG;
  for (uint32_t i = 0; i < n_ids; ++i)
    if (ids_host[i] >= x_dim) return B200_ERR_INVALID_ARG;
  DeviceIds ids(ctx);
  int rc = ids.put(ids_host, n_ids, s);
  if (rc) return rc;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, pick_fw_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), ids.get(), static_cast<T *>(y), base, skip, per_batch, skip * repeat, total,
        x_batched, n_ids > 1);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_pick_bw(b200_ctx *ctx, int mode, const void *gy, const uint32_t *ids_host, uint32_t n_ids, void *gx,
                 uint64_t base, uint32_t x_dim, uint64_t repeat, uint32_t batch, int gx_batched, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 per_batch = base * repeat, skip = base * x_dim;
  if (per_batch == 0 || batch == 0) return B200_OK;
  if (!gx || !gy || !ids_host || (n_ids != 1 && n_ids != batch)) return B200_ERR_INVALID_ARG;
  for (uint32_t i = 0; i < n_ids; ++i)
    if (ids_host[i] >= x_dim) return B200_ERR_INVALID_ARG;
  DeviceIds ids(ctx);
  int rc = ids.put(ids_host, n_ids, s);
  if (rc) return rc;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    if (gx_batched) {
      const u64 total = per_batch * batch;
      b200::launch(ctx, pick_bw_flat_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(gy), ids.get(), static_cast<T *>(gx), base, skip, per_batch, skip * repeat, total,
          n_ids > 1);
    } else {
      // a batch-1 gx can receive several items at the same place: one thread per (r, i), items in order
      b200::launch(ctx, pick_bw_kernel<T>, dim3(grid_for(ctx, per_batch, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(gy), ids.get(), static_cast<T *>(gx), base, skip, per_batch, skip * repeat, batch,
          gx_batched, n_ids > 1);
    }
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_broadcast_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t total, uint64_t skip1,
                      uint32_t size, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 total_out = total * size;
  if (total_out == 0) return B200_OK;
  if (!x || !y || skip1 == 0) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, broadcast_fw_kernel<T>, dim3(grid_for(ctx, total_out, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), skip1, size, total_out);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_batch_pick_fw(b200_ctx *ctx, int mode, const void *x, const uint32_t *ids_host, uint32_t n_ids,
                       void *y, uint64_t volume, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const u64 total = volume * n_ids;
  if (total == 0) return B200_OK;
  if (!x || !y || !ids_host) return B200_ERR_INVALID_ARG;
  DeviceIds ids(ctx);
  int rc = ids.put(ids_host, n_ids, s);
  if (rc) return rc;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, batch_pick_fw_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), ids.get(), static_cast<T *>(y), volume, total);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_batch_pick_bw(b200_ctx *ctx, int mode, const void *gy, const uint32_t *ids_host, uint32_t n_ids,
                       void *gx, uint64_t volume, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (volume == 0 || n_ids == 0) return B200_OK;
  if (!gx || !gy || !ids_host) return B200_ERR_INVALID_ARG;
  DeviceIds ids(ctx);
  int rc = ids.put(ids_host, n_ids, s);
  if (rc) return rc;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, batch_pick_bw_kernel<T>, dim3(grid_for(ctx, volume, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(gy), ids.get(), static_cast<T *>(gx), volume, n_ids);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_transpose(b200_ctx *ctx, int mode, const void *x, void *y, uint32_t d1, uint32_t d2, uint32_t batch,
                   int accumulate, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (d1 == 0 || d2 == 0 || batch == 0) return B200_OK;
  if (!x || !y) return B200_ERR_INVALID_ARG;
  const uint32_t t1 = (d1 + 31u) / 32u, t2 = (d2 + 31u) / 32u;
  const u64 tiles = static_cast<u64>(t1) * t2 * batch;
  const u64 cap = static_cast<u64>(ctx->sm_count) * 16ull;
  const unsigned grid = static_cast<unsigned>(tiles < cap ? tiles : cap);
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, transpose_kernel<T>, dim3(grid), dim3(256), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y), d1, d2, t1, t2, tiles,
                                             accumulate);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_permute_dims(b200_ctx *ctx, int mode, const void *x, void *y, uint32_t ndims, const uint32_t *x_dims,
                      const uint32_t *perm, uint32_t batch, int backward, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (!x || !y || ndims > 8 || (ndims && (!x_dims || !perm))) return B200_ERR_INVALID_ARG;
  // strides exactly as primitiv/devices/naive/ops/permute_dims.cc:17-28 builds them;
  // x_dims are the extents of the tensor whose linear index is decomposed (x forward, gx backward)
  PermuteArgs a;
  a.ndims = ndims;
  uint32_t y_dims[8];
  for (uint32_t i = 0; i < ndims; ++i) {
    if (perm[i] >= ndims) return B200_ERR_INVALID_ARG;
    y_dims[i] = x_dims[perm[i]];
  }
  uint32_t xs = 1, ys = 1;
  u64 volume = 1;
  for (uint32_t i = 0; i < ndims; ++i) {
    a.x_strides[ndims - i - 1] = xs;
    a.y_strides[ndims - perm[i] - 1] = ys;
    xs *= x_dims[i];
    ys *= y_dims[i];
    volume *= x_dims[i];
  }
  const u64 total = volume * batch;
  if (total == 0) return B200_OK;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, permute_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y),
                                                                      a, volume, total, backward);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_flip(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t skip, uint32_t n, uint64_t total,
              int accumulate, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (total == 0) return B200_OK;
  if (!x || !y || skip == 0 || n == 0) return B200_ERR_INVALID_ARG;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, flip_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(y),
                                                                   skip, n, total, accumulate);
  });
  B200_OPS_EPILOGUE(ctx);
}

}  // extern "C"
