// 2-D convolution as a matrix product, and 2-D max pooling.
//
// The reference's conv2d (primitiv/devices/naive/ops/conv2d.cc; cuDNN in its CUDA devices)
// takes x {H, W, C} x batch and w {kh, kw, C, Cout} x batch, column-major with H fastest,
// and computes a true convolution (the kernel is flipped):
//   y[yy, yx, co] = sum_{c, wy, wx} x[yy*s0 - p0 + wy*d0, yx*s1 - p1 + wx*d1, c]
//                                   * w[kh-1-wy, kw-1-wx, c, co]
// With K = kh*kw*C and the K index ordered exactly as w is stored,
//   kk = (c*kw + (kw-1-wx))*kh + (kh-1-wy),
// w is already a column-major {K, Cout} matrix, and with P = Hout*Wout rows p = yx*Hout + yy
// the gathered input Col {P, K} gives  y {P, Cout} = Col . w : one call of the batched,
// broadcasting matrix product of this library per convolution (tensor cores included), and
// its backward gives gCol = gy . w^T and gw += Col^T . gy.  im2col_kernel builds Col,
// col2im_kernel adds gCol back into gx as a gather (each gx element sums the window
// positions that read it, in a fixed order: no atomics, same bits every run).
#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr unsigned kBlock = 256;

struct ConvGeom {
  uint32_t H, W, C, kh, kw, Ho, Wo;
  uint32_t p0, p1, s0, s1, d0, d1;
};

// Col[n][p + P*kk] = x[n or 0][xy + H*(xx + W*c)] or 0 outside the image
template <typename T>
__global__ void __launch_bounds__(kBlock) im2col_kernel(const T *__restrict__ x, T *__restrict__ col, ConvGeom g,
                                                        u64 per_batch, u64 total, u64 x_volume, int x_batched) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 P = static_cast<u64>(g.Ho) * g.Wo;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / per_batch, e = t - n * per_batch;
    const u64 kk = e / P, p = e - kk * P;
    const uint32_t yx = static_cast<uint32_t>(p / g.Ho), yy = static_cast<uint32_t>(p - static_cast<u64>(yx) * g.Ho);
    const uint32_t wyi = static_cast<uint32_t>(kk % g.kh);
    const uint32_t wxi = static_cast<uint32_t>((kk / g.kh) % g.kw);
    const uint32_t c = static_cast<uint32_t>(kk / (static_cast<u64>(g.kh) * g.kw));
    const long long xy = static_cast<long long>(yy) * g.s0 - g.p0 + static_cast<long long>(g.kh - 1u - wyi) * g.d0;
    const long long xx = static_cast<long long>(yx) * g.s1 - g.p1 + static_cast<long long>(g.kw - 1u - wxi) * g.d1;
    float v = 0.f;
    if (xy >= 0 && xy < g.H && xx >= 0 && xx < g.W)
      v = ld(x, (x_batched ? n * x_volume : 0) + static_cast<u64>(xy) + g.H * (static_cast<u64>(xx) + static_cast<u64>(g.W) * c));
    st(col, t, v);
  }
}

// gx[n][xy, xx, c] += sum over the window positions (wy, wx) and outputs (yy, yx) with
// yy*s0 - p0 + wy*d0 == xy and yx*s1 - p1 + wx*d1 == xx of gCol[n][p, kk]
template <typename T>
__global__ void __launch_bounds__(kBlock) col2im_kernel(const T *__restrict__ gcol, T *gx, ConvGeom g, u64 x_volume,
                                                        u64 total, u64 col_per_batch) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 P = static_cast<u64>(g.Ho) * g.Wo;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 n = t / x_volume, e = t - n * x_volume;
    const uint32_t xy = static_cast<uint32_t>(e % g.H);
    const uint32_t xx = static_cast<uint32_t>((e / g.H) % g.W);
    const uint32_t c = static_cast<uint32_t>(e / (static_cast<u64>(g.H) * g.W));
    const T *src = gcol + n * col_per_batch;
    float acc = 0.f;
    for (uint32_t wx = 0; wx < g.kw; ++wx) {
      const long long nx = static_cast<long long>(xx) + g.p1 - static_cast<long long>(wx) * g.d1;
      if (nx < 0 || nx % g.s1 != 0) continue;
      const long long yx = nx / g.s1;
      if (yx >= g.Wo) continue;
      for (uint32_t wy = 0; wy < g.kh; ++wy) {
        const long long ny = static_cast<long long>(xy) + g.p0 - static_cast<long long>(wy) * g.d0;
        if (ny < 0 || ny % g.s0 != 0) continue;
        const long long yy = ny / g.s0;
        if (yy >= g.Ho) continue;
        const u64 kk = (static_cast<u64>(c) * g.kw + (g.kw - 1u - wx)) * g.kh + (g.kh - 1u - wy);
        acc += ld(src, static_cast<u64>(yx) * g.Ho + static_cast<u64>(yy) + P * kk);
      }
    }
    st(gx, t, ld(gx, t) + acc);
  }
}

struct PoolGeom {
  uint32_t H, W, Ho, Wo, w0, w1, p0, p1, s0, s1;
};

// y[r][yy, yx] = max over the window (primitiv/devices/naive/ops/max_pool2d.cc:10-57)
template <typename T>
__global__ void __launch_bounds__(kBlock) max_pool2d_fw_kernel(const T *__restrict__ x, T *__restrict__ y, PoolGeom g,
                                                               u64 total) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 ys = static_cast<u64>(g.Ho) * g.Wo, xs = static_cast<u64>(g.H) * g.W;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 r = t / ys, e = t - r * ys;
    const uint32_t yx = static_cast<uint32_t>(e / g.Ho), yy = static_cast<uint32_t>(e - static_cast<u64>(yx) * g.Ho);
    float best = -3.402823466e38f;  // numeric_limits<float>::lowest(), as the reference starts
    for (uint32_t wx = 0; wx < g.w1; ++wx) {
      const long long xx = static_cast<long long>(yx) * g.s1 - g.p1 + wx;
      if (xx < 0 || xx >= g.W) continue;
      for (uint32_t wy = 0; wy < g.w0; ++wy) {
        const long long xy = static_cast<long long>(yy) * g.s0 - g.p0 + wy;
        if (xy < 0 || xy >= g.H) continue;
        const float v = ld(x, r * xs + static_cast<u64>(xx) * g.H + static_cast<u64>(xy));
        if (v > best) best = v;
      }
    }
    st(y, t, best);
  }
}

// gx[r][xy, xx] += sum of gy over the windows whose FIRST maximal element (scan order: wx
// outer, wy inner, as max_pool2d.cc:84-121) is this one.  A gather over the windows that
// contain the element, so overlapping windows add in a fixed order.
template <typename T>
__global__ void __launch_bounds__(kBlock) max_pool2d_bw_kernel(const T *__restrict__ x, const T *__restrict__ y,
                                                               const T *__restrict__ gy, T *gx, PoolGeom g, u64 total) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 ys = static_cast<u64>(g.Ho) * g.Wo, xs = static_cast<u64>(g.H) * g.W;
  for (u64 t = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
    const u64 r = t / xs, e = t - r * xs;
    const uint32_t xx = static_cast<uint32_t>(e / g.H), xy = static_cast<uint32_t>(e - static_cast<u64>(xx) * g.H);
    const float mine = ld(x, t);
    float acc = 0.f;
    // windows (yy, yx) with yx*s1 - p1 <= xx < yx*s1 - p1 + w1, likewise for y
    for (uint32_t wx = 0; wx < g.w1; ++wx) {
      const long long nx = static_cast<long long>(xx) + g.p1 - wx;
      if (nx < 0 || nx % g.s1 != 0) continue;
      const long long yx = nx / g.s1;
      if (yx >= g.Wo) continue;
      for (uint32_t wy = 0; wy < g.w0; ++wy) {
        const long long ny = static_cast<long long>(xy) + g.p0 - wy;
        if (ny < 0 || ny % g.s0 != 0) continue;
        const long long yy = ny / g.s0;
        if (yy >= g.Ho) continue;
        const u64 ya = r * ys + static_cast<u64>(yx) * g.Ho + static_cast<u64>(yy);
        if (mine != ld(y, ya)) continue;
        // is an earlier element of that window maximal as well?  (wx, wy) is this element's position
        bool first = true;
        for (uint32_t ex = 0; first && ex <= wx; ++ex) {
          const long long fx = yx * g.s1 - g.p1 + ex;
          if (fx < 0 || fx >= g.W) continue;
          const uint32_t ey_end = ex == wx ? wy : g.w0;
          for (uint32_t ey = 0; ey < ey_end; ++ey) {
            const long long fy = yy * g.s0 - g.p0 + ey;
            if (fy < 0 || fy >= g.H) continue;
            if (ld(x, r * xs + static_cast<u64>(fx) * g.H + static_cast<u64>(fy)) == mine) {
              first = false;
              break;
            }
          }
        }
        if (first) acc += ld(gy, ya);
      }
    }
    if (acc != 0.f) st(gx, t, ld(gx, t) + acc);
  }
}

bool geom_ok(const ConvGeom &g) {
  return g.H && g.W && g.C && g.kh && g.kw && g.Ho && g.Wo && g.s0 && g.s1 && g.d0 && g.d1;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_im2col(b200_ctx *ctx, int mode, const void *x, void *col, uint32_t H, uint32_t W, uint32_t C,
                uint32_t kh, uint32_t kw, uint32_t Ho, uint32_t Wo, uint32_t pad0, uint32_t pad1,
                uint32_t stride0, uint32_t stride1, uint32_t dil0, uint32_t dil1, uint32_t batch, int x_batched,
                void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const ConvGeom g{H, W, C, kh, kw, Ho, Wo, pad0, pad1, stride0, stride1, dil0, dil1};
  if (!x || !col || !geom_ok(g)) return B200_ERR_INVALID_ARG;
  if (batch == 0) return B200_OK;
  const u64 per_batch = static_cast<u64>(Ho) * Wo * kh * kw * C, total = per_batch * batch;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, im2col_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<T *>(col), g, per_batch, total, static_cast<u64>(H) * W * C, x_batched);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_col2im(b200_ctx *ctx, int mode, const void *gcol, void *gx, uint32_t H, uint32_t W, uint32_t C,
                uint32_t kh, uint32_t kw, uint32_t Ho, uint32_t Wo, uint32_t pad0, uint32_t pad1,
                uint32_t stride0, uint32_t stride1, uint32_t dil0, uint32_t dil1, uint32_t batch, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const ConvGeom g{H, W, C, kh, kw, Ho, Wo, pad0, pad1, stride0, stride1, dil0, dil1};
  if (!gcol || !gx || !geom_ok(g)) return B200_ERR_INVALID_ARG;
  if (batch == 0) return B200_OK;
  const u64 x_volume = static_cast<u64>(H) * W * C, total = x_volume * batch;
  const u64 col_per_batch = static_cast<u64>(Ho) * Wo * kh * kw * C;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, col2im_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(gcol), static_cast<T *>(gx),
                                                                   g, x_volume, total, col_per_batch);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_max_pool2d_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint32_t H, uint32_t W, uint32_t Ho,
                       uint32_t Wo, uint32_t window0, uint32_t window1, uint32_t pad0, uint32_t pad1,
                       uint32_t stride0, uint32_t stride1, uint64_t repeat, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const PoolGeom g{H, W, Ho, Wo, window0, window1, pad0, pad1, stride0, stride1};
  if (!x || !y || !H || !W || !Ho || !Wo || !window0 || !window1 || !stride0 || !stride1) return B200_ERR_INVALID_ARG;
  const u64 total = static_cast<u64>(Ho) * Wo * repeat;
  if (total == 0) return B200_OK;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, max_pool2d_fw_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x),
                                                                           static_cast<T *>(y), g, total);
  });
  B200_OPS_EPILOGUE(ctx);
}

int b200_max_pool2d_bw(b200_ctx *ctx, int mode, const void *x, const void *y, const void *gy, void *gx, uint32_t H,
                       uint32_t W, uint32_t Ho, uint32_t Wo, uint32_t window0, uint32_t window1, uint32_t pad0,
                       uint32_t pad1, uint32_t stride0, uint32_t stride1, uint64_t repeat, void *stream) {
  B200_OPS_PROLOGUE(ctx);
  const PoolGeom g{H, W, Ho, Wo, window0, window1, pad0, pad1, stride0, stride1};
  if (!x || !y || !gy || !gx || !H || !W || !Ho || !Wo || !window0 || !window1 || !stride0 || !stride1)
    return B200_ERR_INVALID_ARG;
  const u64 total = static_cast<u64>(H) * W * repeat;
  if (total == 0) return B200_OK;
  ProfScope prof(ctx, kProfElementwise, s);
  B200_DISPATCH_MODE(mode, {
    b200::launch(ctx, max_pool2d_bw_kernel<T>, dim3(grid_for(ctx, total, kBlock)), dim3(kBlock), 0, s, 1u, static_cast<const T *>(x), static_cast<const T *>(y), static_cast<const T *>(gy), static_cast<T *>(gx), g, total);
  });
  B200_OPS_EPILOGUE(ctx);
}

}  // extern "C"
