/*
 * primitiv_b200 -- C ABI of the device operations either side of the matrix product:
 * what primitiv::devices::B200 calls for every Device virtual other than matmul.
 *
 * Semantics follow the reference's Naive device (primitiv/devices/naive/ops/<op>.cc, the
 * op named in each comment); the GPU shape of each kernel replaces
 * primitiv/devices/cuda/ops/<op>.cu.  Same conventions as primitiv_b200.h: device
 * pointers, return codes, `mode` selects the storage type (float for the fp32 modes, IEEE
 * half for B200_MODE_FP16; arithmetic is always fp32, rounded once on store, as in
 * primitiv/devices/cuda16/ops/common.h:16-47), launches go to `stream`.
 *
 * Batch broadcasting: a tensor argument flagged "not batched" has one volume that is
 * read for every batch index; a gradient flagged "not batched" receives the SUM over the
 * batch.  Sums over the batch are computed by one thread walking the batch in order, so
 * every kernel here is deterministic and none uses atomics (the reference CUDA kernels
 * use atomicAdd, e.g. primitiv/devices/cuda/ops/add.cu:16-27).
 * No kernel puts the batch index in grid.y: batches beyond 65535 are fine.
 */
#ifndef PRIMITIV_B200_OPS_H_
#define PRIMITIV_B200_OPS_H_

#include "primitiv_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Elementwise functions of one tensor (and a constant).  y = f(x, k);  gx += f'(x, y, gy, k). */
enum {
  B200_OP_NEGATE = 0,   /* negate.cc */
  B200_OP_ABS,          /* abs.cc */
  B200_OP_SQRT,         /* sqrt.cc */
  B200_OP_EXP,          /* exp.cc */
  B200_OP_LOG,          /* log.cc */
  B200_OP_TANH,         /* tanh.cc */
  B200_OP_SIGMOID,      /* sigmoid.cc: .5 + .5 tanh(.5 x) */
  B200_OP_SOFTPLUS,     /* softplus.cc */
  B200_OP_SIN,          /* sin.cc */
  B200_OP_COS,          /* cos.cc */
  B200_OP_TAN,          /* tan.cc */
  B200_OP_ADD_CONST,    /* add.cc        x + k */
  B200_OP_SUB_CONST_R,  /* subtract.cc   x - k */
  B200_OP_SUB_CONST_L,  /* subtract.cc   k - x */
  B200_OP_MUL_CONST,    /* multiply.cc   x * k */
  B200_OP_DIV_CONST_R,  /* divide.cc     x / k */
  B200_OP_DIV_CONST_L,  /* divide.cc     k / x */
  B200_OP_POW_CONST_R,  /* pow.cc        x ^ k */
  B200_OP_POW_CONST_L,  /* pow.cc        k ^ x */
  B200_OP_PRELU,        /* prelu.cc      x (x > 0) + k x (x <= 0) */
  B200_OP_ELU,          /* elu.cc */
  B200_OP_POWN,         /* pown.cc       x ^ ik, integer exponent by squaring */
  B200_OP_UNARY_COUNT
};

/* Elementwise functions of two tensors. */
enum {
  B200_OP_ADD = 0,      /* add.cc */
  B200_OP_SUBTRACT,     /* subtract.cc */
  B200_OP_MULTIPLY,     /* multiply.cc */
  B200_OP_DIVIDE,       /* divide.cc */
  B200_OP_POW,          /* pow.cc */
  /* scalar-operand forms only (x op k with k a {} x batch tensor): */
  B200_OP_SUBTRACT_L,   /* k - x */
  B200_OP_DIVIDE_L,     /* k / x */
  B200_OP_POW_L,        /* k ^ x */
  B200_OP_BINARY_COUNT
};

/* Device::<op>_fw_impl(x, [k], y) and <op>_bw_impl(x, y, gy, [k], gx) for the unary list above.
 * The reference's backward kernels add into gx; `accumulate` = 0 writes gx instead, which is what
 * a caller wants when gx is known to hold zeros (primitiv zero-fills every gradient before its
 * first use, primitiv/core/graph.cc:191-212: the device class defers that fill and turns the
 * first `+=` into a store). */
B200_API int b200_unary_fw(b200_ctx *ctx, int mode, int op, const void *x, void *y, uint64_t n,
                           float k, int32_t ik, void *stream);
B200_API int b200_unary_bw(b200_ctx *ctx, int mode, int op, const void *x, const void *y,
                           const void *gy, void *gx, uint64_t n, float k, int32_t ik, int accumulate,
                           void *stream);

/* Device::<op>_scalar_*_fw_impl: y[b][i] = x[b or 0][i] op k[b or 0]   (CPUDEV_FW_X_SCALAR,
 * primitiv/devices/naive/ops/common.h:50-66). */
B200_API int b200_scalar_fw(b200_ctx *ctx, int mode, int op, const void *x, const void *k, void *y,
                            uint64_t volume, uint32_t batch, int x_batched, int k_batched, void *stream);

/* Device::<op>_fw_impl(a, b, y) and <op>_bw_impl(a, b, y, gy, ga, gb) for ADD .. POW. */
B200_API int b200_binary_fw(b200_ctx *ctx, int mode, int op, const void *a, const void *b, void *y,
                            uint64_t volume, uint32_t batch, int a_batched, int b_batched, void *stream);
/* ga and gb may be the same array (x + x); accumulate_a / accumulate_b as for b200_unary_bw,
 * applied in that order. */
B200_API int b200_binary_bw(b200_ctx *ctx, int mode, int op, const void *a, const void *b,
                            const void *y, const void *gy, void *ga, void *gb,
                            uint64_t volume, uint32_t batch, int a_batched, int b_batched,
                            int accumulate_a, int accumulate_b, void *stream);

/* inplace_add.cc / inplace_subtract.cc: y[b or 0] += sign * x[b or 0] over max(bx, by) batches. */
B200_API int b200_inplace_add(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t volume,
                              uint32_t bx, uint32_t by, float sign, void *stream);
/* The same with an `accumulate` flag: 0 for a y that holds nothing yet (a gradient whose zero-fill
 * the caller has deferred): y[n or 0] = sign * x[n or 0], summed over the batch for a batch-1 y. */
B200_API int b200_inplace_add_ex(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t volume,
                                 uint32_t bx, uint32_t by, float sign, int accumulate, void *stream);
/* inplace_multiply_const.cc, reset_tensor.cc, identity.cc */
B200_API int b200_inplace_multiply_const(b200_ctx *ctx, int mode, void *x, uint64_t n, float k, void *stream);
B200_API int b200_fill(b200_ctx *ctx, int mode, void *y, uint64_t n, float value, void *stream);
B200_API int b200_identity(b200_ctx *ctx, int mode, void *y, uint32_t size, void *stream);

/* Host I/O (reset_tensor_by_array.cc, tensor_to_vector.cc) and device copies (copy_tensor.cc).
 * Host arrays are always float; in fp16 mode the conversion runs on the device.
 * b200_upload copies the array into pinned staging memory of the context and returns: the
 * array may be reused at once, the device copy is ordered on the stream like a kernel, and
 * the stream is not waited for.  b200_download returns when the values are in the host array
 * (it synchronises the stream, like the reference's blocking cudaMemcpy); if a kernel's bounded
 * wait ran out before that point it returns B200_ERR_KERNEL_TIMEOUT once, see b200_status_poll. */
B200_API int b200_upload(b200_ctx *ctx, int mode, const float *values_host, void *y, uint64_t n, void *stream);
B200_API int b200_download(b200_ctx *ctx, int mode, const void *x, float *values_host, uint64_t n, void *stream);
/* y = x, converting between storage types when the modes differ (a copy between two B200 devices). */
B200_API int b200_copy(b200_ctx *ctx, int src_mode, const void *x, int dst_mode, void *y, uint64_t n, void *stream);

/* slice.cc: y = x[..., offset : offset + y_dim, ...] along `dim`.
 *   base = lower_volume(dim), x_dim / y_dim = extents along dim, repeat = x.size() / (base * x_dim). */
B200_API int b200_slice_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t base,
                           uint32_t x_dim, uint32_t y_dim, uint32_t offset, uint64_t repeat, void *stream);
/* slice_bw: gx[b or 0][.., offset + j, ..] += gy[b or 0][.., j, ..]; repeat counts per batch element. */
B200_API int b200_slice_bw(b200_ctx *ctx, int mode, const void *gy, void *gx, uint64_t base,
                           uint32_t x_dim, uint32_t y_dim, uint32_t offset, uint64_t repeat,
                           uint32_t bx, uint32_t by, void *stream);
/* The same with an `accumulate` flag: 0 for a gx that holds nothing yet (a gradient whose zero-fill
 * the caller has deferred): every element of gx is stored, the slice from gy, the rest as zeros. */
B200_API int b200_slice_bw_ex(b200_ctx *ctx, int mode, const void *gy, void *gx, uint64_t base,
                              uint32_t x_dim, uint32_t y_dim, uint32_t offset, uint64_t repeat,
                              uint32_t bx, uint32_t by, int accumulate, void *stream);
/* concat.cc, one input at a time: y[b][.., offset + j, ..] = x[b or 0][.., j, ..] (x_dim rows of y_dim). */
B200_API int b200_concat_part(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t base,
                              uint32_t x_dim, uint32_t y_dim, uint32_t offset, uint64_t repeat,
                              uint32_t batch, int x_batched, void *stream);
/* pick.cc: ids on the HOST (n_ids = 1 or batch). */
B200_API int b200_pick_fw(b200_ctx *ctx, int mode, const void *x, const uint32_t *ids_host, uint32_t n_ids,
                          void *y, uint64_t base, uint32_t x_dim, uint64_t repeat, uint32_t batch,
                          int x_batched, void *stream);
B200_API int b200_pick_bw(b200_ctx *ctx, int mode, const void *gy, const uint32_t *ids_host, uint32_t n_ids,
                          void *gx, uint64_t base, uint32_t x_dim, uint64_t repeat, uint32_t batch,
                          int gx_batched, void *stream);
/* broadcast.cc: y[.., j, ..] = x[.., 0, ..] for j < size; total = x.size(), skip1 = lower_volume(dim). */
B200_API int b200_broadcast_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t total,
                               uint64_t skip1, uint32_t size, void *stream);
/* batch_pick.cc / batch_slice.cc (bw only; fw is b200_copy of a sub-range) */
B200_API int b200_batch_pick_fw(b200_ctx *ctx, int mode, const void *x, const uint32_t *ids_host,
                                uint32_t n_ids, void *y, uint64_t volume, void *stream);
B200_API int b200_batch_pick_bw(b200_ctx *ctx, int mode, const void *gy, const uint32_t *ids_host,
                                uint32_t n_ids, void *gx, uint64_t volume, void *stream);
/* transpose.cc ({d1,d2} x batch), permute_dims.cc (ndims <= 8), flip.cc; accumulate != 0 gives the bw forms */
B200_API int b200_transpose(b200_ctx *ctx, int mode, const void *x, void *y, uint32_t d1, uint32_t d2,
                            uint32_t batch, int accumulate, void *stream);
B200_API int b200_permute_dims(b200_ctx *ctx, int mode, const void *x, void *y, uint32_t ndims,
                               const uint32_t *x_dims, const uint32_t *perm, uint32_t batch,
                               int backward, void *stream);
B200_API int b200_flip(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t skip, uint32_t n,
                       uint64_t total, int accumulate, void *stream);

/* Reductions along one dimension (sum.cc, logsumexp.cc, max.cc, min.cc, argmax.cc, argmin.cc):
 *   n = extent along dim, skip1 = lower_volume(dim), outputs = x.size() / n. */
enum { B200_RED_SUM = 0, B200_RED_LOGSUMEXP, B200_RED_MAX, B200_RED_MIN };
B200_API int b200_reduce_fw(b200_ctx *ctx, int mode, int red, const void *x, void *y, uint32_t n,
                            uint64_t skip1, uint64_t outputs, void *stream);
/* max_bw / min_bw: gx[first position equal to y] += gy */
B200_API int b200_minmax_bw(b200_ctx *ctx, int mode, const void *x, const void *y, const void *gy,
                            void *gx, uint32_t n, uint64_t skip1, uint64_t outputs, void *stream);
/* argmax / argmin: indices to the HOST; synchronises, and reports a wait that ran out like b200_download. */
B200_API int b200_argminmax(b200_ctx *ctx, int mode, int want_max, const void *x, uint32_t *ids_host,
                            uint32_t n, uint64_t skip1, uint64_t outputs, void *stream);
/* batch_sum.cc */
B200_API int b200_batch_sum_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint64_t volume,
                               uint32_t batch, void *stream);

/* conv2d.cc as a matrix product.  x {H, W, C} x batch, w {kh, kw, C, Cout} x batch, y {Ho, Wo, Cout},
 * column-major, the kernel flipped as the reference does.  b200_im2col gathers
 *     col[n][p + Ho*Wo * kk] = x[n or 0][yy*s0 - p0 + wy*d0, yx*s1 - p1 + wx*d1, c]   (0 outside the image)
 * with p = yy + Ho*yx and kk = (c*kw + (kw-1-wx))*kh + (kh-1-wy), the order in which w is stored, so that
 *     y = b200_matmul_fw(col {Ho*Wo, K}, w {K, Cout})      and
 *     gcol, gw from b200_matmul_bw(col, w, gy)             with K = kh*kw*C,
 * and b200_col2im adds gcol back: gx[n][xy, xx, c] += sum of the gcol entries that were read from
 * there (a gather in a fixed order: deterministic).  `batch` counts the items of col / gcol. */
B200_API int b200_im2col(b200_ctx *ctx, int mode, const void *x, void *col, uint32_t H, uint32_t W, uint32_t C,
                         uint32_t kh, uint32_t kw, uint32_t Ho, uint32_t Wo, uint32_t pad0, uint32_t pad1,
                         uint32_t stride0, uint32_t stride1, uint32_t dil0, uint32_t dil1, uint32_t batch,
                         int x_batched, void *stream);
B200_API int b200_col2im(b200_ctx *ctx, int mode, const void *gcol, void *gx, uint32_t H, uint32_t W, uint32_t C,
                         uint32_t kh, uint32_t kw, uint32_t Ho, uint32_t Wo, uint32_t pad0, uint32_t pad1,
                         uint32_t stride0, uint32_t stride1, uint32_t dil0, uint32_t dil1, uint32_t batch,
                         void *stream);

/* max_pool2d.cc: x {H, W} x repeat (channels x batch), y {Ho, Wo} x repeat; padding never wins the
 * maximum; the backward adds gy to the first maximal element of each window (scan order: columns
 * of the window outer, rows inner), overlapping windows in a fixed order. */
B200_API int b200_max_pool2d_fw(b200_ctx *ctx, int mode, const void *x, void *y, uint32_t H, uint32_t W,
                                uint32_t Ho, uint32_t Wo, uint32_t window0, uint32_t window1, uint32_t pad0,
                                uint32_t pad1, uint32_t stride0, uint32_t stride1, uint64_t repeat, void *stream);
B200_API int b200_max_pool2d_bw(b200_ctx *ctx, int mode, const void *x, const void *y, const void *gy, void *gx,
                                uint32_t H, uint32_t W, uint32_t Ho, uint32_t Wo, uint32_t window0,
                                uint32_t window1, uint32_t pad0, uint32_t pad1, uint32_t stride0, uint32_t stride1,
                                uint64_t repeat, void *stream);

/* Random fills (random_*.cc).  Counter-based Philox4x32-10 keyed by the context's seed and a
 * call counter: the stream of values depends only on (seed, call order, element index), not
 * on the launch geometry.  This is a generator of this library, not cuRAND's XORWOW. */
enum { B200_RAND_BERNOULLI = 0, B200_RAND_UNIFORM, B200_RAND_NORMAL, B200_RAND_LOG_NORMAL };
B200_API int b200_seed(b200_ctx *ctx, uint64_t seed);
B200_API int b200_random(b200_ctx *ctx, int mode, int kind, float p0, float p1, void *y, uint64_t n,
                         void *stream);

/* ---- several GPUs driven by one host thread (the device-group class) ----
 *
 * No counterpart in the reference: primitiv binds a tensor to one device (core/parameter.cc:80-97).
 * These three calls are what a device object that keeps one shard per GPU needs besides the
 * per-GPU operations above: peer mappings, an ordering point between the GPUs' streams that does
 * not block the host, and the sum of per-GPU partial results (the gradient of a broadcast
 * operand, a sum over the batch) read over NVLink with plain loads. */

/* Lets kernels and copies of ctx's GPU read peer's memory.  Same GPU, or already enabled: no-op. */
B200_API int b200_peer_enable(b200_ctx *ctx, b200_ctx *peer);
/* Work queued later on any of the n contexts' default streams starts only after all work queued
 * so far on every one of them has finished.  Asynchronous; contexts on the same GPU share a
 * stream and need nothing. */
B200_API int b200_stream_barrier(b200_ctx *const *ctxs, int n);
/* dst[i] = (accumulate ? dst[i] : 0) + (srcs[0][i] + srcs[1][i] + ...) (in that order, fp32
 * arithmetic, one rounding to the storage type), on ctx's GPU; srcs may live on peers
 * (b200_peer_enable first, and a b200_stream_barrier between their producers and this call).
 * 1 <= nsrc <= 16. */
B200_API int b200_peer_sum(b200_ctx *ctx, int mode, const void *const *srcs, int nsrc, void *dst,
                           uint64_t n, int accumulate, void *stream);

#ifdef __cplusplus
}
#endif

#endif  /* PRIMITIV_B200_OPS_H_ */
