// Packing pre-pass of the tensor-core matrix product: operand views, the K-major TF32 planes of
// the 3xTF32 / TF32 modes and the row-scaled half planes of the 3xFP16 mode.
#ifndef PRIMITIV_B200_CSRC_PACK_H_
#define PRIMITIV_B200_CSRC_PACK_H_

#include "ctx.h"

namespace b200 {

struct OperandView {
  const void *ptr;
  uint32_t mn, k;         // extents
  bool mn_major;          // true: mn contiguous; false: k contiguous
  uint64_t ld;            // elements between consecutive lines of the slow axis
  uint64_t batch_stride;  // elements between consecutive matrices
  uint32_t nbatch;
};

#ifdef __CUDACC__
// 3xFP16 mode: 1/s for a row whose largest magnitude is amax (see the pre-pass further down).
__device__ __forceinline__ float inv_scale_for(float amax) {
  int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2(amax)) for normal values
  e = e < -100 ? -100 : (e > 127 ? 127 : e);
  return __uint_as_float(static_cast<uint32_t>(e - 14 + 127) << 23);  // 2^(e-14), so that amax / it is in [2^14, 2^15)
}
#endif

// ---- TF32 planes: dst[b][i][p], i < mn, p < k, row stride kpad (k rounded up to 4) ----
struct Tf32Planes {
  uint64_t plane_elems;  // floats per plane, rounded up to 64
  uint32_t kpad;
};
Tf32Planes tf32_planes(const OperandView &v);
// Writes hi = rn_tf32(x) at dst and, when two_planes, lo = rn_tf32(x - hi) at dst + plane_elems;
// planes_out receives the two plane pointers and v is rewritten to describe the packed operand.
void pack_tf32(b200_ctx *ctx, cudaStream_t stream, OperandView &v, bool two_planes, float *dst,
               const Tf32Planes &lay, const void *planes_out[2]);

// ---- half planes of the 3xFP16 mode: [row maxima][h0 plane][h1 plane], rows of kpad halves ----
struct F16Planes {
  uint64_t plane_halves;  // halves per plane, rounded up to 128
  uint64_t scale_floats;  // row maxima, rounded up to 64
  uint32_t kpad;          // k rounded up to 8
  bool shared;            // one maximum per row for all batches (the batch is a contraction axis)
  uint64_t bytes() const { return scale_floats * sizeof(float) + 2 * plane_halves * 2; }
};
F16Planes f16_planes(const OperandView &v, bool shared);
void pack_f16(b200_ctx *ctx, cudaStream_t stream, OperandView &v, const F16Planes &lay, char *dst,
              const void *planes_out[2], const float **amax_out);

}  // namespace b200

#endif  // PRIMITIV_B200_CSRC_PACK_H_
