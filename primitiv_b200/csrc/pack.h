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

// ---- planes of the fp32 mode whose correction passes run on the bf16 pipe -------------------
// x = hi + lo with hi = rn_tf32(x) exactly as above; the product a.b ~ a_hi.b_hi + a_lo.b_hi + a_hi.b_lo
// needs the two small terms only to a few digits (they are 2^-11 of the result), so their operands
// are carried as bf16, which the tensor core multiplies at twice the TF32 rate:
//   hi  = rn_tf32(x)        float plane, operand of the kind::tf32 pass
//   hi8 = rn_bf16(x)        bf16 plane,  operand of the kind::f16 correction passes
//   lo8 = rn_bf16(x - hi)   bf16 plane
// Same 8 bytes per element as two TF32 planes.  All three are K-major [b][i][kpad] with kpad = k
// rounded up to 8 (16-byte rows in the bf16 planes), laid out [hi][hi8][lo8] in one block.
struct MixPlanes {
  uint64_t hi_elems;   // floats in the hi plane, rounded up to 64
  uint64_t h8_elems;   // bf16 elements in each of the two bf16 planes, rounded up to 128
  uint32_t kpad;
  uint64_t floats() const { return hi_elems + h8_elems; }  // the whole block, in floats
};
MixPlanes mix_planes(const OperandView &v);
// planes_out = {hi, hi8, lo8}; v is rewritten to describe the packed operand (K-major, ld = kpad).
// With hi_only the TF32 plane alone is written (dst holds lay.hi_elems floats; planes_out[1], [2] are null).
void pack_mix(b200_ctx *ctx, cudaStream_t stream, OperandView &v, float *dst, const MixPlanes &lay,
              const void *planes_out[3], bool hi_only = false);

// Flat form of the same three planes: element e of the caller's array <-> element e of each plane,
// so the planes keep the operand's major-ness and serve any later use of the same array.  Possible
// when the operand is dense and every stride is a multiple of 8 elements (TMA needs 16-byte rows in
// the bf16 planes too).
bool mix_flat_ok(const OperandView &v);
// Whether the context's plane cache already holds the flat planes of this operand.
bool mix_flat_cached(const b200_ctx *ctx, const OperandView &v);
// Finds the operand's flat planes in the context's plane cache, or packs them (one elementwise
// pass) and offers them to the cache.  planes_out = {hi, hi8, lo8}.  *owned_block is the block the
// caller has to return to the pool after its launch, or null when the cache keeps it.
int mix_flat_planes(b200_ctx *ctx, cudaStream_t stream, const OperandView &v, const void *planes_out[3],
                    void **owned_block);

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
