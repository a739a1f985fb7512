// Tensor-core matrix product for sm_100a: tcgen05.mma with the accumulator in
// tensor memory (TMEM), operands staged in shared memory by TMA, one persistent
// CTA per SM walking a static tile list.
//
//   C[g] = (acc ? C[g] : 0) + sum_{r<red} opA(A[g*a_gs + r*a_rs]) . opB(B[g*b_gs + r*b_rs])
//
// primitiv tensors are column-major, so of the three contractions on the path
//   forward     y  = a . b        A is MN-major (m contiguous), B is K-major
//   backward-a  ga += gy . b^T    A and B are both MN-major
//   backward-b  gb += a^T . gy    A and B are both K-major
// every major-ness combination occurs.  The shared-memory matrix descriptors, the
// instruction descriptor and the TMA boxes are computed on the host and passed in;
// nothing about the operand layout is compiled into the kernel.
//
// fp16 operands, and fp32 operands in single-pass TF32 mode, are fed to the tensor
// core in either major-ness straight from the caller's memory when they meet TMA's
// 16-byte alignment rules (the tensor core ignores the 13 low mantissa bits of an
// fp32 word).  Otherwise (unaligned fp32, or the 3xTF32 accuracy mode) a packing
// pre-pass writes K-major planes [matrix][mn][k padded to 4] into pool scratch,
// transposing if needed and rounding to TF32: hi = rn_tf32(x) and, for 3xTF32,
// lo = rn_tf32(x - hi).  The main loop then runs one pass (hi,hi) or three passes
// (lo,hi), (hi,lo), (hi,hi) per k-block into the same accumulator.
//
// Shared-memory layouts (stage bases 1024-aligned):
//   K-major operand : [rows][128 B of k]              one TMA box {BK, rows}
//   MN-major operand: [chunk][BK k-rows][128 B of mn] one TMA box {128 B, BK} per chunk
// BK is 32 fp32 / 64 fp16 elements (128 bytes) per pipeline stage.  The swizzle is
// the 128-byte pattern on 16-byte units, except for 32-bit MN-major operands:
// kind::tf32 reads those correctly only under the 128-byte pattern on 32-byte
// units (TMA SWIZZLE_128B_ATOM_32B, descriptor layout 1) with k-groups of 4 rows,
// i.e. a stride-byte-offset of 512; under the plain pattern it returns zeros.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2-9 = epilogue.  Both pipeline warps walk their loops converged:
// all 32 lanes wait on the barriers, the boxes of a stage are issued side by side
// (one per lane), and the MMAs of a stage are one straight-line block issued under
// elect.sync with everything they need in registers.  (A lone lane looping in a
// diverged warp, parameter re-reads after each asm statement, and branches between
// MMAs each left the tensor pipe idle for 100-200 ns per stage; with them gone the
// issue path alone sustains the tensor peak, and MN-major operands, which need more
// and smaller boxes, load as fast as K-major ones.)  A pipeline stage is one k-block
// with hi and lo planes (3xTF32: 12 MMAs) or two k-blocks (single pass: 8 MMAs).
// Output row i of the tile lives in TMEM lane i, so
// for a fixed output column the 32 lanes of a warp hold 32 consecutive rows:
// column-major C is written (and, for +=, read) with coalesced 128-byte accesses
// straight from registers.
//
// Accumulation accuracy.  The tensor core truncates when it adds into its fp32
// accumulator, which biases a long contraction (measured: 7e-6 normwise after
// 384 accumulation steps).  In 3xTF32 mode the contraction is therefore cut into
// chunks of kChunkKBlocks k-blocks; each chunk accumulates in TMEM from zero, and
// the epilogue warps add finished chunks into fp32 registers with round-to-nearest
// while the tensor core works on the next chunk (two TMEM buffers).  The error
// then no longer grows with the contraction length.  The single-pass modes use one
// chunk per tile, and the two TMEM buffers overlap a tile's epilogue with the next
// tile's main loop.
//
// Every device-side wait is bounded (a few seconds, counted in SM clock cycles).  A wait that runs
// out raises a CTA-wide abort flag, writes B200_ERR_KERNEL_TIMEOUT into the
// context's status word, drains the CTA's own TMA copies and MMAs with bounded
// waits, frees TMEM and returns.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "ctx.h"
#include "pack.h"

namespace b200 {
namespace {

// Development knobs (environment variables that switch parts of the kernel off, cap the stage
// count, change the tile band or forbid split-K) exist only in builds made with
// -DPRIMITIV_B200_DEV_KNOBS; in the product build the flags below are constant zero and the
// branches on them are compiled out.
#ifdef PRIMITIV_B200_DEV_KNOBS
constexpr bool kDevKnobs = true;
#else
constexpr bool kDevKnobs = false;
#endif

constexpr uint32_t kBM = 128;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kKSteps = 4;  // MMAs per 128-byte k-block: 32 bytes of k each (8 tf32 / 16 fp16)
constexpr uint32_t kThreads = 320;
constexpr uint32_t kEpilogueWarps = 8;
constexpr uint32_t kChunkKBlocks = 8;  // 3xTF32: promote to registers every 8 k-blocks (256 k)
constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s at boost clock, 4 s at the lowest

struct MixDesc {
  uint32_t hi, lo_fixed, kstep;
};
struct MixBox {
  uint32_t dst;      // byte offset inside the stage
  int32_t mn_off;    // element offset along mn from the CTA's first row
  uint32_t map;      // index into the tensor maps, in the order they lie in TcParams
  uint32_t flags;    // bit 0: operand B; bit 1: the box is MN-major (coordinates {mn, k} instead of {k, mn})
};

struct alignas(64) TcParams {
  CUtensorMap mapA[2];  // [0] = values (or hi plane), [1] = lo plane
  CUtensorMap mapB[2];
  CUtensorMap mapA8[2];  // kind 4: bf16 planes of the correction passes, [0] = hi8, [1] = lo8
  CUtensorMap mapB8[2];
  void *C;
  unsigned long long c_gs;
  uint32_t m, n, k;
  uint32_t kblocks, red, groups;
  uint32_t tiles_m, tiles_n;
  uint32_t bn, bk, stages;
  uint32_t a_chunks, b_chunks;
  uint32_t a_chunk_elems, b_chunk_elems;
  uint32_t a_chunk_bytes, b_chunk_bytes;
  uint32_t a_mn_major, b_mn_major;
  uint32_t a_gmul, a_rmul, b_gmul, b_rmul;
  uint32_t kstep_a_bytes, kstep_b_bytes, ksteps;
  uint32_t lbo_a, sbo_a, lbo_b, sbo_b;
  uint32_t layout_a, layout_b;  // descriptor swizzle field
  uint32_t idesc;
  uint32_t idesc8;          // kind 4: instruction descriptor of the bf16 correction passes
  uint32_t a8_bytes, b8_bytes;  // kind 4: bytes of one bf16 plane of A / of B in a stage (per CTA)
  // kind 4: the planes of an operand are either K-major repacks or flat copies of the caller's
  // layout (then MN-major operands stay MN-major), so every plane has its own descriptor fields
  // ({high half, fixed low bits, k-step in 16-byte units}; [0] = the TF32 plane, [1] = the bf16 planes)
  // and the TMA boxes of a stage come from a host-built table, one entry per producer lane.
  MixDesc mix_a[2], mix_b[2];
  MixBox mix_box[32];
  uint32_t mix_boxes;
  uint32_t passes;
  uint32_t chunk_kblocks;  // k-blocks per accumulation chunk
  uint32_t accumulate, out_half, kind_f16;
  uint32_t band_m;  // tile-rows per band of the tile order
  // 3xFP16 mode: row maxima of A and B; the epilogue multiplies by 1/s of the output row (from A) and column (from B);
  // per group when the operand has one matrix per group, else one set (stride 0)
  const float *scale_a, *scale_b;
  uint32_t scale_a_gs, scale_b_gs;
  uint32_t splits;  // k-splits per output tile (split-K): `groups` then counts groups x splits,
                    // kblocks is per split and C is the fp32 partial buffer [group][split][m x n]
  uint32_t a_stage_bytes, b_stage_bytes, stage_bytes;  // per plane, per CTA; stage = subs * planes * (a + b)
  uint32_t subs, sub_bytes;  // k-blocks per pipeline stage and the bytes of one (planes * (a + b))
  uint32_t tmem_cols;
  uint32_t debug;  // development switches: 1 = no global stores, 2 = no MMA, 4 = no TMA loads
  int *status;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait.  Returns false if the CTA is aborting or the limit ran out (in
// which case it raises the abort flag itself).  The limit is counted in SM clock
// cycles (%clock64 is a few cycles to read; %globaltimer costs hundreds of nanoseconds
// per read and, on the path every pipeline stage takes, was itself the bottleneck),
// and the clock is only consulted after a run of failed polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *s_abort,
                                          uint32_t sleep_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  uint32_t spins = 0;
  long long t0 = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (sleep_ns) __nanosleep(sleep_ns);  // leave the issue slots to the warps that are not waiting
    if (++spins == 256u) t0 = clock64();
    if (spins > 256u && (spins & 255u) == 0u) {
      if (*s_abort) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *s_abort = 1;
        return false;
      }
    }
  }
}

// A whole warp waits, but only lane 0 polls the barrier (32 pollers per warp on one
// shared-memory word slow everyone else's barrier traffic down).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int *s_abort, uint32_t lane) {
  uint32_t ok = 1u;
  if (lane == 0) {
    // The epilogue waits for a whole chunk of main loop: sleep between polls so that the
    // MMA issuer, which shares a scheduler with two epilogue warps, keeps its issue slots.
    ok = mbar_wait(bar, parity, s_abort, 256u) ? 1u : 0u;
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0u;
}

// Wait used only on the abort path: never raises anything, just gives up.
__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitLimitCycles / 4) return;
  }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// One tcgen05.mma.  The 64-bit shared-memory descriptors are passed as 32-bit halves and
// assembled inside the asm block: the high half (stride offset, version, swizzle) never
// changes during a launch and the low half only advances by a constant per k-step, so the
// issuing thread spends a handful of instructions per MMA.  (With the descriptors rebuilt
// from scratch for every MMA the single issuing thread, sharing its scheduler with polling
// warps, could not feed the tensor core: ~190 ns per MMA whatever the tile width.)
#define B200_MMA_ASM(GROUP, KIND)                                                      \
  asm volatile(                                                                        \
      "{\n\t"                                                                          \
      ".reg .pred p, e;\n\t"                                                           \
      ".reg .b64 da, db;\n\t"                                                          \
      "elect.sync _|e, 0xffffffff;\n\t"                                                \
      "setp.ne.b32 p, %6, 0;\n\t"                                                      \
      "mov.b64 da, {%1, %2};\n\t"                                                      \
      "mov.b64 db, {%3, %4};\n\t"                                                      \
      "@e tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %5, p;\n\t"    \
      "}\n" ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) \
      : "memory")

// Called by ALL 32 lanes of the converged MMA warp with warp-uniform arguments; the
// instruction itself is issued by the one lane elect.sync picks (the same lane every
// time for a full mask, so tcgen05.commit from that lane tracks these MMAs).
template <int kCtas, bool kF16>
__device__ __forceinline__ void mma_issue(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                          uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kCtas == 2) {
    if constexpr (kF16) B200_MMA_ASM("2", "f16"); else B200_MMA_ASM("2", "tf32");
  } else {
    if constexpr (kF16) B200_MMA_ASM("1", "f16"); else B200_MMA_ASM("1", "tf32");
  }
}

// Runs the k-steps (and, for 3xTF32, the three hi/lo pass combinations) of one pipeline stage.
// Runs the k-steps (and, for 3xTF32, the three hi/lo pass combinations) of one k-block as
// straight-line code: every transfer of control between two MMAs showed up as a gap in the
// tensor pipe, so a pipeline stage is one basic block of 8 (single-pass, two k-blocks) or 12
// (3xTF32) MMAs.
template <int kCtas, bool kF16, int kPasses>
__device__ __forceinline__ void mma_stage(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t a_plane, uint32_t b_plane,
                                          uint32_t a_hi, uint32_t b_hi, uint32_t a_lo_fixed, uint32_t b_lo_fixed,
                                          uint32_t kstep_a, uint32_t kstep_b, uint32_t idesc, bool first) {
  uint32_t acc = first ? 0u : 1u;
#pragma unroll
  for (int ps = 0; ps < kPasses; ++ps) {
    // 3xTF32: (lo, hi), (hi, lo), (hi, hi) -- small terms first
    const uint32_t ia = (kPasses == 3 && ps == 0) ? a_plane : 0u;
    const uint32_t ib = (kPasses == 3 && ps == 1) ? b_plane : 0u;
    uint32_t a_lo = a_lo_fixed | (((sa + ia) & 0x3FFFFu) >> 4);
    uint32_t b_lo = b_lo_fixed | (((sb + ib) & 0x3FFFFu) >> 4);
#pragma unroll
    for (uint32_t ks = 0; ks < kKSteps; ++ks) {
      mma_issue<kCtas, kF16>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, acc);
      acc = 1u;
      a_lo += kstep_a;  // in 16-byte units; never carries out of the 14-bit address field within a stage
      b_lo += kstep_b;
    }
  }
}

// One k-block of the fp32 mode with bf16 correction passes (kind 4), as one basic block of
// 8 MMAs: (lo8, hi8) and (hi8, lo8) on the bf16 pipe, two k-steps of 16 each, then (hi, hi) in
// TF32, four k-steps of 8 -- small terms first, all into the same fp32 accumulator.  A stage
// holds [A hi | A hi8 | A lo8 | B hi | B hi8 | B lo8]; the bf16 planes are K-major rows of 64
// bytes under the 64-byte swizzle (descriptor layout 4, 8-row groups 512 bytes apart).
template <int kCtas>
__device__ __forceinline__ void mma_stage_mix(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t a_plane,
                                              uint32_t b_plane, uint32_t a8, uint32_t b8, const MixDesc &a32,
                                              const MixDesc &ad8, const MixDesc &b32, const MixDesc &bd8,
                                              uint32_t idesc, uint32_t idesc8, bool first) {
  uint32_t acc = first ? 0u : 1u;
  {
    uint32_t a_lo = ad8.lo_fixed | (((sa + a_plane + a8) & 0x3FFFFu) >> 4);   // A lo8
    uint32_t b_lo = bd8.lo_fixed | (((sb + b_plane) & 0x3FFFFu) >> 4);        // B hi8
#pragma unroll
    for (uint32_t ks = 0; ks < 2u; ++ks) {
      mma_issue<kCtas, true>(d_tmem, a_lo, ad8.hi, b_lo, bd8.hi, idesc8, acc);
      acc = 1u;
      a_lo += ad8.kstep;
      b_lo += bd8.kstep;
    }
  }
  {
    uint32_t a_lo = ad8.lo_fixed | (((sa + a_plane) & 0x3FFFFu) >> 4);        // A hi8
    uint32_t b_lo = bd8.lo_fixed | (((sb + b_plane + b8) & 0x3FFFFu) >> 4);   // B lo8
#pragma unroll
    for (uint32_t ks = 0; ks < 2u; ++ks) {
      mma_issue<kCtas, true>(d_tmem, a_lo, ad8.hi, b_lo, bd8.hi, idesc8, 1u);
      a_lo += ad8.kstep;
      b_lo += bd8.kstep;
    }
  }
  {
    uint32_t a_lo = a32.lo_fixed | ((sa & 0x3FFFFu) >> 4);                    // A hi
    uint32_t b_lo = b32.lo_fixed | ((sb & 0x3FFFFu) >> 4);                    // B hi
#pragma unroll
    for (uint32_t ks = 0; ks < kKSteps; ++ks) {
      mma_issue<kCtas, false>(d_tmem, a_lo, a32.hi, b_lo, b32.hi, idesc, 1u);
      a_lo += a32.kstep;
      b_lo += b32.kstep;
    }
  }
}

__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same load without the wait, and the wait as a statement that "produces" the registers, so
// that nothing which uses them can be scheduled in front of it: several loads can then be in
// flight behind one wait.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// ---- CTA-pair (cta_group::2) forms.  Two CTAs of a cluster share one MMA: the leader
// (cluster rank 0) issues it for both, each CTA stages its own 128 rows of A and its own
// half of B's rows, and holds the 128 accumulator rows of its half of M in its own TMEM. ----

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA load whose completion is signalled on a barrier that may live in the peer CTA.
// The data itself lands only in the issuing CTA's shared memory: every CTA fetches its own tiles.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1),
        "r"(c2)
      : "memory");
}

// arrives (once) on the barrier at this shared-memory offset in BOTH CTAs of the pair when
// the MMAs issued so far have retired
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
      "}\n" ::"r"(bar),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

// Writes 32 consecutive output columns of one row (this lane's) to column-major C.
// For += all 32 old values are fetched before the first store: written as one
// load-add-store per column the stores would order the loads behind them (the compiler
// must assume they alias) and the epilogue would pay one memory latency per column.
// kWide = old values in flight per thread: 8 where registers are tight (the chunked kernel holds
// a whole tile row in registers), 32 elsewhere.
template <uint32_t kWide, bool kAccumulate, typename T>
__device__ __forceinline__ void store_cols_as(T *C, unsigned long long base, uint32_t m, uint32_t n,
                                              uint32_t col0, const float (&x)[32]) {
  T *q = C + base + static_cast<unsigned long long>(col0) * m;
  const uint32_t left = n - col0;  // caller guarantees col0 < n
#pragma unroll
  for (uint32_t h = 0; h < 32u; h += kWide) {  // kWide loads in flight per thread, then kWide stores
    float old[kWide];
#pragma unroll
    for (uint32_t j = 0; j < kWide; ++j) {
      old[j] = 0.f;
      if (kAccumulate && h + j < left) {
        if constexpr (sizeof(T) == 2) old[j] = __half2float(q[static_cast<unsigned long long>(h + j) * m]);
        else old[j] = q[static_cast<unsigned long long>(h + j) * m];
      }
    }
#pragma unroll
    for (uint32_t j = 0; j < kWide; ++j) {
      if (h + j < left) {
        const float v = x[h + j] + old[j];
        if constexpr (sizeof(T) == 2) q[static_cast<unsigned long long>(h + j) * m] = __float2half_rn(v);
        else q[static_cast<unsigned long long>(h + j) * m] = v;
      }
    }
  }
}

// The two cases are separate code: with `accumulate` as a run-time operand of one loop the
// compiler has at times interleaved the loads with the stores again (27 % on an fp16 launch).
template <uint32_t kWide, typename T>
__device__ __forceinline__ void store_cols(T *C, unsigned long long base, uint32_t m, uint32_t n,
                                           uint32_t col0, const float (&x)[32], bool accumulate) {
  if (accumulate) store_cols_as<kWide, true>(C, base, m, n, col0, x);
  else store_cols_as<kWide, false>(C, base, m, n, col0, x);
}

// Tile order.  Tiles of one group (one output matrix) are walked in bands of kBandTilesM
// row-tiles: inside a band the row-tile index runs fastest, then the column-tile index.
// The CTAs of one wave therefore work on a roughly square patch of the output (8 row-tiles
// by sm_count/8 column-tiles) and share both operand panels through L2, instead of
// sweeping all of A for a couple of B panels (which for an A larger than L2, e.g.
// 8192 x 8192 halves, re-reads A from HBM for every column-tile).
constexpr uint32_t kBandTilesM = 8;

__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t band_m,
                                            uint32_t &g, uint32_t &mt, uint32_t &nt) {
  const uint32_t per_group = tiles_m * tiles_n;
  g = tile / per_group;
  const uint32_t rem = tile - g * per_group;
  const uint32_t band_tiles = band_m * tiles_n;
  const uint32_t band = rem / band_tiles;
  const uint32_t in_band = rem - band * band_tiles;
  const uint32_t first_m = band * band_m;
  const uint32_t rows = tiles_m - first_m < band_m ? tiles_m - first_m : band_m;
  mt = first_m + in_band % rows;
  nt = in_band / rows;
}

// kCtas == 1: one CTA per 128 x bn tile.  kCtas == 2: a cluster of two CTAs per 256 x bn
// tile (tcgen05 cta_group::2): CTA r of the pair stages rows [128 r, 128 r + 128) of A and
// rows [bn/2 r, bn/2 r + bn/2) of B, the leader (r = 0) issues every MMA for both, and each
// CTA's TMEM receives the 128 accumulator rows of its half of M for all bn columns.  Per
// CTA that is a third less shared-memory fill and operand traffic per FLOP than the
// single-CTA tile, which is what bounds this kernel.
//
// kWide (half storage, pairs only): a 256 x 512 tile per pair.  Each CTA stages its 128 rows of A and
// 128 rows of B for each of the two 256-column halves; a k-block is two runs of four MMAs (left half
// into TMEM columns 0-255, right half into 256-511) that share the A tile.  Per FLOP that is a
// quarter less to take in from L2, which is what bounds the 256 x 256 form (an SM takes in 56-58
// bytes per clock where that form needs 64).  The accumulator fills the tensor memory, so there is
// no second buffer to hide the epilogue behind: the epilogue warps therefore first drain their 256
// columns into registers (as packed halves), hand the tensor memory back, and only then go to
// global memory while the next tile's main loop is already running.
template <bool kChunked, int kCtas, int kKind, bool kWide = false>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ TcParams p) {
  // kind 0 = 3xTF32 (hi / lo TF32 planes), 1 = TF32, 2 = FP16, 3 = 3xFP16,
  // 4 = fp32 via one TF32 pass plus two bf16 correction passes (hi, hi8, lo8 planes)
  constexpr int kPasses = (kKind == 0 || kKind == 3 || kKind == 4) ? 3 : 1;
  constexpr uint32_t kSubs = (kPasses == 1 && !kWide) ? 2u : 1u;  // k-blocks per pipeline stage
  constexpr bool kF16 = kKind == 2 || kKind == 3;
  constexpr bool kMix = kKind == 4;
  constexpr bool kTable = kMix || kWide;   // the TMA boxes of a stage come from the host-built table
  static_assert(!kChunked || kPasses == 3, "only the three-pass products are chunked");
  static_assert(!kWide || (kCtas == 2 && kKind == 2 && !kChunked), "the wide tile is a pair form for half storage");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ __align__(8) uint64_t drain_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  pdl_release_next();   // the grid queued behind this one may be scheduled as room becomes free
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int *abort_flag = &s_abort;
  const uint32_t cta_rank = kCtas == 2 ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  const uint32_t first_tile = blockIdx.x / kCtas;   // tiles are dealt to CTAs (kCtas == 1) or to pairs
  const uint32_t tile_step = gridDim.x / kCtas;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), kEpilogueWarps * kCtas);  // only the leader's copy is waited on
    }
    mbar_init(smem_u32(&drain_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (kCtas == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&tmem_slot)),
                   "r"(p.tmem_cols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&tmem_slot)),
                   "r"(p.tmem_cols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (kCtas == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // barriers and tensor memory are set up; nothing above touched global memory.  From here on the
  // operands (and the old C) must be what the grid in front of this one left behind.
  pdl_wait_previous();

  const uint32_t tiles_per_group = p.tiles_m * p.tiles_n;
  const uint32_t total_tiles = tiles_per_group * p.groups;
  const uint32_t kb_per_tile = p.red * p.kblocks;  // k-blocks of one tile, over both contraction axes
  const uint32_t chunks_per_tile = (kb_per_tile + p.chunk_kblocks - 1) / p.chunk_kblocks;
  constexpr uint32_t planes = kPasses == 3 ? 2u : 1u;  // hi and lo planes share a stage
  const uint32_t b_rows = p.bn / kCtas;               // rows of B this CTA stages

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp walks the loop; the boxes of one pipeline stage are issued side by side,
    // one per lane (each lane keeps its box's shared-memory offset, tensor map and coordinate
    // offsets in registers), so a stage costs one wait and one issue slot, not a serial chain.
    {
      uint32_t stage = 0, phase = 0;
      uint32_t armed_mask = 0, armed_parity = 0;
      bool ok = true;
      const uint32_t stage_bytes = p.stage_bytes, nstages = p.stages, dbg = kDevKnobs ? p.debug : 0u, kblocks = p.kblocks,
                     red = p.red, kstage = kSubs * p.bk;
      const uint32_t tx_bytes = p.stage_bytes * kCtas;
      const uint32_t splits = p.splits;
      // this lane's box: [sub][plane][A boxes..., B boxes...]
      const uint32_t a_boxes = p.a_mn_major ? p.a_chunks : 1u, b_boxes = p.b_mn_major ? p.b_chunks : 1u;
      const uint32_t per_plane = a_boxes + b_boxes;
      // kind 4: this lane's box comes from the host-built table
      const MixBox mbox = (kTable && lane < p.mix_boxes) ? p.mix_box[lane] : MixBox{0u, 0, 0u, 0u};
      const uint32_t nboxes = kTable ? p.mix_boxes : kSubs * planes * per_plane;  // <= 32, checked on the host
      const bool has_box = lane < nboxes;
      const uint32_t bsub = kTable ? 0u : lane / (planes * per_plane), brem = lane % (planes * per_plane);
      const uint32_t bpl = (brem / per_plane) & 1u, bidx = brem % per_plane;
      const bool is_b = kTable ? (mbox.flags & 1u) != 0u : bidx >= a_boxes;
      const uint32_t bchunk = is_b ? bidx - a_boxes : bidx;
      const bool box_mn = kTable ? (mbox.flags & 2u) != 0u : (is_b ? p.b_mn_major != 0u : p.a_mn_major != 0u);
      const uint32_t box_dst =
          kTable ? mbox.dst
               : bsub * p.sub_bytes +
                     (is_b ? planes * p.a_stage_bytes + bpl * p.b_stage_bytes + bchunk * p.b_chunk_bytes
                           : bpl * p.a_stage_bytes + bchunk * p.a_chunk_bytes);
      const int box_k = static_cast<int>(bsub * p.bk);
      const int box_mn_off = kTable ? mbox.mn_off
                                    : static_cast<int>(box_mn ? bchunk * (is_b ? p.b_chunk_elems : p.a_chunk_elems) : 0u);
      // the eight tensor maps lie back to back at the head of the parameter block
      const CUtensorMap *box_map = kTable ? &p.mapA[0] + mbox.map : (is_b ? &p.mapB[bpl] : &p.mapA[bpl]);
      // rows of B this CTA contributes to one MMA (the wide tile stages two such sets, 256 columns apart)
      const uint32_t b_rank_rows = kWide ? b_rows / 2u : b_rows;
      for (uint32_t tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        uint32_t vg, mt, nt;
        tile_coords(tile, p.tiles_m, p.tiles_n, p.band_m, vg, mt, nt);
        const uint32_t g = vg / splits, split = vg - g * splits;  // split-K: this tile's slice of k
        const int m0 = static_cast<int>(mt * (kBM * kCtas) + cta_rank * kBM);
        const int n0 = static_cast<int>(nt * p.bn + cta_rank * b_rank_rows);
        const int mn = (is_b ? n0 : m0) + box_mn_off;
        for (uint32_t r = 0; ok && r < red; ++r) {
          const int z = static_cast<int>(is_b ? g * p.b_gmul + r * p.b_rmul : g * p.a_gmul + r * p.a_rmul);
          int k0 = box_k + static_cast<int>(split * kblocks * kstage);
          for (uint32_t kb = 0; kb < kblocks; ++kb, k0 += static_cast<int>(kstage)) {
            if (dbg & 16u) continue;  // development: the MMA thread runs without stage hand-offs
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag))) {
              ok = false;
              break;
            }
            const uint32_t own_bar = smem_u32(&full_bar[stage]);
            // both CTAs of a pair report their bytes to the leader's barrier
            const uint32_t bar = kCtas == 2 ? map_to_cta(own_bar, 0u) : own_bar;
            if (dbg & 4u) {
              if (leader && lane == 0) mbar_arrive(own_bar);
            } else {
              if (leader) {
                if (lane == 0) mbar_arrive_expect_tx(own_bar, tx_bytes);
                armed_mask |= 1u << stage;
                armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
              }
              if (has_box) {
                const uint32_t dst = smem_base + stage * stage_bytes + box_dst;
                const int c0 = box_mn ? mn : k0, c1 = box_mn ? k0 : mn;
                if constexpr (kCtas == 2) tma_load_3d_pair(dst, box_map, bar, c0, c1, z);
                else tma_load_3d(dst, box_map, bar, c0, c1, z);
              }
            }
            __syncwarp();
            if (++stage == nstages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (*abort_flag && leader && lane == 0) {
        // let the copies in flight (this CTA's and, for a pair, the peer's, which report to
        // the same barriers) land before shared memory is given up
        for (uint32_t s = 0; s < p.stages; ++s)
          if (armed_mask & (1u << s))
            mbar_wait_quiet(smem_u32(&full_bar[s]), (armed_parity >> s) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp walks the loop and waits on the barriers together; one lane issues.
    // (A lone lane looping inside a diverged warp pays a scheduling penalty at every loop
    // back-edge, which showed as ~200 ns per pipeline stage.)
    if (leader) {
      uint32_t stage = 0, phase = 0;
      uint32_t chunk_no = 0;  // chunks this CTA has started, over all its tiles
      bool ok = true;
      // descriptor halves that do not change during the launch
      const uint32_t a_hi = ((p.sbo_a >> 4) & 0x3FFFu) | (1u << 14) | ((p.layout_a & 7u) << 29);
      const uint32_t b_hi = ((p.sbo_b >> 4) & 0x3FFFu) | (1u << 14) | ((p.layout_b & 7u) << 29);
      const uint32_t a_lo_fixed = ((p.lbo_a >> 4) & 0x3FFFu) << 16;
      const uint32_t b_lo_fixed = ((p.lbo_b >> 4) & 0x3FFFu) << 16;
      const uint32_t kstep_a = p.kstep_a_bytes >> 4, kstep_b = p.kstep_b_bytes >> 4;
      // Everything the loop needs sits in registers: the asm statements below clobber memory,
      // and a parameter re-read after each of them is latency the tensor core waits out
      // (the issue queue is shallow, so a gap between two MMAs is a gap in the pipe).
      const uint32_t stage_bytes = p.stage_bytes, sub_bytes = p.sub_bytes;
      const uint32_t a_plane = p.a_stage_bytes, b_plane = p.b_stage_bytes, b_off = planes * p.a_stage_bytes;
      const uint32_t idesc = p.idesc, nstages = p.stages, dbg = kDevKnobs ? p.debug : 0u;
      const uint32_t chunk_kblocks = p.chunk_kblocks, bn = p.bn;
      // kind 4: descriptor fields of each plane kind of each operand, in registers
      const MixDesc mxa32 = p.mix_a[0], mxa8 = p.mix_a[1], mxb32 = p.mix_b[0], mxb8 = p.mix_b[1];
      const uint32_t idesc8 = p.idesc8, a8 = p.a8_bytes, b8 = p.b8_bytes;
      for (uint32_t tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        uint32_t kb_left = kb_per_tile;
        for (uint32_t c = 0; ok && c < chunks_per_tile; ++c, ++chunk_no) {
          const uint32_t buf = kWide ? 0u : chunk_no & 1u;   // the wide tile's accumulator is the whole tensor memory
          const uint32_t buf_phase = kWide ? chunk_no & 1u : (chunk_no >> 1) & 1u;
          if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abort_flag))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * bn;
          const uint32_t kbs = kb_left < chunk_kblocks ? kb_left : chunk_kblocks;
          kb_left -= kbs;
          uint32_t sa = smem_base + stage * stage_bytes;
          for (uint32_t it = 0; it < kbs; ++it) {
            // No tcgen05 fence after this wait: the barrier orders the TMA writes (async proxy)
            // before the MMA's reads (async proxy); the fence is for tcgen05.ld/st of other threads.
            if (!(dbg & 24u) && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag))) {
              ok = false;
              break;
            }
            if (!(dbg & 2u)) {
#pragma unroll
              for (uint32_t sub = 0; sub < kSubs; ++sub) {
                const uint32_t ssa = sa + sub * sub_bytes;
                if constexpr (kMix) {
                  mma_stage_mix<kCtas>(d_tmem, ssa, ssa + b_off, a_plane, b_plane, a8, b8, mxa32, mxa8, mxb32, mxb8,
                                       idesc, idesc8, it == 0u);
                } else if constexpr (kWide) {
                  // left and right 256 columns: same A tile, B rows 0-127 and 128-255 of the stage
                  mma_stage<kCtas, kF16, kPasses>(d_tmem, ssa, ssa + b_off, a_plane, b_plane, a_hi, b_hi, a_lo_fixed,
                                                  b_lo_fixed, kstep_a, kstep_b, idesc, it == 0u);
                  mma_stage<kCtas, kF16, kPasses>(d_tmem + 256u, ssa, ssa + b_off + (b_plane >> 1), a_plane, b_plane, a_hi,
                                                  b_hi, a_lo_fixed, b_lo_fixed, kstep_a, kstep_b, idesc, it == 0u);
                } else
                  mma_stage<kCtas, kF16, kPasses>(d_tmem, ssa, ssa + b_off, a_plane, b_plane, a_hi, b_hi, a_lo_fixed,
                                                  b_lo_fixed, kstep_a, kstep_b, idesc, (it | sub) == 0u);
              }
            }
            // frees the stage (in both CTAs of a pair) when these MMAs retire
            if (!(dbg & 16u)) {
              if constexpr (kCtas == 2) mma_commit_pair(smem_u32(&empty_bar[stage]));
              else mma_commit(smem_u32(&empty_bar[stage]));
            }
            sa += stage_bytes;
            if (++stage == nstages) {
              stage = 0;
              phase ^= 1u;
              sa = smem_base;
            }
          }
          if (ok) {
            if constexpr (kCtas == 2) mma_commit_pair(smem_u32(&tmem_full_bar[buf]));
            else mma_commit(smem_u32(&tmem_full_bar[buf]));
          }
        }
      }
      if (*abort_flag) {
        // retire whatever was issued before TMEM is freed
        __syncwarp();
        if constexpr (kCtas == 2) mma_commit_pair(smem_u32(&drain_bar));
        else mma_commit(smem_u32(&drain_bar));
        mbar_wait_quiet(smem_u32(&drain_bar), 0);
      }
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue --------------------------------
    const uint32_t quarter = warp & 3u;         // TMEM lanes this warp may touch
    const uint32_t half = (warp - 2u) >> 2;     // which half of the tile's columns
    const uint32_t cols_per = p.bn >> 1;        // 32, 64 or 128 columns per thread
    const uint32_t col_base = half * cols_per;
    const uint32_t row_in_tile = cta_rank * kBM + quarter * 32u + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    uint32_t chunk_no = 0;
    bool ok = true;
    // the accumulator buffers are handed back to the leader's MMA thread
    const uint32_t empty0 = kCtas == 2 ? map_to_cta(smem_u32(&tmem_empty_bar[0]), 0u) : smem_u32(&tmem_empty_bar[0]);
    const uint32_t empty1 = kCtas == 2 ? map_to_cta(smem_u32(&tmem_empty_bar[1]), 0u) : smem_u32(&tmem_empty_bar[1]);
    for (uint32_t tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
      uint32_t g, mt, nt;
      tile_coords(tile, p.tiles_m, p.tiles_n, p.band_m, g, mt, nt);
      const uint32_t m0 = mt * (kBM * kCtas);
      const uint32_t n0 = nt * p.bn;
      const uint32_t row = m0 + row_in_tile;
      const bool row_ok = row < p.m && !(kDevKnobs && (p.debug & 1u));
      const unsigned long long base =
          static_cast<unsigned long long>(g) * p.c_gs + static_cast<unsigned long long>(row);
      // 3xFP16: undo the power-of-two scales of this output row (from A) and of each column (from B)
      float row_scale = 1.f;
      const float *col_scale = nullptr;
      if constexpr (kKind == 3) {
        const uint32_t g_real = g / p.splits;
        if (row < p.m) row_scale = inv_scale_for(p.scale_a[static_cast<unsigned long long>(g_real) * p.scale_a_gs + row]);
        col_scale = p.scale_b + static_cast<unsigned long long>(g_real) * p.scale_b_gs;
      }
      if constexpr (kWide) {
        if (!warp_wait(smem_u32(&tmem_full_bar[0]), chunk_no & 1u, abort_flag, lane)) {
          ok = false;
          break;
        }
        ++chunk_no;
        tc_fence_after();
        // this thread's 256 columns of its row, rounded to half and packed in pairs: 128 registers
        uint32_t pk[8][16];
#pragma unroll
        for (uint32_t j = 0; j < 8u; j += 2u) {   // two loads of 32 columns in flight behind each wait
          uint32_t v0[32], v1[32];
          tmem_ld32_issue(tmem_base + lane_addr + col_base + j * 32u, v0);
          tmem_ld32_issue(tmem_base + lane_addr + col_base + j * 32u + 32u, v1);
          tmem_ld_wait(v0);
          tmem_ld_wait(v1);
#pragma unroll
          for (uint32_t i = 0; i < 16u; ++i) {
            const __half2 h0 = __floats2half2_rn(__uint_as_float(v0[2u * i]), __uint_as_float(v0[2u * i + 1u]));
            const __half2 h1 = __floats2half2_rn(__uint_as_float(v1[2u * i]), __uint_as_float(v1[2u * i + 1u]));
            pk[j][i] = *reinterpret_cast<const uint32_t *>(&h0);
            pk[j + 1u][i] = *reinterpret_cast<const uint32_t *>(&h1);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(empty0);   // the next tile's main loop may start
        if (row_ok) {
          const bool acc_now = p.accumulate != 0u;
#pragma unroll
          for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t col0 = n0 + col_base + j * 32u;
            if (col0 < p.n) {
              float x[32];
#pragma unroll
              for (uint32_t i = 0; i < 16u; ++i) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pk[j][i]));
                x[2u * i] = f.x;
                x[2u * i + 1u] = f.y;
              }
              store_cols<8>(static_cast<__half *>(p.C), base, p.m, p.n, col0, x, acc_now);
            }
          }
        }
      } else if constexpr (kChunked) {
        float acc[4][32];
        for (uint32_t c = 0; ok && c < chunks_per_tile; ++c, ++chunk_no) {
          const uint32_t buf = chunk_no & 1u;
          if (p.accumulate && c + 1u == chunks_per_tile && row_ok && !(kDevKnobs && (p.debug & 32u))) {
            // The tile's last chunk is in flight: ask L2 for this thread's part of the old C tile,
            // which the final read-add-write would otherwise fetch from HBM with the tensor core
            // waiting.  One request per thread and column measured better than one per line or per
            // sector, and one chunk ahead better than two.
            const unsigned long long ebytes = p.out_half ? 2u : 4u;
            const uint32_t first = n0 + col_base;
            const uint32_t ncols = first < p.n ? (p.n - first < cols_per ? p.n - first : cols_per) : 0u;
            const char *q = static_cast<const char *>(p.C) + (base + static_cast<unsigned long long>(first) * p.m) * ebytes;
            for (uint32_t col = 0; col < ncols; ++col)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(q + static_cast<unsigned long long>(col) * p.m * ebytes));
          }
          if (!warp_wait(smem_u32(&tmem_full_bar[buf]), (chunk_no >> 1) & 1u, abort_flag, lane)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (uint32_t j = 0; j < 4u; ++j) {
            if (j * 32u < cols_per) {
              uint32_t v[32];
              tmem_ld32(tmem_base + lane_addr + buf * p.bn + col_base + j * 32u, v);
              if (c == 0) {
#pragma unroll
                for (uint32_t i = 0; i < 32u; ++i) acc[j][i] = __uint_as_float(v[i]);
              } else {
#pragma unroll
                for (uint32_t i = 0; i < 32u; ++i) acc[j][i] += __uint_as_float(v[i]);
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtas == 2) mbar_arrive_cluster(buf ? empty1 : empty0);
            else mbar_arrive(buf ? empty1 : empty0);
          }
        }
        if (ok && row_ok) {
#pragma unroll
          for (uint32_t j = 0; j < 4u; ++j) {
            const uint32_t col0 = n0 + col_base + j * 32u;
            if (j * 32u < cols_per && col0 < p.n) {
              if constexpr (kKind == 3) {
#pragma unroll
                for (uint32_t i = 0; i < 32u; ++i)
                  if (col0 + i < p.n) acc[j][i] *= row_scale * inv_scale_for(col_scale[col0 + i]);
              }
              // the three-pass kinds always store fp32 (half storage is the single-pass fp16 kind)
              store_cols<8>(static_cast<float *>(p.C), base, p.m, p.n, col0, acc[j], p.accumulate != 0u);
            }
          }
        }
      } else {
        const uint32_t buf = chunk_no & 1u;
        if (!warp_wait(smem_u32(&tmem_full_bar[buf]), (chunk_no >> 1) & 1u, abort_flag, lane)) {
          ok = false;
          break;
        }
        ++chunk_no;
        tc_fence_after();
        const bool acc_now = p.accumulate != 0u;  // read once: the store loops below are compiled per case
        for (uint32_t c0 = 0; c0 < cols_per; c0 += 32u) {
          const uint32_t col0 = n0 + col_base + c0;
          if (col0 >= p.n) break;  // warp-uniform
          uint32_t v[32];
          tmem_ld32(tmem_base + lane_addr + buf * p.bn + col_base + c0, v);
          if (row_ok) {
            float x[32];
#pragma unroll
            for (uint32_t i = 0; i < 32u; ++i) x[i] = __uint_as_float(v[i]);
            if constexpr (kKind == 3) {
#pragma unroll
              for (uint32_t i = 0; i < 32u; ++i)
                if (col0 + i < p.n) x[i] *= row_scale * inv_scale_for(col_scale[col0 + i]);
            }
            if (p.out_half)
              store_cols<32>(static_cast<__half *>(p.C), base, p.m, p.n, col0, x, acc_now);
            else
              store_cols<32>(static_cast<float *>(p.C), base, p.m, p.n, col0, x, acc_now);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtas == 2) mbar_arrive_cluster(buf ? empty1 : empty0);
          else mbar_arrive(buf ? empty1 : empty0);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  // neither CTA of a pair may leave (or free TMEM) while the other can still signal its
  // barriers or read accumulators the shared MMA wrote
  if constexpr (kCtas == 2) cluster_sync_all();
  if (threadIdx.x == 0 && s_abort) report_status(p.status, B200_ERR_KERNEL_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    if constexpr (kCtas == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                   : "memory");
  }
}

// ------------------------------ split-K reduction ------------------------------
//
// A product with few output tiles and a long contraction (the gradient of a broadcast weight:
// m x n small, k = everything in the minibatch) would leave most SMs idle.  Its k range is cut
// into `splits` slices, every (tile, slice) is a work item of the main kernel writing an fp32
// partial tile, and this kernel adds the slices in a fixed order (no atomics: results are the
// same bits every run) into C.
template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ partial, T *__restrict__ C,
                                                            unsigned long long mn, uint32_t groups, uint32_t splits,
                                                            unsigned long long c_gs, int accumulate) {
  pdl_enter();
  const unsigned long long total = mn * groups;
  for (unsigned long long idx = blockIdx.x * 256ull + threadIdx.x; idx < total;
       idx += static_cast<unsigned long long>(gridDim.x) * 256ull) {
    const unsigned long long g = idx / mn, i = idx - g * mn;
    const float *src = partial + g * splits * mn + i;
    float sum = src[0];
    for (uint32_t sidx = 1; sidx < splits; ++sidx) sum += src[sidx * mn];
    T *dst = C + g * c_gs + i;
    if (accumulate) sum += static_cast<float>(*dst);
    *dst = static_cast<T>(sum);
  }
}

int encode_map(const b200_ctx *ctx, CUtensorMap *map, const void *ptr, const OperandView &v,
               int ebytes, uint32_t box_mn, uint32_t box_k, CUtensorMapSwizzle swz, bool bf16 = false) {
  const uint64_t d0 = v.mn_major ? v.mn : v.k;
  const uint64_t d1 = v.mn_major ? v.k : v.mn;
  const uint32_t nb = v.nbatch > 0 ? v.nbatch : 1;
  cuuint64_t dims[3] = {d0, d1, nb};
  cuuint64_t strides[2] = {v.ld * ebytes, (nb > 1 ? v.batch_stride : v.ld * d1) * ebytes};
  cuuint32_t box[3] = {v.mn_major ? box_mn : box_k, v.mn_major ? box_k : box_mn, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = bf16          ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : ebytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUresult r = ctx->encode_tiled(map, dt, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_DRIVER;
}

// Batch-stride pattern of one operand: (g, r) -> matrix index g*gmul + r*rmul.
bool stride_pattern(uint64_t gs, uint64_t rs, uint32_t groups, uint32_t red, uint64_t *stride,
                    uint32_t *nbatch, uint32_t *gmul, uint32_t *rmul) {
  const bool g_on = groups > 1 && gs != 0, r_on = red > 1 && rs != 0;
  *gmul = g_on ? 1u : 0u;
  *rmul = r_on ? 1u : 0u;
  if (g_on && r_on) return false;  // two independent batch axes: not needed by primitiv's matmul
  *stride = g_on ? gs : (r_on ? rs : 0);
  *nbatch = g_on ? groups : (r_on ? red : 1u);
  return true;
}

// Can this operand be handed to TMA as it lies in the caller's memory?
bool direct_ok(const void *ptr, uint64_t ld, uint64_t bstride, uint32_t nbatch, int eb) {
  const uint64_t al = 16 / eb;
  if (reinterpret_cast<uintptr_t>(ptr) % 16) return false;
  if (ld % al) return false;
  if (nbatch > 1 && bstride % al) return false;
  return true;
}

}  // namespace

bool gemm_tc_eligible(const b200_ctx *ctx, const GemmArgs &g) {
  if (!ctx->encode_tiled) return false;
  if (g.m == 0 || g.n == 0 || g.k == 0 || g.groups == 0 || g.red == 0) return false;
  uint64_t sta, stb;
  uint32_t nba, nbb, gm, rm;
  if (!stride_pattern(g.a_gs, g.a_rs, g.groups, g.red, &sta, &nba, &gm, &rm)) return false;
  if (!stride_pattern(g.b_gs, g.b_rs, g.groups, g.red, &stb, &nbb, &gm, &rm)) return false;
  if (g.mode == B200_MODE_FP16) {
    // half operands are never repacked: they must satisfy TMA's alignment rules as they lie
    const uint64_t lda = g.trans_a ? g.k : g.m, ldb = g.trans_b ? g.n : g.k;
    return direct_ok(g.A, lda, sta, nba, 2) && direct_ok(g.B, ldb, stb, nbb, 2);
  }
  return true;  // fp32: whatever is not directly loadable goes through the packing pre-pass
}

namespace {

// Shared body of gemm_tc and of the allocation-free entry point.  With
// fixed_scratch == nullptr the packing planes come from the context's pool; otherwise
// they are laid out in the caller-supplied device buffer of fixed_elems floats and
// nothing is allocated.
int gemm_tc_run(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream, float *fixed_scratch,
                uint64_t fixed_elems) {
  if (!gemm_tc_eligible(ctx, g)) return B200_ERR_INVALID_ARG;
  const bool half_store = g.mode == B200_MODE_FP16;        // operands and C are half in memory
  const bool split16 = g.mode == B200_MODE_FP32_3XFP16;    // fp32 in memory, two half planes per operand
  const bool f16 = half_store || split16;                  // what the tensor core is fed: kind::f16
  const int eb = f16 ? 2 : 4;                              // bytes of a tensor-core operand element
  const uint32_t passes = (g.mode == B200_MODE_FP32_3XTF32 || split16) ? 3u : 1u;
  // fp32 mode: the two correction passes on the bf16 pipe (hi / hi8 / lo8 planes) unless the
  // context asks for TF32 planes throughout
  const bool mix = g.mode == B200_MODE_FP32_3XTF32 && ctx->correction_policy != 1;

  TcParams p;
  memset(&p, 0, sizeof(p));
  p.bk = 128u / eb;                       // 128 bytes of k per stage
  const uint32_t umma_k = 32u / eb;       // 8 (tf32) or 16 (fp16)
  const uint32_t chunk = 128u / eb;       // mn elements per 128-byte swizzle row
  p.bn = g.n > 128 ? 256u : (g.n > 64 ? 128u : 64u);
  p.m = g.m;
  p.n = g.n;
  p.k = g.k;
  p.kblocks = (g.k + p.bk - 1) / p.bk;
  p.red = g.red;
  p.groups = g.groups;
  // A pair of CTAs per 256-row tile when the problem has the rows and columns for it
  // (each CTA then stages bn/2 >= 64 rows of B) and the context allows it.
  const uint32_t ctas = (ctx->pair_policy != 1 && g.m > kBM && p.bn >= 128u && ctx->sm_count >= 2) ? 2u : 1u;
  const uint32_t tile_m = kBM * ctas;
  p.tiles_m = (g.m + tile_m - 1) / tile_m;
  // Half storage, pairs: a 256 x 512 tile per pair (see gemm_tc_kernel, kWide) for long contractions
  // of problems that still fill the GPU four times over with tiles of that size.  Each tile pays
  // about 6 us at its end that the 256 x 256 form hides behind its second accumulator buffer, and
  // earns 5 % in its main loop: measured on 8192 x 8192 x 65536 halves, +4 % at k = 65536, -2.5 % at
  // k = 8192, break-even near 12 K.  pair_policy 2 = never, 3 = whenever n allows (tests).
  bool wide = false;
  if (half_store && ctas == 2u && !fixed_scratch && g.n >= 512u && ctx->pair_policy != 2) {
    const uint64_t wide_tiles = static_cast<uint64_t>(p.tiles_m) * ((g.n + 511u) / 512u) * g.groups;
    const uint64_t k_total = static_cast<uint64_t>(g.k) * g.red;
    wide = ctx->pair_policy == 3 ||
           (k_total >= 16384u && wide_tiles >= 4ull * static_cast<uint64_t>(ctx->sm_count / 2));
  }
  if (wide) p.bn = 512u;
  p.tiles_n = (g.n + p.bn - 1) / p.bn;
  const uint64_t total_tiles = static_cast<uint64_t>(p.tiles_m) * p.tiles_n * g.groups;
  if (total_tiles > 0x7fffffffull) return B200_ERR_TOO_LARGE;

  // ---- operand views, packing where needed ----
  OperandView va, vb;
  va.ptr = g.A; va.mn = g.m; va.k = g.k; va.mn_major = !g.trans_a; va.ld = g.trans_a ? g.k : g.m;
  stride_pattern(g.a_gs, g.a_rs, g.groups, g.red, &va.batch_stride, &va.nbatch, &p.a_gmul, &p.a_rmul);
  vb.ptr = g.B; vb.mn = g.n; vb.k = g.k; vb.mn_major = g.trans_b != 0; vb.ld = g.trans_b ? g.n : g.k;
  stride_pattern(g.b_gs, g.b_rs, g.groups, g.red, &vb.batch_stride, &vb.nbatch, &p.b_gmul, &p.b_rmul);

  const void *a_src[2] = {g.A, nullptr}, *b_src[2] = {g.B, nullptr};
  const void *a_mix[3] = {nullptr, nullptr, nullptr}, *b_mix[3] = {nullptr, nullptr, nullptr};
  void *flat_blocks[2] = {nullptr, nullptr};  // flat planes that the cache did not take: freed after the launch
  void *scratch = nullptr;
  auto release = [&]() {   // stream-ordered reuse: later work queues behind this product
    if (scratch) ctx->pool.free(scratch);
    for (void *&blk : flat_blocks) {
      if (blk) ctx->pool.free(blk);
      blk = nullptr;
    }
    scratch = nullptr;
  };
  // kind 4 bookkeeping: the plane pointers of each operand and whether they are flat copies
  bool a_flat = false, b_flat = false;
  // ... and the one mixed case: B's TF32 plane transposed into K-major scratch, its bf16 planes taken
  // flat (MN-major) from the cache.  vb8 is then the view of those bf16 planes.
  bool b_hybrid = false;
  OperandView vb8;
  if (mix) {
    // An operand that is dense and 32-byte aligned in every stride is packed "flat": the three
    // planes repeat the caller's layout element for element (the kernel reads either
    // major-ness), the pre-pass is purely elementwise, and the planes can serve every later
    // use of the same array, whichever side of whichever product it is on: they go through the
    // context's plane cache.  Anything else is repacked K-major into scratch for this launch.
    OperandView *views[2] = {&va, &vb};
    const void **outs[2] = {a_mix, b_mix};
    bool *flat[2] = {&a_flat, &b_flat};
    uint64_t repack_floats = 0;
    MixPlanes lay[2];
    for (int o = 0; o < 2; ++o) {
      // (measured: an MN-major A costs nothing, an MN-major B 20 % of the main loop -- 3.84 against 3.16 ms
      // on 8 x 4096^3 -- so a B operand that is MN-major in memory is still transposed into K-major planes.
      // Unless its flat planes are already cached and the product has few rows: transposing B costs
      // 12 bytes per element of B whatever m is, a fifth of the main loop shrinks with m, and the two
      // meet near m = 1800.  That is the weight gradient of a layer, gW = gZ . H^T over a large
      // minibatch, whose H was split flat for the forward product.)
      const bool b_mn = o == 1 && views[o]->mn_major;
      const bool flat_possible = !fixed_scratch && ctx->correction_policy == 0 && mix_flat_ok(*views[o]);
      const bool cached = flat_possible && b_mn && mix_flat_cached(ctx, *views[o]);
      // (a small B as well, whatever m: its transposing pre-pass would be one more launch in a chain of
      // few-microsecond kernels, more than a fifth of such a product's main loop)
      const bool small_b = static_cast<uint64_t>(views[o]->mn) * views[o]->k * (views[o]->nbatch ? views[o]->nbatch : 1u) < (1ull << 20);
      *flat[o] = flat_possible && (!b_mn || ((g.m <= 1536u || small_b) && cached));
      // Only the TF32 plane of an MN-major B is slow to read; its bf16 planes are not.  With the flat
      // planes already cached, the transposing pre-pass therefore writes the TF32 plane alone (8
      // instead of 12 bytes per element) and the correction passes read the cached bf16 planes.
      if (b_mn && !*flat[o] && cached) b_hybrid = true;
      if (!*flat[o]) {
        lay[o] = mix_planes(*views[o]);
        repack_floats += (o == 1 && b_hybrid) ? lay[o].hi_elems : lay[o].floats();
      }
    }
    float *cursor = nullptr;
    if (repack_floats && fixed_scratch) {
      if (repack_floats > fixed_elems) return B200_ERR_TOO_LARGE;
      cursor = fixed_scratch;
    } else if (repack_floats) {
      int rc = ctx->pool.alloc(repack_floats * sizeof(float), &scratch, nullptr);
      if (rc != B200_OK) return rc;
      cursor = static_cast<float *>(scratch);
    }
    for (int o = 0; o < 2; ++o) {
      if (*flat[o]) {
        const int rc = mix_flat_planes(ctx, stream, *views[o], outs[o], &flat_blocks[o]);
        if (rc != B200_OK) {
          release();
          return rc;
        }
      } else if (o == 1 && b_hybrid) {
        vb8 = vb;   // the caller's layout: what the cached bf16 planes repeat
        const void *flat_planes[3];
        void *unused = nullptr;
        const int rc = mix_flat_planes(ctx, stream, vb, flat_planes, &unused);   // a cache hit: nothing is packed
        if (rc != B200_OK || unused) {
          if (unused) ctx->pool.free(unused);
          release();
          return rc != B200_OK ? rc : B200_ERR_INVALID_ARG;
        }
        pack_mix(ctx, stream, vb, cursor, lay[o], outs[o], /*hi_only=*/true);
        cursor += lay[o].hi_elems;
        b_mix[1] = flat_planes[1];
        b_mix[2] = flat_planes[2];
      } else {
        pack_mix(ctx, stream, *views[o], cursor, lay[o], outs[o]);
        cursor += lay[o].floats();
      }
    }
    a_src[0] = a_mix[0];
    b_src[0] = b_mix[0];
  } else if (split16) {
    // row maxima and two half planes per operand, all in one scratch block
    if (fixed_scratch) return B200_ERR_INVALID_ARG;  // the allocation-free entry point is 3xTF32 only
    const F16Planes la = f16_planes(va, p.a_rmul != 0u), lb = f16_planes(vb, p.b_rmul != 0u);
    int rc = ctx->pool.alloc(la.bytes() + lb.bytes(), &scratch, nullptr);
    if (rc != B200_OK) return rc;
    char *base = static_cast<char *>(scratch);
    pack_f16(ctx, stream, va, la, base, a_src, &p.scale_a);
    pack_f16(ctx, stream, vb, lb, base + la.bytes(), b_src, &p.scale_b);
    p.scale_a_gs = (!la.shared && p.a_gmul) ? g.m : 0u;
    p.scale_b_gs = (!lb.shared && p.b_gmul) ? g.n : 0u;
  } else if (!f16) {
    // 3xTF32 always repacks, even operands the tensor core could read where they lie (it
    // truncates fp32 words to TF32, so the caller's array could serve as the hi plane and only
    // lo = rn(x - trunc(x)) be written).  That was tried: the pre-pass got a third cheaper, but
    // the main loop, which runs against the power cap, slowed by as much with un-rounded
    // operand words (and by more with MN-major 4 KB boxes).
    OperandView *views[2] = {&va, &vb};
    const void **srcs[2] = {a_src, b_src};
    Tf32Planes lay[2];
    bool pack[2];
    uint64_t total = 0;
    const uint64_t planes = passes == 3 ? 2 : 1;
    for (int o = 0; o < 2; ++o) {
      const OperandView &v = *views[o];
      // (single pass: an MN-major B is the one layout the kernel reads slowly, a fifth of the main
      // loop; from about 2600 output rows up that costs more than transposing B once into K-major
      // scratch, 8 bytes of traffic per element)
      // (and only for a B of 4 Mi elements or more: for a small product the extra launch costs more)
      const bool slow_b = passes == 1 && o == 1 && v.mn_major && g.m >= 2560u && !fixed_scratch &&
                          static_cast<uint64_t>(v.mn) * v.k * (v.nbatch ? v.nbatch : 1u) >= (1ull << 22);
      pack[o] = passes == 3 || slow_b || !direct_ok(v.ptr, v.ld, v.batch_stride, v.nbatch, 4);
      lay[o] = tf32_planes(v);
      if (pack[o]) total += planes * lay[o].plane_elems;
    }
    float *cursor = nullptr;
    if (total && fixed_scratch) {
      if (total > fixed_elems) return B200_ERR_TOO_LARGE;
      cursor = fixed_scratch;
    } else if (total) {
      int rc = ctx->pool.alloc(total * sizeof(float), &scratch, nullptr);
      if (rc != B200_OK) return rc;
      cursor = static_cast<float *>(scratch);
    }
    for (int o = 0; o < 2; ++o) {
      if (!pack[o]) continue;
      pack_tf32(ctx, stream, *views[o], passes == 3, cursor, lay[o], srcs[o]);
      cursor += planes * lay[o].plane_elems;
    }
  }

  p.a_mn_major = va.mn_major ? 1u : 0u;   // (after packing: a K-major repack has cleared the flag, flat planes keep it)
  p.b_mn_major = vb.mn_major ? 1u : 0u;
  p.ksteps = p.bk / umma_k;
  const uint32_t planes = passes == 3 ? 2u : 1u;
  const uint32_t b_rows = p.bn / ctas;  // rows of B each CTA stages
  p.a_stage_bytes = kBM * 128u;
  p.b_stage_bytes = b_rows * 128u;
  p.sub_bytes = planes * (p.a_stage_bytes + p.b_stage_bytes);
  p.a8_bytes = kBM * 64u;     // kind 4: the two bf16 planes of an operand together fill one TF32 plane's room
  p.b8_bytes = b_rows * 64u;
  // Single-pass modes issue only four MMAs per k-block: their pipeline stage holds two k-blocks
  // (a k-block past the end of k is zero-filled by TMA and adds nothing), 3xTF32 stages hold one.
  p.subs = (passes == 1 && !wide) ? 2u : 1u;   // (a wide stage is one k-block: 16 KB of A, 32 KB of B)
  {
    // the producer warp issues one TMA box per lane and stage
    const uint32_t boxes = planes * ((p.a_mn_major ? kBM / chunk : 1u) + (p.b_mn_major ? b_rows / chunk : 1u));
    if (p.subs * boxes > 32u) {
      release();
      return B200_ERR_INVALID_ARG;
    }
  }
  p.stage_bytes = p.subs * p.sub_bytes;
  p.kblocks = (g.k + p.bk * p.subs - 1) / (p.bk * p.subs);  // pipeline-stage iterations along k
  // Split-K: with fewer tiles than half the CTAs (or pairs) and a long contraction, slices of k go
  // to the idle ones (at least four pipeline stages each) and splitk_reduce_kernel adds them up.
  uint32_t splits = 1;
  void *partial = nullptr;
  {
    const uint64_t units = static_cast<uint64_t>(ctx->sm_count) / ctas;
    static const char *sp = kDevKnobs ? std::getenv("PRIMITIV_B200_TC_SPLIT") : nullptr;  // 0 = never split
    const bool allow = !(sp && std::atoi(sp) == 0) && ctx->split_policy != 1 && !wide;   // (the wide epilogue stores halves only)
    if (!fixed_scratch && allow && total_tiles * 2 <= units && p.kblocks >= 16u) {
      uint64_t want = units / total_tiles;
      if (want > p.kblocks / 4u) want = p.kblocks / 4u;
      if (want > 64u) want = 64u;
      if (want >= 2u) {
        const uint32_t per = (p.kblocks + static_cast<uint32_t>(want) - 1u) / static_cast<uint32_t>(want);
        splits = (p.kblocks + per - 1u) / per;  // no empty slices
        p.kblocks = per;
      }
    }
  }
  p.splits = splits;
  p.groups = g.groups * splits;
  const uint64_t launch_tiles = total_tiles * splits;
  p.layout_a = p.layout_b = 2u;  // 128-byte swizzle
  CUtensorMapSwizzle swz_a = CU_TENSOR_MAP_SWIZZLE_128B, swz_b = CU_TENSOR_MAP_SWIZZLE_128B;
  if (p.a_mn_major) {
    p.a_chunks = kBM / chunk;
    p.a_chunk_elems = chunk;
    p.a_chunk_bytes = p.bk * 128u;
    p.lbo_a = p.a_chunk_bytes;
    p.sbo_a = 1024u;
    p.kstep_a_bytes = (umma_k / 8u) * 1024u;
    if (!f16) {  // 32-bit MN-major: 32-byte swizzle atoms, k-groups of 4 rows
      swz_a = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
      p.layout_a = 1u;
      p.sbo_a = 512u;
    }
  } else {
    p.a_chunks = 1;
    p.lbo_a = 0;
    p.sbo_a = 1024u;
    p.kstep_a_bytes = umma_k * eb;
  }
  if (p.b_mn_major) {
    p.b_chunks = b_rows / chunk;
    p.b_chunk_elems = chunk;
    p.b_chunk_bytes = p.bk * 128u;
    p.lbo_b = p.b_chunk_bytes;
    p.sbo_b = 1024u;
    p.kstep_b_bytes = (umma_k / 8u) * 1024u;
    if (!f16) {
      swz_b = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
      p.layout_b = 1u;
      p.sbo_b = 512u;
    }
  } else {
    p.b_chunks = 1;
    p.lbo_b = 0;
    p.sbo_b = 1024u;
    p.kstep_b_bytes = umma_k * eb;
  }
  const uint32_t fmt = f16 ? 0u : 2u;  // F16 = 0 (kind::f16), TF32 = 2 (kind::tf32)
  const uint32_t mma_n = wide ? 256u : p.bn;   // columns of one instruction
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (p.a_mn_major << 15) | (p.b_mn_major << 16) |
            ((mma_n >> 3) << 17) | ((tile_m >> 4) << 24);
  // bf16 x bf16 -> fp32 (kind::f16 with format 1 = BF16), same operand major-ness as the TF32 pass
  const bool b8_mn = b_hybrid ? true : vb.mn_major;   // major-ness of B's bf16 planes
  p.idesc8 = (1u << 4) | (1u << 7) | (1u << 10) | (p.a_mn_major << 15) | ((b8_mn ? 1u : 0u) << 16) |
             ((p.bn >> 3) << 17) | ((tile_m >> 4) << 24);
  if (mix) {
    // Descriptor fields per plane kind.  K-major: rows of 128 bytes (TF32, 128-byte swizzle, 8-row groups
    // 1024 bytes apart) or 64 bytes (bf16, 64-byte swizzle, groups 512 bytes apart), 32 bytes per k-step.
    // MN-major: chunks of 128 bytes of mn by bk k-rows, 4096 bytes apart; TF32 under the 32-byte-atom
    // pattern with k-groups of 4 rows (512 bytes), a k-step of 8 rows = 1024 bytes; bf16 under the
    // plain 128-byte pattern with k-groups of 8 rows (1024 bytes), a k-step of 16 rows = 2048 bytes.
    auto desc = [&](bool mn_major, bool tf32) {
      MixDesc d;
      const uint32_t sbo = mn_major ? (tf32 ? 512u : 1024u) : (tf32 ? 1024u : 512u);
      const uint32_t layout = mn_major ? (tf32 ? 1u : 2u) : (tf32 ? 2u : 4u);
      const uint32_t lbo = mn_major ? p.bk * 128u : 0u;
      d.hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);
      d.lo_fixed = ((lbo >> 4) & 0x3FFFu) << 16;
      d.kstep = (mn_major ? (tf32 ? 1024u : 2048u) : 32u) >> 4;
      return d;
    };
    p.mix_a[0] = desc(va.mn_major, true);
    p.mix_a[1] = desc(va.mn_major, false);
    p.mix_b[0] = desc(vb.mn_major, true);
    p.mix_b[1] = desc(b8_mn, false);
    // TMA boxes of one stage: [A hi | A hi8 | A lo8 | B hi | B hi8 | B lo8]; a K-major plane is one box,
    // an MN-major plane one box per 128 bytes of mn (32 floats, 64 bf16)
    uint32_t nb = 0;
    for (uint32_t o = 0; o < 2u; ++o) {
      const uint32_t rows = o ? b_rows : kBM;
      const uint32_t plane32 = o ? p.b_stage_bytes : p.a_stage_bytes, plane8 = o ? p.b8_bytes : p.a8_bytes;
      const uint32_t base = o ? 2u * p.a_stage_bytes : 0u;
      for (uint32_t t = 0; t < 3u; ++t) {
        const bool mn = o ? (t == 0 ? vb.mn_major : b8_mn) : va.mn_major;
        const uint32_t off = base + (t == 0 ? 0u : plane32 + (t - 1u) * plane8);
        const uint32_t map = t == 0 ? (o ? 2u : 0u) : (o ? 6u : 4u) + (t - 1u);
        const uint32_t per = t == 0 ? 32u : 64u;   // mn elements per 128-byte chunk
        const uint32_t count = mn ? rows / per : 1u;
        for (uint32_t c = 0; c < count; ++c) {
          if (nb >= 32u) {
            release();
            return B200_ERR_INVALID_ARG;
          }
          p.mix_box[nb].dst = off + c * p.bk * 128u;
          p.mix_box[nb].mn_off = static_cast<int32_t>(c * per);
          p.mix_box[nb].map = map;
          p.mix_box[nb].flags = o | (mn ? 2u : 0u);
          ++nb;
        }
      }
    }
    p.mix_boxes = nb;
  }
  if (wide) {
    // TMA boxes of one stage: [A | B rows for the left 256 columns | B rows for the right 256 columns];
    // a K-major tile is one box of 128 rows, an MN-major tile one box per 64 elements (128 bytes) of mn
    uint32_t nb = 0;
    auto add = [&](uint32_t dst, uint32_t mn_off, uint32_t map, uint32_t flags) {
      p.mix_box[nb].dst = dst;
      p.mix_box[nb].mn_off = static_cast<int32_t>(mn_off);
      p.mix_box[nb].map = map;
      p.mix_box[nb].flags = flags;
      ++nb;
    };
    const uint32_t a_cnt = va.mn_major ? kBM / chunk : 1u, b_cnt = vb.mn_major ? 128u / chunk : 1u;
    for (uint32_t c = 0; c < a_cnt; ++c) add(c * p.bk * 128u, c * chunk, 0u, va.mn_major ? 2u : 0u);
    for (uint32_t h = 0; h < 2u; ++h)
      for (uint32_t c = 0; c < b_cnt; ++c)
        add(p.a_stage_bytes + h * (p.b_stage_bytes >> 1) + c * p.bk * 128u, h * 256u + c * chunk, 2u,
            1u | (vb.mn_major ? 2u : 0u));
    p.mix_boxes = nb;
  }
  p.passes = passes;
  const bool chunked = passes == 3 && static_cast<uint64_t>(g.red) * p.kblocks > kChunkKBlocks;
  p.chunk_kblocks = chunked ? kChunkKBlocks : g.red * p.kblocks;
  p.accumulate = g.accumulate ? 1u : 0u;
  p.out_half = half_store ? 1u : 0u;
  p.kind_f16 = f16 ? 1u : 0u;
  p.C = g.C;
  p.c_gs = g.c_gs;
  if (splits > 1) {
    const uint64_t mn = static_cast<uint64_t>(g.m) * g.n;
    const int arc = ctx->pool.alloc(mn * g.groups * splits * sizeof(float), &partial, nullptr);
    if (arc != B200_OK) {
      release();
      return arc;
    }
    p.C = partial;
    p.c_gs = mn;
    p.accumulate = 0u;
    p.out_half = 0u;
  }
  p.status = ctx->d_status;
  p.tmem_cols = wide ? 512u : p.bn * 2u;  // 128, 256 or 512: powers of two
  p.debug = 0u;
  p.band_m = kBandTilesM;
  if (kDevKnobs) {
    const char *dbg = std::getenv("PRIMITIV_B200_TC_DEBUG");  // read per call: A/B runs inside one process
    if (dbg) p.debug = static_cast<uint32_t>(std::atoi(dbg));
    static const char *bd = std::getenv("PRIMITIV_B200_TC_BAND");
    if (bd && std::atoi(bd) > 0) p.band_m = static_cast<uint32_t>(std::atoi(bd));
    static const char *st = std::getenv("PRIMITIV_B200_TC_STAGES");
    if (st) ctx->debug_stage_cap = std::atoi(st);
  }

  // everything the SM offers minus the kernel's static shared memory (barriers, ~200 B) and some slack
  const size_t budget = ctx->smem_optin > 8192 ? ctx->smem_optin - 1024 : 0;
  uint32_t stages = budget > 1024 ? static_cast<uint32_t>((budget - 1024) / p.stage_bytes) : 0;
  if (stages > kMaxStages) stages = kMaxStages;
  if (ctx->debug_stage_cap > 0 && stages > (uint32_t)ctx->debug_stage_cap) stages = ctx->debug_stage_cap;
  int rc = stages >= 2 ? B200_OK : B200_ERR_INVALID_ARG;
  p.stages = stages;
  const size_t smem_bytes = static_cast<size_t>(stages) * p.stage_bytes + 1024;

  for (int i = 0; i < ((passes == 3 && !mix) ? 2 : 1) && rc == B200_OK; ++i) {
    rc = encode_map(ctx, &p.mapA[i], a_src[i], va, eb, p.a_mn_major ? chunk : kBM, p.bk, swz_a);
    if (rc == B200_OK)
      rc = encode_map(ctx, &p.mapB[i], b_src[i], vb, eb, p.b_mn_major ? chunk : (wide ? 128u : b_rows), p.bk, swz_b);
  }
  for (int i = 0; mix && i < 2 && rc == B200_OK; ++i) {
    // the bf16 planes share the packed operand's indexing.  K-major: rows of bk elements = 64 bytes under
    // the 64-byte swizzle; MN-major: boxes of 64 mn elements = 128 bytes by bk rows, plain 128-byte swizzle
    rc = encode_map(ctx, &p.mapA8[i], a_mix[1 + i], va, 2, va.mn_major ? 64u : kBM, p.bk,
                    va.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, true);
    if (rc == B200_OK)
      rc = encode_map(ctx, &p.mapB8[i], b_mix[1 + i], b_hybrid ? vb8 : vb, 2, b8_mn ? 64u : b_rows, p.bk,
                      b8_mn ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, true);
  }
  if (rc == B200_OK && !ctx->tc_smem_configured) {
    const int max_dyn = static_cast<int>(ctx->smem_optin - 512);
    cudaError_t e = cudaSuccess;
    auto allow = [&](auto kernel) {
      if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dyn);
    };
    allow(gemm_tc_kernel<true, 1, 0>);
    allow(gemm_tc_kernel<false, 1, 0>);
    allow(gemm_tc_kernel<false, 1, 1>);
    allow(gemm_tc_kernel<false, 1, 2>);
    allow(gemm_tc_kernel<true, 2, 0>);
    allow(gemm_tc_kernel<false, 2, 0>);
    allow(gemm_tc_kernel<false, 2, 1>);
    allow(gemm_tc_kernel<false, 2, 2>);
    allow(gemm_tc_kernel<true, 1, 3>);
    allow(gemm_tc_kernel<false, 1, 3>);
    allow(gemm_tc_kernel<true, 2, 3>);
    allow(gemm_tc_kernel<false, 2, 3>);
    allow(gemm_tc_kernel<true, 1, 4>);
    allow(gemm_tc_kernel<false, 1, 4>);
    allow(gemm_tc_kernel<true, 2, 4>);
    allow(gemm_tc_kernel<false, 2, 4>);
    allow(gemm_tc_kernel<false, 2, 2, true>);
    if (e != cudaSuccess) rc = static_cast<int>(e);
    ctx->tc_smem_configured = (e == cudaSuccess);
  }
  if (rc == B200_OK) {
    // persistent: one CTA (or one pair) per tile up to one CTA per SM
    const uint64_t units = static_cast<uint64_t>(ctx->sm_count) / ctas;
    const unsigned grid = static_cast<unsigned>((launch_tiles < units ? launch_tiles : units) * ctas);
    ProfScope prof(ctx, kProfGemmTc, stream);
    if (ctas == 2) {
      // clusters of two CTAs along x (a pair per 256-row tile)
      const dim3 gd(grid), bd(kThreads);
      if (mix && chunked) b200::launch(ctx, gemm_tc_kernel<true, 2, 4>, gd, bd, smem_bytes, stream, 2u, p);
      else if (mix) b200::launch(ctx, gemm_tc_kernel<false, 2, 4>, gd, bd, smem_bytes, stream, 2u, p);
      else if (split16 && chunked) b200::launch(ctx, gemm_tc_kernel<true, 2, 3>, gd, bd, smem_bytes, stream, 2u, p);
      else if (split16) b200::launch(ctx, gemm_tc_kernel<false, 2, 3>, gd, bd, smem_bytes, stream, 2u, p);
      else if (chunked) b200::launch(ctx, gemm_tc_kernel<true, 2, 0>, gd, bd, smem_bytes, stream, 2u, p);
      else if (passes == 3) b200::launch(ctx, gemm_tc_kernel<false, 2, 0>, gd, bd, smem_bytes, stream, 2u, p);
      else if (!f16) b200::launch(ctx, gemm_tc_kernel<false, 2, 1>, gd, bd, smem_bytes, stream, 2u, p);
      else if (wide) b200::launch(ctx, gemm_tc_kernel<false, 2, 2, true>, gd, bd, smem_bytes, stream, 2u, p);
      else b200::launch(ctx, gemm_tc_kernel<false, 2, 2>, gd, bd, smem_bytes, stream, 2u, p);
    } else if (mix && chunked) {
      b200::launch(ctx, gemm_tc_kernel<true, 1, 4>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else if (mix) {
      b200::launch(ctx, gemm_tc_kernel<false, 1, 4>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else if (split16 && chunked) {
      b200::launch(ctx, gemm_tc_kernel<true, 1, 3>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else if (split16) {
      b200::launch(ctx, gemm_tc_kernel<false, 1, 3>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else if (chunked) {
      b200::launch(ctx, gemm_tc_kernel<true, 1, 0>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else if (passes == 3) {
      b200::launch(ctx, gemm_tc_kernel<false, 1, 0>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else if (!f16) {
      b200::launch(ctx, gemm_tc_kernel<false, 1, 1>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    } else {
      b200::launch(ctx, gemm_tc_kernel<false, 1, 2>, dim3(grid), dim3(kThreads), smem_bytes, stream, 1u, p);
    }
    ++ctx->launches;
    if (rc == B200_OK) rc = static_cast<int>(cudaGetLastError());
    if (rc == B200_OK && splits > 1) {
      const unsigned long long mn = static_cast<unsigned long long>(g.m) * g.n;
      const unsigned long long need = (mn * g.groups + 255ull) / 256ull;
      const unsigned long long cap = static_cast<unsigned long long>(ctx->sm_count) * 8ull;
      const unsigned blocks = static_cast<unsigned>(need < cap ? need : cap);
      if (half_store)
        b200::launch(ctx, splitk_reduce_kernel<__half>, dim3(blocks), dim3(256), 0, stream, 1u, static_cast<const float *>(partial),
                                                                   static_cast<__half *>(g.C), mn, g.groups, splits,
                                                                   g.c_gs, g.accumulate);
      else
        b200::launch(ctx, splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1u, static_cast<const float *>(partial),
                                                                  static_cast<float *>(g.C), mn, g.groups, splits,
                                                                  g.c_gs, g.accumulate);
      ++ctx->launches;
      rc = static_cast<int>(cudaGetLastError());
    }
  }
  if (partial) ctx->pool.free(partial);
  release();
  return rc;
}

}  // namespace

int gemm_tc(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream) {
  return gemm_tc_run(ctx, g, stream, nullptr, 0);
}

// ---------------- self-test of the bounded-wait machinery ----------------
namespace {

// Waits on a barrier that nothing ever arrives at, with a limit of `limit_cycles`, then
// reports through the status word exactly as gemm_tc_kernel does when one of its waits
// runs out.  Nothing faults or traps: the kernel returns normally.
__global__ void wait_timeout_selftest_kernel(int *status, long long limit_cycles) {
  pdl_enter();
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const long long t0 = clock64();
    bool timed_out = false;
    while (!mbar_try_wait(smem_u32(&bar), 0)) {
      if (clock64() - t0 > limit_cycles) {
        timed_out = true;
        break;
      }
    }
    if (timed_out) report_status(status, B200_ERR_KERNEL_TIMEOUT);
  }
}

}  // namespace

int selftest_wait_timeout(b200_ctx *ctx, cudaStream_t stream) {
  b200::launch(ctx, wait_timeout_selftest_kernel, dim3(1), dim3(32), 0, stream, 1u, ctx->d_status, 2000000ll);  // about a millisecond
  ++ctx->launches;
  return static_cast<int>(cudaGetLastError());
}

// ---------------- allocation-free 3xTF32 product (b200_gemm_3xtf32_noalloc) ----------------
//
// The packing planes of this variant live in a file-scope device array instead of
// pool memory.  Every GPU that loads the library carries the array until the process
// exits, so it is kept modest: 8 Mi floats = 32 MiB, which holds the hi and lo planes
// of both operands as long as  2 * (m + n) * round_up(k, 4) <= 8 Mi  (with 64-float
// rounding per plane), e.g. 1024 x 1024 x 2048 or 2048 x 2048 x 1024.
constexpr uint64_t kStaticScratchFloats = 8ull << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is looked up once per device, with that device
// current, and cached here.
constexpr int kMaxDevices = 64;
static float *g_static_scratch_addr[kMaxDevices] = {};

int gemm_3xtf32_noalloc(b200_ctx *ctx, const GemmArgs &g, cudaStream_t stream) {
  if (ctx->device < 0 || ctx->device >= kMaxDevices) return B200_ERR_INVALID_ARG;
  {
    // The documented limit, checked here so that it does not depend on how the operands end up
    // being packed: 8 bytes per operand element (a float plane and two bf16 planes, or two float
    // planes), k padded to 8, each plane rounded up to 128 elements.
    const uint64_t kpad = (static_cast<uint64_t>(g.k) + 7ull) & ~7ull;
    const uint64_t pa = (static_cast<uint64_t>(g.m) * kpad + 127ull) & ~127ull;
    const uint64_t pb = (static_cast<uint64_t>(g.n) * kpad + 127ull) & ~127ull;
    if (2ull * (pa + pb) > kStaticScratchFloats) return B200_ERR_TOO_LARGE;
  }
  float *&addr = g_static_scratch_addr[ctx->device];
  if (!addr) {
    void *sym = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&sym, g_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    addr = static_cast<float *>(sym);
  }
  // Per-launch timing creates events, which is an allocation of sorts: keep it off here.
  const bool was_profiling = ctx->profiling;
  ctx->profiling = false;
  const int rc = gemm_tc_run(ctx, g, stream, addr, kStaticScratchFloats);
  ctx->profiling = was_profiling;
  return rc;
}

}  // namespace b200
