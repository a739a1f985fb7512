/*
 * primitiv_b200 -- C ABI of the Blackwell (sm_100a) backend for primitiv's
 * minibatch-broadcasting matrix product and the device operations around it.
 *
 * This is the only surface that crosses from host code into the CUDA kernels.
 * primitiv::devices::B200 (primitiv_b200/device/) is written on top of it, and so
 * is anything that binds the library from another language.
 *
 * Conventions
 *   - Every function returns 0 on success, otherwise a non-zero B200_ERR_* /
 *     cudaError code; b200_error_string() explains it.  Nothing throws.
 *   - All tensors are primitiv tensors: column-major, densely packed, minibatch
 *     outermost (primitiv/core/device.h:298-299).  Element (i, j, n) of a
 *     Shape({r, c}, batch) tensor is at  i + j*r + n*r*c.
 *   - Pointers are DEVICE pointers unless the parameter name ends in `_host`.
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default
 *     stream, which is what the reference CUDA device uses for every launch.
 *   - Calls are asynchronous with respect to the host unless stated otherwise.
 *   - One host thread at a time per context (the contract of primitiv::Device).
 *   - One stream per context at a time.  The pool hands a freed block to the next request
 *     without waiting for the GPU: reuse is safe because the next user's work is queued on the
 *     same stream, behind the last reader.  The matrix product frees its packing and split-k
 *     scratch this way right after its launch.  A caller that moves a context from one stream
 *     to another must order the two itself (an event, or a synchronisation) at the switch;
 *     two streams used in alternation on one context race on recycled scratch.  (The reference
 *     device works on the legacy default stream only, primitiv/devices/cuda/ops/matmul.cu.)
 *   - There is no CPU fallback: if no sm_100 GPU is present, context creation fails.
 */
#ifndef PRIMITIV_B200_H_
#define PRIMITIV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

typedef struct b200_ctx b200_ctx;

/* Numeric modes of the matrix product. */
enum {
  B200_MODE_FP32_3XTF32 = 0, /* fp32 storage; each product = 3 tensor-core passes on hi/lo splits (hi.hi in TF32, the two
                              * correction terms in TF32 or bf16, see b200_set_correction_policy); fp32 accuracy */
  B200_MODE_TF32        = 1, /* fp32 storage; one TF32 pass */
  B200_MODE_FP16        = 2, /* half storage, fp32 accumulation, one rounding on store (mirrors primitiv::devices::CUDA16) */
  /* fp32 storage and fp32-grade results on the fp16 tensor pipe: every operand row is scaled by a
   * power of two and split into two half planes, x*s = h0 + h1 (11 + 11 mantissa bits, as TF32 hi + lo),
   * a product is three fp16 passes (h1,h0), (h0,h1), (h0,h0) at twice the TF32 rate, and the scales
   * are undone in the epilogue.  Same normwise accuracy class as 3xTF32 (<= 1e-5); elements more than
   * ~2^18 below the largest of their row lose relative (not absolute) precision, which 3xTF32, with
   * TF32's 8-bit exponent, does not.  No counterpart in the reference. */
  B200_MODE_FP32_3XFP16 = 3
};

/* Error codes (values >= 1000; smaller non-zero values are cudaError_t). */
enum {
  B200_OK                 = 0,
  B200_ERR_INVALID_ARG    = 1001,
  B200_ERR_NO_DEVICE      = 1002, /* no CUDA device / not compute capability 10.x */
  B200_ERR_OUT_OF_MEMORY  = 1003,
  B200_ERR_KERNEL_TIMEOUT = 1004, /* a bounded device-side wait gave up; see b200_status_poll */
  B200_ERR_DRIVER         = 1005, /* driver entry point for tensor-map encoding unavailable or failed */
  B200_ERR_TOO_LARGE      = 1006  /* size beyond a documented maximum */
};

B200_API const char *b200_error_string(int code);

/* ---- context ------------------------------------------------------------------
 * Replaces primitiv::cuda::InternalState (primitiv/internal/cuda/utils.h:320-350):
 * device properties, the caching memory pool and the kernels' status word.  No
 * cuBLAS / cuRAND / cuDNN handle exists: every kernel is in this library. */
B200_API int b200_ctx_create(int device_id, b200_ctx **ctx);
B200_API int b200_ctx_destroy(b200_ctx *ctx);
B200_API int b200_ctx_device(const b200_ctx *ctx, int *device_id, int *sm_count);

/* Every device-side wait of this library is bounded.  A kernel whose wait ran out gives up,
 * returns normally and stores B200_ERR_KERNEL_TIMEOUT in the context's status word, which lives
 * in pinned host memory.  This plays the part of the reference's CUDA_CALL checks
 * (primitiv/internal/cuda/utils.h:20-48): every entry point that hands results to the host
 * after waiting for the GPU (b200_download, b200_argminmax, the *_host products) reads the word
 * and, if it is set, clears it and returns B200_ERR_KERNEL_TIMEOUT instead of 0.
 *
 * b200_status_poll waits for `stream`, then reads and clears the word into *code (0 = nothing
 * was reported).  b200_status_peek does the same without waiting: for callers that have just
 * synchronised by other means. */
B200_API int b200_status_poll(b200_ctx *ctx, void *stream, int *code);
B200_API int b200_status_peek(b200_ctx *ctx, int *code);

/* Exercises the failure-reporting path without any failure: launches a one-warp kernel that
 * waits about a millisecond on a barrier nothing arrives at, gives up, and writes
 * B200_ERR_KERNEL_TIMEOUT to the status word.  The kernel returns normally and the context stays
 * usable; b200_status_poll then returns 1004 once. */
B200_API int b200_selftest_wait_timeout(b200_ctx *ctx, void *stream);

/* ---- caching memory pool --------------------------------------------------------
 * Replaces primitiv::MemoryPool (primitiv/core/memory_pool.cc:35-94) as configured
 * by the CUDA device (primitiv/internal/cuda/utils.h:327-342).  Blocks are 256-byte
 * aligned; freed blocks are cached per size class (geometric classes with four
 * steps per octave, so at most ~19% round-up instead of up to 100%); when
 * cudaMalloc fails every cached block is released and the allocation retried once,
 * as the reference pool does. */
B200_API int b200_pool_alloc(b200_ctx *ctx, size_t bytes, void **ptr, size_t *allocated_bytes);
B200_API int b200_pool_free(b200_ctx *ctx, void *ptr);
B200_API int b200_pool_release_cached(b200_ctx *ctx);
/* stats[0]=bytes in use, [1]=bytes cached, [2]=cudaMalloc calls, [3]=cache hits */
B200_API int b200_pool_stats(const b200_ctx *ctx, uint64_t stats[4]);
/* Pure host function: the block size a request of `bytes` is rounded up to. */
B200_API size_t b200_pool_size_class(size_t bytes);
/* Host-side fault injection for tests: a soft capacity in bytes (0 = none).  A
 * request that would push in-use + cached bytes past it is treated exactly like
 * a failed cudaMalloc (release cached blocks, retry once, then
 * B200_ERR_OUT_OF_MEMORY), without touching the GPU's real memory limit. */
B200_API int b200_pool_set_limit(b200_ctx *ctx, size_t bytes);
/* Debugging aid for out-of-bounds writes: with `bytes` > 0 (rounded up to 256) every block
 * the pool takes from the driver carries that many bytes of a fixed pattern in front of and
 * behind the part the caller sees; 0 switches it off.  Only while no block is handed out
 * (B200_ERR_INVALID_ARG otherwise); cached blocks are released.  b200_pool_check_guards waits
 * for `stream`, inspects the bands of every block, handed out or cached, restores the
 * pattern, and reports the number of blocks with a damaged band, the lowest such block (the
 * pointer b200_pool_alloc returned) and which side was hit (1 front, 2 back, 3 both).
 * Blocks come from cudaMalloc, so a store a little past the end of an output does not
 * fault; this is how such a store is found.  primitiv::devices::B200 switches the bands on
 * when PRIMITIV_B200_POOL_GUARD is set and checks them at every host synchronisation
 * (=1) or before every operation as well (=2), throwing primitiv::Error. */
B200_API int b200_pool_set_guard(b200_ctx *ctx, size_t bytes);
B200_API int b200_pool_check_guards(b200_ctx *ctx, void *stream, uint64_t *damaged_blocks, void **first_block, int *side);

/* ---- the hot path -----------------------------------------------------------------
 * b200_matmul_fw replaces Device::matmul_fw_impl (primitiv/core/device.h:464;
 * CUDA: primitiv/devices/cuda/ops/matmul.cu:26-65; CUDA16: cuda16/ops/matmul.cu:46-129):
 *     y[n] = a[n or 0] . b[n or 0]                      (overwrite)
 * a: Shape({di,dj}, ba), b: Shape({dj,dk}, bb), y: Shape({di,dk}, max(ba,bb));
 * ba, bb in {1, N}; an operand with batch 1 is broadcast.
 *
 * b200_matmul_bw replaces Device::matmul_bw_impl (primitiv/core/device.h:481-483;
 * CUDA: matmul.cu:67-138; CUDA16: cuda16/ops/matmul.cu:131-266):
 *     ga[n or 0] += gy[n] . b[n or 0]^T ;   gb[n or 0] += a[n or 0]^T . gy[n]
 * accumulating in place, and summing over the batch into a broadcast operand's
 * gradient.  Either of ga / gb may be NULL to skip that product.
 *
 * Element type is float for the two fp32 modes and IEEE half for B200_MODE_FP16.
 * The tensor-core path needs 16-byte aligned pointers and leading dimensions
 * that are multiples of 16 bytes; anything else (e.g. 123x123, {10,1024}) runs
 * on the CUDA-core kernel of this library, which computes in plain fp32 FMA. */
B200_API int b200_matmul_fw(b200_ctx *ctx, int mode,
                            const void *a, const void *b, void *y,
                            uint32_t di, uint32_t dj, uint32_t dk,
                            uint32_t ba, uint32_t bb, void *stream);

B200_API int b200_matmul_bw(b200_ctx *ctx, int mode,
                            const void *a, const void *b, const void *gy,
                            void *ga, void *gb,
                            uint32_t di, uint32_t dj, uint32_t dk,
                            uint32_t ba, uint32_t bb, void *stream);

/* b200_matmul_bw with a choice per gradient between `+=` (1, the reference's semantics) and
 * `=` (0, for a gradient known to hold zeros: saves reading it and the fill that zeroed it). */
B200_API int b200_matmul_bw_ex(b200_ctx *ctx, int mode,
                               const void *a, const void *b, const void *gy,
                               void *ga, void *gb,
                               uint32_t di, uint32_t dj, uint32_t dk,
                               uint32_t ba, uint32_t bb,
                               int accumulate_a, int accumulate_b, void *stream);

/* Same two operations with HOST buffers: copies the operands to the device
 * (pool memory), runs the kernels, copies the result back and synchronises.
 * This is what a caller holding host data pays end to end
 * (Device::new_tensor_by_array + matmul + Tensor::to_vector in primitiv terms). */
B200_API int b200_matmul_fw_host(b200_ctx *ctx, int mode,
                                 const void *a_host, const void *b_host, void *y_host,
                                 uint32_t di, uint32_t dj, uint32_t dk,
                                 uint32_t ba, uint32_t bb);

B200_API int b200_matmul_bw_host(b200_ctx *ctx, int mode,
                                 const void *a_host, const void *b_host, const void *gy_host,
                                 void *ga_host, void *gb_host,
                                 uint32_t di, uint32_t dj, uint32_t dk,
                                 uint32_t ba, uint32_t bb);

/* Forward and both gradients of one product from HOST buffers in a single pipelined pass, the
 * end-to-end form of a training step's use of the path (Device::new_tensor_by_array, matmul_fw,
 * matmul_bw, Tensor::to_vector in primitiv terms):
 *     y = a . b ;   ga (+)= gy . b^T ;   gb (+)= a^T . gy
 * a, b and gy cross the bus once each (the two separate calls above upload a and b twice).
 * accumulate_a / accumulate_b: 1 = `+=` into the values ga_host / gb_host hold on entry (the
 * reference's semantics, matmul.cu:67-138; the gradient is uploaded first), 0 = the gradient is
 * known to start from zeros: it is not uploaded and the kernels store instead of adding.
 * y_host may be NULL (no forward product); ga_host / gb_host may be NULL (that gradient is
 * skipped); gy_host may be NULL when both gradients are.  Synchronous: returns when every result
 * is in host memory.  Pinned host buffers give full bus speed; pageable ones work. */
B200_API int b200_matmul_fw_bw_host(b200_ctx *ctx, int mode,
                                    const void *a_host, const void *b_host, const void *gy_host,
                                    void *y_host, void *ga_host, void *gb_host,
                                    uint32_t di, uint32_t dj, uint32_t dk,
                                    uint32_t ba, uint32_t bb,
                                    int accumulate_a, int accumulate_b);

/* ---- the general contraction underneath (what cublasSgemm / SgemmBatched /
 * Hgemm were to the reference devices) --------------------------------------------------
 *   C[g] = (accumulate ? C[g] : 0) + sum_{r < red} opA(A[g*a_gs + r*a_rs]) . opB(B[g*b_gs + r*b_rs])
 * for g < groups; all strides in ELEMENTS.  C is m x n, column-major, ld = m.
 *   trans_a == 0: A is m x k column-major (ld m);  trans_a != 0: A is k x m (ld k), used transposed
 *   trans_b == 0: B is k x n column-major (ld k);  trans_b != 0: B is n x k (ld n), used transposed
 * `red` > 1 sums several operand pairs into one C without atomics (the
 * "a batched, b broadcast" gradient that the reference computes with a serial
 * loop of Sgemm calls, matmul.cu:113-123).
 * force_path: 0 = choose; 1 = CUDA-core kernel; 2 = tensor-core kernel (error if ineligible);
 * 3 = the CUDA-core kernels for one tiny extent (m <= 16 or k <= 16) against large ones (error if
 * the shape and layout are not one of theirs). */
B200_API int b200_gemm(b200_ctx *ctx, int mode, int trans_a, int trans_b,
                       const void *A, const void *B, void *C,
                       uint32_t m, uint32_t n, uint32_t k,
                       uint32_t groups, uint32_t red,
                       uint64_t a_gs, uint64_t a_rs, uint64_t b_gs, uint64_t b_rs, uint64_t c_gs,
                       int accumulate, int force_path, void *stream);

/* ---- one product without any allocation (no counterpart in the reference) -----------------
 * Some hosts of this library may not allocate device memory on the path that calls it: an
 * application that handed the whole GPU to its own allocator at start-up, or a serving loop
 * that forbids cudaMalloc / cudaFree between requests because both synchronise the device.
 * For them this entry point computes one fp32 product in 3xTF32 mode,
 *     C = (accumulate ? C : 0) + opA(A) . opB(B)        (same operand conventions as b200_gemm,
 *                                                        groups = red = 1, tensor-core kernel)
 * with the hi/lo packing planes, which b200_gemm takes from the pool, placed in a fixed
 * 32 MiB array inside the library's device image (B200_NOALLOC_SCRATCH_BYTES; every GPU that
 * loads the library holds it until the process exits).  It calls no cudaMalloc, cudaFree,
 * pool routine or event creation.  It runs the same kernel in the same accuracy class as
 * b200_gemm (<= 1e-5 normwise), but always as one pass over k: b200_gemm may cut a long
 * contraction with few output tiles into k-slices (which needs pool scratch) or pick another
 * kernel for a small or skinny shape, so the two results can differ in their last bits.
 *
 * Limit: 2 planes x (m + n) x round_up(k, 4) floats, each plane rounded up to 64 floats, must
 * fit the array, i.e. roughly (m + n) * k <= 4 Mi elements (1024 x 1024 x 2048, 2048 x 2048 x
 * 1024, ...).  Larger products return B200_ERR_TOO_LARGE and launch nothing.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress)
 * and keeps it.  All calls share the one array: it keeps
 * whatever the previous call packed, nothing in it needs clearing because the packing pass
 * rewrites every element the product reads, and two calls whose kernels can overlap on the
 * GPU (different streams, or different contexts on the same device) race on it. */
#define B200_NOALLOC_SCRATCH_BYTES (32u << 20)
B200_API int b200_gemm_3xtf32_noalloc(b200_ctx *ctx, int trans_a, int trans_b,
                                      const void *A, const void *B, void *C,
                                      uint32_t m, uint32_t n, uint32_t k,
                                      int accumulate, void *stream);

/* Kernel choice for b200_matmul_* and for b200_gemm calls with force_path == 0:
 * 0 = per problem (default), 1 = always the CUDA-core kernel, 2 = the tensor-core
 * kernel whenever the operands are eligible, however small the problem. */
B200_API int b200_set_path_policy(b200_ctx *ctx, int policy);

/* Tile shape of the tensor-core kernel: 0 (default) = a pair of CTAs per 256-row tile
 * (tcgen05 cta_group::2) whenever the problem has more than 128 rows and at least 128
 * columns, 256 x 512 per pair for large half-precision products and 256 x 256 otherwise;
 * 1 = always one CTA per 128-row tile; 2 = pairs, never the 256 x 512 tile; 3 = pairs, the
 * 256 x 512 tile whenever the product has 512 columns (test hook). */
B200_API int b200_set_pair_policy(b200_ctx *ctx, int policy);

/* ---- launch policy (no counterpart in the reference, which pays one blocking-free but serial launch per
 * operation on the caller's thread) -------------------------------------------------------------------------
 * b200_set_async_launch(ctx, 1): kernel launches of this context are issued by a worker thread.  An entry
 * point then does its bookkeeping on the caller's thread as before, copies the kernel arguments into a
 * ring and returns; the worker issues the launches in program order.  A graph-level step of thousands of
 * 3-microsecond kernels is bound by the driver's launch call; this takes that call off the caller's thread
 * (the recurrent loop of the benchmark: 13.2 -> 9 ms).  Everything else that is ordered on a stream (copies,
 * b200_download, b200_status_poll, the *_host products) first lets the worker catch up, so results never
 * depend on the setting.  What does: work the CALLER queues on the same stream by other means (its own
 * kernels, another library) is ordered against this library's launches only after a call that drains the
 * queue (b200_status_poll, b200_download).  Hence off by default; primitiv::devices::B200, whose tensors
 * nothing else touches, switches it on.  A launch that fails is reported by the next draining call.
 *
 * b200_set_dependent_launch(ctx, on): programmatic dependent launch, on by default.  Every kernel of the
 * library begins by releasing the grid queued behind it and then waits for the grid in front of it to
 * finish (griddepcontrol), and is launched with the programmatic-serialization attribute: a chain of small
 * kernels overlaps each launch latency with the predecessor's execution.  Results do not depend on it. */
B200_API int b200_set_async_launch(b200_ctx *ctx, int on);
/* Returns when every launch queued so far has been handed to the driver (it does not wait for the GPU):
 * from then on, work queued on the same stream by anyone else runs after it.  Two contexts on one GPU
 * share the default stream but not a launch queue; whoever makes one read what the other computed calls
 * this on the producer first.  A no-op without the queue. */
B200_API int b200_launch_flush(b200_ctx *ctx);
B200_API int b200_set_dependent_launch(b200_ctx *ctx, int on);

/* ---- operand-plane cache (fp32 mode; no counterpart in the reference) ------------------------------
 * In B200_MODE_FP32_3XTF32 every fp32 operand is split into three planes before the tensor cores see it
 * (4 bytes read and 8 written per element).  A dense operand whose strides are multiples of 8 elements
 * is split "flat": the planes repeat the array's own layout, so the same planes serve every use of the
 * array, as either operand of any product.  Inside one call this is automatic (gy feeds both products
 * of b200_matmul_bw; a, b and gy feed two products each in b200_matmul_fw_bw_host).  Across calls the
 * library cannot know whether the array has changed in between, so the caller opts in:
 *
 *   b200_operand_cache_enable(ctx, max_bytes)   keep planes after the call that packed them, least
 *        recently used first out above max_bytes of plane memory (pool memory, twice the operands'
 *        size); 0 switches the cache off and frees it.  Typical use: a training step, where the
 *        backward product receives the very arrays the forward product read.
 *   b200_operand_cache_invalidate(ctx, ptr, bytes)   forget planes packed from any array that overlaps
 *        [ptr, ptr + bytes); ptr == NULL forgets everything.  The caller MUST do this for every
 *        array it (or anything other than the products of this library) writes while the cache is
 *        on.  Two cases are handled inside: the output of b200_gemm / b200_matmul_*, and blocks
 *        returned through b200_pool_free.  primitiv::devices::B200 calls it from the one place
 *        where it hands out a mutable tensor pointer.
 *   b200_operand_cache_stats   [0] hits, [1] misses, [2] bytes of planes held, [3] entries. */
B200_API int b200_operand_cache_enable(b200_ctx *ctx, size_t max_bytes);
B200_API int b200_operand_cache_invalidate(b200_ctx *ctx, const void *ptr, size_t bytes);
B200_API int b200_operand_cache_stats(const b200_ctx *ctx, uint64_t stats[4]);

/* Arithmetic of the two correction passes of B200_MODE_FP32_3XTF32.  With x = hi + lo, hi = x rounded
 * to TF32, a product is hi.hi + lo.hi + hi.lo.  The last two terms are 2^-11 of the result and need only
 * a few digits, so by default (0) their operands are carried as bf16 planes and multiplied on the
 * bf16 pipe, at twice the TF32 rate: 8 tensor-core instructions per 32 elements of k instead of 12,
 * the same bytes per packed element, and the same <= 1e-5 normwise bound (measured 2e-6).
 * 1 = all three passes on TF32 planes (the textbook 3xTF32 form; per-product error 2^-22 instead of
 * 2^-19, which matters only where a single product, not a sum of many, must be right to the last
 * bits). */
B200_API int b200_set_correction_policy(b200_ctx *ctx, int policy);

/* Optional per-launch timing.  While enabled, every kernel launch of this context is
 * bracketed by a pair of CUDA events on its stream.  b200_profile_read synchronises the
 * device, sums elapsed milliseconds and launch counts per kernel kind since the last
 * read, and clears the records:
 *   [0] tensor-core GEMM   [1] TF32 packing pre-pass   [2] CUDA-core GEMM   [3] elementwise */
B200_API int b200_profile_enable(b200_ctx *ctx, int on);
B200_API int b200_profile_read(b200_ctx *ctx, double ms[4], uint64_t launches[4]);

/* Measurement aid: how fast an SM of this GPU takes data in from the L2 cache.  Every SM streams
 * 32 KB blocks of a 64 MB buffer into a four-stage shared-memory ring with bulk copies and does
 * nothing else; reported are bytes per SM clock (slowest SM) and GB/s per SM (CUDA events), about
 * two milliseconds of GPU time.  The tensor-core products need 64 bytes per SM clock at full
 * tensor rate with their 256 x 256 tiles; the benchmark reports this figure beside their
 * roofline.  Waits for `stream`. */
B200_API int b200_measure_l2_ingest(b200_ctx *ctx, void *stream, double *bytes_per_clock_per_sm, double *gb_per_s_per_sm);

/* Number of kernel launches this context has issued (all kernels of this library). */
B200_API int b200_launch_count(const b200_ctx *ctx, uint64_t *launches);

#ifdef __cplusplus
}
#endif

#endif  /* PRIMITIV_B200_H_ */
