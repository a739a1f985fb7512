// Measures how fast one SM can take operand tiles in from the L2 cache: the second roofline of the
// tensor-core products beside the tensor pipe itself.
//
// The tcgen05 kernels move every operand byte L2 -> shared memory with bulk copies, and with
// 256 x 256 tiles per CTA pair the single-pass kinds and the fp32 kind ask for 64 bytes per SM
// clock at full tensor rate.  This kernel does nothing but such copies: every SM streams 32 KB
// blocks of a 64 MB buffer (it fits in L2) through a four-stage shared-memory ring, a producer
// thread issuing bulk copies, a consumer thread releasing each stage as soon as it has landed.
// The rate it reaches is what that much shared memory in flight can be fed when every block is an
// L2 hit; a product whose operands partly come from HBM is fed less per byte in flight.
#include <vector>

#include "ctx.h"
#include "mbar.cuh"

namespace b200 {
namespace {

constexpr int kStages = 4;
constexpr uint32_t kStageBytes = 32768;

__global__ void l2_ingest_probe_kernel(const unsigned char *src, unsigned long long span, int iters, int *status,
                                       long long *cycles) {
  pdl_enter();
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(8) uint64_t full[kStages], empty[kStages];
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ring::init(ring::smem_addr(&full[s]), 1);
      ring::init(ring::smem_addr(&empty[s]), 1);
    }
    ring::fence_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  if (threadIdx.x == 0) {
    unsigned long long off = (static_cast<unsigned long long>(blockIdx.x) * 7919ull * kStageBytes) % span;
    for (int it = 0; it < iters; ++it) {
      const int s = it % kStages;
      const uint32_t phase = (it / kStages) & 1u;
      if (it >= kStages && !ring::wait(ring::smem_addr(&empty[s]), phase ^ 1u, &abort_flag)) break;
      ring::arrive_expect_tx(ring::smem_addr(&full[s]), kStageBytes);
      ring::bulk_load(ring::smem_addr(ring_mem + static_cast<size_t>(s) * kStageBytes), src + off, kStageBytes,
                      ring::smem_addr(&full[s]));
      off = (off + static_cast<unsigned long long>(gridDim.x) * kStageBytes) % span;
    }
  } else if (threadIdx.x == 32) {
    int it = 0;
    for (; it < iters; ++it) {
      const int s = it % kStages;
      if (!ring::wait(ring::smem_addr(&full[s]), (it / kStages) & 1u, &abort_flag)) break;
      ring::arrive(ring::smem_addr(&empty[s]));
    }
    if (it < iters) {   // gave up: let the copies that are still in flight land before the CTA goes
      const long long t = clock64();
      while (clock64() - t < 4000000ll) {
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    cycles[blockIdx.x] = clock64() - t0;
    if (abort_flag) report_status(status, B200_ERR_KERNEL_TIMEOUT);
  }
}

}  // namespace

int measure_l2_ingest(b200_ctx *ctx, cudaStream_t stream, double *bytes_per_clock_per_sm, double *gb_per_s_per_sm) {
  constexpr size_t kBuffer = 64u << 20;
  constexpr int kIters = 4000;       // 131 MB per SM, 19 GB in all: a millisecond or two
  const int sms = ctx->sm_count;
  void *buf = nullptr, *cyc = nullptr;
  int rc = ctx->pool.alloc(kBuffer, &buf, nullptr);
  if (rc != B200_OK) return rc;
  rc = ctx->pool.alloc(sizeof(long long) * sms, &cyc, nullptr);
  if (rc != B200_OK) {
    ctx->pool.free(buf);
    return rc;
  }
  const size_t smem = static_cast<size_t>(kStages) * kStageBytes;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaError_t e = cudaFuncSetAttribute(l2_ingest_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  queue_drain(ctx);
  if (e == cudaSuccess) e = cudaMemsetAsync(buf, 1, kBuffer, stream);
  float ms = 0.f;
  std::vector<long long> cycles(sms, 0);
  for (int rep = 0; rep < 3 && e == cudaSuccess; ++rep) {   // the last repetition is the one reported
    e = cudaEventRecord(e0, stream);
    launch(ctx, l2_ingest_probe_kernel, dim3(sms), dim3(64), smem, stream, 1u, static_cast<const unsigned char *>(buf),
           static_cast<unsigned long long>(kBuffer - kStageBytes), kIters, ctx->d_status, static_cast<long long *>(cyc));
    ++ctx->launches;
    queue_drain(ctx);
    if (e == cudaSuccess) e = cudaEventRecord(e1, stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  }
  if (e == cudaSuccess) e = cudaMemcpy(cycles.data(), cyc, sizeof(long long) * sms, cudaMemcpyDeviceToHost);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  ctx->pool.free(buf);
  ctx->pool.free(cyc);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int status = take_status(ctx);
  if (status != 0) return status;
  long long slowest = 1;
  for (long long c : cycles) slowest = c > slowest ? c : slowest;
  const double per_sm = static_cast<double>(kIters) * kStageBytes;
  if (bytes_per_clock_per_sm) *bytes_per_clock_per_sm = per_sm / static_cast<double>(slowest);
  if (gb_per_s_per_sm) *gb_per_s_per_sm = ms > 0.f ? per_sm / (ms * 1e-3) / 1e9 : 0.0;
  return B200_OK;
}

}  // namespace b200
