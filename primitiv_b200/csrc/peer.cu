// What a device object spanning several GPUs needs besides the per-GPU operations: peer
// mappings, a stream barrier across GPUs, and the ordered sum of per-GPU partial results.
#include <cstdint>

#include "ops_common.cuh"

namespace b200 {
namespace {

constexpr int kMaxPeerSources = 16;

struct PeerSources {
  const void *p[kMaxPeerSources];
};

// dst[i] = (accumulate ? dst[i] : 0) + sum over sources in list order.  Sources may be peer memory: plain 128-bit loads,
// one per source and thread in flight, so a launch keeps nsrc x grid x 16 B outstanding on NVLink.
template <typename T>
__global__ void __launch_bounds__(256) peer_sum_kernel(PeerSources srcs, int nsrc, T *__restrict__ dst, u64 n,
                                                       int vector_ok, int accumulate) {
  pdl_enter();
  const u64 stride = static_cast<u64>(gridDim.x) * blockDim.x;
  const u64 tid = static_cast<u64>(blockIdx.x) * blockDim.x + threadIdx.x;
  constexpr int N = Vec<T>::N;
  const u64 nvec = vector_ok ? n / N : 0;
  for (u64 v = tid; v < nvec; v += stride) {
    float acc[N];
    Vec<T> x;
    x.load(static_cast<const T *>(srcs.p[0]) + v * N);
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = x.get(i);
    for (int s = 1; s < nsrc; ++s) {
      x.load(static_cast<const T *>(srcs.p[s]) + v * N);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += x.get(i);
    }
    if (accumulate) {
      x.load(dst + v * N);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += x.get(i);
    }
#pragma unroll
    for (int i = 0; i < N; ++i) x.set(i, acc[i]);
    x.store(dst + v * N);
  }
  for (u64 i = nvec * N + tid; i < n; i += stride) {
    float acc = ld(static_cast<const T *>(srcs.p[0]), i);
    for (int s = 1; s < nsrc; ++s) acc += ld(static_cast<const T *>(srcs.p[s]), i);
    if (accumulate) acc += ld(dst, i);
    st(dst, i, acc);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_peer_enable(b200_ctx *ctx, b200_ctx *peer) {
  if (!ctx || !peer) return B200_ERR_INVALID_ARG;
  if (ctx->device == peer->device) return B200_OK;
  DeviceGuard guard(ctx->device);
  int can = 0;
  B200_CUDA_TRY(cudaDeviceCanAccessPeer(&can, ctx->device, peer->device));
  if (!can) return B200_ERR_NO_DEVICE;
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // not an error for the caller: clear it
    return B200_OK;
  }
  return static_cast<int>(e);
}

int b200_stream_barrier(b200_ctx *const *ctxs, int n) {
  if (!ctxs || n < 1) return B200_ERR_INVALID_ARG;
  for (int i = 0; i < n; ++i)
    if (!ctxs[i]) return B200_ERR_INVALID_ARG;
  for (int i = 0; i < n; ++i) b200::queue_drain(ctxs[i]);   // launches still waiting in a context's launch queue
  bool one_gpu = true;
  for (int i = 1; i < n; ++i) one_gpu = one_gpu && ctxs[i]->device == ctxs[0]->device;
  if (one_gpu) return B200_OK;  // one default stream: already ordered
  for (int i = 0; i < n; ++i) {
    b200_ctx *c = ctxs[i];
    DeviceGuard guard(c->device);
    if (!c->barrier_event) B200_CUDA_TRY(cudaEventCreateWithFlags(&c->barrier_event, cudaEventDisableTiming));
    B200_CUDA_TRY(cudaEventRecord(c->barrier_event, nullptr));
  }
  for (int i = 0; i < n; ++i) {
    DeviceGuard guard(ctxs[i]->device);
    for (int j = 0; j < n; ++j)
      if (ctxs[j]->device != ctxs[i]->device) B200_CUDA_TRY(cudaStreamWaitEvent(nullptr, ctxs[j]->barrier_event, 0));
  }
  return B200_OK;
}

int b200_peer_sum(b200_ctx *ctx, int mode, const void *const *srcs, int nsrc, void *dst, uint64_t n, int accumulate,
                  void *stream) {
  B200_OPS_PROLOGUE(ctx);
  if (!srcs || nsrc < 1 || nsrc > kMaxPeerSources || (!dst && n)) return B200_ERR_INVALID_ARG;
  if (n == 0) return B200_OK;
  PeerSources ps;
  int vector_ok = aligned16(dst);
  for (int i = 0; i < kMaxPeerSources; ++i) ps.p[i] = i < nsrc ? srcs[i] : nullptr;
  for (int i = 0; i < nsrc; ++i) {
    if (!srcs[i]) return B200_ERR_INVALID_ARG;
    vector_ok = vector_ok && aligned16(srcs[i]);
  }
  B200_DISPATCH_MODE(mode, {
    ProfScope prof(ctx, kProfElementwise, s);
    b200::launch(ctx, peer_sum_kernel<T>, dim3(grid_for(ctx, n / Vec<T>::N + 1, 256)), dim3(256), 0, s, 1u, ps, nsrc, static_cast<T *>(dst), n,
                                                                            vector_ok, accumulate);
  });
  B200_OPS_EPILOGUE(ctx);
}

}  // extern "C"
