// Guard bands round the blocks of the memory pool: a debugging aid for out-of-bounds writes.
//
// With b200_pool_set_guard(ctx, n) every block the pool takes from the driver carries n bytes
// of a fixed pattern in front of and behind the part a caller sees.  Blocks come from
// cudaMalloc, so a kernel that stores a few elements past the end of its output does not
// fault: it lands in the neighbour's data or in allocator padding and shows up much later as
// wrong numbers.  With the bands in place it lands in the pattern, and the check below finds
// it: one small kernel over the bands of every block (handed out or cached), which also
// restores the pattern so that the next check reports new damage only.
#include <utility>
#include <vector>

#include "ctx.h"

namespace b200 {
namespace {

struct GuardBlock {
  unsigned char *user;    // what the caller sees; the bands are [user - guard, user) and [user + size, + guard)
  unsigned long long size;
};

// out[2 * i + side] = number of damaged 4-byte words of block i's front (0) / back (1) band.
__global__ void pool_guard_check_kernel(const GuardBlock *blocks, unsigned n_blocks, unsigned guard_words,
                                        unsigned *out) {
  pdl_enter();
  const unsigned want = 0x01010101u * Pool::kGuardByte;
  for (unsigned b = blockIdx.x; b < n_blocks; b += gridDim.x) {
    const GuardBlock blk = blocks[b];
    unsigned *front = reinterpret_cast<unsigned *>(blk.user) - guard_words;
    unsigned *back = reinterpret_cast<unsigned *>(blk.user + blk.size);
    unsigned bad[2] = {0u, 0u};
    for (unsigned w = threadIdx.x; w < guard_words; w += blockDim.x) {
      if (front[w] != want) { ++bad[0]; front[w] = want; }
      if (back[w] != want) { ++bad[1]; back[w] = want; }
    }
    if (bad[0]) atomicAdd(&out[2 * b], bad[0]);
    if (bad[1]) atomicAdd(&out[2 * b + 1], bad[1]);
  }
}

}  // namespace

int pool_check_guards(b200_ctx *ctx, cudaStream_t stream, std::uint64_t *damaged, void **first, int *side) {
  if (damaged) *damaged = 0;
  if (first) *first = nullptr;
  if (side) *side = 0;
  const std::size_t guard = ctx->pool.guard();
  if (guard == 0) return B200_OK;
  std::vector<std::pair<void *, std::size_t>> blocks;
  ctx->pool.blocks(&blocks);
  if (blocks.empty()) return B200_OK;
  std::vector<GuardBlock> list(blocks.size());
  for (std::size_t i = 0; i < blocks.size(); ++i)
    list[i] = GuardBlock{static_cast<unsigned char *>(blocks[i].first), blocks[i].second};
  // plain driver allocations, outside the pool: the check must not change what it checks
  GuardBlock *d_list = nullptr;
  unsigned *d_out = nullptr;
  const std::size_t list_bytes = list.size() * sizeof(GuardBlock), out_bytes = list.size() * 2 * sizeof(unsigned);
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&d_list), list_bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&d_out), out_bytes);
  std::vector<unsigned> counts(list.size() * 2, 0u);
  if (e == cudaSuccess) {
    queue_drain(ctx);
    e = cudaMemcpyAsync(d_list, list.data(), list_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_out, 0, out_bytes, stream);
  }
  if (e == cudaSuccess) {
    const unsigned n = static_cast<unsigned>(list.size());
    launch(ctx, pool_guard_check_kernel, dim3(n < 1184u ? n : 1184u), dim3(64), 0, stream, 1u,
           static_cast<const GuardBlock *>(d_list), n, static_cast<unsigned>(guard / 4), d_out);
    ++ctx->launches;
    queue_drain(ctx);
    e = cudaMemcpyAsync(counts.data(), d_out, out_bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  }
  cudaFree(d_list);
  cudaFree(d_out);
  if (e != cudaSuccess) return static_cast<int>(e);
  std::uint64_t n_bad = 0;
  for (std::size_t i = 0; i < list.size(); ++i) {
    const int s = (counts[2 * i] ? 1 : 0) | (counts[2 * i + 1] ? 2 : 0);
    if (!s) continue;
    ++n_bad;
    if (first && (*first == nullptr || list[i].user < static_cast<unsigned char *>(*first))) {
      *first = list[i].user;
      if (side) *side = s;
    }
  }
  if (damaged) *damaged = n_bad;
  return B200_OK;
}

}  // namespace b200
