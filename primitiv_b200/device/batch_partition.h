// How devices::B200Group cuts a minibatch over its shards.  Header-only and free of CUDA and of
// primitiv types, so that the rule can be checked on a machine without a GPU.
//
// A batch of one is not cut: every shard holds a replica.  A batch of n > 1 is cut into
// min(g, n) contiguous ranges whose sizes differ by at most one; shards past the n-th hold
// nothing.  For a batch that the shard count divides this is the cut of
// functions::batch::split (primitiv/core/tensor_funcs.cc:366-384).
#ifndef PRIMITIV_DEVICES_B200_BATCH_PARTITION_H_
#define PRIMITIV_DEVICES_B200_BATCH_PARTITION_H_

#include <cstdint>

namespace primitiv {
namespace devices {
namespace batch_partition {

// shards that hold a part of a tensor with this batch size
inline std::uint32_t active(std::uint32_t shards, std::uint32_t batch) {
  return batch == 1 ? shards : (batch < shards ? batch : shards);
}

// [*lo, *hi): the batch items shard r holds; r < active(shards, batch)
inline void range(std::uint32_t shards, std::uint32_t batch, std::uint32_t r, std::uint32_t *lo, std::uint32_t *hi) {
  if (batch == 1) {
    *lo = 0;
    *hi = 1;
    return;
  }
  const std::uint64_t n = active(shards, batch);
  *lo = static_cast<std::uint32_t>(static_cast<std::uint64_t>(r) * batch / n);
  *hi = static_cast<std::uint32_t>(static_cast<std::uint64_t>(r + 1) * batch / n);
}

// the shard that holds batch item `item` of a cut batch (batch > 1)
inline std::uint32_t owner(std::uint32_t shards, std::uint32_t batch, std::uint32_t item) {
  const std::uint32_t n = active(shards, batch);
  std::uint32_t r = static_cast<std::uint32_t>((static_cast<std::uint64_t>(item) * n) / batch);
  std::uint32_t lo, hi;
  for (range(shards, batch, r, &lo, &hi); item < lo; range(shards, batch, r, &lo, &hi)) --r;
  for (; item >= hi; range(shards, batch, r, &lo, &hi)) ++r;
  return r;
}

}  // namespace batch_partition
}  // namespace devices
}  // namespace primitiv

#endif  // PRIMITIV_DEVICES_B200_BATCH_PARTITION_H_
