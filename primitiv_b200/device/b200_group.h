// primitiv::devices::B200Group -- one primitiv Device spread over several GPUs of a box.
//
// primitiv binds every tensor and parameter to one Device object
// (primitiv/core/parameter.cc:80-97) and knows nothing of data parallelism.  This class keeps
// that contract and hides the GPUs below it: a tensor's handle (an opaque shared_ptr<void> to
// primitiv's core, primitiv/core/tensor.h:213-227) is a table with one part per GPU.
//
//   * a tensor with a minibatch (batch > 1) is cut along the batch axis into contiguous,
//     balanced ranges, one per GPU (the first `batch` GPUs when there are fewer items);
//   * a tensor without one (parameters, their gradients, optimiser state, scalars) is
//     replicated, and every replica is kept bit-identical.
//
// Every operation of the Device interface runs part by part on the per-GPU B200 devices through
// their public Device methods.  Exactly the operations that sum over the batch meet between
// GPUs: the gradient of a broadcast operand (matmul_bw and the elementwise backward passes),
// inplace_add of a minibatch into a tensor without one, batch_sum, and the backward of slice /
// pick into an unbatched tensor.  Each GPU computes its partial sum into a scratch tensor; then
// every GPU reads all partials over NVLink (plain peer loads) and adds them, in GPU order, straight
// into its replica of the result, so the replicas stay equal bit for bit (large sums: each GPU
// does this for one slice and the slices are then copied between the replicas).  The batch-moving operations (batch_pick / slice / concat) copy
// items between GPUs as needed.  The host thread never blocks except for those copies and for
// reads to the host.
//
// Graphs, optimisers and the examples run on a group unchanged: make it the default device.
#ifndef PRIMITIV_DEVICES_B200_GROUP_H_
#define PRIMITIV_DEVICES_B200_GROUP_H_

#include <cstdint>
#include <memory>
#include <vector>

#include <primitiv/core/device.h>

#include "b200_device.h"

namespace primitiv {
namespace devices {

class B200Group : public Device {
  B200Group() = delete;

public:
  /**
   * @param device_ids CUDA ordinals, one shard each.  An ordinal may repeat (several shards
   *                   on one GPU): useful to exercise the sharding logic on a single GPU.
   * @param rng_seed Shard i seeds its random fills with rng_seed + i.
   * @param mode Numeric mode of every shard; PRIMITIV_B200_MODE applies when not given.
   * @throw primitiv::Error if a GPU is missing or two of them cannot map each other's memory.
   */
  explicit B200Group(const std::vector<std::uint32_t> &device_ids);
  B200Group(const std::vector<std::uint32_t> &device_ids, std::uint32_t rng_seed);
  B200Group(const std::vector<std::uint32_t> &device_ids, std::uint32_t rng_seed, B200::Mode mode);
  ~B200Group() override;

  void dump_description() const override;
  DeviceType type() const override { return shards_.front()->type(); }

  std::uint32_t num_shards() const { return static_cast<std::uint32_t>(shards_.size()); }
  B200 &shard(std::uint32_t i) { return *shards_.at(i); }

  /** The part of x that shard i holds (its share of the minibatch, or its replica): read-only. */
  Tensor part(const Tensor &x, std::uint32_t i) const;

  /** Blocks until every GPU has finished its queued work; throws if a kernel reported a timeout. */
  void synchronize();

  /** Sums over GPUs performed so far (each: kernels on every GPU between stream barriers, no host block). */
  std::uint64_t cross_gpu_sums() const { return cross_gpu_sums_; }

private:
  struct Table;    // the handle: one Tensor per shard
  class GradSink;  // where a backward pass adds one gradient

  std::vector<std::unique_ptr<B200>> shards_;
  std::vector<b200_ctx *> ctxs_;
  std::uint64_t cross_gpu_sums_ = 0;

  void initialize(const std::vector<std::uint32_t> &ids, std::uint32_t rng_seed, const B200::Mode *mode);

  std::uint32_t g() const { return static_cast<std::uint32_t>(shards_.size()); }
  // shards that hold a part of a tensor or take part in an operation of this batch size
  std::uint32_t active(std::uint32_t batch) const;
  void range(std::uint32_t batch, std::uint32_t r, std::uint32_t *lo, std::uint32_t *hi) const;
  Shape local(const Shape &s, std::uint32_t r) const;
  std::uint32_t owner(std::uint32_t batch, std::uint32_t item) const;

  Tensor view(const Tensor &x, std::uint32_t r) const;   // read-only part with its local shape
  Table &table(Tensor &x);                               // for writing; may clone a shared tensor
  Tensor take(Table &t, const Shape &xs, std::uint32_t r);
  void sum_into(std::vector<Tensor> &partials, std::uint32_t count, const std::vector<char *> &dst,
                const std::vector<int> &accumulate);
  std::vector<Tensor> sum_over_shards(std::vector<Tensor> &partials, std::uint32_t count);
  Tensor gather(const Tensor &x, const std::vector<std::uint32_t> &items, std::uint32_t r);

  template <typename F> void random_fill(Tensor &y, F make);

#include "device_overrides.inc"
};

}  // namespace devices
}  // namespace primitiv

#endif  // PRIMITIV_DEVICES_B200_GROUP_H_
