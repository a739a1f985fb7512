// primitiv::devices::B200 -- a primitiv Device backed by libprimitiv_b200.so.
//
// Plugs into primitiv exactly where devices::CUDA / devices::CUDA16 do
// (primitiv/devices/cuda/device.h): it subclasses primitiv::Device and overrides every
// pure virtual of primitiv/core/device.h:52-58,368-534.  All device work goes through the C
// ABI of include/primitiv_b200.h and include/primitiv_b200_ops.h; this class only turns
// Tensors and Shapes into pointers and extents.  No CUDA header is needed to compile it.
#ifndef PRIMITIV_DEVICES_B200_DEVICE_H_
#define PRIMITIV_DEVICES_B200_DEVICE_H_

#include <cstdint>
#include <memory>
#include <vector>

#include <primitiv/core/device.h>

struct b200_ctx;

namespace primitiv {
namespace devices {

class B200 : public Device {
  B200() = delete;

public:
  /**
   * Numeric mode of the device.  The storage type of every tensor follows from it.
   */
  enum class Mode : std::uint32_t {
    FP32_3XTF32 = 0,  // float storage; matmul = 3 TF32 tensor-core passes, fp32 accuracy (default)
    TF32_FAST = 1,    // float storage; matmul = 1 TF32 pass
    FP16 = 2,         // half storage, fp32 arithmetic, like devices::CUDA16
    FP32_3XFP16 = 3,  // float storage; matmul = 3 fp16 tensor-core passes on row-scaled half planes, fp32 accuracy
  };

  /** Number of GPUs this backend can drive (compute capability 10.x only). */
  static std::uint32_t num_devices();

  /**
   * @param device_id CUDA ordinal of the GPU.
   * @param rng_seed Seed of the device's random fills; without it the seed comes from
   *                 std::random_device, as in the reference's CUDA device.
   * @param mode Numeric mode; the environment variable PRIMITIV_B200_MODE
   *             (3xtf32 | tf32 | fp16 | 3xfp16) overrides the default when `mode` is not given.
   * @throw primitiv::Error if the GPU does not exist or is not a Blackwell part.
   */
  explicit B200(std::uint32_t device_id);
  B200(std::uint32_t device_id, std::uint32_t rng_seed);
  B200(std::uint32_t device_id, std::uint32_t rng_seed, Mode mode);
  ~B200() override;

  void dump_description() const override;

  /**
   * Reports CUDA for the fp32 modes and CUDA16 for the fp16 mode, so that code keyed on
   * the device type (e.g. the tolerances of primitiv's own tests) treats this device like
   * the reference GPU device of the same storage type.
   */
  DeviceType type() const override {
    return mode_ == Mode::FP16 ? DeviceType::CUDA16 : DeviceType::CUDA;
  }

  Mode mode() const { return mode_; }
  std::uint32_t device_id() const { return device_id_; }
  b200_ctx *context() const;

  /**
   * Blocks until the device's queued work is done.
   * @throw primitiv::Error if a kernel reported that one of its bounded waits ran out (once;
   *        the report is cleared and the device stays usable).  The calls that hand values to
   *        the host (to_vector, argmax, argmin, copies between GPUs) make the same check.
   */
  void wait_and_check();

  /**
   * Whether kernel launches are issued by the library's worker thread (see b200_set_async_launch;
   * also switched on by PRIMITIV_B200_ASYNC=1) or on the calling thread (default).  Results are
   * the same either way.
   */
  void set_async_launch(bool on);

  /** Kernel choice for matmul: 0 per problem, 1 CUDA cores, 2 tensor cores whenever eligible. */
  void set_matmul_path_policy(int policy);

  /**
   * Device pointer of a tensor of this device, for code that launches its own work on it (the
   * device group's sum over GPUs).  `data` makes a deferred zero-fill happen first;
   * `data_for_overwrite` drops it, for a caller that writes every element;
   * `data_for_accumulate` drops it too and then reports *accumulate = 0: a caller that would
   * add to every element stores instead.
   */
  const void *data(const Tensor &x);
  void *data_for_overwrite(Tensor &x);
  void *data_for_accumulate(Tensor &x, int *accumulate);

private:
  struct State;
  std::shared_ptr<State> state_;
  std::uint32_t device_id_;
  Mode mode_;
  int guard_level_ = 0;  // PRIMITIV_B200_POOL_GUARD: 0 off, 1 check at host synchronisation, 2 before every operation too

  void initialize(std::uint32_t rng_seed);
  void check_pool_guards();

  // Tensor -> device pointer.  primitiv zero-fills every gradient right before the first `+=`
  // into it (primitiv/core/graph.cc:191-212).  reset_tensor(0) therefore only notes the
  // tensor as "zero pending"; the fill is launched when something reads it or writes part of
  // it (in / out), and never if the first writer is an accumulating kernel that can store
  // instead of add (out_acc).
  const void *in(const Tensor &x);
  void *out(Tensor &x);
  void *out_acc(Tensor &x, int *accumulate);
  void materialize(const void *ptr);
  void written(const void *p, const Tensor &x);  // x is about to be written: planes packed from it are stale
  void unary_bw(int op, const Tensor &x, const Tensor &y, const Tensor &gy, float k, std::int32_t ik, Tensor &gx);
  int imode() const { return static_cast<int>(mode_); }
  std::size_t elem_size() const { return mode_ == Mode::FP16 ? 2 : 4; }

#include "device_overrides.inc"
};

}  // namespace devices
}  // namespace primitiv

#endif  // PRIMITIV_DEVICES_B200_DEVICE_H_
