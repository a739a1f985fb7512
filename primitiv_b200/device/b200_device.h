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
   * @param rng_seed Seed of the device's random fills.
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

  /** Kernel choice for matmul: 0 per problem, 1 CUDA cores, 2 tensor cores whenever eligible. */
  void set_matmul_path_policy(int policy);

private:
  struct State;
  std::shared_ptr<State> state_;
  std::uint32_t device_id_;
  Mode mode_;

  void initialize(std::uint32_t rng_seed);

  // Tensor -> device pointer.  primitiv zero-fills every gradient right before the first `+=`
  // into it (primitiv/core/graph.cc:191-212).  reset_tensor(0) therefore only notes the
  // tensor as "zero pending"; the fill is launched when something reads it or writes part of
  // it (in / out), and never if the first writer is an accumulating kernel that can store
  // instead of add (out_acc).
  const void *in(const Tensor &x);
  void *out(Tensor &x);
  void *out_acc(Tensor &x, int *accumulate);
  void materialize(const void *ptr);
  void unary_bw(int op, const Tensor &x, const Tensor &y, const Tensor &gy, float k, std::int32_t ik, Tensor &gx);
  int imode() const { return static_cast<int>(mode_); }
  std::size_t elem_size() const { return mode_ == Mode::FP16 ? 2 : 4; }

  std::shared_ptr<void> new_handle(const Shape &shape, std::size_t *const allocated_size) override;

  std::vector<float> tensor_to_vector_impl(const Tensor &x) override;
  std::vector<std::uint32_t> argmax_impl(const Tensor &x, std::uint32_t dim) override;
  std::vector<std::uint32_t> argmin_impl(const Tensor &x, std::uint32_t dim) override;

  void reset_tensor_impl(float k, Tensor &x) override;
  void reset_tensor_by_array_impl(const float values[], Tensor &x) override;
  void copy_tensor_impl(const Tensor &x, Tensor &y) override;
  void identity_impl(Tensor &y) override;

  void random_bernoulli_impl(float p, Tensor &y) override;
  void random_uniform_impl(float lower, float upper, Tensor &y) override;
  void random_normal_impl(float mean, float sd, Tensor &y) override;
  void random_log_normal_impl(float mean, float sd, Tensor &y) override;

  void pick_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &ids, std::uint32_t dim, Tensor &y) override;
  void slice_fw_impl(const Tensor &x, std::uint32_t dim, std::uint32_t offset, Tensor &y) override;
  void concat_fw_impl(const std::vector<const Tensor *> &xs, std::uint32_t dim, Tensor &y) override;
  void pick_bw_impl(const Tensor &gy, const std::vector<std::uint32_t> &ids, std::uint32_t dim, Tensor &gx) override;
  void slice_bw_impl(const Tensor &gy, std::uint32_t dim, std::uint32_t offset, Tensor &gx) override;

#define B200_DECL_X(name)                                        \
  void name##_fw_impl(const Tensor &x, Tensor &y) override;      \
  void name##_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, Tensor &gx) override;
  void negate_fw_impl(const Tensor &x, Tensor &y) override;
  B200_DECL_X(abs) B200_DECL_X(sqrt) B200_DECL_X(exp) B200_DECL_X(log) B200_DECL_X(tanh)
  B200_DECL_X(sigmoid) B200_DECL_X(softplus) B200_DECL_X(sin) B200_DECL_X(cos) B200_DECL_X(tan)
  B200_DECL_X(transpose)
#undef B200_DECL_X

  void permute_dims_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &perm, Tensor &y) override;
  void permute_dims_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy,
                            const std::vector<std::uint32_t> &perm, Tensor &gx) override;
  void flip_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) override;
  void flip_bw_impl(const Tensor &gy, std::uint32_t dim, Tensor &gx) override;

#define B200_DECL_X_CONST(name)                                           \
  void name##_fw_impl(const Tensor &x, float k, Tensor &y) override;      \
  void name##_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, float k, Tensor &gx) override;
  B200_DECL_X_CONST(add_const) B200_DECL_X_CONST(subtract_const_r) B200_DECL_X_CONST(subtract_const_l)
  B200_DECL_X_CONST(multiply_const) B200_DECL_X_CONST(divide_const_r) B200_DECL_X_CONST(divide_const_l)
  B200_DECL_X_CONST(pow_const_r) B200_DECL_X_CONST(pow_const_l) B200_DECL_X_CONST(prelu) B200_DECL_X_CONST(elu)
#undef B200_DECL_X_CONST

  void pown_fw_impl(const Tensor &x, std::int32_t k, Tensor &y) override;
  void pown_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::int32_t k, Tensor &gx) override;

#define B200_DECL_X_SCALAR(name) \
  void name##_fw_impl(const Tensor &x, const Tensor &k, Tensor &y) override;
  B200_DECL_X_SCALAR(add_scalar) B200_DECL_X_SCALAR(subtract_scalar_r) B200_DECL_X_SCALAR(subtract_scalar_l)
  B200_DECL_X_SCALAR(multiply_scalar) B200_DECL_X_SCALAR(divide_scalar_r) B200_DECL_X_SCALAR(divide_scalar_l)
  B200_DECL_X_SCALAR(pow_scalar_r) B200_DECL_X_SCALAR(pow_scalar_l)
#undef B200_DECL_X_SCALAR

#define B200_DECL_AB(name)                                                    \
  void name##_fw_impl(const Tensor &a, const Tensor &b, Tensor &y) override;  \
  void name##_bw_impl(const Tensor &a, const Tensor &b, const Tensor &y, const Tensor &gy, \
                      Tensor &ga, Tensor &gb) override;
  B200_DECL_AB(add) B200_DECL_AB(subtract) B200_DECL_AB(multiply) B200_DECL_AB(divide) B200_DECL_AB(pow)
  B200_DECL_AB(matmul)
#undef B200_DECL_AB

  void max_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) override;
  void min_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) override;
  void max_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t dim, Tensor &gx) override;
  void min_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t dim, Tensor &gx) override;
  void sum_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) override;
  void logsumexp_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) override;
  void broadcast_fw_impl(const Tensor &x, std::uint32_t dim, std::uint32_t size, Tensor &y) override;

  void batch_pick_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &ids, Tensor &y) override;
  void batch_slice_fw_impl(const Tensor &x, std::uint32_t offset, Tensor &y) override;
  void batch_concat_fw_impl(const std::vector<const Tensor *> &xs, Tensor &y) override;
  void batch_sum_fw_impl(const Tensor &x, Tensor &y) override;
  void batch_pick_bw_impl(const Tensor &gy, const std::vector<std::uint32_t> &ids, Tensor &gx) override;
  void batch_slice_bw_impl(const Tensor &gy, std::uint32_t offset, Tensor &gx) override;

  void conv2d_fw_impl(const Tensor &x, const Tensor &w, std::uint32_t padding0, std::uint32_t padding1,
                      std::uint32_t stride0, std::uint32_t stride1, std::uint32_t dilation0,
                      std::uint32_t dilation1, Tensor &y) override;
  void conv2d_bw_impl(const Tensor &x, const Tensor &w, const Tensor &y, const Tensor &gy,
                      std::uint32_t padding0, std::uint32_t padding1, std::uint32_t stride0,
                      std::uint32_t stride1, std::uint32_t dilation0, std::uint32_t dilation1, Tensor &gx,
                      Tensor &gw) override;
  void max_pool2d_fw_impl(const Tensor &x, std::uint32_t window0, std::uint32_t window1, std::uint32_t padding0,
                          std::uint32_t padding1, std::uint32_t stride0, std::uint32_t stride1, Tensor &y) override;
  void max_pool2d_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t window0,
                          std::uint32_t window1, std::uint32_t padding0, std::uint32_t padding1,
                          std::uint32_t stride0, std::uint32_t stride1, Tensor &gx) override;

  void inplace_multiply_const_impl(float k, Tensor &x) override;
  void inplace_add_impl(const Tensor &x, Tensor &y) override;
  void inplace_subtract_impl(const Tensor &x, Tensor &y) override;
};

}  // namespace devices
}  // namespace primitiv

#endif  // PRIMITIV_DEVICES_B200_DEVICE_H_
