// primitiv::devices::B200: every Device virtual expressed as a call into the C ABI.
//
// What the base class has already done before any *_impl runs (primitiv/core/device.cc):
// checked that all tensors live on this device, validated and inferred shapes, allocated
// the output.  So nothing here validates shapes; it only derives the flat extents
// (base / repeat / skip, volumes, batch flags) that the kernels take, with the same
// definitions as the reference's Naive device (primitiv/devices/naive/ops/<op>.cc).
#include "b200_device.h"

#include <cstdlib>
#include <cstring>
#include <iostream>
#include <random>
#include <string>
#include <unordered_map>

#include <primitiv/core/error.h>

#include "../../include/primitiv_b200_ops.h"

// A non-zero return code of the C ABI becomes primitiv::Error, the way CUDA_CALL and
// CUBLAS_CALL do for the reference device (primitiv/internal/cuda/utils.h:20-48).
#define B200_CALL(expr)                                                       \
  do {                                                                        \
    const int rc__ = (expr);                                                  \
    if (rc__ != 0) {                                                          \
      PRIMITIV_THROW_ERROR("B200 call `" #expr "` failed: "                   \
                           << ::b200_error_string(rc__) << " [" << rc__ << "]"); \
    }                                                                         \
  } while (0)

#define CDATA(x) (in(x))
#define MDATA(x) (out(x))

namespace primitiv {
namespace devices {

// Owns the context.  Handles keep a weak reference: a Tensor may outlive its device
// (primitiv/test/cuda_device_test.cc:66-78 requires that destroying it then is safe); once
// the state is gone the block has already been released together with the pool.
struct B200::State {
  ::b200_ctx *ctx = nullptr;
  int mode = 0;
  // tensors whose zero-fill has been deferred: device pointer -> element count
  std::unordered_map<const void *, std::uint64_t> zero_pending;
  ~State() {
    if (ctx) ::b200_ctx_destroy(ctx);
  }
};

namespace {

// plane memory the device may keep between products (pool memory; least recently used out first)
const std::size_t kPlaneCacheBytes = std::size_t(8) << 30;
const std::size_t kPoolGuardBytes = 256;

B200::Mode mode_from_environment() {
  const char *e = std::getenv("PRIMITIV_B200_MODE");
  if (!e) return B200::Mode::FP32_3XTF32;
  const std::string v(e);
  if (v == "tf32" || v == "TF32" || v == "tf32_fast") return B200::Mode::TF32_FAST;
  if (v == "fp16" || v == "FP16" || v == "half") return B200::Mode::FP16;
  if (v == "3xtf32" || v == "3XTF32" || v == "fp32") return B200::Mode::FP32_3XTF32;
  if (v == "3xfp16" || v == "3XFP16") return B200::Mode::FP32_3XFP16;
  PRIMITIV_THROW_ERROR("Unknown PRIMITIV_B200_MODE: '" << v << "' (3xtf32 | tf32 | fp16 | 3xfp16)");
}

}  // namespace

std::uint32_t B200::num_devices() {
  // Probe ordinals until context creation reports that the ordinal does not exist.
  std::uint32_t n = 0;
  for (; n < 64; ++n) {
    ::b200_ctx *c = nullptr;
    const int rc = ::b200_ctx_create(static_cast<int>(n), &c);
    if (rc != 0) break;
    ::b200_ctx_destroy(c);
  }
  return n;
}

// Without a seed the random fills start from the system's entropy source, as the reference's
// one-argument constructors do (primitiv/devices/cuda/device.cu:111-112): two unseeded devices
// must not draw the same dropout masks and initial weights.
B200::B200(std::uint32_t device_id) : device_id_(device_id), mode_(mode_from_environment()) {
  initialize(std::random_device()());
}

B200::B200(std::uint32_t device_id, std::uint32_t rng_seed)
    : device_id_(device_id), mode_(mode_from_environment()) {
  initialize(rng_seed);
}

B200::B200(std::uint32_t device_id, std::uint32_t rng_seed, Mode mode) : device_id_(device_id), mode_(mode) {
  initialize(rng_seed);
}

void B200::initialize(std::uint32_t rng_seed) {
  state_ = std::make_shared<State>();
  const int rc = ::b200_ctx_create(static_cast<int>(device_id_), &state_->ctx);
  if (rc != 0) {
    state_.reset();
    PRIMITIV_THROW_ERROR("Could not create a B200 device on GPU " << device_id_ << ": "
                         << ::b200_error_string(rc) << " [" << rc << "]");
  }
  state_->mode = imode();
  // Debugging aid: PRIMITIV_B200_POOL_GUARD=1 puts guard bands round every block of the memory pool
  // and checks them whenever the host waits for the device; =2 checks before every operation as
  // well, so that a store outside a tensor is reported at the operation after the one that did it.
  const char *guard = std::getenv("PRIMITIV_B200_POOL_GUARD");
  if (guard && (std::string(guard) == "1" || std::string(guard) == "2")) {
    B200_CALL(::b200_pool_set_guard(state_->ctx, kPoolGuardBytes));
    guard_level_ = guard[0] - '0';
  }
  B200_CALL(::b200_seed(state_->ctx, rng_seed));
  // The split planes of an fp32 operand are kept from the forward product for the backward one
  // (and for any other product that reads the same tensor); every write goes through out() /
  // out_acc() below, which forget the planes of what is written.
  B200_CALL(::b200_operand_cache_enable(state_->ctx, kPlaneCacheBytes));
  // PRIMITIV_B200_ASYNC=1 moves the kernel launches to the library's worker thread (nothing but this
  // class queues work on the device's stream, and every call that hands values to the host drains
  // the queue).  Off by default: with dependent launches on, the graph-level loops measured here are
  // no longer bound by the launch call, and the worker costs a spinning core.
  const char *async = std::getenv("PRIMITIV_B200_ASYNC");
  if (async && std::string(async) == "1") set_async_launch(true);
  const char *pdl = std::getenv("PRIMITIV_B200_DEPENDENT_LAUNCH");   // 0 switches programmatic dependent launch off
  if (pdl && std::string(pdl) == "0") B200_CALL(::b200_set_dependent_launch(state_->ctx, 0));
}

void B200::check_pool_guards() {
  std::uint64_t damaged = 0;
  void *first = nullptr;
  int side = 0;
  B200_CALL(::b200_pool_check_guards(state_->ctx, nullptr, &damaged, &first, &side));
  if (damaged != 0) {
    PRIMITIV_THROW_ERROR("B200: a kernel on GPU " << device_id_ << " wrote outside its tensor: " << damaged
                         << " block(s) of the memory pool have a damaged guard band, the lowest at " << first
                         << (side == 1 ? " (in front of it)" : side == 2 ? " (behind it)" : " (on both sides)"));
  }
}

void B200::set_async_launch(bool on) { B200_CALL(::b200_set_async_launch(state_->ctx, on ? 1 : 0)); }

void B200::written(const void *p, const Tensor &x) {
  if (guard_level_ >= 2) check_pool_guards();
  ::b200_operand_cache_invalidate(state_->ctx, p, elem_size() * static_cast<std::size_t>(x.shape().size()));
}

void B200::materialize(const void *ptr) {
  auto &pending = state_->zero_pending;
  if (pending.empty()) return;
  const auto it = pending.find(ptr);
  if (it == pending.end()) return;
  const std::uint64_t n = it->second;
  pending.erase(it);
  B200_CALL(::b200_fill(state_->ctx, imode(), const_cast<void *>(ptr), n, 0.f, nullptr));
}

const void *B200::in(const Tensor &x) {
  const void *p = get_handle(x);
  materialize(p);
  return p;
}

void *B200::out(Tensor &x) {
  void *p = get_mutable_handle(x);  // may clone a shared tensor (copy-on-write) through copy_tensor_impl
  materialize(p);
  written(p, x);
  return p;
}

void *B200::out_acc(Tensor &x, int *accumulate) {
  void *p = get_mutable_handle(x);
  auto &pending = state_->zero_pending;
  *accumulate = 1;
  if (!pending.empty()) {
    const auto it = pending.find(p);
    if (it != pending.end()) {
      pending.erase(it);
      *accumulate = 0;  // the kernel stores where it would have added to zeros
    }
  }
  written(p, x);
  return p;
}

B200::~B200() {
  // Outstanding handles only hold weak references, so this releases the context now.
  state_.reset();
}

::b200_ctx *B200::context() const { return state_->ctx; }

// Waits for the device's stream and turns a bounded wait that ran out in some kernel into
// primitiv::Error, the way the reference's CUDA_CALL does for any failed CUDA call
// (primitiv/internal/cuda/utils.h:20-48).  The status word is cleared by the read, so the
// device stays usable: the error is reported once.
void B200::wait_and_check() {
  int code = 0;
  B200_CALL(::b200_status_poll(state_->ctx, nullptr, &code));
  if (code != 0) {
    PRIMITIV_THROW_ERROR("B200: a kernel on GPU " << device_id_ << " gave up waiting: "
                         << ::b200_error_string(code) << " [" << code << "]");
  }
  if (guard_level_ >= 1) check_pool_guards();
}

const void *B200::data(const Tensor &x) {
  if (&x.device() != this) PRIMITIV_THROW_ERROR("B200::data: the tensor lives on another device.");
  return in(x);
}

void *B200::data_for_accumulate(Tensor &x, int *accumulate) {
  if (&x.device() != this) PRIMITIV_THROW_ERROR("B200::data_for_accumulate: the tensor lives on another device.");
  return out_acc(x, accumulate);
}

void *B200::data_for_overwrite(Tensor &x) {
  if (&x.device() != this) PRIMITIV_THROW_ERROR("B200::data_for_overwrite: the tensor lives on another device.");
  void *p = get_mutable_handle(x);
  state_->zero_pending.erase(p);
  written(p, x);
  return p;
}

void B200::set_matmul_path_policy(int policy) { B200_CALL(::b200_set_path_policy(state_->ctx, policy)); }

void B200::dump_description() const {
  int dev = 0, sms = 0;
  ::b200_ctx_device(state_->ctx, &dev, &sms);
  std::uint64_t st[4] = {0, 0, 0, 0};
  ::b200_pool_stats(state_->ctx, st);
  static const char *names[] = {"FP32 (3xTF32)", "TF32 (single pass)", "FP16", "FP32 (3xFP16)"};
  std::cerr << "Device " << this << std::endl;
  std::cerr << "  Type: B200 (sm_100a, libprimitiv_b200)" << std::endl;
  std::cerr << "  GPU ordinal ........ " << dev << std::endl;
  std::cerr << "  SMs ................ " << sms << std::endl;
  std::cerr << "  Numeric mode ....... " << names[imode()] << std::endl;
  std::cerr << "  Pool in use ........ " << st[0] << " bytes" << std::endl;
  std::cerr << "  Pool cached ........ " << st[1] << " bytes" << std::endl;
}

// ---------------------------------------------------------------- memory and host I/O

std::shared_ptr<void> B200::new_handle(const Shape &shape, std::size_t *const allocated_size) {
  void *ptr = nullptr;
  std::size_t got = 0;
  B200_CALL(::b200_pool_alloc(state_->ctx, elem_size() * shape.size(), &ptr, &got));
  if (allocated_size) *allocated_size = got;
  std::weak_ptr<State> weak = state_;
  return std::shared_ptr<void>(ptr, [weak](void *p) {
    if (std::shared_ptr<State> st = weak.lock()) {
      st->zero_pending.erase(p);  // a fill that nobody needed
      ::b200_pool_free(st->ctx, p);
    }
  });
}

std::vector<float> B200::tensor_to_vector_impl(const Tensor &x) {
  std::vector<float> ret(x.shape().size());
  B200_CALL(::b200_download(state_->ctx, imode(), CDATA(x), ret.data(), ret.size(), nullptr));
  if (guard_level_ >= 1) check_pool_guards();
  return ret;
}

std::vector<std::uint32_t> B200::argmax_impl(const Tensor &x, std::uint32_t dim) {
  const Shape &s = x.shape();
  const std::uint32_t n = s[dim];
  std::vector<std::uint32_t> ret(s.size() / n);
  B200_CALL(::b200_argminmax(state_->ctx, imode(), 1, CDATA(x), ret.data(), n, s.lower_volume(dim), ret.size(),
                             nullptr));
  return ret;
}

std::vector<std::uint32_t> B200::argmin_impl(const Tensor &x, std::uint32_t dim) {
  const Shape &s = x.shape();
  const std::uint32_t n = s[dim];
  std::vector<std::uint32_t> ret(s.size() / n);
  B200_CALL(::b200_argminmax(state_->ctx, imode(), 0, CDATA(x), ret.data(), n, s.lower_volume(dim), ret.size(),
                             nullptr));
  return ret;
}

void B200::reset_tensor_impl(float k, Tensor &x) {
  void *p = get_mutable_handle(x);
  written(p, x);
  if (k == 0.f) {
    state_->zero_pending[p] = x.shape().size();  // deferred: see in() / out_acc()
    return;
  }
  state_->zero_pending.erase(p);  // overwritten as a whole
  B200_CALL(::b200_fill(state_->ctx, imode(), p, x.shape().size(), k, nullptr));
}

void B200::reset_tensor_by_array_impl(const float values[], Tensor &x) {
  B200_CALL(::b200_upload(state_->ctx, imode(), values, MDATA(x), x.shape().size(), nullptr));
}

void B200::copy_tensor_impl(const Tensor &x, Tensor &y) {
  // This device reports CUDA / CUDA16 as its type, so the source is identified by its class,
  // not by type(): another B200 (any GPU, any mode) is copied on the device, a Naive tensor is
  // read straight from its host buffer (primitiv/devices/cuda/ops/copy_tensor.cu:12-14), anything
  // else goes through to_vector().
  const std::uint64_t n = x.shape().size();
  if (const B200 *src = dynamic_cast<const B200 *>(&x.device())) {
    if (src->device_id_ == device_id_ || src->mode_ == mode_) {
      // a zero-fill still pending on x is the source device's to launch
      const void *px = const_cast<B200 *>(src)->in(x);
      if (src != this) {
        // whatever still computes x may be waiting in the source device's launch queue: hand it to the
        // driver before this device queues the copy behind it (one GPU: one default stream)
        B200_CALL(::b200_launch_flush(src->state_->ctx));
      }
      if (src->device_id_ != device_id_) {
        // The two GPUs' default streams do not order against each other: let the source
        // device finish whatever still writes x before this device reads it.
        const_cast<B200 *>(src)->wait_and_check();
      }
      B200_CALL(::b200_copy(state_->ctx, src->imode(), px, imode(), MDATA(y), n, nullptr));
      // ... and the copy itself (a converting kernel when the modes differ) is handed to the driver before
      // the source device may queue anything that overwrites x
      if (src != this) B200_CALL(::b200_launch_flush(state_->ctx));
      if (src->device_id_ != device_id_) {
        // ... and finish the copy before the caller may release x: the source GPU's pool
        // orders reuse on its own stream only.
        wait_and_check();
      }
      return;
    }
  } else if (x.device().type() == DeviceType::NAIVE) {
    reset_tensor_by_array(static_cast<const float *>(CDATA(x)), y);
    return;
  }
  reset_tensor_by_vector(x.to_vector(), y);
}

void B200::identity_impl(Tensor &y) {
  B200_CALL(::b200_identity(state_->ctx, imode(), MDATA(y), y.shape()[0], nullptr));
}

// ---------------------------------------------------------------- random fills

void B200::random_bernoulli_impl(float p, Tensor &y) {
  B200_CALL(::b200_random(state_->ctx, imode(), B200_RAND_BERNOULLI, p, 0.f, MDATA(y), y.shape().size(), nullptr));
}
void B200::random_uniform_impl(float lower, float upper, Tensor &y) {
  B200_CALL(::b200_random(state_->ctx, imode(), B200_RAND_UNIFORM, lower, upper, MDATA(y), y.shape().size(), nullptr));
}
void B200::random_normal_impl(float mean, float sd, Tensor &y) {
  B200_CALL(::b200_random(state_->ctx, imode(), B200_RAND_NORMAL, mean, sd, MDATA(y), y.shape().size(), nullptr));
}
void B200::random_log_normal_impl(float mean, float sd, Tensor &y) {
  B200_CALL(::b200_random(state_->ctx, imode(), B200_RAND_LOG_NORMAL, mean, sd, MDATA(y), y.shape().size(), nullptr));
}

// ---------------------------------------------------------------- pick / slice / concat

void B200::pick_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &ids, std::uint32_t dim, Tensor &y) {
  const std::uint64_t base = y.shape().lower_volume(dim);
  B200_CALL(::b200_pick_fw(state_->ctx, imode(), CDATA(x), ids.data(), static_cast<std::uint32_t>(ids.size()),
                           MDATA(y), base, x.shape()[dim], y.shape().volume() / base, y.shape().batch(),
                           x.shape().has_batch(), nullptr));
}

void B200::pick_bw_impl(const Tensor &gy, const std::vector<std::uint32_t> &ids, std::uint32_t dim, Tensor &gx) {
  const std::uint64_t base = gy.shape().lower_volume(dim);
  B200_CALL(::b200_pick_bw(state_->ctx, imode(), CDATA(gy), ids.data(), static_cast<std::uint32_t>(ids.size()),
                           MDATA(gx), base, gx.shape()[dim], gy.shape().volume() / base, gy.shape().batch(),
                           gx.shape().has_batch(), nullptr));
}

void B200::slice_fw_impl(const Tensor &x, std::uint32_t dim, std::uint32_t offset, Tensor &y) {
  const std::uint64_t base = y.shape().lower_volume(dim);
  const std::uint32_t y_dim = y.shape()[dim];
  B200_CALL(::b200_slice_fw(state_->ctx, imode(), CDATA(x), MDATA(y), base, x.shape()[dim], y_dim, offset,
                            y.shape().size() / (base * y_dim), nullptr));
}

void B200::slice_bw_impl(const Tensor &gy, std::uint32_t dim, std::uint32_t offset, Tensor &gx) {
  const Shape &sx = gx.shape();
  const std::uint64_t base = sx.lower_volume(dim);
  const std::uint32_t x_dim = sx[dim];
  // a gradient whose zero-fill is still pending is stored as a whole (slice from gy, zeros elsewhere)
  int accumulate = 1;
  void *dst = out_acc(gx, &accumulate);
  B200_CALL(::b200_slice_bw_ex(state_->ctx, imode(), CDATA(gy), dst, base, x_dim, gy.shape()[dim], offset,
                               sx.volume() / (base * x_dim), sx.batch(), gy.shape().batch(), accumulate, nullptr));
}

void B200::concat_fw_impl(const std::vector<const Tensor *> &xs, std::uint32_t dim, Tensor &y) {
  const Shape &sy = y.shape();
  const std::uint64_t base = sy.lower_volume(dim);
  const std::uint32_t y_dim = sy[dim];
  const std::uint64_t repeat = sy.volume() / (base * y_dim);
  void *dest = MDATA(y);
  std::uint32_t offset = 0;
  for (const Tensor *x : xs) {
    const std::uint32_t x_dim = x->shape()[dim];
    B200_CALL(::b200_concat_part(state_->ctx, imode(), CDATA(*x), dest, base, x_dim, y_dim, offset, repeat,
                                 sy.batch(), x->shape().has_batch(), nullptr));
    offset += x_dim;
  }
}

// ---------------------------------------------------------------- elementwise, one tensor

// gx (+)= d op(x, y) * gy: the operands are resolved first, then gx, which stores instead of
// adding when its zero-fill is still pending.
void B200::unary_bw(int op, const Tensor &x, const Tensor &y, const Tensor &gy, float k, std::int32_t ik,
                    Tensor &gx) {
  const void *px = in(x), *py = in(y), *pgy = in(gy);
  int acc = 1;
  void *pgx = out_acc(gx, &acc);
  B200_CALL(::b200_unary_bw(state_->ctx, imode(), op, px, py, pgy, pgx, x.shape().size(), k, ik, acc, nullptr));
}

#define B200_IMPL_X_FW(name, op)                                                                   \
  void B200::name##_fw_impl(const Tensor &x, Tensor &y) {                                          \
    B200_CALL(::b200_unary_fw(state_->ctx, imode(), op, CDATA(x), MDATA(y), x.shape().size(), 0.f, 0, nullptr)); \
  }
#define B200_IMPL_X_BW(name, op)                                                                   \
  void B200::name##_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, Tensor &gx) {      \
    unary_bw(op, x, y, gy, 0.f, 0, gx);                                                            \
  }
#define B200_IMPL_X(name, op) B200_IMPL_X_FW(name, op) B200_IMPL_X_BW(name, op)

B200_IMPL_X_FW(negate, B200_OP_NEGATE)
B200_IMPL_X(abs, B200_OP_ABS)
B200_IMPL_X(sqrt, B200_OP_SQRT)
B200_IMPL_X(exp, B200_OP_EXP)
B200_IMPL_X(log, B200_OP_LOG)
B200_IMPL_X(tanh, B200_OP_TANH)
B200_IMPL_X(sigmoid, B200_OP_SIGMOID)
B200_IMPL_X(softplus, B200_OP_SOFTPLUS)
B200_IMPL_X(sin, B200_OP_SIN)
B200_IMPL_X(cos, B200_OP_COS)
B200_IMPL_X(tan, B200_OP_TAN)

#define B200_IMPL_X_CONST(name, op)                                                                \
  void B200::name##_fw_impl(const Tensor &x, float k, Tensor &y) {                                 \
    B200_CALL(::b200_unary_fw(state_->ctx, imode(), op, CDATA(x), MDATA(y), x.shape().size(), k, 0, nullptr)); \
  }                                                                                                \
  void B200::name##_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, float k, Tensor &gx) { \
    unary_bw(op, x, y, gy, k, 0, gx);                                                              \
  }

B200_IMPL_X_CONST(add_const, B200_OP_ADD_CONST)
B200_IMPL_X_CONST(subtract_const_r, B200_OP_SUB_CONST_R)
B200_IMPL_X_CONST(subtract_const_l, B200_OP_SUB_CONST_L)
B200_IMPL_X_CONST(multiply_const, B200_OP_MUL_CONST)
B200_IMPL_X_CONST(divide_const_r, B200_OP_DIV_CONST_R)
B200_IMPL_X_CONST(divide_const_l, B200_OP_DIV_CONST_L)
B200_IMPL_X_CONST(pow_const_r, B200_OP_POW_CONST_R)
B200_IMPL_X_CONST(pow_const_l, B200_OP_POW_CONST_L)
B200_IMPL_X_CONST(prelu, B200_OP_PRELU)
B200_IMPL_X_CONST(elu, B200_OP_ELU)

void B200::pown_fw_impl(const Tensor &x, std::int32_t k, Tensor &y) {
  B200_CALL(::b200_unary_fw(state_->ctx, imode(), B200_OP_POWN, CDATA(x), MDATA(y), x.shape().size(), 0.f, k, nullptr));
}
void B200::pown_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::int32_t k, Tensor &gx) {
  unary_bw(B200_OP_POWN, x, y, gy, 0.f, k, gx);
}

// ---------------------------------------------------------------- transpose / permute / flip

void B200::transpose_fw_impl(const Tensor &x, Tensor &y) {
  B200_CALL(::b200_transpose(state_->ctx, imode(), CDATA(x), MDATA(y), x.shape()[0], x.shape()[1],
                             x.shape().batch(), 0, nullptr));
}
void B200::transpose_bw_impl(const Tensor &, const Tensor &, const Tensor &gy, Tensor &gx) {
  B200_CALL(::b200_transpose(state_->ctx, imode(), CDATA(gy), MDATA(gx), gy.shape()[0], gy.shape()[1],
                             gy.shape().batch(), 1, nullptr));
}

void B200::permute_dims_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &perm, Tensor &y) {
  std::uint32_t dims[8];
  const std::uint32_t nd = static_cast<std::uint32_t>(perm.size());
  for (std::uint32_t i = 0; i < nd && i < 8; ++i) dims[i] = x.shape()[i];
  B200_CALL(::b200_permute_dims(state_->ctx, imode(), CDATA(x), MDATA(y), nd, dims, perm.data(),
                                x.shape().batch(), 0, nullptr));
}
void B200::permute_dims_bw_impl(const Tensor &, const Tensor &, const Tensor &gy,
                                const std::vector<std::uint32_t> &perm, Tensor &gx) {
  std::uint32_t dims[8];
  const std::uint32_t nd = static_cast<std::uint32_t>(perm.size());
  for (std::uint32_t i = 0; i < nd && i < 8; ++i) dims[i] = gx.shape()[i];
  B200_CALL(::b200_permute_dims(state_->ctx, imode(), CDATA(gy), MDATA(gx), nd, dims, perm.data(),
                                gx.shape().batch(), 1, nullptr));
}

void B200::flip_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) {
  const Shape &s = x.shape();
  B200_CALL(::b200_flip(state_->ctx, imode(), CDATA(x), MDATA(y), s.lower_volume(dim), s[dim], s.size(), 0, nullptr));
}
void B200::flip_bw_impl(const Tensor &gy, std::uint32_t dim, Tensor &gx) {
  const Shape &s = gx.shape();
  B200_CALL(::b200_flip(state_->ctx, imode(), CDATA(gy), MDATA(gx), s.lower_volume(dim), s[dim], s.size(), 1, nullptr));
}

// ---------------------------------------------------------------- elementwise, tensor and scalar tensor

#define B200_IMPL_X_SCALAR(name, op)                                                               \
  void B200::name##_fw_impl(const Tensor &x, const Tensor &k, Tensor &y) {                         \
    B200_CALL(::b200_scalar_fw(state_->ctx, imode(), op, CDATA(x), CDATA(k), MDATA(y), y.shape().volume(), \
                               y.shape().batch(), x.shape().has_batch(), k.shape().has_batch(), nullptr)); \
  }

B200_IMPL_X_SCALAR(add_scalar, B200_OP_ADD)
B200_IMPL_X_SCALAR(subtract_scalar_r, B200_OP_SUBTRACT)
B200_IMPL_X_SCALAR(subtract_scalar_l, B200_OP_SUBTRACT_L)
B200_IMPL_X_SCALAR(multiply_scalar, B200_OP_MULTIPLY)
B200_IMPL_X_SCALAR(divide_scalar_r, B200_OP_DIVIDE)
B200_IMPL_X_SCALAR(divide_scalar_l, B200_OP_DIVIDE_L)
B200_IMPL_X_SCALAR(pow_scalar_r, B200_OP_POW)
B200_IMPL_X_SCALAR(pow_scalar_l, B200_OP_POW_L)

// ---------------------------------------------------------------- elementwise, two tensors

#define B200_IMPL_AB(name, op)                                                                     \
  void B200::name##_fw_impl(const Tensor &a, const Tensor &b, Tensor &y) {                         \
    B200_CALL(::b200_binary_fw(state_->ctx, imode(), op, CDATA(a), CDATA(b), MDATA(y), y.shape().volume(), \
                               y.shape().batch(), a.shape().has_batch(), b.shape().has_batch(), nullptr)); \
  }                                                                                                \
  void B200::name##_bw_impl(const Tensor &a, const Tensor &b, const Tensor &y, const Tensor &gy,   \
                            Tensor &ga, Tensor &gb) {                                              \
    const void *pa = in(a), *pb = in(b), *py = in(y), *pgy = in(gy);                               \
    int acc_a = 1, acc_b = 1;                                                                      \
    void *pga = out_acc(ga, &acc_a);                                                               \
    void *pgb = out_acc(gb, &acc_b); /* the same tensor as ga for x op x: then it accumulates */   \
    B200_CALL(::b200_binary_bw(state_->ctx, imode(), op, pa, pb, py, pgy, pga, pgb, gy.shape().volume(), \
                               gy.shape().batch(), a.shape().has_batch(), b.shape().has_batch(), acc_a, \
                               acc_b, nullptr));                                                   \
  }

B200_IMPL_AB(add, B200_OP_ADD)
B200_IMPL_AB(subtract, B200_OP_SUBTRACT)
B200_IMPL_AB(multiply, B200_OP_MULTIPLY)
B200_IMPL_AB(divide, B200_OP_DIVIDE)
B200_IMPL_AB(pow, B200_OP_POW)

// ---------------------------------------------------------------- the hot path

void B200::matmul_fw_impl(const Tensor &a, const Tensor &b, Tensor &y) {
  B200_CALL(::b200_matmul_fw(state_->ctx, imode(), CDATA(a), CDATA(b), MDATA(y), a.shape()[0], a.shape()[1],
                             b.shape()[1], a.shape().batch(), b.shape().batch(), nullptr));
}

void B200::matmul_bw_impl(const Tensor &a, const Tensor &b, const Tensor &, const Tensor &gy, Tensor &ga,
                          Tensor &gb) {
  const void *pa = in(a), *pb = in(b), *pgy = in(gy);
  int acc_a = 1, acc_b = 1;
  void *pga = out_acc(ga, &acc_a);
  void *pgb = out_acc(gb, &acc_b);
  B200_CALL(::b200_matmul_bw_ex(state_->ctx, imode(), pa, pb, pgy, pga, pgb, a.shape()[0], a.shape()[1],
                                b.shape()[1], a.shape().batch(), b.shape().batch(), acc_a, acc_b, nullptr));
}

// ---------------------------------------------------------------- reductions and broadcast

#define B200_IMPL_REDUCE(name, red)                                                                \
  void B200::name##_fw_impl(const Tensor &x, std::uint32_t dim, Tensor &y) {                       \
    B200_CALL(::b200_reduce_fw(state_->ctx, imode(), red, CDATA(x), MDATA(y), x.shape()[dim],      \
                               y.shape().lower_volume(dim), y.shape().size(), nullptr));           \
  }

B200_IMPL_REDUCE(max, B200_RED_MAX)
B200_IMPL_REDUCE(min, B200_RED_MIN)
B200_IMPL_REDUCE(sum, B200_RED_SUM)
B200_IMPL_REDUCE(logsumexp, B200_RED_LOGSUMEXP)

void B200::max_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t dim, Tensor &gx) {
  B200_CALL(::b200_minmax_bw(state_->ctx, imode(), CDATA(x), CDATA(y), CDATA(gy), MDATA(gx), x.shape()[dim],
                             y.shape().lower_volume(dim), y.shape().size(), nullptr));
}
void B200::min_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t dim, Tensor &gx) {
  B200_CALL(::b200_minmax_bw(state_->ctx, imode(), CDATA(x), CDATA(y), CDATA(gy), MDATA(gx), x.shape()[dim],
                             y.shape().lower_volume(dim), y.shape().size(), nullptr));
}

void B200::broadcast_fw_impl(const Tensor &x, std::uint32_t dim, std::uint32_t size, Tensor &y) {
  B200_CALL(::b200_broadcast_fw(state_->ctx, imode(), CDATA(x), MDATA(y), x.shape().size(),
                                y.shape().lower_volume(dim), size, nullptr));
}

// ---------------------------------------------------------------- batch operations

void B200::batch_pick_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &ids, Tensor &y) {
  B200_CALL(::b200_batch_pick_fw(state_->ctx, imode(), CDATA(x), ids.data(), static_cast<std::uint32_t>(ids.size()),
                                 MDATA(y), x.shape().volume(), nullptr));
}
void B200::batch_pick_bw_impl(const Tensor &gy, const std::vector<std::uint32_t> &ids, Tensor &gx) {
  B200_CALL(::b200_batch_pick_bw(state_->ctx, imode(), CDATA(gy), ids.data(), static_cast<std::uint32_t>(ids.size()),
                                 MDATA(gx), gx.shape().volume(), nullptr));
}

void B200::batch_slice_fw_impl(const Tensor &x, std::uint32_t offset, Tensor &y) {
  const std::uint64_t volume = y.shape().volume();
  const char *src = static_cast<const char *>(CDATA(x)) + elem_size() * volume * offset;
  B200_CALL(::b200_copy(state_->ctx, imode(), src, imode(), MDATA(y), volume * y.shape().batch(), nullptr));
}
void B200::batch_slice_bw_impl(const Tensor &gy, std::uint32_t offset, Tensor &gx) {
  const std::uint64_t volume = gy.shape().volume();
  char *dest = static_cast<char *>(MDATA(gx)) + elem_size() * volume * offset;
  B200_CALL(::b200_inplace_add(state_->ctx, imode(), CDATA(gy), dest, volume * gy.shape().batch(), 1, 1, 1.f, nullptr));
}

void B200::batch_concat_fw_impl(const std::vector<const Tensor *> &xs, Tensor &y) {
  char *dest = static_cast<char *>(MDATA(y));
  for (const Tensor *x : xs) {
    const std::uint64_t span = x->shape().size();
    B200_CALL(::b200_copy(state_->ctx, imode(), CDATA(*x), imode(), dest, span, nullptr));
    dest += elem_size() * span;
  }
}

void B200::batch_sum_fw_impl(const Tensor &x, Tensor &y) {
  B200_CALL(::b200_batch_sum_fw(state_->ctx, imode(), CDATA(x), MDATA(y), y.shape().size(), x.shape().batch(), nullptr));
}

// ---------------------------------------------------------------- convolution and pooling

namespace {

// Pool memory for the lifetime of one operation (the gathered input of a convolution).
struct Scratch {
  ::b200_ctx *ctx;
  void *p = nullptr;
  Scratch(::b200_ctx *c, std::size_t bytes) : ctx(c) {
    std::size_t got = 0;
    const int rc = ::b200_pool_alloc(ctx, bytes, &p, &got);
    if (rc != 0) PRIMITIV_THROW_ERROR("B200: scratch allocation of " << bytes << " bytes failed: "
                                      << ::b200_error_string(rc) << " [" << rc << "]");
  }
  ~Scratch() { if (p) ::b200_pool_free(ctx, p); }  // stream-ordered reuse: later work queues behind its readers
  Scratch(const Scratch &) = delete;
  Scratch &operator=(const Scratch &) = delete;
};

}  // namespace

// conv2d = gather (im2col) + the matrix product of the hot path: y {P, Cout} = col {P, K} . w {K, Cout}
// with P = Ho*Wo, K = kh*kw*C; the batch of x becomes the batch of col, a batch of w stays one
// (the reference lets either operand broadcast, primitiv/devices/naive/ops/conv2d.cc:29-31).
void B200::conv2d_fw_impl(const Tensor &x, const Tensor &w, std::uint32_t padding0, std::uint32_t padding1,
                          std::uint32_t stride0, std::uint32_t stride1, std::uint32_t dilation0,
                          std::uint32_t dilation1, Tensor &y) {
  const Shape &xs = x.shape(), &ws = w.shape(), &ys = y.shape();
  const std::uint32_t P = ys[0] * ys[1], K = ws[0] * ws[1] * xs[2], bx = xs.batch();
  const void *px = in(x), *pw = in(w);
  void *py = out(y);
  Scratch col(state_->ctx, static_cast<std::size_t>(P) * K * bx * elem_size());
  B200_CALL(::b200_im2col(state_->ctx, imode(), px, col.p, xs[0], xs[1], xs[2], ws[0], ws[1], ys[0], ys[1],
                          padding0, padding1, stride0, stride1, dilation0, dilation1, bx, xs.has_batch(), nullptr));
  B200_CALL(::b200_matmul_fw(state_->ctx, imode(), col.p, pw, py, P, K, ys[2], bx, ws.batch(), nullptr));
}

void B200::conv2d_bw_impl(const Tensor &x, const Tensor &w, const Tensor &, const Tensor &gy,
                          std::uint32_t padding0, std::uint32_t padding1, std::uint32_t stride0,
                          std::uint32_t stride1, std::uint32_t dilation0, std::uint32_t dilation1, Tensor &gx,
                          Tensor &gw) {
  const Shape &xs = x.shape(), &ws = w.shape(), &ys = gy.shape();
  const std::uint32_t P = ys[0] * ys[1], K = ws[0] * ws[1] * xs[2], bx = xs.batch();
  const void *px = in(x), *pw = in(w), *pgy = in(gy);
  int acc_w = 1;
  void *pgw = out_acc(gw, &acc_w);
  void *pgx = out(gx);
  const std::size_t col_bytes = static_cast<std::size_t>(P) * K * bx * elem_size();
  Scratch col(state_->ctx, col_bytes), gcol(state_->ctx, col_bytes);
  B200_CALL(::b200_im2col(state_->ctx, imode(), px, col.p, xs[0], xs[1], xs[2], ws[0], ws[1], ys[0], ys[1],
                          padding0, padding1, stride0, stride1, dilation0, dilation1, bx, xs.has_batch(), nullptr));
  // gcol = gy . w^T (written, summed over the batch when x is broadcast); gw += col^T . gy
  B200_CALL(::b200_matmul_bw_ex(state_->ctx, imode(), col.p, pw, pgy, gcol.p, pgw, P, K, ys[2], bx, ws.batch(),
                                0, acc_w, nullptr));
  B200_CALL(::b200_col2im(state_->ctx, imode(), gcol.p, pgx, xs[0], xs[1], xs[2], ws[0], ws[1], ys[0], ys[1],
                          padding0, padding1, stride0, stride1, dilation0, dilation1, bx, nullptr));
}

void B200::max_pool2d_fw_impl(const Tensor &x, std::uint32_t window0, std::uint32_t window1,
                              std::uint32_t padding0, std::uint32_t padding1, std::uint32_t stride0,
                              std::uint32_t stride1, Tensor &y) {
  const Shape &xs = x.shape(), &ys = y.shape();
  const std::uint64_t repeat = xs.size() / (static_cast<std::uint64_t>(xs[0]) * xs[1]);
  B200_CALL(::b200_max_pool2d_fw(state_->ctx, imode(), CDATA(x), MDATA(y), xs[0], xs[1], ys[0], ys[1], window0,
                                 window1, padding0, padding1, stride0, stride1, repeat, nullptr));
}

void B200::max_pool2d_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t window0,
                              std::uint32_t window1, std::uint32_t padding0, std::uint32_t padding1,
                              std::uint32_t stride0, std::uint32_t stride1, Tensor &gx) {
  const Shape &xs = x.shape(), &ys = y.shape();
  const std::uint64_t repeat = xs.size() / (static_cast<std::uint64_t>(xs[0]) * xs[1]);
  const void *px = in(x), *py = in(y), *pgy = in(gy);
  void *pgx = out(gx);
  B200_CALL(::b200_max_pool2d_bw(state_->ctx, imode(), px, py, pgy, pgx, xs[0], xs[1], ys[0], ys[1], window0,
                                 window1, padding0, padding1, stride0, stride1, repeat, nullptr));
}

// ---------------------------------------------------------------- in place

void B200::inplace_multiply_const_impl(float k, Tensor &x) {
  B200_CALL(::b200_inplace_multiply_const(state_->ctx, imode(), MDATA(x), x.shape().size(), k, nullptr));
}
void B200::inplace_add_impl(const Tensor &x, Tensor &y) {
  const void *px = in(x);
  int acc = 1;
  void *py = out_acc(y, &acc);   // acc == 0: y held (deferred) zeros and is stored, not added to
  B200_CALL(::b200_inplace_add_ex(state_->ctx, imode(), px, py, y.shape().volume(), x.shape().batch(), y.shape().batch(),
                                  1.f, acc, nullptr));
}
void B200::inplace_subtract_impl(const Tensor &x, Tensor &y) {
  const void *px = in(x);
  int acc = 1;
  void *py = out_acc(y, &acc);
  B200_CALL(::b200_inplace_add_ex(state_->ctx, imode(), px, py, y.shape().volume(), x.shape().batch(), y.shape().batch(),
                                  -1.f, acc, nullptr));
}

}  // namespace devices
}  // namespace primitiv
