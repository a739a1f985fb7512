// primitiv::devices::B200Group: every Device virtual as a loop over per-GPU B200 devices.
//
// The base class has validated shapes and allocated the output before any *_impl runs
// (primitiv/core/device.cc), on the *global* shapes.  Each part carries the same dimensions with
// its share of the batch, so the per-GPU call goes through the public Device method of the
// shard and is validated once more there, on the local shapes.
#include "b200_group.h"

#include <algorithm>
#include <iostream>
#include <random>
#include <string>

#include <primitiv/core/error.h>

#include "../../include/primitiv_b200_ops.h"
#include "batch_partition.h"

#define GROUP_CALL(expr)                                                                     \
  do {                                                                                       \
    const int rc__ = (expr);                                                                 \
    if (rc__ != 0) {                                                                         \
      PRIMITIV_THROW_ERROR("B200Group call `" #expr "` failed: " << ::b200_error_string(rc__) \
                                                                 << " [" << rc__ << "]");    \
    }                                                                                        \
  } while (0)

namespace primitiv {
namespace devices {

// One Tensor per shard, each owned by that shard's B200 device.  An entry is invalid when the
// shard holds no part (a minibatch smaller than the group) or nothing has been written yet.
// reshape() / flatten() share the table between tensors of different dimensions
// (primitiv/core/tensor.cc:58-69), so a part's own shape is only a hint: view() and take()
// re-shape it to what the asking tensor says.
struct B200Group::Table {
  std::vector<Tensor> parts;
};

namespace {
// sums over GPUs of at least this many bytes are done slice by slice (see sum_over_shards)
const std::uint64_t kSlicedSumBytes = 1ull << 20;
}  // namespace

// ---------------------------------------------------------------- construction

// unseeded: entropy from the system, like the reference's one-argument CUDA constructor
// (primitiv/devices/cuda/device.cu:111-112); shard i then draws from seed + i
B200Group::B200Group(const std::vector<std::uint32_t> &device_ids) {
  initialize(device_ids, std::random_device()(), nullptr);
}

B200Group::B200Group(const std::vector<std::uint32_t> &device_ids, std::uint32_t rng_seed) {
  initialize(device_ids, rng_seed, nullptr);
}

B200Group::B200Group(const std::vector<std::uint32_t> &device_ids, std::uint32_t rng_seed, B200::Mode mode) {
  initialize(device_ids, rng_seed, &mode);
}

void B200Group::initialize(const std::vector<std::uint32_t> &ids, std::uint32_t rng_seed, const B200::Mode *mode) {
  if (ids.empty() || ids.size() > 16) {
    PRIMITIV_THROW_ERROR("B200Group needs between 1 and 16 device ids, got " << ids.size() << ".");
  }
  for (std::size_t i = 0; i < ids.size(); ++i) {
    const std::uint32_t seed = rng_seed + static_cast<std::uint32_t>(i);
    shards_.emplace_back(mode ? new B200(ids[i], seed, *mode) : new B200(ids[i], seed));
    // the group orders its GPUs' streams against each other with events and launches peer sums itself:
    // its shards launch on the calling thread
    shards_.back()->set_async_launch(false);
    ctxs_.push_back(shards_.back()->context());
  }
  for (std::size_t i = 0; i < ids.size(); ++i) {
    for (std::size_t j = 0; j < ids.size(); ++j) {
      if (i == j) continue;
      const int rc = ::b200_peer_enable(ctxs_[i], ctxs_[j]);
      if (rc != 0) {
        PRIMITIV_THROW_ERROR("B200Group: GPU " << ids[i] << " cannot map the memory of GPU " << ids[j] << ": "
                                               << ::b200_error_string(rc) << " [" << rc << "]");
      }
    }
  }
}

B200Group::~B200Group() {
  // Finish everything that may still read a peer's memory before any shard releases its pool.
  for (b200_ctx *c : ctxs_) {
    int code = 0;
    ::b200_status_poll(c, nullptr, &code);
  }
}

void B200Group::synchronize() {
  // every GPU is waited for before the first report is thrown, so that no shard is left running
  std::string failed;
  for (auto &s : shards_) {
    try {
      s->wait_and_check();
    } catch (const primitiv::Error &e) {
      if (failed.empty()) failed = e.what();
    }
  }
  if (!failed.empty()) PRIMITIV_THROW_ERROR("B200Group: " << failed);
}

void B200Group::dump_description() const {
  std::cerr << "Device " << this << std::endl;
  std::cerr << "  Type: B200Group, " << shards_.size() << " shard(s); minibatches are cut along the batch axis,"
            << " everything else is replicated" << std::endl;
  for (const auto &s : shards_) s->dump_description();
}

// ---------------------------------------------------------------- partition

std::uint32_t B200Group::active(std::uint32_t batch) const { return batch_partition::active(g(), batch); }

void B200Group::range(std::uint32_t batch, std::uint32_t r, std::uint32_t *lo, std::uint32_t *hi) const {
  batch_partition::range(g(), batch, r, lo, hi);
}

Shape B200Group::local(const Shape &s, std::uint32_t r) const {
  std::uint32_t lo, hi;
  range(s.batch(), r, &lo, &hi);
  return s.resize_batch(hi - lo);
}

std::uint32_t B200Group::owner(std::uint32_t batch, std::uint32_t item) const {
  return batch_partition::owner(g(), batch, item);
}

// ---------------------------------------------------------------- parts of a tensor

Tensor B200Group::view(const Tensor &x, std::uint32_t r) const {
  const Table *t = static_cast<const Table *>(get_handle(x));
  const Tensor &p = t->parts[r];
  if (!p.valid()) {
    PRIMITIV_THROW_ERROR("B200Group: shard " << r << " holds no part of a tensor of shape "
                                             << x.shape().to_string() << " (read before written?)");
  }
  const Shape want = local(x.shape(), r);
  return p.shape() == want ? p : p.reshape(want);
}

Tensor B200Group::part(const Tensor &x, std::uint32_t i) const {
  if (&x.device() != this) PRIMITIV_THROW_ERROR("B200Group::part: the tensor lives on another device.");
  if (i >= g()) PRIMITIV_THROW_ERROR("B200Group::part: no shard " << i << ".");
  return view(x, i);
}

B200Group::Table &B200Group::table(Tensor &x) {
  return *static_cast<Table *>(get_mutable_handle(x));  // copy-on-write through copy_tensor_impl
}

// Moves a part out of its table so that the shard sees a tensor nobody else refers to (otherwise
// its own copy-on-write would clone it); the caller puts it back.
Tensor B200Group::take(Table &t, const Shape &xs, std::uint32_t r) {
  Tensor p = std::move(t.parts[r]);
  if (!p.valid()) {
    PRIMITIV_THROW_ERROR("B200Group: shard " << r << " holds no part of a tensor of shape " << xs.to_string()
                                             << " (updated before written?)");
  }
  const Shape want = local(xs, r);
  if (p.shape() != want) {
    Tensor q = p.reshape(want);
    p.invalidate();
    p = std::move(q);
  }
  return p;
}

std::shared_ptr<void> B200Group::new_handle(const Shape &shape, std::size_t *const allocated_size) {
  // Parts are made by the operation that writes the tensor first.
  if (allocated_size) *allocated_size = static_cast<std::size_t>(shape.size()) * (type() == DeviceType::CUDA16 ? 2 : 4);
  Table *t = new Table;
  t->parts.resize(shards_.size());
  return std::shared_ptr<void>(t, [](void *p) { delete static_cast<Table *>(p); });
}

// ---------------------------------------------------------------- the meeting point of the GPUs

// partials[0 .. count) live on shards 0 .. count-1 and have one shape; dst[r] is memory of that
// shape on shard r (every shard, also those without a partial).  On every shard
//   dst[r] = (accumulate[r] ? dst[r] : 0) + (partials[0] + partials[1] + ...)
// with the partials added in that order: replicas that were equal stay equal, bit for bit.
//
// Small sums (and two GPUs): every GPU reads all partials and adds them itself; (g - 1) x bytes
// cross NVLink per GPU, in one step.  Large sums on three or more GPUs: GPU r does this only for
// the r-th slice, then copies the other slices from the GPUs that made them; 2 (g - 1) / g x
// bytes per GPU, in two steps.
void B200Group::sum_into(std::vector<Tensor> &partials, std::uint32_t count, const std::vector<char *> &dst,
                         const std::vector<int> &accumulate) {
  const Shape shape = partials[0].shape();
  const std::uint64_t n = shape.size();
  const std::size_t es = type() == DeviceType::CUDA16 ? 2 : 4;
  const int imode = static_cast<int>(shards_[0]->mode());
  std::vector<const void *> srcs(count);
  for (std::uint32_t s = 0; s < count; ++s) srcs[s] = shards_[s]->data(partials[s]);
  GROUP_CALL(::b200_stream_barrier(ctxs_.data(), static_cast<int>(ctxs_.size())));  // partials complete everywhere
  if (g() < 3 || n * es < kSlicedSumBytes) {
    for (std::uint32_t r = 0; r < g(); ++r) {
      GROUP_CALL(::b200_peer_sum(ctxs_[r], imode, srcs.data(), static_cast<int>(count), dst[r], n, accumulate[r],
                                 nullptr));
    }
  } else {
    // slice boundaries on multiples of 8 elements keep every 128-bit access aligned
    auto cut = [&](std::uint32_t r) { return r >= g() ? n : (static_cast<std::uint64_t>(r) * n / g()) & ~std::uint64_t(7); };
    std::vector<const void *> shifted(count);
    for (std::uint32_t r = 0; r < g(); ++r) {
      for (std::uint32_t s = 0; s < count; ++s) shifted[s] = static_cast<const char *>(srcs[s]) + cut(r) * es;
      GROUP_CALL(::b200_peer_sum(ctxs_[r], imode, shifted.data(), static_cast<int>(count), dst[r] + cut(r) * es,
                                 cut(r + 1) - cut(r), accumulate[r], nullptr));
    }
    GROUP_CALL(::b200_stream_barrier(ctxs_.data(), static_cast<int>(ctxs_.size())));  // every slice is final
    for (std::uint32_t r = 0; r < g(); ++r) {
      for (std::uint32_t s = 0; s < g(); ++s) {
        if (s == r || cut(s + 1) == cut(s)) continue;
        const void *from = dst[s] + cut(s) * es;
        GROUP_CALL(::b200_peer_sum(ctxs_[r], imode, &from, 1, dst[r] + cut(s) * es, cut(s + 1) - cut(s), 0, nullptr));
      }
    }
  }
  // nobody reuses a partial's (or a slice's) memory before every reader is done with it
  GROUP_CALL(::b200_stream_barrier(ctxs_.data(), static_cast<int>(ctxs_.size())));
  ++cross_gpu_sums_;
}

// The same into fresh tensors, one per shard.
std::vector<Tensor> B200Group::sum_over_shards(std::vector<Tensor> &partials, std::uint32_t count) {
  std::vector<Tensor> sums(g());
  if (g() == 1) {
    sums[0] = std::move(partials[0]);
    return sums;
  }
  std::vector<char *> dst(g());
  for (std::uint32_t r = 0; r < g(); ++r) {
    sums[r] = shards_[r]->new_tensor_by_constant(partials[0].shape(), 0);  // the fill is deferred and dropped right here
    dst[r] = static_cast<char *>(shards_[r]->data_for_overwrite(sums[r]));
  }
  sum_into(partials, count, dst, std::vector<int>(g(), 0));
  return sums;
}

// Where a backward pass adds one gradient.  When the operation runs over a minibatch but the
// gradient has none (a broadcast operand), each shard adds into a zeroed scratch tensor
// instead; finish() adds the scratch tensors of all shards, in shard order, into every replica.
class B200Group::GradSink {
public:
  GradSink(B200Group &dev, Tensor &gx, std::uint32_t op_batch)
      : dev_(dev), shape_(gx.shape()), table_(dev.table(gx)), op_batch_(op_batch),
        meet_(dev.g() > 1 && op_batch > 1 && shape_.batch() == 1), cur_(dev.g()) {}

  Tensor &at(std::uint32_t r) {
    if (!cur_[r].valid()) {
      cur_[r] = meet_ ? dev_.shards_[r]->new_tensor_by_constant(shape_, 0) : dev_.take(table_, shape_, r);
    }
    return cur_[r];
  }

  void finish() {
    if (!meet_) {
      for (std::uint32_t r = 0; r < dev_.g(); ++r)
        if (cur_[r].valid()) table_.parts[r] = std::move(cur_[r]);
      return;
    }
    const std::uint32_t count = dev_.active(op_batch_);
    for (std::uint32_t r = 0; r < count; ++r) at(r);  // a shard that was skipped contributes zeros
    // the total lands in the gradient itself: stored where its zero-fill was still pending, added otherwise
    std::vector<Tensor> parts(dev_.g());
    std::vector<char *> dst(dev_.g());
    std::vector<int> accumulate(dev_.g(), 1);
    for (std::uint32_t r = 0; r < dev_.g(); ++r) {
      parts[r] = dev_.take(table_, shape_, r);
      dst[r] = static_cast<char *>(dev_.shards_[r]->data_for_accumulate(parts[r], &accumulate[r]));
    }
    dev_.sum_into(cur_, count, dst, accumulate);
    for (std::uint32_t r = 0; r < dev_.g(); ++r) table_.parts[r] = std::move(parts[r]);
  }

private:
  B200Group &dev_;
  const Shape shape_;
  Table &table_;
  const std::uint32_t op_batch_;
  const bool meet_;
  std::vector<Tensor> cur_;
};

// A tensor on shard r holding the given items (global batch indices) of x, in that order.
Tensor B200Group::gather(const Tensor &x, const std::vector<std::uint32_t> &items, std::uint32_t r) {
  const std::uint32_t bx = x.shape().batch();
  std::vector<Tensor> pieces;
  std::size_t i = 0;
  while (i < items.size()) {
    if (bx == 1) {  // replicated: the local copy, once per request
      pieces.push_back(view(x, r));
      ++i;
      continue;
    }
    // a run of consecutive items inside one source part
    const std::uint32_t s = owner(bx, items[i]);
    std::uint32_t lo, hi;
    range(bx, s, &lo, &hi);
    std::size_t j = i + 1;
    while (j < items.size() && items[j] == items[j - 1] + 1 && items[j] < hi) ++j;
    const std::uint32_t a = items[i] - lo, b = items[j - 1] + 1 - lo;
    Tensor part = view(x, s);
    Tensor piece = (a == 0 && b == hi - lo) ? part : shards_[s]->batch_slice_fw(part, a, b);
    if (s != r) piece = shards_[r]->copy_tensor(piece);  // between GPUs; waits for both ends
    pieces.push_back(std::move(piece));
    i = j;
  }
  if (pieces.size() == 1) return pieces[0];
  std::vector<const Tensor *> ptrs;
  for (const Tensor &p : pieces) ptrs.push_back(&p);
  return shards_[r]->batch_concat_fw(ptrs);
}

// ---------------------------------------------------------------- host I/O, fills, copies

std::vector<float> B200Group::tensor_to_vector_impl(const Tensor &x) {
  const std::uint32_t n = x.shape().has_batch() ? active(x.shape().batch()) : 1;
  std::vector<float> ret;
  ret.reserve(x.shape().size());
  for (std::uint32_t r = 0; r < n; ++r) {
    const std::vector<float> part = view(x, r).to_vector();
    ret.insert(ret.end(), part.begin(), part.end());
  }
  return ret;
}

std::vector<std::uint32_t> B200Group::argmax_impl(const Tensor &x, std::uint32_t dim) {
  const std::uint32_t n = x.shape().has_batch() ? active(x.shape().batch()) : 1;
  std::vector<std::uint32_t> ret;
  for (std::uint32_t r = 0; r < n; ++r) {
    const std::vector<std::uint32_t> part = view(x, r).argmax(dim);
    ret.insert(ret.end(), part.begin(), part.end());
  }
  return ret;
}

std::vector<std::uint32_t> B200Group::argmin_impl(const Tensor &x, std::uint32_t dim) {
  const std::uint32_t n = x.shape().has_batch() ? active(x.shape().batch()) : 1;
  std::vector<std::uint32_t> ret;
  for (std::uint32_t r = 0; r < n; ++r) {
    const std::vector<std::uint32_t> part = view(x, r).argmin(dim);
    ret.insert(ret.end(), part.begin(), part.end());
  }
  return ret;
}

void B200Group::reset_tensor_impl(float k, Tensor &x) {
  Table &t = table(x);
  const Shape xs = x.shape();
  for (std::uint32_t r = 0; r < active(xs.batch()); ++r) t.parts[r] = shards_[r]->new_tensor_by_constant(local(xs, r), k);
}

void B200Group::reset_tensor_by_array_impl(const float values[], Tensor &x) {
  Table &t = table(x);
  const Shape xs = x.shape();
  for (std::uint32_t r = 0; r < active(xs.batch()); ++r) {
    std::uint32_t lo, hi;
    range(xs.batch(), r, &lo, &hi);
    t.parts[r] = shards_[r]->new_tensor_by_array(local(xs, r), values + static_cast<std::size_t>(lo) * xs.volume());
  }
}

void B200Group::copy_tensor_impl(const Tensor &x, Tensor &y) {
  if (&x.device() == this) {
    Table &t = table(y);
    for (std::uint32_t r = 0; r < active(x.shape().batch()); ++r) t.parts[r] = shards_[r]->copy_tensor(view(x, r));
    return;
  }
  // from any other device (another group included): through the host
  const std::vector<float> values = x.to_vector();
  reset_tensor_by_array_impl(values.data(), y);
}

void B200Group::identity_impl(Tensor &y) {
  Table &t = table(y);
  for (std::uint32_t r = 0; r < g(); ++r) t.parts[r] = shards_[r]->identity(y.shape()[0]);
}

// A minibatch is drawn part by part (every shard has its own seed); a tensor without one is
// drawn on shard 0 and copied, so that replicas agree.
template <typename F>
void B200Group::random_fill(Tensor &y, F make) {
  Table &t = table(y);
  const Shape ys = y.shape();
  if (ys.has_batch()) {
    for (std::uint32_t r = 0; r < active(ys.batch()); ++r) t.parts[r] = make(*shards_[r], local(ys, r));
    return;
  }
  t.parts[0] = make(*shards_[0], ys);
  for (std::uint32_t r = 1; r < g(); ++r) t.parts[r] = shards_[r]->copy_tensor(t.parts[0]);
}

void B200Group::random_bernoulli_impl(float p, Tensor &y) {
  random_fill(y, [p](B200 &d, const Shape &s) { return d.random_bernoulli(s, p); });
}
void B200Group::random_uniform_impl(float lower, float upper, Tensor &y) {
  random_fill(y, [lower, upper](B200 &d, const Shape &s) { return d.random_uniform(s, lower, upper); });
}
void B200Group::random_normal_impl(float mean, float sd, Tensor &y) {
  random_fill(y, [mean, sd](B200 &d, const Shape &s) { return d.random_normal(s, mean, sd); });
}
void B200Group::random_log_normal_impl(float mean, float sd, Tensor &y) {
  random_fill(y, [mean, sd](B200 &d, const Shape &s) { return d.random_log_normal(s, mean, sd); });
}

// ---------------------------------------------------------------- pick / slice / concat

namespace {

// ids carry one entry per batch item, or a single entry for all of them
std::vector<std::uint32_t> ids_of_range(const std::vector<std::uint32_t> &ids, std::uint32_t lo, std::uint32_t hi) {
  std::vector<std::uint32_t> part;
  if (ids.size() == 1) part = ids;
  else part.assign(ids.begin() + lo, ids.begin() + hi);
  return part;
}

std::uint32_t max3(std::uint32_t a, std::uint32_t b, std::uint32_t c) { return std::max(a, std::max(b, c)); }

}  // namespace

void B200Group::pick_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &ids, std::uint32_t dim, Tensor &y) {
  Table &t = table(y);
  const std::uint32_t batch = y.shape().batch();
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    std::uint32_t lo, hi;
    range(batch, r, &lo, &hi);
    t.parts[r] = shards_[r]->pick_fw(view(x, r), ids_of_range(ids, lo, hi), dim);
  }
}

void B200Group::pick_bw_impl(const Tensor &gy, const std::vector<std::uint32_t> &ids, std::uint32_t dim, Tensor &gx) {
  const std::uint32_t batch = max3(gy.shape().batch(), gx.shape().batch(), static_cast<std::uint32_t>(ids.size()));
  GradSink sink(*this, gx, batch);
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    std::uint32_t lo, hi;
    range(batch, r, &lo, &hi);
    shards_[r]->pick_bw(view(gy, r), ids_of_range(ids, lo, hi), dim, sink.at(r));
  }
  sink.finish();
}

void B200Group::slice_fw_impl(const Tensor &x, std::uint32_t dim, std::uint32_t offset, Tensor &y) {
  Table &t = table(y);
  const std::uint32_t upper = offset + y.shape()[dim];
  for (std::uint32_t r = 0; r < active(y.shape().batch()); ++r) t.parts[r] = shards_[r]->slice_fw(view(x, r), dim, offset, upper);
}

void B200Group::slice_bw_impl(const Tensor &gy, std::uint32_t dim, std::uint32_t offset, Tensor &gx) {
  const std::uint32_t batch = std::max(gy.shape().batch(), gx.shape().batch());
  GradSink sink(*this, gx, batch);
  for (std::uint32_t r = 0; r < active(batch); ++r) shards_[r]->slice_bw(view(gy, r), dim, offset, sink.at(r));
  sink.finish();
}

void B200Group::concat_fw_impl(const std::vector<const Tensor *> &xs, std::uint32_t dim, Tensor &y) {
  Table &t = table(y);
  for (std::uint32_t r = 0; r < active(y.shape().batch()); ++r) {
    std::vector<Tensor> views;
    for (const Tensor *x : xs) views.push_back(view(*x, r));
    std::vector<const Tensor *> ptrs;
    for (const Tensor &v : views) ptrs.push_back(&v);
    t.parts[r] = shards_[r]->concat_fw(ptrs, dim);
  }
}

// ---------------------------------------------------------------- elementwise, one tensor

#define GROUP_FW(name, decl_args, call_args)                                                  \
  void B200Group::name##_fw_impl decl_args {                                                  \
    Table &t = table(y);                                                                      \
    for (std::uint32_t r = 0; r < active(y.shape().batch()); ++r) t.parts[r] = shards_[r]->name##_fw call_args; \
  }
// the gradient has the shape of x
#define GROUP_BW(name, decl_args, call_args)                                                  \
  void B200Group::name##_bw_impl decl_args {                                                  \
    const std::uint32_t batch = std::max(gy.shape().batch(), gx.shape().batch());             \
    GradSink sink(*this, gx, batch);                                                          \
    for (std::uint32_t r = 0; r < active(batch); ++r) shards_[r]->name##_bw call_args;        \
    sink.finish();                                                                            \
  }

#define GROUP_X_FW(name) GROUP_FW(name, (const Tensor &x, Tensor &y), (view(x, r)))
#define GROUP_X_BW(name)                                                                      \
  GROUP_BW(name, (const Tensor &x, const Tensor &y, const Tensor &gy, Tensor &gx),            \
           (view(x, r), view(y, r), view(gy, r), sink.at(r)))
#define GROUP_X(name) GROUP_X_FW(name) GROUP_X_BW(name)

GROUP_X_FW(negate)
GROUP_X(abs) GROUP_X(sqrt) GROUP_X(exp) GROUP_X(log) GROUP_X(tanh) GROUP_X(sigmoid) GROUP_X(softplus)
GROUP_X(sin) GROUP_X(cos) GROUP_X(tan) GROUP_X(transpose)

#define GROUP_X_CONST(name)                                                                   \
  GROUP_FW(name, (const Tensor &x, float k, Tensor &y), (view(x, r), k))                      \
  GROUP_BW(name, (const Tensor &x, const Tensor &y, const Tensor &gy, float k, Tensor &gx),   \
           (view(x, r), view(y, r), view(gy, r), k, sink.at(r)))

GROUP_X_CONST(add_const) GROUP_X_CONST(subtract_const_r) GROUP_X_CONST(subtract_const_l)
GROUP_X_CONST(multiply_const) GROUP_X_CONST(divide_const_r) GROUP_X_CONST(divide_const_l)
GROUP_X_CONST(pow_const_r) GROUP_X_CONST(pow_const_l) GROUP_X_CONST(prelu) GROUP_X_CONST(elu)

GROUP_FW(pown, (const Tensor &x, std::int32_t k, Tensor &y), (view(x, r), k))
GROUP_BW(pown, (const Tensor &x, const Tensor &y, const Tensor &gy, std::int32_t k, Tensor &gx),
         (view(x, r), view(y, r), view(gy, r), k, sink.at(r)))

GROUP_FW(permute_dims, (const Tensor &x, const std::vector<std::uint32_t> &perm, Tensor &y), (view(x, r), perm))
GROUP_BW(permute_dims, (const Tensor &x, const Tensor &y, const Tensor &gy, const std::vector<std::uint32_t> &perm,
                        Tensor &gx),
         (view(x, r), view(y, r), view(gy, r), perm, sink.at(r)))

GROUP_FW(flip, (const Tensor &x, std::uint32_t dim, Tensor &y), (view(x, r), dim))
GROUP_BW(flip, (const Tensor &gy, std::uint32_t dim, Tensor &gx), (view(gy, r), dim, sink.at(r)))

// ---------------------------------------------------------------- two tensors

#define GROUP_X_SCALAR(name) GROUP_FW(name, (const Tensor &x, const Tensor &k, Tensor &y), (view(x, r), view(k, r)))

GROUP_X_SCALAR(add_scalar) GROUP_X_SCALAR(subtract_scalar_r) GROUP_X_SCALAR(subtract_scalar_l)
GROUP_X_SCALAR(multiply_scalar) GROUP_X_SCALAR(divide_scalar_r) GROUP_X_SCALAR(divide_scalar_l)
GROUP_X_SCALAR(pow_scalar_r) GROUP_X_SCALAR(pow_scalar_l)

// ga and gb are one tensor for x op x (the graph hands out the same gradient twice)
#define GROUP_AB(name)                                                                        \
  GROUP_FW(name, (const Tensor &a, const Tensor &b, Tensor &y), (view(a, r), view(b, r)))     \
  void B200Group::name##_bw_impl(const Tensor &a, const Tensor &b, const Tensor &y, const Tensor &gy, Tensor &ga, \
                                 Tensor &gb) {                                                \
    const std::uint32_t batch = gy.shape().batch();                                           \
    if (&ga == &gb) {                                                                         \
      GradSink sink(*this, ga, batch);                                                        \
      for (std::uint32_t r = 0; r < active(batch); ++r)                                       \
        shards_[r]->name##_bw(view(a, r), view(b, r), view(y, r), view(gy, r), sink.at(r), sink.at(r)); \
      sink.finish();                                                                          \
      return;                                                                                 \
    }                                                                                         \
    GradSink sink_a(*this, ga, batch), sink_b(*this, gb, batch);                              \
    for (std::uint32_t r = 0; r < active(batch); ++r)                                         \
      shards_[r]->name##_bw(view(a, r), view(b, r), view(y, r), view(gy, r), sink_a.at(r), sink_b.at(r)); \
    sink_a.finish();                                                                          \
    sink_b.finish();                                                                          \
  }

GROUP_AB(add) GROUP_AB(subtract) GROUP_AB(multiply) GROUP_AB(divide) GROUP_AB(pow)
// The hot path: forward is purely local; backward meets between GPUs only for a broadcast operand.
GROUP_AB(matmul)

// ---------------------------------------------------------------- reductions and broadcast

GROUP_FW(max, (const Tensor &x, std::uint32_t dim, Tensor &y), (view(x, r), dim))
GROUP_FW(min, (const Tensor &x, std::uint32_t dim, Tensor &y), (view(x, r), dim))
GROUP_FW(sum, (const Tensor &x, std::uint32_t dim, Tensor &y), (view(x, r), dim))
GROUP_FW(logsumexp, (const Tensor &x, std::uint32_t dim, Tensor &y), (view(x, r), dim))
GROUP_BW(max, (const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t dim, Tensor &gx),
         (view(x, r), view(y, r), view(gy, r), dim, sink.at(r)))
GROUP_BW(min, (const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t dim, Tensor &gx),
         (view(x, r), view(y, r), view(gy, r), dim, sink.at(r)))
GROUP_FW(broadcast, (const Tensor &x, std::uint32_t dim, std::uint32_t size, Tensor &y), (view(x, r), dim, size))

// ---------------------------------------------------------------- batch operations: items move between GPUs

void B200Group::batch_pick_fw_impl(const Tensor &x, const std::vector<std::uint32_t> &ids, Tensor &y) {
  Table &t = table(y);
  const std::uint32_t batch = y.shape().batch();
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    std::uint32_t lo, hi;
    range(batch, r, &lo, &hi);
    t.parts[r] = gather(x, std::vector<std::uint32_t>(ids.begin() + lo, ids.begin() + hi), r);
  }
}

void B200Group::batch_slice_fw_impl(const Tensor &x, std::uint32_t offset, Tensor &y) {
  Table &t = table(y);
  const std::uint32_t batch = y.shape().batch();
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    std::uint32_t lo, hi;
    range(batch, r, &lo, &hi);
    std::vector<std::uint32_t> items;
    for (std::uint32_t i = lo; i < hi; ++i) items.push_back(offset + i);
    t.parts[r] = gather(x, items, r);
  }
}

void B200Group::batch_concat_fw_impl(const std::vector<const Tensor *> &xs, Tensor &y) {
  Table &t = table(y);
  const std::uint32_t batch = y.shape().batch();
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    std::uint32_t lo, hi;
    range(batch, r, &lo, &hi);
    std::vector<Tensor> pieces;
    std::uint32_t first = 0;  // global index in y of the current tensor's item 0
    for (const Tensor *x : xs) {
      const std::uint32_t bx = x->shape().batch();
      const std::uint32_t a = std::max(lo, first), b = std::min(hi, first + bx);
      if (a < b) {
        std::vector<std::uint32_t> items;
        for (std::uint32_t i = a; i < b; ++i) items.push_back(i - first);
        pieces.push_back(gather(*x, items, r));
      }
      first += bx;
    }
    if (pieces.size() == 1) {
      t.parts[r] = std::move(pieces[0]);
    } else {
      std::vector<const Tensor *> ptrs;
      for (const Tensor &p : pieces) ptrs.push_back(&p);
      t.parts[r] = shards_[r]->batch_concat_fw(ptrs);
    }
  }
}

void B200Group::batch_sum_fw_impl(const Tensor &x, Tensor &y) {
  Table &t = table(y);
  const std::uint32_t batch = x.shape().batch();
  std::vector<Tensor> partials(g());
  for (std::uint32_t r = 0; r < active(batch); ++r) partials[r] = shards_[r]->batch_sum_fw(view(x, r));
  if (batch == 1 || g() == 1) {
    t.parts = std::move(partials);
    return;
  }
  t.parts = sum_over_shards(partials, active(batch));
}

void B200Group::batch_pick_bw_impl(const Tensor &gy, const std::vector<std::uint32_t> &ids, Tensor &gx) {
  Table &t = table(gx);
  const Shape xs = gx.shape();
  for (std::uint32_t r = 0; r < active(xs.batch()); ++r) {
    std::uint32_t lo, hi;
    range(xs.batch(), r, &lo, &hi);
    std::vector<std::uint32_t> items, local_ids;  // entries of gy that land in this part
    for (std::uint32_t i = 0; i < ids.size(); ++i) {
      if (ids[i] >= lo && ids[i] < hi) {
        items.push_back(i);
        local_ids.push_back(ids[i] - lo);
      }
    }
    if (items.empty()) continue;
    const Tensor piece = gather(gy, items, r);
    Tensor p = take(t, xs, r);
    shards_[r]->batch_pick_bw(piece, local_ids, p);
    t.parts[r] = std::move(p);
  }
}

void B200Group::batch_slice_bw_impl(const Tensor &gy, std::uint32_t offset, Tensor &gx) {
  Table &t = table(gx);
  const Shape xs = gx.shape();
  const std::uint32_t by = gy.shape().batch();
  for (std::uint32_t r = 0; r < active(xs.batch()); ++r) {
    std::uint32_t lo, hi;
    range(xs.batch(), r, &lo, &hi);
    const std::uint32_t a = std::max(lo, offset), b = std::min(hi, offset + by);
    if (a >= b) continue;
    std::vector<std::uint32_t> items;
    for (std::uint32_t i = a; i < b; ++i) items.push_back(i - offset);
    const Tensor piece = gather(gy, items, r);
    Tensor p = take(t, xs, r);
    shards_[r]->batch_slice_bw(piece, a - lo, p);
    t.parts[r] = std::move(p);
  }
}

// ---------------------------------------------------------------- convolution and pooling

void B200Group::conv2d_fw_impl(const Tensor &x, const Tensor &w, std::uint32_t padding0, std::uint32_t padding1,
                               std::uint32_t stride0, std::uint32_t stride1, std::uint32_t dilation0,
                               std::uint32_t dilation1, Tensor &y) {
  Table &t = table(y);
  for (std::uint32_t r = 0; r < active(y.shape().batch()); ++r) {
    t.parts[r] = shards_[r]->conv2d_fw(view(x, r), view(w, r), padding0, padding1, stride0, stride1, dilation0,
                                       dilation1);
  }
}

void B200Group::conv2d_bw_impl(const Tensor &x, const Tensor &w, const Tensor &y, const Tensor &gy,
                               std::uint32_t padding0, std::uint32_t padding1, std::uint32_t stride0,
                               std::uint32_t stride1, std::uint32_t dilation0, std::uint32_t dilation1, Tensor &gx,
                               Tensor &gw) {
  const std::uint32_t batch = gy.shape().batch();
  GradSink sink_x(*this, gx, batch), sink_w(*this, gw, batch);
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    shards_[r]->conv2d_bw(view(x, r), view(w, r), view(y, r), view(gy, r), padding0, padding1, stride0, stride1,
                          dilation0, dilation1, sink_x.at(r), sink_w.at(r));
  }
  sink_x.finish();
  sink_w.finish();
}

void B200Group::max_pool2d_fw_impl(const Tensor &x, std::uint32_t window0, std::uint32_t window1,
                                   std::uint32_t padding0, std::uint32_t padding1, std::uint32_t stride0,
                                   std::uint32_t stride1, Tensor &y) {
  Table &t = table(y);
  for (std::uint32_t r = 0; r < active(y.shape().batch()); ++r) {
    t.parts[r] = shards_[r]->max_pool2d_fw(view(x, r), window0, window1, padding0, padding1, stride0, stride1);
  }
}

void B200Group::max_pool2d_bw_impl(const Tensor &x, const Tensor &y, const Tensor &gy, std::uint32_t window0,
                                   std::uint32_t window1, std::uint32_t padding0, std::uint32_t padding1,
                                   std::uint32_t stride0, std::uint32_t stride1, Tensor &gx) {
  const std::uint32_t batch = std::max(gy.shape().batch(), gx.shape().batch());
  GradSink sink(*this, gx, batch);
  for (std::uint32_t r = 0; r < active(batch); ++r) {
    shards_[r]->max_pool2d_bw(view(x, r), view(y, r), view(gy, r), window0, window1, padding0, padding1, stride0,
                              stride1, sink.at(r));
  }
  sink.finish();
}

// ---------------------------------------------------------------- in place

void B200Group::inplace_multiply_const_impl(float k, Tensor &x) {
  Table &t = table(x);
  const Shape xs = x.shape();
  for (std::uint32_t r = 0; r < active(xs.batch()); ++r) {
    Tensor p = take(t, xs, r);
    shards_[r]->inplace_multiply_const(k, p);
    t.parts[r] = std::move(p);
  }
}

// y += x.  A minibatch added into a tensor without one is a sum over the batch: each shard sums
// its items, the totals meet between the GPUs.
void B200Group::inplace_add_impl(const Tensor &x, Tensor &y) {
  const std::uint32_t batch = std::max(x.shape().batch(), y.shape().batch());
  GradSink sink(*this, y, batch);
  for (std::uint32_t r = 0; r < active(batch); ++r) shards_[r]->inplace_add(view(x, r), sink.at(r));
  sink.finish();
}

void B200Group::inplace_subtract_impl(const Tensor &x, Tensor &y) {
  const std::uint32_t batch = std::max(x.shape().batch(), y.shape().batch());
  GradSink sink(*this, y, batch);
  for (std::uint32_t r = 0; r < active(batch); ++r) shards_[r]->inplace_subtract(view(x, r), sink.at(r));
  sink.finish();
}

}  // namespace devices
}  // namespace primitiv
