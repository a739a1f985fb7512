// Parity of primitiv::devices::B200Group (one Device over several shards / GPUs) against the
// reference's Naive device, on the operations where shards meet or items move between them,
// with minibatches that do not divide evenly and minibatches smaller than the group; then a
// few training steps of a small perceptron through primitiv's Graph, where every replica of
// every parameter must stay bit-identical.  The Naive device is the checker only.
//
//   group_parity <mode: 3xtf32|tf32|fp16|3xfp16> <ordinal,ordinal,...>
// Exit status 0 = all checks passed.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include <primitiv/core/error.h>
#include <primitiv/core/functions.h>
#include <primitiv/core/graph.h>
#include <primitiv/core/initializer_impl.h>
#include <primitiv/core/optimizer_impl.h>
#include <primitiv/core/parameter.h>
#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>
#include <primitiv/devices/naive/device.h>

#include "b200_group.h"
#include "../../include/primitiv_b200.h"

using primitiv::Device;
using primitiv::Graph;
using primitiv::Node;
using primitiv::Parameter;
using primitiv::Shape;
using primitiv::Tensor;
using primitiv::devices::B200;
using primitiv::devices::B200Group;
using primitiv::devices::Naive;
using std::vector;
namespace F = primitiv::functions;

namespace {

int g_checks = 0, g_failures = 0;
float g_tol = 1e-5f, g_mm_tol = 1e-5f;
bool g_half = false;
std::mt19937 g_rng(2024);

float to_grid(float x) {  // exactly representable in half when the device stores half
  if (!g_half) return x;
  int e;
  const float m = std::frexp(x, &e);
  return std::ldexp(std::round(m * 2048.f) / 2048.f, e);
}

vector<float> rnd(std::size_t n, float lo = -1.f, float hi = 1.f) {
  std::uniform_real_distribution<float> d(lo, hi);
  vector<float> v(n);
  for (float &x : v) x = to_grid(d(g_rng));
  return v;
}

void expect(bool ok, const std::string &what) {
  ++g_checks;
  if (!ok) { ++g_failures; std::cerr << "FAIL: " << what << std::endl; }
}

void expect_close(const vector<float> &want, const vector<float> &got, const std::string &what, float tol) {
  ++g_checks;
  if (want.size() != got.size()) { ++g_failures; std::cerr << "FAIL: " << what << ": size" << std::endl; return; }
  double num = 0, den = 0;
  for (std::size_t i = 0; i < want.size(); ++i) {
    const double d = double(want[i]) - got[i];
    num += d * d;
    den += double(want[i]) * want[i];
  }
  const double rel = den > 0 ? std::sqrt(num / den) : std::sqrt(num);
  if (!(rel <= tol)) { ++g_failures; std::cerr << "FAIL: " << what << ": normwise error " << rel << " > " << tol << std::endl; }
}

struct Pair {  // the same values on both devices
  Tensor ref, got;
  Pair(const Shape &s, const vector<float> &v, Naive &n, B200Group &g)
      : ref(n.new_tensor_by_vector(s, v)), got(g.new_tensor_by_vector(s, v)) {}
};

// Every replica of an unbatched tensor holds the same bits.
void expect_replicas_equal(B200Group &g, const Tensor &x, const std::string &what) {
  const vector<float> first = g.part(x, 0).to_vector();
  for (std::uint32_t i = 1; i < g.num_shards(); ++i) {
    const vector<float> other = g.part(x, i).to_vector();
    expect(other.size() == first.size() && std::memcmp(other.data(), first.data(), first.size() * sizeof(float)) == 0,
           what + ": replica " + std::to_string(i) + " differs from replica 0");
  }
}

void test_matmul(Naive &n, B200Group &g, std::uint32_t batch) {
  const std::uint32_t di = 48, dj = 40, dk = 24;
  for (int ba = 0; ba < 2; ++ba) {
    for (int bb = 0; bb < 2; ++bb) {
      const std::uint32_t na = ba ? batch : 1, nb = bb ? batch : 1, ny = std::max(na, nb);
      const std::string tag = "matmul batch " + std::to_string(batch) + " a" + std::to_string(ba) + " b" + std::to_string(bb);
      Pair a(Shape({di, dj}, na), rnd(di * dj * na), n, g), b(Shape({dj, dk}, nb), rnd(dj * dk * nb), n, g);
      Pair gy(Shape({di, dk}, ny), rnd(di * dk * ny), n, g);
      Pair ga(Shape({di, dj}, na), rnd(di * dj * na), n, g), gb(Shape({dj, dk}, nb), rnd(dj * dk * nb), n, g);
      const Tensor yr = n.matmul_fw(a.ref, b.ref), yg = g.matmul_fw(a.got, b.got);
      expect_close(yr.to_vector(), yg.to_vector(), tag + " fw", g_mm_tol);
      n.matmul_bw(a.ref, b.ref, yr, gy.ref, ga.ref, gb.ref);
      g.matmul_bw(a.got, b.got, yg, gy.got, ga.got, gb.got);
      expect_close(ga.ref.to_vector(), ga.got.to_vector(), tag + " ga", g_mm_tol);
      expect_close(gb.ref.to_vector(), gb.got.to_vector(), tag + " gb", g_mm_tol);
      if (na == 1) expect_replicas_equal(g, ga.got, tag + " ga");
      if (nb == 1) expect_replicas_equal(g, gb.got, tag + " gb");
    }
  }
}

void test_sums(Naive &n, B200Group &g, std::uint32_t batch) {
  const Shape s({5, 7}, batch), s1({5, 7});
  const std::string tag = "batch " + std::to_string(batch);
  Pair x(s, rnd(s.size()), n, g), w(s1, rnd(s1.size()), n, g), gy(s, rnd(s.size()), n, g);
  expect_close(n.batch_sum_fw(x.ref).to_vector(), g.batch_sum_fw(x.got).to_vector(), tag + " batch_sum", g_tol);
  {  // y (no batch) += x (batch)
    Pair y(s1, rnd(s1.size()), n, g);
    n.inplace_add(x.ref, y.ref);
    g.inplace_add(x.got, y.got);
    expect_close(y.ref.to_vector(), y.got.to_vector(), tag + " inplace_add into unbatched", g_tol);
    expect_replicas_equal(g, y.got, tag + " inplace_add");
    n.inplace_subtract(x.ref, y.ref);
    g.inplace_subtract(x.got, y.got);
    expect_close(y.ref.to_vector(), y.got.to_vector(), tag + " inplace_subtract into unbatched", 10 * g_tol);
  }
  {  // y (batch) += w (no batch)
    Pair y(s, rnd(s.size()), n, g);
    n.inplace_add(w.ref, y.ref);
    g.inplace_add(w.got, y.got);
    expect_close(y.ref.to_vector(), y.got.to_vector(), tag + " inplace_add of unbatched", g_tol);
  }
  {  // multiply_bw with a broadcast operand: its gradient is summed over the batch
    const Tensor yr = n.multiply_fw(x.ref, w.ref), yg = g.multiply_fw(x.got, w.got);
    expect_close(yr.to_vector(), yg.to_vector(), tag + " multiply_fw", g_tol);
    Pair gx(s, rnd(s.size()), n, g), gw(s1, rnd(s1.size()), n, g);
    n.multiply_bw(x.ref, w.ref, yr, gy.ref, gx.ref, gw.ref);
    g.multiply_bw(x.got, w.got, yg, gy.got, gx.got, gw.got);
    expect_close(gx.ref.to_vector(), gx.got.to_vector(), tag + " multiply_bw gx", g_tol);
    expect_close(gw.ref.to_vector(), gw.got.to_vector(), tag + " multiply_bw gw (broadcast)", 10 * g_tol);
    expect_replicas_equal(g, gw.got, tag + " multiply_bw gw");
  }
  {  // x + x: both gradients are one tensor
    Pair gx(s, rnd(s.size()), n, g);
    const Tensor yr = n.add_fw(x.ref, x.ref), yg = g.add_fw(x.got, x.got);
    n.add_bw(x.ref, x.ref, yr, gy.ref, gx.ref, gx.ref);
    g.add_bw(x.got, x.got, yg, gy.got, gx.got, gx.got);
    expect_close(gx.ref.to_vector(), gx.got.to_vector(), tag + " add_bw x+x", g_tol);
  }
  {  // slice_bw / pick_bw into an unbatched gradient
    Pair gs(Shape({5, 3}, batch), rnd(15 * batch), n, g), gx(s1, rnd(s1.size()), n, g);
    n.slice_bw(gs.ref, 1, 2, gx.ref);
    g.slice_bw(gs.got, 1, 2, gx.got);
    expect_close(gx.ref.to_vector(), gx.got.to_vector(), tag + " slice_bw into unbatched", 10 * g_tol);
    vector<std::uint32_t> ids(batch);
    for (std::uint32_t i = 0; i < batch; ++i) ids[i] = (i * 3 + 1) % 7;
    Pair gp(Shape({5}, batch), rnd(5 * batch), n, g), gx2(s1, rnd(s1.size()), n, g);
    n.pick_bw(gp.ref, ids, 1, gx2.ref);
    g.pick_bw(gp.got, ids, 1, gx2.got);
    expect_close(gx2.ref.to_vector(), gx2.got.to_vector(), tag + " pick_bw into unbatched", 10 * g_tol);
    expect_close(n.pick_fw(x.ref, ids, 1).to_vector(), g.pick_fw(x.got, ids, 1).to_vector(), tag + " pick_fw per item", g_tol);
    expect_close(n.pick_fw(w.ref, ids, 1).to_vector(), g.pick_fw(w.got, ids, 1).to_vector(), tag + " pick_fw of unbatched", g_tol);
  }
  {  // reads to the host keep the batch order
    const vector<std::uint32_t> ar = x.ref.argmax(1), ag = x.got.argmax(1);
    expect(ar == ag, tag + " argmax");
    const Tensor rs = x.got.reshape(Shape({35}, batch));  // shares the table, other dimensions
    expect_close(n.sum_fw(x.ref.reshape(Shape({35}, batch)), 0).to_vector(), g.sum_fw(rs, 0).to_vector(), tag + " sum of reshaped", 10 * g_tol);
  }
}

// A sum over shards large enough (> 1 MiB in either storage type) for the slice-by-slice form
// that groups of three or more use, with a length that is not a multiple of the slice alignment.
void test_large_sum(Naive &n, B200Group &g) {
  const Shape s({1021, 601}, 5), s1({1021, 601});
  Pair x(s, rnd(s.size()), n, g), y(s1, rnd(s1.size()), n, g);
  n.inplace_add(x.ref, y.ref);
  g.inplace_add(x.got, y.got);
  expect_close(y.ref.to_vector(), y.got.to_vector(), "large inplace_add into unbatched", 10 * g_tol);
  expect_replicas_equal(g, y.got, "large inplace_add");
  expect_close(n.batch_sum_fw(x.ref).to_vector(), g.batch_sum_fw(x.got).to_vector(), "large batch_sum", 10 * g_tol);
}

void test_batch_moves(Naive &n, B200Group &g, std::uint32_t batch) {
  const Shape s({3, 4}, batch);
  const std::string tag = "batch " + std::to_string(batch);
  Pair x(s, rnd(s.size()), n, g);
  for (std::uint32_t lower : {0u, 1u, batch / 2}) {
    for (std::uint32_t upper : {lower + 1, batch}) {
      if (upper <= lower || upper > batch) continue;
      const std::string t2 = tag + " [" + std::to_string(lower) + "," + std::to_string(upper) + ")";
      expect_close(n.batch_slice_fw(x.ref, lower, upper).to_vector(), g.batch_slice_fw(x.got, lower, upper).to_vector(),
                   t2 + " batch_slice_fw", 0.f);
      const Shape sg({3, 4}, upper - lower);
      Pair gy(sg, rnd(sg.size()), n, g), gx(s, rnd(s.size()), n, g);
      n.batch_slice_bw(gy.ref, lower, gx.ref);
      g.batch_slice_bw(gy.got, lower, gx.got);
      expect_close(gx.ref.to_vector(), gx.got.to_vector(), t2 + " batch_slice_bw", g_tol);
    }
  }
  vector<std::uint32_t> ids;
  for (std::uint32_t i = 0; i < batch + 3; ++i) ids.push_back((i * 5 + 2) % batch);
  expect_close(n.batch_pick_fw(x.ref, ids).to_vector(), g.batch_pick_fw(x.got, ids).to_vector(), tag + " batch_pick_fw", 0.f);
  expect_close(n.batch_pick_fw(x.ref, {batch - 1}).to_vector(), g.batch_pick_fw(x.got, {batch - 1}).to_vector(),
               tag + " batch_pick_fw one item", 0.f);
  {
    const Shape sg({3, 4}, static_cast<std::uint32_t>(ids.size()));
    Pair gy(sg, rnd(sg.size()), n, g), gx(s, rnd(s.size()), n, g);
    n.batch_pick_bw(gy.ref, ids, gx.ref);
    g.batch_pick_bw(gy.got, ids, gx.got);
    expect_close(gx.ref.to_vector(), gx.got.to_vector(), tag + " batch_pick_bw", 10 * g_tol);
  }
  {
    Pair a(Shape({3, 4}, 1), rnd(12), n, g), b(Shape({3, 4}, batch), rnd(12 * batch), n, g), c(Shape({3, 4}, 2), rnd(24), n, g);
    expect_close(n.batch_concat_fw({&a.ref, &b.ref, &c.ref, &x.ref}).to_vector(),
                 g.batch_concat_fw({&a.got, &b.got, &c.got, &x.got}).to_vector(), tag + " batch_concat_fw", 0.f);
  }
}

struct Mlp {
  Parameter w1, b1, w2, b2;
  primitiv::optimizers::SGD opt;
  Mlp(const vector<float> &v1, const vector<float> &v2, Device &dev)
      : w1({32, 20}, v1, dev), b1({32}, primitiv::initializers::Constant(0), dev), w2({6, 32}, v2, dev),
        b2({6}, primitiv::initializers::Constant(0), dev), opt(0.1f) {
    opt.add(w1, b1, w2, b2);
  }
  float step(const vector<float> &x, const vector<std::uint32_t> &labels, std::uint32_t batch, Device &dev) {
    Device::set_default(dev);
    Graph gr;
    Graph::set_default(gr);
    const Node in = F::input<Node>(Shape({20}, batch), x, dev);
    const Node h = F::tanh(F::matmul(F::parameter<Node>(w1), in) + F::parameter<Node>(b1));
    const Node y = F::matmul(F::parameter<Node>(w2), F::dropout(h, 0.f, true)) + F::parameter<Node>(b2);
    const Node loss = F::batch::mean(F::softmax_cross_entropy(y, labels, 0));
    const float l = loss.to_float();
    opt.reset_gradients();
    loss.backward();
    opt.update();
    return l;
  }
};

void test_training(Naive &n, B200Group &g, std::uint32_t batch) {
  const vector<float> v1 = rnd(32 * 20, -0.3f, 0.3f), v2 = rnd(6 * 32, -0.3f, 0.3f), x = rnd(20 * batch);
  vector<std::uint32_t> labels(batch);
  for (auto &l : labels) l = g_rng() % 6;
  Mlp ref(v1, v2, n), got(v1, v2, g);
  const std::string tag = "training batch " + std::to_string(batch);
  for (int step = 0; step < 3; ++step) {
    const float lr = ref.step(x, labels, batch, n), lg = got.step(x, labels, batch, g);
    expect(std::fabs(lr - lg) <= 50 * g_mm_tol * std::fabs(lr), tag + " step " + std::to_string(step) + " loss " +
                                                                   std::to_string(lr) + " vs " + std::to_string(lg));
  }
  expect_close(ref.w1.value().to_vector(), got.w1.value().to_vector(), tag + " w1", 50 * g_mm_tol);
  expect_close(ref.w2.value().to_vector(), got.w2.value().to_vector(), tag + " w2", 50 * g_mm_tol);
  expect_close(ref.b1.value().to_vector(), got.b1.value().to_vector(), tag + " b1", 50 * g_mm_tol);
  for (Parameter *p : {&got.w1, &got.b1, &got.w2, &got.b2}) {
    expect_replicas_equal(g, p->value(), tag + " parameter");
    expect_replicas_equal(g, p->gradient(), tag + " gradient");
  }
}

// A bounded wait that ran out on any shard surfaces as primitiv::Error from the group, once
// (the wait here is the library's self-test kernel, which returns normally after a millisecond).
void test_kernel_timeout_is_reported(B200Group &group) {
  const std::uint32_t last = group.num_shards() - 1;
  const Shape s({3, 2}, 2 * group.num_shards());
  vector<float> v(s.size(), 0.25f);
  Tensor t = group.new_tensor_by_vector(s, v);
  auto thrown_by = [&](const std::function<void()> &f) {
    try { f(); } catch (const primitiv::Error &) { return true; }
    return false;
  };
  expect(::b200_selftest_wait_timeout(group.shard(last).context(), nullptr) == 0, "timeout self-test launches");
  expect(thrown_by([&] { t.to_vector(); }), "group to_vector() throws after a shard's kernel gave up waiting");
  expect(!thrown_by([&] { t.to_vector(); }), "the report is delivered once");
  expect(::b200_selftest_wait_timeout(group.shard(0).context(), nullptr) == 0, "timeout self-test launches again");
  expect(thrown_by([&] { group.synchronize(); }), "group synchronize() throws after a shard's kernel gave up waiting");
  expect(!thrown_by([&] { group.synchronize(); }), "and not a second time");
  expect(t.to_vector() == v, "the group still works after the report");
}

}  // namespace

int main(int argc, char **argv) {
  const std::string mode_name = argc > 1 ? argv[1] : "3xtf32";
  const std::string id_list = argc > 2 ? argv[2] : "0,0";
  B200::Mode mode = B200::Mode::FP32_3XTF32;
  if (mode_name == "tf32") { mode = B200::Mode::TF32_FAST; g_mm_tol = 2e-3f; }
  else if (mode_name == "fp16") { mode = B200::Mode::FP16; g_half = true; g_tol = 2e-3f; g_mm_tol = 2e-3f; }
  else if (mode_name == "3xfp16") mode = B200::Mode::FP32_3XFP16;
  else if (mode_name != "3xtf32") { std::cerr << "usage: group_parity <mode> <ordinals>" << std::endl; return 2; }
  vector<std::uint32_t> ids;
  for (char c : id_list) if (c >= '0' && c <= '9') ids.push_back(static_cast<std::uint32_t>(c - '0'));
  try {
    Naive naive(0);
    B200Group group(ids, 7, mode);
    group.dump_description();
    const std::uint32_t shards = group.num_shards();
    for (std::uint32_t batch : {2u, shards, shards + 1, 37u}) {
      if (batch < 2) continue;
      test_matmul(naive, group, batch);
      test_sums(naive, group, batch);
      test_batch_moves(naive, group, batch);
      test_training(naive, group, batch);
    }
    test_large_sum(naive, group);
    group.synchronize();
    test_kernel_timeout_is_reported(group);
    std::printf("{\"mode\": \"%s\", \"shards\": %u, \"checks\": %d, \"failures\": %d, \"cross_gpu_sums\": %llu}\n",
                mode_name.c_str(), shards, g_checks, g_failures, static_cast<unsigned long long>(group.cross_gpu_sums()));
  } catch (const std::exception &e) {
    std::cerr << "EXCEPTION: " << e.what() << std::endl;
    return 3;
  }
  return g_failures == 0 ? 0 : 1;
}
