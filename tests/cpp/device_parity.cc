// Parity of primitiv::devices::B200 against the reference's own Naive device, op by op,
// through primitiv's public Device / Tensor / Graph API.
//
// The reference's device tests (test/tensor_forward_test.cc, tensor_backward_test.cc,
// tensor_test.cc) loop over every available device and hold all of them to the same
// answers.  Here the Naive device, compiled from the reference sources, supplies the
// answers: every operation is run on both devices from the same seeded inputs, all batch
// broadcasting combinations included, and the results are compared.  The Naive device is
// the checker only; the B200 device never touches it.
//
//   device_parity [mode]      mode: 3xtf32 (default) | tf32 | fp16
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
#include <primitiv/core/model.h>
#include <primitiv/core/optimizer_impl.h>
#include <primitiv/core/parameter.h>
#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>
#include <primitiv/devices/naive/device.h>

#include "b200_device.h"
#include "../../include/primitiv_b200.h"

using primitiv::Device;
using primitiv::Shape;
using primitiv::Tensor;
using primitiv::devices::B200;
using primitiv::devices::Naive;
using std::vector;

namespace {

int g_checks = 0, g_failures = 0;
float g_tol = 1e-5f;      // elementwise ops: relative + absolute
float g_mm_tol = 1e-5f;   // matmul: normwise
std::mt19937 g_rng(12345);

vector<float> rnd(std::size_t n, float lo = -1.f, float hi = 1.f) {
  std::uniform_real_distribution<float> d(lo, hi);
  vector<float> v(n);
  for (float &x : v) x = d(g_rng);
  return v;
}

// In fp16 mode the device stores half: give both devices inputs that are exactly
// representable so that the comparison measures the operation, not the storage.
bool g_half = false;
float to_half_grid(float x) {
  if (!g_half) return x;
  int e;
  const float m = std::frexp(x, &e);
  return std::ldexp(std::round(m * 2048.f) / 2048.f, e);
}
vector<float> on_grid(vector<float> v) {
  for (float &x : v) x = to_half_grid(x);
  return v;
}

void expect(bool ok, const std::string &what) {
  ++g_checks;
  if (!ok) {
    ++g_failures;
    std::cerr << "FAIL: " << what << std::endl;
  }
}

void expect_close(const vector<float> &want, const vector<float> &got, const std::string &what, float tol) {
  ++g_checks;
  if (want.size() != got.size()) {
    ++g_failures;
    std::cerr << "FAIL: " << what << ": size " << got.size() << " != " << want.size() << std::endl;
    return;
  }
  for (std::size_t i = 0; i < want.size(); ++i) {
    const float err = std::fabs(want[i] - got[i]);
    const float lim = tol * (1.f + std::fabs(want[i]));
    if (!(err <= lim)) {
      ++g_failures;
      std::cerr << "FAIL: " << what << ": [" << i << "] want " << want[i] << " got " << got[i] << std::endl;
      return;
    }
  }
}

void expect_normwise(const vector<float> &want, const vector<float> &got, const std::string &what, float tol) {
  ++g_checks;
  double num = 0, den = 0;
  if (want.size() != got.size()) { ++g_failures; std::cerr << "FAIL: " << what << ": size" << std::endl; return; }
  for (std::size_t i = 0; i < want.size(); ++i) {
    const double d = double(want[i]) - got[i];
    num += d * d;
    den += double(want[i]) * want[i];
  }
  const double rel = den > 0 ? std::sqrt(num / den) : std::sqrt(num);
  if (!(rel <= tol)) {
    ++g_failures;
    std::cerr << "FAIL: " << what << ": normwise error " << rel << " > " << tol << std::endl;
  }
}

struct Pair {
  Naive naive;
  B200 dev;
  explicit Pair(B200::Mode m) : naive(7), dev(0, 7, m) {}
  Tensor on(Device &d, const Shape &s, const vector<float> &v) { return d.new_tensor_by_vector(s, v); }
};

const std::uint32_t kBatches[4][2] = {{1, 1}, {3, 3}, {1, 3}, {3, 1}};

// ---------------------------------------------------------------------------------------------

void test_memory_and_io(Pair &p) {
  const Shape s({5, 3}, 2);
  const vector<float> v = on_grid(rnd(s.size()));
  Tensor t = p.dev.new_tensor_by_vector(s, v);
  expect(t.valid() && &t.device() == &p.dev, "tensor belongs to the B200 device");
  expect_close(v, t.to_vector(), "upload/download round trip", 0.f);
  Tensor c = p.dev.new_tensor_by_constant(Shape({7}, 3), 2.5f);
  expect_close(vector<float>(21, 2.5f), c.to_vector(), "new_tensor_by_constant", 0.f);
  // copy between devices, both directions, and on the device
  Tensor from_naive = p.dev.copy_tensor(p.naive.new_tensor_by_vector(s, v));
  expect_close(v, from_naive.to_vector(), "copy_tensor Naive -> B200", 0.f);
  Tensor to_naive = p.naive.copy_tensor(t);
  expect_close(v, to_naive.to_vector(), "copy_tensor B200 -> Naive", 0.f);
  Tensor same = p.dev.copy_tensor(t);
  expect_close(v, same.to_vector(), "copy_tensor B200 -> B200", 0.f);
  // copy-on-write: a copy of the Tensor object shares the handle until one side is written
  Tensor alias = t;
  alias.reset(1.f);
  expect_close(v, t.to_vector(), "copy-on-write keeps the original", 0.f);
  expect_close(vector<float>(s.size(), 1.f), alias.to_vector(), "copy-on-write writes the clone", 0.f);
  // reshape / flatten share the handle
  expect_close(v, t.reshape(Shape({15}, 2)).to_vector(), "reshape", 0.f);
  expect_close(v, t.flatten().to_vector(), "flatten", 0.f);
  expect_close(p.naive.identity(4).to_vector(), p.dev.identity(4).to_vector(), "identity", 0.f);
  // scalar read-back
  expect(p.dev.new_tensor_by_constant({}, 3.f).to_float() == 3.f, "to_float");
  // a tensor may outlive its device; destroying it afterwards must be safe
  Tensor orphan;
  {
    B200 shortlived(0, 1, p.dev.mode());
    orphan = shortlived.new_tensor_by_constant({4}, 1.f);
  }
  orphan = Tensor();
  expect(true, "tensor outliving its device is destroyed safely");
  bool threw = false;
  try { B200 bad(12345); } catch (const primitiv::Error &) { threw = true; }
  expect(threw, "invalid device id throws primitiv::Error");
}

typedef Tensor (Device::*FwX)(const Tensor &);
typedef void (Device::*BwX)(const Tensor &, const Tensor &, const Tensor &, Tensor &);
typedef Tensor (Device::*FwXC)(const Tensor &, float);
typedef void (Device::*BwXC)(const Tensor &, const Tensor &, const Tensor &, float, Tensor &);
typedef Tensor (Device::*FwXS)(const Tensor &, const Tensor &);
typedef void (Device::*BwAB)(const Tensor &, const Tensor &, const Tensor &, const Tensor &, Tensor &, Tensor &);

void test_unary(Pair &p) {
  struct Case { const char *name; FwX fw; BwX bw; float lo, hi; };
  const Case cases[] = {
    {"negate", &Device::negate_fw, nullptr, -2, 2},   {"abs", &Device::abs_fw, &Device::abs_bw, -2, 2},
    {"sqrt", &Device::sqrt_fw, &Device::sqrt_bw, .1f, 4}, {"exp", &Device::exp_fw, &Device::exp_bw, -2, 2},
    {"log", &Device::log_fw, &Device::log_bw, .1f, 4}, {"tanh", &Device::tanh_fw, &Device::tanh_bw, -2, 2},
    {"sigmoid", &Device::sigmoid_fw, &Device::sigmoid_bw, -3, 3},
    {"softplus", &Device::softplus_fw, &Device::softplus_bw, -3, 3},
    {"sin", &Device::sin_fw, &Device::sin_bw, -3, 3}, {"cos", &Device::cos_fw, &Device::cos_bw, -3, 3},
    {"tan", &Device::tan_fw, &Device::tan_bw, -1, 1},
  };
  for (const Shape &s : {Shape({5, 3}, 2), Shape({129}, 1), Shape({8, 4, 2}, 3)}) {
    for (const Case &c : cases) {
      const vector<float> xv = on_grid(rnd(s.size(), c.lo, c.hi)), gv = on_grid(rnd(s.size()));
      vector<float> ys[2], gxs[2];
      Device *devs[2] = {&p.naive, &p.dev};
      for (int d = 0; d < 2; ++d) {
        Tensor x = p.on(*devs[d], s, xv), gy = p.on(*devs[d], s, gv);
        Tensor y = (devs[d]->*c.fw)(x);
        ys[d] = y.to_vector();
        if (c.bw) {
          Tensor gx = devs[d]->new_tensor_by_constant(s, g_half ? 0.5f : 0.25f);
          (devs[d]->*c.bw)(x, y, gy, gx);
          gxs[d] = gx.to_vector();
        }
      }
      expect_close(ys[0], ys[1], std::string(c.name) + "_fw " + s.to_string(), g_tol);
      if (c.bw) expect_close(gxs[0], gxs[1], std::string(c.name) + "_bw " + s.to_string(), g_tol * 4);
    }
  }
}

void test_const_ops(Pair &p) {
  struct Case { const char *name; FwXC fw; BwXC bw; float lo, hi, k; };
  const Case cases[] = {
    {"add_const", &Device::add_const_fw, &Device::add_const_bw, -2, 2, 1.5f},
    {"subtract_const_r", &Device::subtract_const_r_fw, &Device::subtract_const_r_bw, -2, 2, 1.5f},
    {"subtract_const_l", &Device::subtract_const_l_fw, &Device::subtract_const_l_bw, -2, 2, 1.5f},
    {"multiply_const", &Device::multiply_const_fw, &Device::multiply_const_bw, -2, 2, -0.75f},
    {"divide_const_r", &Device::divide_const_r_fw, &Device::divide_const_r_bw, -2, 2, 4.f},
    {"divide_const_l", &Device::divide_const_l_fw, &Device::divide_const_l_bw, .5f, 2, 3.f},
    {"pow_const_r", &Device::pow_const_r_fw, &Device::pow_const_r_bw, .5f, 2, 2.5f},
    {"pow_const_l", &Device::pow_const_l_fw, &Device::pow_const_l_bw, -2, 2, 1.5f},
    {"prelu", &Device::prelu_fw, &Device::prelu_bw, -2, 2, .25f},
    {"elu", &Device::elu_fw, &Device::elu_bw, -2, 2, 1.5f},
  };
  const Shape s({6, 5}, 3);
  Device *devs[2] = {&p.naive, &p.dev};
  for (const Case &c : cases) {
    const vector<float> xv = on_grid(rnd(s.size(), c.lo, c.hi)), gv = on_grid(rnd(s.size()));
    vector<float> ys[2], gxs[2];
    for (int d = 0; d < 2; ++d) {
      Tensor x = p.on(*devs[d], s, xv), gy = p.on(*devs[d], s, gv);
      Tensor y = (devs[d]->*c.fw)(x, c.k);
      Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
      (devs[d]->*c.bw)(x, y, gy, c.k, gx);
      ys[d] = y.to_vector();
      gxs[d] = gx.to_vector();
    }
    expect_close(ys[0], ys[1], std::string(c.name) + "_fw", g_tol);
    expect_close(gxs[0], gxs[1], std::string(c.name) + "_bw", g_tol * 4);
  }
  for (std::int32_t k : {3, -2, 0}) {
    const vector<float> xv = on_grid(rnd(s.size(), .5f, 2)), gv = on_grid(rnd(s.size()));
    vector<float> ys[2], gxs[2];
    for (int d = 0; d < 2; ++d) {
      Tensor x = p.on(*devs[d], s, xv), gy = p.on(*devs[d], s, gv);
      Tensor y = devs[d]->pown_fw(x, k);
      Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
      devs[d]->pown_bw(x, y, gy, k, gx);
      ys[d] = y.to_vector();
      gxs[d] = gx.to_vector();
    }
    expect_close(ys[0], ys[1], "pown_fw k=" + std::to_string(k), g_tol * 2);
    expect_close(gxs[0], gxs[1], "pown_bw k=" + std::to_string(k), g_tol * 8);
  }
}

void test_scalar_and_binary(Pair &p) {
  struct SCase { const char *name; FwXS fw; float lo, hi; };
  const SCase scalars[] = {
    {"add_scalar", &Device::add_scalar_fw, -2, 2}, {"subtract_scalar_r", &Device::subtract_scalar_r_fw, -2, 2},
    {"subtract_scalar_l", &Device::subtract_scalar_l_fw, -2, 2}, {"multiply_scalar", &Device::multiply_scalar_fw, -2, 2},
    {"divide_scalar_r", &Device::divide_scalar_r_fw, .5f, 2}, {"divide_scalar_l", &Device::divide_scalar_l_fw, .5f, 2},
    {"pow_scalar_r", &Device::pow_scalar_r_fw, .5f, 2}, {"pow_scalar_l", &Device::pow_scalar_l_fw, .5f, 2},
  };
  struct BCase { const char *name; FwXS fw; BwAB bw; float lo, hi; };
  const BCase binaries[] = {
    {"add", &Device::add_fw, &Device::add_bw, -2, 2}, {"subtract", &Device::subtract_fw, &Device::subtract_bw, -2, 2},
    {"multiply", &Device::multiply_fw, &Device::multiply_bw, -2, 2},
    {"divide", &Device::divide_fw, &Device::divide_bw, .5f, 2}, {"pow", &Device::pow_fw, &Device::pow_bw, .5f, 2},
  };
  Device *devs[2] = {&p.naive, &p.dev};
  for (const auto &bb : kBatches) {
    const Shape sx({4, 3}, bb[0]), sk({}, bb[1]), sb({4, 3}, bb[1]);
    const Shape sy({4, 3}, std::max(bb[0], bb[1]));
    const std::string tag = " x" + std::to_string(bb[0]) + "," + std::to_string(bb[1]);
    for (const SCase &c : scalars) {
      const vector<float> xv = on_grid(rnd(sx.size(), c.lo, c.hi)), kv = on_grid(rnd(sk.size(), c.lo, c.hi));
      vector<float> ys[2];
      for (int d = 0; d < 2; ++d) ys[d] = (devs[d]->*c.fw)(p.on(*devs[d], sx, xv), p.on(*devs[d], sk, kv)).to_vector();
      expect_close(ys[0], ys[1], std::string(c.name) + "_fw" + tag, g_tol);
    }
    for (const BCase &c : binaries) {
      const vector<float> av = on_grid(rnd(sx.size(), c.lo, c.hi)), bv = on_grid(rnd(sb.size(), c.lo, c.hi));
      const vector<float> gv = on_grid(rnd(sy.size()));
      vector<float> ys[2], gas[2], gbs[2];
      for (int d = 0; d < 2; ++d) {
        Tensor a = p.on(*devs[d], sx, av), b = p.on(*devs[d], sb, bv), gy = p.on(*devs[d], sy, gv);
        Tensor y = (devs[d]->*c.fw)(a, b);
        Tensor ga = devs[d]->new_tensor_by_constant(sx, 0.5f), gb = devs[d]->new_tensor_by_constant(sb, 0.5f);
        (devs[d]->*c.bw)(a, b, y, gy, ga, gb);
        ys[d] = y.to_vector(); gas[d] = ga.to_vector(); gbs[d] = gb.to_vector();
      }
      expect_close(ys[0], ys[1], std::string(c.name) + "_fw" + tag, g_tol);
      expect_close(gas[0], gas[1], std::string(c.name) + "_bw ga" + tag, g_tol * 8);
      expect_close(gbs[0], gbs[1], std::string(c.name) + "_bw gb" + tag, g_tol * 8);
    }
  }
}

void test_matmul(Pair &p) {
  Device *devs[2] = {&p.naive, &p.dev};
  struct Dim { std::uint32_t di, dj, dk; };
  for (int policy : {0, 2}) {
    p.dev.set_matmul_path_policy(policy);
    for (const Dim &dm : {Dim{2, 2, 2}, Dim{3, 4, 6}, Dim{64, 48, 40}, Dim{136, 72, 104}, Dim{123, 123, 123}}) {
      if (g_half && policy == 2 && (dm.di % 8 || dm.dj % 8)) continue;  // half operands are never repacked
      for (const auto &bb : kBatches) {
        const std::uint32_t bs = std::max(bb[0], bb[1]);
        const Shape sa({dm.di, dm.dj}, bb[0]), sb({dm.dj, dm.dk}, bb[1]), sy({dm.di, dm.dk}, bs);
        const vector<float> av = on_grid(rnd(sa.size())), bv = on_grid(rnd(sb.size())), gv = on_grid(rnd(sy.size()));
        vector<float> ys[2], gas[2], gbs[2];
        for (int d = 0; d < 2; ++d) {
          Tensor a = p.on(*devs[d], sa, av), b = p.on(*devs[d], sb, bv), gy = p.on(*devs[d], sy, gv);
          Tensor y = devs[d]->matmul_fw(a, b);
          Tensor ga = devs[d]->new_tensor_by_constant(sa, 0.5f), gb = devs[d]->new_tensor_by_constant(sb, 0.5f);
          devs[d]->matmul_bw(a, b, y, gy, ga, gb);
          ys[d] = y.to_vector(); gas[d] = ga.to_vector(); gbs[d] = gb.to_vector();
        }
        const std::string tag = " " + sa.to_string() + " . " + sb.to_string() + " policy " + std::to_string(policy);
        expect_normwise(ys[0], ys[1], "matmul_fw" + tag, g_mm_tol);
        expect_normwise(gas[0], gas[1], "matmul_bw ga" + tag, g_mm_tol);
        expect_normwise(gbs[0], gbs[1], "matmul_bw gb" + tag, g_mm_tol);
      }
    }
  }
  p.dev.set_matmul_path_policy(0);
  // the shape checks stay with the base class: an invalid product throws before any kernel runs
  bool threw = false;
  try { p.dev.matmul_fw(p.dev.new_tensor_by_constant({2, 3}, 0), p.dev.new_tensor_by_constant({2, 3}, 0)); }
  catch (const primitiv::Error &) { threw = true; }
  expect(threw, "matmul of {2,3} and {2,3} throws");
}

void test_movement(Pair &p) {
  Device *devs[2] = {&p.naive, &p.dev};
  const Shape s({4, 3, 5}, 2);
  const vector<float> xv = on_grid(rnd(s.size()));
  for (std::uint32_t dim = 0; dim < 4; ++dim) {
    // slice fw / bw
    const std::uint32_t n = s[dim];
    const std::uint32_t lo = n > 1 ? 1 : 0, hi = n;
    vector<float> ys[2], gxs[2], gxs1[2];
    for (int d = 0; d < 2; ++d) {
      Tensor x = p.on(*devs[d], s, xv);
      Tensor y = devs[d]->slice_fw(x, dim, lo, hi);
      ys[d] = y.to_vector();
      Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
      devs[d]->slice_bw(y, dim, lo, gx);
      gxs[d] = gx.to_vector();
      Tensor gx1 = devs[d]->new_tensor_by_constant(Shape({4, 3, 5}), 0.5f);  // gradient without batch: summed
      devs[d]->slice_bw(y, dim, lo, gx1);
      gxs1[d] = gx1.to_vector();
    }
    expect_close(ys[0], ys[1], "slice_fw dim " + std::to_string(dim), 0.f);
    expect_close(gxs[0], gxs[1], "slice_bw dim " + std::to_string(dim), g_tol);
    expect_close(gxs1[0], gxs1[1], "slice_bw (batch-summed) dim " + std::to_string(dim), g_tol);
    // flip
    for (int d = 0; d < 2; ++d) {
      Tensor x = p.on(*devs[d], s, xv);
      ys[d] = devs[d]->flip_fw(x, dim).to_vector();
      Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
      devs[d]->flip_bw(x, dim, gx);
      gxs[d] = gx.to_vector();
    }
    expect_close(ys[0], ys[1], "flip_fw dim " + std::to_string(dim), 0.f);
    expect_close(gxs[0], gxs[1], "flip_bw dim " + std::to_string(dim), g_tol);
    // sum / logsumexp / max / min fw, max / min bw, argmax / argmin
    for (int d = 0; d < 2; ++d) ys[d] = devs[d]->sum_fw(p.on(*devs[d], s, xv), dim).to_vector();
    expect_close(ys[0], ys[1], "sum_fw dim " + std::to_string(dim), g_tol * 4);
    for (int d = 0; d < 2; ++d) ys[d] = devs[d]->logsumexp_fw(p.on(*devs[d], s, xv), dim).to_vector();
    expect_close(ys[0], ys[1], "logsumexp_fw dim " + std::to_string(dim), g_tol * 4);
    for (int which = 0; which < 2; ++which) {
      vector<std::uint32_t> ids[2];
      for (int d = 0; d < 2; ++d) {
        Tensor x = p.on(*devs[d], s, xv);
        Tensor y = which ? devs[d]->max_fw(x, dim) : devs[d]->min_fw(x, dim);
        ys[d] = y.to_vector();
        Tensor gy = devs[d]->new_tensor_by_constant(y.shape(), 2.f);
        Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
        if (which) devs[d]->max_bw(x, y, gy, dim, gx); else devs[d]->min_bw(x, y, gy, dim, gx);
        gxs[d] = gx.to_vector();
        ids[d] = which ? x.argmax(dim) : x.argmin(dim);
      }
      const std::string nm = which ? "max" : "min";
      expect_close(ys[0], ys[1], nm + "_fw dim " + std::to_string(dim), 0.f);
      expect_close(gxs[0], gxs[1], nm + "_bw dim " + std::to_string(dim), g_tol);
      expect(ids[0] == ids[1], "arg" + nm + " dim " + std::to_string(dim));
    }
    // broadcast along a dimension of extent 1
    Shape s1 = s;
    s1.update_dim(dim, 1);
    const vector<float> v1 = on_grid(rnd(s1.size()));
    for (int d = 0; d < 2; ++d) ys[d] = devs[d]->broadcast_fw(p.on(*devs[d], s1, v1), dim, 3).to_vector();
    expect_close(ys[0], ys[1], "broadcast_fw dim " + std::to_string(dim), 0.f);
  }
  // long reduction along the leading dimension (the softmax case): warp-per-output path
  {
    const Shape big({300, 7}, 5);
    const vector<float> bv = on_grid(rnd(big.size()));
    vector<float> ys[2];
    for (int d = 0; d < 2; ++d) ys[d] = devs[d]->logsumexp_fw(p.on(*devs[d], big, bv), 0).to_vector();
    expect_close(ys[0], ys[1], "logsumexp_fw 300-long", g_tol * 8);
    for (int d = 0; d < 2; ++d) ys[d] = devs[d]->sum_fw(p.on(*devs[d], big, bv), 0).to_vector();
    expect_close(ys[0], ys[1], "sum_fw 300-long", g_tol * 32);
    for (int d = 0; d < 2; ++d) ys[d] = devs[d]->max_fw(p.on(*devs[d], big, bv), 0).to_vector();
    expect_close(ys[0], ys[1], "max_fw 300-long", 0.f);
  }
  // pick fw / bw with one id and with one id per batch, repeated ids included
  for (std::uint32_t dim = 0; dim < 3; ++dim) {
    for (const vector<std::uint32_t> &ids : {vector<std::uint32_t>{1}, vector<std::uint32_t>{2, 2}}) {
      for (const Shape &sx : {s, Shape({4, 3, 5})}) {
        vector<float> ys[2], gxs[2];
        const vector<float> v = on_grid(rnd(sx.size()));
        for (int d = 0; d < 2; ++d) {
          Tensor x = p.on(*devs[d], sx, v);
          Tensor y = devs[d]->pick_fw(x, ids, dim);
          ys[d] = y.to_vector();
          Tensor gx = devs[d]->new_tensor_by_constant(sx, 0.5f);
          devs[d]->pick_bw(y, ids, dim, gx);
          gxs[d] = gx.to_vector();
        }
        expect_close(ys[0], ys[1], "pick_fw dim " + std::to_string(dim), 0.f);
        expect_close(gxs[0], gxs[1], "pick_bw dim " + std::to_string(dim), g_tol);
      }
    }
  }
  // concat along each dimension, mixing batched and broadcast inputs
  for (std::uint32_t dim = 0; dim < 3; ++dim) {
    Shape sa({4, 3, 5}, 2), sb({4, 3, 5}, 1);
    sb.update_dim(dim, 2);
    const vector<float> av = on_grid(rnd(sa.size())), bv = on_grid(rnd(sb.size()));
    vector<float> ys[2];
    for (int d = 0; d < 2; ++d) {
      Tensor a = p.on(*devs[d], sa, av), b = p.on(*devs[d], sb, bv);
      ys[d] = devs[d]->concat_fw({&a, &b, &a}, dim).to_vector();
    }
    expect_close(ys[0], ys[1], "concat_fw dim " + std::to_string(dim), 0.f);
  }
  // transpose and permute_dims
  {
    const Shape st({37, 50}, 3);
    const vector<float> v = on_grid(rnd(st.size()));
    vector<float> ys[2], gxs[2];
    for (int d = 0; d < 2; ++d) {
      Tensor x = p.on(*devs[d], st, v);
      Tensor y = devs[d]->transpose_fw(x);
      ys[d] = y.to_vector();
      Tensor gx = devs[d]->new_tensor_by_constant(st, 0.5f);
      devs[d]->transpose_bw(x, y, y, gx);
      gxs[d] = gx.to_vector();
    }
    expect_close(ys[0], ys[1], "transpose_fw", 0.f);
    expect_close(gxs[0], gxs[1], "transpose_bw", g_tol);
    for (const vector<std::uint32_t> &perm : {vector<std::uint32_t>{2, 0, 1}, vector<std::uint32_t>{1, 0, 2}}) {
      for (int d = 0; d < 2; ++d) {
        Tensor x = p.on(*devs[d], s, xv);
        Tensor y = devs[d]->permute_dims_fw(x, perm);
        ys[d] = y.to_vector();
        Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
        devs[d]->permute_dims_bw(x, y, y, perm, gx);
        gxs[d] = gx.to_vector();
      }
      expect_close(ys[0], ys[1], "permute_dims_fw", 0.f);
      expect_close(gxs[0], gxs[1], "permute_dims_bw", g_tol);
    }
  }
}

void test_batch_ops_and_inplace(Pair &p) {
  Device *devs[2] = {&p.naive, &p.dev};
  const Shape s({3, 4}, 5);
  const vector<float> xv = on_grid(rnd(s.size()));
  vector<float> ys[2], gxs[2];
  const vector<std::uint32_t> ids{4, 0, 0, 2};
  for (int d = 0; d < 2; ++d) {
    Tensor x = p.on(*devs[d], s, xv);
    Tensor y = devs[d]->batch_pick_fw(x, ids);
    ys[d] = y.to_vector();
    Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
    devs[d]->batch_pick_bw(y, ids, gx);
    gxs[d] = gx.to_vector();
  }
  expect_close(ys[0], ys[1], "batch_pick_fw", 0.f);
  expect_close(gxs[0], gxs[1], "batch_pick_bw (repeated ids)", g_tol);
  for (int d = 0; d < 2; ++d) {
    Tensor x = p.on(*devs[d], s, xv);
    Tensor y = devs[d]->batch_slice_fw(x, 1, 4);
    ys[d] = y.to_vector();
    Tensor gx = devs[d]->new_tensor_by_constant(s, 0.5f);
    devs[d]->batch_slice_bw(y, 1, gx);
    gxs[d] = gx.to_vector();
  }
  expect_close(ys[0], ys[1], "batch_slice_fw", 0.f);
  expect_close(gxs[0], gxs[1], "batch_slice_bw", g_tol);
  for (int d = 0; d < 2; ++d) {
    Tensor x = p.on(*devs[d], s, xv), z = p.on(*devs[d], Shape({3, 4}), on_grid(vector<float>(12, 0.125f)));
    ys[d] = devs[d]->batch_concat_fw({&x, &z, &x}).to_vector();
    gxs[d] = devs[d]->batch_sum_fw(x).to_vector();
  }
  expect_close(ys[0], ys[1], "batch_concat_fw", 0.f);
  expect_close(gxs[0], gxs[1], "batch_sum_fw", g_tol * 4);
  // in-place add / subtract with every batch combination (a batch-1 destination receives the sum)
  for (const auto &bb : kBatches) {
    const Shape sx({3, 4}, bb[0]), sy({3, 4}, bb[1]);
    const vector<float> a = on_grid(rnd(sx.size())), b = on_grid(rnd(sy.size()));
    for (int sign = 0; sign < 2; ++sign) {
      for (int d = 0; d < 2; ++d) {
        Tensor x = p.on(*devs[d], sx, a), y = p.on(*devs[d], sy, b);
        if (sign) y.inplace_subtract(x); else y.inplace_add(x);
        y.inplace_multiply_const(-1.5f);
        ys[d] = y.to_vector();
      }
      expect_close(ys[0], ys[1], std::string(sign ? "inplace_subtract" : "inplace_add") + " + scale", g_tol * 4);
    }
  }
}

// Sums over the batch in their large forms: volumes that take the 128-bit vector kernels (a multiple
// of 8 elements, at least 256), ragged ones that do not, batches long enough to be cut into slices,
// and a tiny volume under a very long batch (hundreds of slices, combined by the warp form of the
// final pass).  Binary operators with one broadcast operand, batch::sum, and in-place addition
// into a batch-1 tensor all go through them.
void test_large_batch_sums(Pair &p) {
  Device *devs[2] = {&p.naive, &p.dev};
  struct BCase { const char *name; FwXS fw; BwAB bw; float lo, hi; };
  const BCase binaries[] = {
    {"add", &Device::add_fw, &Device::add_bw, -2, 2}, {"subtract", &Device::subtract_fw, &Device::subtract_bw, -2, 2},
    {"multiply", &Device::multiply_fw, &Device::multiply_bw, -2, 2},
    {"divide", &Device::divide_fw, &Device::divide_bw, .5f, 2}, {"pow", &Device::pow_fw, &Device::pow_bw, .5f, 2},
  };
  struct Dim { std::uint32_t rows, cols, batch; };
  const Dim dims[] = {{40, 8, 70}, {33, 5, 300}, {64, 16, 300}, {8, 1, 16384}};
  for (const Dim &dm : dims) {
    for (int which = 0; which < 2; ++which) {   // which operand is broadcast
      const Shape sa({dm.rows, dm.cols}, which == 0 ? 1 : dm.batch), sb({dm.rows, dm.cols}, which == 0 ? dm.batch : 1);
      const Shape sy({dm.rows, dm.cols}, dm.batch);
      const std::string tag = " " + std::to_string(dm.rows) + "x" + std::to_string(dm.cols) + " batch " +
                              std::to_string(dm.batch) + (which == 0 ? " (a broadcast)" : " (b broadcast)");
      for (const BCase &c : binaries) {
        const vector<float> av = on_grid(rnd(sa.size(), c.lo, c.hi)), bv = on_grid(rnd(sb.size(), c.lo, c.hi));
        const vector<float> gv = on_grid(rnd(sy.size()));
        vector<float> gas[2], gbs[2];
        for (int d = 0; d < 2; ++d) {
          Tensor a = p.on(*devs[d], sa, av), b = p.on(*devs[d], sb, bv), gy = p.on(*devs[d], sy, gv);
          Tensor y = (devs[d]->*c.fw)(a, b);
          Tensor ga = devs[d]->new_tensor_by_constant(sa, 0.5f), gb = devs[d]->new_tensor_by_constant(sb, 0.5f);
          (devs[d]->*c.bw)(a, b, y, gy, ga, gb);
          gas[d] = ga.to_vector(); gbs[d] = gb.to_vector();
        }
        // a sum of `batch` terms: the tolerance grows with its square root
        const float t = g_tol * 8 * std::sqrt(static_cast<float>(dm.batch));
        expect_normwise(gas[0], gas[1], std::string(c.name) + "_bw ga" + tag, t);
        expect_normwise(gbs[0], gbs[1], std::string(c.name) + "_bw gb" + tag, t);
      }
    }
    const Shape s({dm.rows, dm.cols}, dm.batch), s1({dm.rows, dm.cols}, 1);
    const vector<float> xv = on_grid(rnd(s.size())), zv = on_grid(rnd(s1.size()));
    vector<float> sums[2], adds[2];
    for (int d = 0; d < 2; ++d) {
      Tensor x = p.on(*devs[d], s, xv), z = p.on(*devs[d], s1, zv);
      sums[d] = devs[d]->batch_sum_fw(x).to_vector();
      z.inplace_add(x);
      adds[d] = z.to_vector();
    }
    const float t = g_tol * 8 * std::sqrt(static_cast<float>(dm.batch));
    const std::string tag = " " + std::to_string(dm.rows) + "x" + std::to_string(dm.cols) + " batch " + std::to_string(dm.batch);
    expect_normwise(sums[0], sums[1], "batch_sum_fw" + tag, t);
    expect_normwise(adds[0], adds[1], "inplace_add into batch 1" + tag, t);
  }
}

void test_random(Pair &p) {
  const Shape s({1000, 100});
  const vector<float> u = p.dev.random_uniform(s, -2.f, 3.f).to_vector();
  double mean = 0, mn = 1e9, mx = -1e9;
  for (float v : u) { mean += v; mn = std::min<double>(mn, v); mx = std::max<double>(mx, v); }
  mean /= u.size();
  expect(mn > -2.0 - 1e-3 && mx <= 3.0 + 1e-3 && std::fabs(mean - 0.5) < 0.02, "random_uniform range and mean");
  const vector<float> nrm = p.dev.random_normal(s, 1.f, 2.f).to_vector();
  double m1 = 0, m2 = 0;
  for (float v : nrm) m1 += v;
  m1 /= nrm.size();
  for (float v : nrm) m2 += (v - m1) * (v - m1);
  expect(std::fabs(m1 - 1.0) < 0.03 && std::fabs(std::sqrt(m2 / nrm.size()) - 2.0) < 0.03, "random_normal moments");
  const vector<float> ber = p.dev.random_bernoulli(s, 0.3f).to_vector();
  double ones = 0;
  bool binary = true;
  for (float v : ber) { ones += v; binary = binary && (v == 0.f || v == 1.f); }
  expect(binary && std::fabs(ones / ber.size() - 0.3) < 0.01, "random_bernoulli values and rate");
  const vector<float> ln = p.dev.random_log_normal(Shape({1000}), 0.f, 0.5f).to_vector();
  bool pos = true;
  for (float v : ln) pos = pos && v > 0.f;
  expect(pos, "random_log_normal positive");
  // same seed, same sequence; successive fills differ
  B200 d1(0, 99, p.dev.mode()), d2(0, 99, p.dev.mode());
  const vector<float> a = d1.random_uniform(Shape({257}), 0, 1).to_vector();
  const vector<float> b = d2.random_uniform(Shape({257}), 0, 1).to_vector();
  const vector<float> c = d2.random_uniform(Shape({257}), 0, 1).to_vector();
  expect(a == b && b != c, "random fills are a function of (seed, call order)");
}

// conv2d and max_pool2d against Naive: paddings, strides, dilations, every batch broadcast
// combination of x and w (primitiv/test/tensor_forward_test.cc:3103-3692, 3702-4068 run the
// same sweeps against hard-coded answers), gradients accumulated into non-zero tensors, pooling
// with ties and overlapping windows.
void test_conv_and_pool(Pair &p) {
  Device *devs[2] = {&p.naive, &p.dev};
  struct Conv { std::uint32_t p0, p1, s0, s1, d0, d1; };
  const Conv convs[] = {{0, 0, 1, 1, 1, 1}, {1, 2, 1, 1, 1, 1}, {0, 1, 2, 1, 1, 1}, {2, 0, 1, 2, 2, 1},
                        {1, 1, 2, 2, 1, 2}, {3, 3, 3, 2, 2, 2}};
  for (const Conv &c : convs) {
    for (const auto &bb : kBatches) {
      const Shape sx({7, 6, 3}, bb[0]), sw({3, 2, 3, 4}, bb[1]);
      const vector<float> xv = on_grid(rnd(sx.size())), wv = on_grid(rnd(sw.size()));
      vector<float> ys[2], gxs[2], gws[2];
      Shape sy;
      for (int d = 0; d < 2; ++d) {
        Device &dev = *devs[d];
        Tensor x = p.on(dev, sx, xv), w = p.on(dev, sw, wv);
        Tensor y = dev.conv2d_fw(x, w, c.p0, c.p1, c.s0, c.s1, c.d0, c.d1);
        sy = y.shape();
        std::mt19937 local(99);
        std::uniform_real_distribution<float> dist(-1.f, 1.f);
        vector<float> gv(sy.size());
        for (float &v : gv) v = to_half_grid(dist(local));
        Tensor gy = p.on(dev, sy, gv);
        Tensor gx = dev.new_tensor_by_constant(sx, 0.5f), gw = dev.new_tensor_by_constant(sw, 0.25f);
        dev.conv2d_bw(x, w, y, gy, c.p0, c.p1, c.s0, c.s1, c.d0, c.d1, gx, gw);
        ys[d] = y.to_vector(); gxs[d] = gx.to_vector(); gws[d] = gw.to_vector();
      }
      const std::string tag = " pad " + std::to_string(c.p0) + "," + std::to_string(c.p1) + " stride " +
                              std::to_string(c.s0) + "," + std::to_string(c.s1) + " dilation " +
                              std::to_string(c.d0) + "," + std::to_string(c.d1) + " batches " +
                              std::to_string(bb[0]) + "," + std::to_string(bb[1]);
      expect_normwise(ys[0], ys[1], "conv2d_fw" + tag, g_mm_tol);
      expect_normwise(gxs[0], gxs[1], "conv2d_bw gx" + tag, g_mm_tol);
      expect_normwise(gws[0], gws[1], "conv2d_bw gw" + tag, g_mm_tol);
    }
  }
  {
    // a convolution big enough for the tensor-core kernel: 32 x 32 x 16 image, 3 x 3 x 16 x 32 kernel, batch 4
    const Shape sx({32, 32, 16}, 4), sw({3, 3, 16, 32});
    const vector<float> xv = on_grid(rnd(sx.size())), wv = on_grid(rnd(sw.size(), -.2f, .2f));
    vector<float> ys[2], gxs[2], gws[2];
    for (int d = 0; d < 2; ++d) {
      Device &dev = *devs[d];
      Tensor x = p.on(dev, sx, xv), w = p.on(dev, sw, wv);
      Tensor y = dev.conv2d_fw(x, w, 1, 1, 1, 1, 1, 1);
      Tensor gy = dev.new_tensor_by_constant(y.shape(), 0.125f);
      Tensor gx = dev.new_tensor_by_constant(sx, 0), gw = dev.new_tensor_by_constant(sw, 0);
      dev.conv2d_bw(x, w, y, gy, 1, 1, 1, 1, 1, 1, gx, gw);
      ys[d] = y.to_vector(); gxs[d] = gx.to_vector(); gws[d] = gw.to_vector();
    }
    expect_normwise(ys[0], ys[1], "conv2d_fw 32x32x16 * 3x3x16x32", g_mm_tol);
    expect_normwise(gxs[0], gxs[1], "conv2d_bw gx 32x32x16 * 3x3x16x32", g_mm_tol);
    expect_normwise(gws[0], gws[1], "conv2d_bw gw 32x32x16 * 3x3x16x32", g_mm_tol);
  }
  struct Pool { std::uint32_t w0, w1, p0, p1, s0, s1; };
  const Pool pools[] = {{2, 2, 0, 0, 2, 2}, {3, 2, 1, 0, 1, 1}, {2, 3, 0, 1, 1, 2}, {3, 3, 1, 1, 2, 1},
                        {7, 6, 0, 0, 1, 1}, {1, 1, 0, 0, 1, 1}, {2, 2, 1, 1, 3, 3}};
  for (const Pool &c : pools) {
    for (std::uint32_t batch : {1u, 3u}) {
      const Shape sx({7, 6, 3}, batch);
      vector<float> xv = rnd(sx.size(), -2.f, 2.f);
      for (float &v : xv) v = std::round(v * 2.f) / 2.f;   // many ties: the first maximal element takes the gradient
      vector<float> ys[2], gxs[2];
      for (int d = 0; d < 2; ++d) {
        Device &dev = *devs[d];
        Tensor x = p.on(dev, sx, xv);
        Tensor y = dev.max_pool2d_fw(x, c.w0, c.w1, c.p0, c.p1, c.s0, c.s1);
        std::mt19937 local(7);
        std::uniform_real_distribution<float> dist(-1.f, 1.f);
        vector<float> gv(y.shape().size());
        for (float &v : gv) v = to_half_grid(dist(local));
        Tensor gy = p.on(dev, y.shape(), gv);
        Tensor gx = dev.new_tensor_by_constant(sx, 0.5f);
        dev.max_pool2d_bw(x, y, gy, c.w0, c.w1, c.p0, c.p1, c.s0, c.s1, gx);
        ys[d] = y.to_vector(); gxs[d] = gx.to_vector();
      }
      const std::string tag = " window " + std::to_string(c.w0) + "," + std::to_string(c.w1) + " pad " +
                              std::to_string(c.p0) + "," + std::to_string(c.p1) + " stride " +
                              std::to_string(c.s0) + "," + std::to_string(c.s1) + " batch " + std::to_string(batch);
      expect_close(ys[0], ys[1], "max_pool2d_fw" + tag, 0.f);
      expect_close(gxs[0], gxs[1], "max_pool2d_bw" + tag, g_tol * 4);
    }
  }
}

// Gradients that start as zeros.  primitiv zero-fills a gradient right before the first `+=`
// into it; the B200 device defers that fill and lets the first accumulating kernel store
// instead.  Everything that can meet such a tensor first is run here from
// new_tensor_by_constant(shape, 0) on both devices: accumulating kernels (store path), a reader,
// a partial writer (the fill must then really happen), x op x (both gradients are one tensor),
// a second accumulation (must add), reset(0) of a live tensor, and a tensor dropped while its
// fill was still pending.
void test_zero_gradients(Pair &p) {
  Device *devs[2] = {&p.naive, &p.dev};
  const float tol = g_tol * 4;
  for (const auto &bb : kBatches) {
    const std::uint32_t bs = std::max(bb[0], bb[1]);
    const Shape sa({6, 5}, bb[0]), sb({6, 5}, bb[1]), sy({6, 5}, bs);
    const vector<float> av = on_grid(rnd(sa.size(), .5f, 2.f)), bv = on_grid(rnd(sb.size(), .5f, 2.f));
    const vector<float> gv = on_grid(rnd(sy.size()));
    vector<float> r[2][6];
    for (int d = 0; d < 2; ++d) {
      Device &dev = *devs[d];
      Tensor a = p.on(dev, sa, av), b = p.on(dev, sb, bv), gy = p.on(dev, sy, gv);
      Tensor y = dev.multiply_fw(a, b);
      Tensor ga = dev.new_tensor_by_constant(sa, 0), gb = dev.new_tensor_by_constant(sb, 0);
      dev.multiply_bw(a, b, y, gy, ga, gb);              // first writer stores
      r[d][0] = ga.to_vector(); r[d][1] = gb.to_vector();
      dev.add_bw(a, b, y, gy, ga, gb);                   // second writer adds
      r[d][2] = ga.to_vector(); r[d][3] = gb.to_vector();
      Tensor acc = dev.new_tensor_by_constant(sa, 0);
      dev.inplace_add(gy, acc);                          // same batch: copy; batch 1 <- 3: batch sum
      dev.inplace_add(gy, acc);
      r[d][4] = acc.to_vector();
      Tensor wide = dev.new_tensor_by_constant(sy, 0);
      dev.inplace_add(a, wide);                          // batch 3 <- 1 when a is broadcast
      r[d][5] = wide.to_vector();
    }
    const std::string tag = " batches " + std::to_string(bb[0]) + "," + std::to_string(bb[1]);
    expect_close(r[0][0], r[1][0], "multiply_bw into zeros: ga" + tag, tol);
    expect_close(r[0][1], r[1][1], "multiply_bw into zeros: gb" + tag, tol);
    expect_close(r[0][2], r[1][2], "add_bw after it: ga" + tag, tol);
    expect_close(r[0][3], r[1][3], "add_bw after it: gb" + tag, tol);
    expect_close(r[0][4], r[1][4], "inplace_add twice into zeros" + tag, tol);
    expect_close(r[0][5], r[1][5], "inplace_add of a (possibly broadcast) tensor into zeros" + tag, tol);
  }
  {
    const Shape s({7, 3}, 2), ss({3, 3}, 2);
    const vector<float> xv = on_grid(rnd(s.size())), gv = on_grid(rnd(s.size())), sv = on_grid(rnd(ss.size()));
    vector<float> r[2][7];
    for (int d = 0; d < 2; ++d) {
      Device &dev = *devs[d];
      Tensor x = p.on(dev, s, xv), gy = p.on(dev, s, gv), gs = p.on(dev, ss, sv);
      Tensor y = dev.tanh_fw(x);
      Tensor gx = dev.new_tensor_by_constant(s, 0);
      dev.tanh_bw(x, y, gy, gx);
      r[d][0] = gx.to_vector();
      dev.prelu_bw(x, y, gy, 0.1f, gx);
      r[d][1] = gx.to_vector();
      Tensor z = dev.new_tensor_by_constant(s, 0);
      r[d][2] = z.to_vector();                           // a reader sees zeros
      Tensor part = dev.new_tensor_by_constant(s, 0);
      dev.slice_bw(gs, 0, 2, part);                      // writes rows 2..4 only
      r[d][3] = part.to_vector();
      Tensor twice = dev.new_tensor_by_constant(s, 0);   // x * x: both gradients are this tensor
      Tensor sq = dev.multiply_fw(x, x);
      dev.multiply_bw(x, x, sq, gy, twice, twice);
      r[d][4] = twice.to_vector();
      Tensor live = p.on(dev, s, xv);
      live.reset(0);
      dev.inplace_add(gy, live);
      r[d][5] = live.to_vector();
      { Tensor dropped = dev.new_tensor_by_constant(s, 0); }   // never used
      Tensor next = p.on(dev, s, gv);                    // may reuse the dropped block
      r[d][6] = next.to_vector();
    }
    expect_close(r[0][0], r[1][0], "tanh_bw into zeros", tol);
    expect_close(r[0][1], r[1][1], "prelu_bw after it", tol);
    expect_close(r[0][2], r[1][2], "zeros read back", 0.f);
    expect_close(r[0][3], r[1][3], "slice_bw into zeros", tol);
    // ... along either axis, with every batch combination, followed by a second slice that must be added
    for (std::uint32_t dim = 0; dim < 2; ++dim) {
      for (const auto &bb : kBatches) {
        const Shape sx({7, 5}, bb[0]);
        const Shape sg(dim == 0 ? std::vector<std::uint32_t>{3, 5} : std::vector<std::uint32_t>{7, 2}, bb[1]);
        if (bb[0] > 1 && bb[1] > 1 && bb[0] != bb[1]) continue;
        const vector<float> g1 = on_grid(rnd(sg.size())), g2 = on_grid(rnd(sg.size()));
        vector<float> got[2];
        for (int d = 0; d < 2; ++d) {
          Device &dev = *devs[d];
          Tensor gx = dev.new_tensor_by_constant(sx, 0);
          dev.slice_bw(p.on(dev, sg, g1), dim, 1, gx);
          dev.slice_bw(p.on(dev, sg, g2), dim, 2, gx);
          got[d] = gx.to_vector();
        }
        expect_close(got[0], got[1], "slice_bw twice into zeros, dim " + std::to_string(dim) + " batches " +
                     std::to_string(bb[0]) + "," + std::to_string(bb[1]), tol * 4);
      }
    }
    expect_close(r[0][4], r[1][4], "multiply_bw with ga == gb into zeros", tol);
    expect_close(r[0][5], r[1][5], "reset(0) of a live tensor, then inplace_add", tol);
    expect_close(r[0][6], r[1][6], "a block reused after a dropped pending fill", 0.f);
  }
  for (const auto &bb : kBatches) {
    const std::uint32_t bs = std::max(bb[0], bb[1]);
    const Shape sa({64, 48}, bb[0]), sb({48, 40}, bb[1]), sy({64, 40}, bs);
    const vector<float> av = on_grid(rnd(sa.size())), bv = on_grid(rnd(sb.size())), gv = on_grid(rnd(sy.size()));
    vector<float> gas[2], gbs[2];
    for (int d = 0; d < 2; ++d) {
      Device &dev = *devs[d];
      Tensor a = p.on(dev, sa, av), b = p.on(dev, sb, bv), gy = p.on(dev, sy, gv);
      Tensor y = dev.matmul_fw(a, b);
      Tensor ga = dev.new_tensor_by_constant(sa, 0), gb = dev.new_tensor_by_constant(sb, 0);
      dev.matmul_bw(a, b, y, gy, ga, gb);   // stores
      dev.matmul_bw(a, b, y, gy, ga, gb);   // adds
      gas[d] = ga.to_vector(); gbs[d] = gb.to_vector();
    }
    const std::string tag = " " + sa.to_string() + " . " + sb.to_string();
    expect_normwise(gas[0], gas[1], "matmul_bw twice into zeros: ga" + tag, g_mm_tol);
    expect_normwise(gbs[0], gbs[1], "matmul_bw twice into zeros: gb" + tag, g_mm_tol);
  }
}

// A small MLP trained through primitiv's Graph, Parameter and SGD on both devices from the
// same initial weights: the loss trajectories must coincide (test/graph_test.cc:362-435 pins
// such a run for the Naive device).
void test_graph_training(Pair &p) {
  namespace F = primitiv::functions;
  using primitiv::Graph;
  using primitiv::Node;
  using primitiv::Parameter;
  const std::uint32_t in = 8, hid = 16, out = 4, bs = 12;
  const vector<float> w1 = on_grid(rnd(hid * in, -.5f, .5f)), w2 = on_grid(rnd(out * hid, -.5f, .5f));
  const vector<float> xs = on_grid(rnd(in * bs)), ts = on_grid(rnd(out * bs));
  vector<float> losses[2];
  Device *devs[2] = {&p.naive, &p.dev};
  for (int d = 0; d < 2; ++d) {
    Device::set_default(*devs[d]);
    Parameter pw1({hid, in}, w1, *devs[d]), pb1({hid}, primitiv::initializers::Constant(0), *devs[d]);
    Parameter pw2({out, hid}, w2, *devs[d]), pb2({out}, primitiv::initializers::Constant(0), *devs[d]);
    primitiv::optimizers::SGD opt(0.1f);
    opt.add(pw1, pb1, pw2, pb2);
    for (int step = 0; step < 6; ++step) {
      Graph g;
      Graph::set_default(g);
      Node x = F::input<Node>(Shape({in}, bs), xs, *devs[d]);
      Node t = F::input<Node>(Shape({out}, bs), ts, *devs[d]);
      Node h = F::tanh(F::matmul(F::parameter<Node>(pw1), x) + F::parameter<Node>(pb1));
      Node y = F::matmul(F::parameter<Node>(pw2), h) + F::parameter<Node>(pb2);
      Node diff = y - t;
      Node loss = F::batch::mean(F::sum(diff * diff, 0));
      losses[d].push_back(loss.to_float());
      opt.reset_gradients();
      loss.backward();
      opt.update();
    }
  }
  expect_close(losses[0], losses[1], "loss trajectory of a 2-layer MLP under SGD", g_half ? 2e-2f : 1e-4f);
  expect(losses[1].back() < losses[1].front(), "training on B200 reduces the loss");
}

// A kernel whose bounded wait ran out must not hand garbage to the host silently: the next call
// that returns values to the host throws primitiv::Error (as the reference's CUDA_CALL does for
// any failed CUDA call, primitiv/internal/cuda/utils.h:20-48), once, and the device stays usable.
// The wait that runs out here is the library's self-test: a one-warp kernel that waits a
// millisecond for a barrier nothing arrives at and returns normally.  Nothing faults.
void test_kernel_timeout_is_reported(Pair &p) {
  const Shape s({4, 3}, 2);
  const vector<float> v = on_grid(rnd(s.size()));
  Tensor t = p.dev.new_tensor_by_vector(s, v);
  auto thrown_by = [&](const std::function<void()> &f) {
    try { f(); } catch (const primitiv::Error &) { return true; }
    return false;
  };
  expect(::b200_selftest_wait_timeout(p.dev.context(), nullptr) == 0, "timeout self-test launches");
  expect(thrown_by([&] { t.to_vector(); }), "to_vector() throws after a kernel's wait ran out");
  expect(!thrown_by([&] { t.to_vector(); }), "the report is delivered once");
  expect_close(v, t.to_vector(), "the device still works after the report", g_tol);
  expect(::b200_selftest_wait_timeout(p.dev.context(), nullptr) == 0, "timeout self-test launches again");
  expect(thrown_by([&] { t.argmax(0); }), "argmax() throws after a kernel's wait ran out");
  expect(t.argmax(0).size() == 6, "argmax works afterwards");
  expect(::b200_selftest_wait_timeout(p.dev.context(), nullptr) == 0, "timeout self-test launches a third time");
  expect(thrown_by([&] { p.dev.wait_and_check(); }), "wait_and_check() throws after a kernel's wait ran out");
  expect(!thrown_by([&] { p.dev.wait_and_check(); }), "and not a second time");
  Tensor y = p.dev.matmul_fw(p.dev.new_tensor_by_vector(Shape({2, 4}), on_grid(rnd(8))), t);
  expect(y.to_vector().size() == 12, "the next product on the same device succeeds");
}

// Checkpoint round trip (primitiv/core/model.cc:16-75 over Parameter::save / load, which go
// through to_vector() and new_tensor_by_array on the device): parameters trained on the B200
// device are written, read back into fresh parameters on the same device, and must be the same
// values bit for bit; a Naive-side load of the same file agrees too.
void test_model_save_load(Pair &p) {
  using primitiv::Model;
  using primitiv::Parameter;
  const std::string path = "/tmp/primitiv_b200_device_parity_model.bin";
  const vector<float> w = on_grid(rnd(6 * 5)), b = on_grid(rnd(6));
  vector<float> saved_w, saved_b;
  {
    Parameter pw({6, 5}, w, p.dev), pb({6}, b, p.dev);
    pw.gradient() += p.dev.new_tensor_by_vector(Shape({6, 5}), on_grid(rnd(30)));
    primitiv::optimizers::SGD opt(0.5f);
    opt.add(pw, pb);
    opt.update();
    Model m;
    m.add("w", pw);
    m.add("b", pb);
    m.save(path, true);
    saved_w = pw.value().to_vector();
    saved_b = pb.value().to_vector();
  }
  Device *devs[2] = {&p.dev, &p.naive};
  for (Device *d : devs) {
    Parameter qw, qb;
    Model m;
    m.add("w", qw);
    m.add("b", qb);
    m.load(path, true, d);
    expect(qw.value().to_vector() == saved_w, "Model::load returns the saved weights bit for bit");
    expect(qb.value().to_vector() == saved_b, "Model::load returns the saved bias bit for bit");
    expect(&qw.device() == d, "loaded parameter lives on the requested device");
  }
  std::remove(path.c_str());
}

// The one-argument constructor takes its seed from the system's entropy source
// (primitiv/devices/cuda/device.cu:111-112): two such devices draw different numbers, two
// devices with the same explicit seed the same ones.
void test_unseeded_devices_differ() {
  const Shape s({64, 4});
  B200 a(0), b(0);
  expect(a.random_uniform(s, 0.f, 1.f).to_vector() != b.random_uniform(s, 0.f, 1.f).to_vector(),
         "unseeded devices draw different numbers");
  B200 c(0, 11), d(0, 11);
  expect(c.random_uniform(s, 0.f, 1.f).to_vector() == d.random_uniform(s, 0.f, 1.f).to_vector(),
         "devices with the same seed draw the same numbers");
}

}  // namespace

int main(int argc, char **argv) {
  B200::Mode mode = B200::Mode::FP32_3XTF32;
  const std::string m = argc > 1 ? argv[1] : "3xtf32";
  if (m == "tf32") { mode = B200::Mode::TF32_FAST; g_mm_tol = 2e-3f; }
  else if (m == "fp16") { mode = B200::Mode::FP16; g_half = true; g_tol = 2e-3f; g_mm_tol = 2e-3f; }
  else if (m == "3xfp16") { mode = B200::Mode::FP32_3XFP16; }
  else if (m != "3xtf32") { std::cerr << "usage: device_parity [3xtf32|tf32|fp16|3xfp16]" << std::endl; return 2; }
  try {
    Pair p(mode);
    p.dev.dump_description();
    expect(p.dev.type() == (g_half ? primitiv::DeviceType::CUDA16 : primitiv::DeviceType::CUDA), "device type");
    expect(B200::num_devices() >= 1, "num_devices");
    test_memory_and_io(p);
    test_unary(p);
    test_const_ops(p);
    test_scalar_and_binary(p);
    test_matmul(p);
    test_movement(p);
    test_batch_ops_and_inplace(p);
    test_large_batch_sums(p);
    test_random(p);
    test_conv_and_pool(p);
    test_zero_gradients(p);
    test_graph_training(p);
    test_model_save_load(p);
    test_kernel_timeout_is_reported(p);
    test_unseeded_devices_differ();
  } catch (const std::exception &e) {
    std::cerr << "EXCEPTION: " << e.what() << std::endl;
    return 3;
  }
  std::printf("device_parity[%s]: %d checks, %d failures\n", m.c_str(), g_checks, g_failures);
  return g_failures == 0 ? 0 : 1;
}
