// The recurrent step loop of an LSTM encoder through primitiv's Graph on the B200 device:
// many small broadcast matrix products with elementwise work between them, the
// latency-bound counterpart of the large batched products.
//
//   u_t = Wx . x_t + Wh . h_{t-1} + b          Wx {4H, E}, Wh {4H, H}, b {4H}; x_t {E} x batch
//   i, f, o = sigmoid(u_t[0:H], [H:2H], [2H:3H]);  j = tanh(u_t[3H:4H])
//   c_t = i * j + f * c_{t-1};  h_t = o * tanh(c_t);  loss = sum_t sum_batch sum h_t^2
//
// the structure of the reference's examples/encdec/lstm.h:46-57 and test/graph_test.cc:586-598,
// with E = 512, H = 1024, batch 64, 50 steps by default.  Forward and backward through time
// are timed on the B200 device (wall clock around graph construction, forward, backward and a
// final device synchronisation); a short prefix of the same loop is run on the reference's
// Naive device from the same inputs to check the loss and the weight gradients and to give
// a CPU time per step.
//
//   lstm_steps [tf32|3xtf32|fp16] [steps] [repeats] [naive_steps]
// Prints one JSON object.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include <primitiv/core/error.h>
#include <primitiv/core/functions.h>
#include <primitiv/core/graph.h>
#include <primitiv/core/initializer_impl.h>
#include <primitiv/core/parameter.h>
#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>
#include <primitiv/devices/naive/device.h>

#include <primitiv_b200.h>

#include "b200_device.h"

using primitiv::Device;
using primitiv::Graph;
using primitiv::Node;
using primitiv::Parameter;
using primitiv::Shape;
using primitiv::devices::B200;
using primitiv::devices::Naive;
using std::vector;
namespace F = primitiv::functions;

namespace {

const std::uint32_t kE = 512, kH = 1024, kBatch = 64;

struct Inputs {
  vector<float> wx, wh;
  vector<vector<float>> xs;
};

Inputs make_inputs(std::uint32_t steps) {
  std::mt19937 rng(0);
  std::uniform_real_distribution<float> w(-0.1f, 0.1f);
  std::normal_distribution<float> e(0.f, 1.f);
  Inputs in;
  in.wx.resize(4 * kH * kE);
  in.wh.resize(4 * kH * kH);
  for (float &v : in.wx) v = w(rng);
  for (float &v : in.wh) v = w(rng);
  in.xs.resize(steps);
  for (auto &x : in.xs) {
    x.resize(kE * kBatch);
    for (float &v : x) v = e(rng);
  }
  return in;
}

struct Model {
  Parameter wx, wh, b;
  Model(const Inputs &in, Device &dev)
      : wx({4 * kH, kE}, in.wx, dev), wh({4 * kH, kH}, in.wh, dev),
        b({4 * kH}, primitiv::initializers::Constant(0), dev) {}
  void reset_gradients() {
    wx.reset_gradient();
    wh.reset_gradient();
    b.reset_gradient();
  }
};

struct Result {
  float loss = 0;
  double forward_ms = 0, total_ms = 0;
};

void sync(Device &dev) {
  B200 *b = dynamic_cast<B200 *>(&dev);
  if (!b) return;
  int code = 0;
  b200_status_poll(b->context(), nullptr, &code);  // waits for the stream, reads the status word
  if (code != 0) throw std::runtime_error("a kernel reported a bounded-wait timeout");
}

// One forward + backward pass over `steps` time steps.
Result run_loop(Model &m, const Inputs &in, std::uint32_t steps, Device &dev) {
  using clock = std::chrono::steady_clock;
  Device::set_default(dev);
  m.reset_gradients();
  sync(dev);
  const auto t0 = clock::now();
  Graph g;
  Graph::set_default(g);
  const Node wx = F::parameter<Node>(m.wx), wh = F::parameter<Node>(m.wh), b = F::parameter<Node>(m.b);
  Node h = F::zeros<Node>(Shape({kH}, kBatch), dev);
  Node c = F::zeros<Node>(Shape({kH}, kBatch), dev);
  Node loss = F::zeros<Node>(Shape({}, 1), dev);
  for (std::uint32_t t = 0; t < steps; ++t) {
    const Node x = F::input<Node>(Shape({kE}, kBatch), in.xs[t], dev);
    const Node u = F::matmul(wx, x) + F::matmul(wh, h) + b;
    const Node i = F::sigmoid(F::slice(u, 0, 0, kH));
    const Node f = F::sigmoid(F::slice(u, 0, kH, 2 * kH));
    const Node o = F::sigmoid(F::slice(u, 0, 2 * kH, 3 * kH));
    const Node j = F::tanh(F::slice(u, 0, 3 * kH, 4 * kH));
    c = i * j + f * c;
    h = o * F::tanh(c);
    loss = loss + F::batch::sum(F::sum(h * h, 0));
  }
  Result r;
  r.loss = loss.to_float();  // runs the forward pass and reads the scalar back
  const auto t1 = clock::now();
  loss.backward();
  sync(dev);
  const auto t2 = clock::now();
  r.forward_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
  r.total_ms = std::chrono::duration<double, std::milli>(t2 - t0).count();
  return r;
}

double rel_diff(const vector<float> &a, const vector<float> &b) {
  double num = 0, den = 0;
  for (std::size_t i = 0; i < a.size(); ++i) {
    const double d = static_cast<double>(a[i]) - b[i];
    num += d * d;
    den += static_cast<double>(b[i]) * b[i];
  }
  return std::sqrt(num / (den > 0 ? den : 1));
}

}  // namespace

int main(int argc, char **argv) {
  const std::string mode_name = argc > 1 ? argv[1] : "tf32";
  const std::uint32_t steps = argc > 2 ? std::atoi(argv[2]) : 50;
  const int repeats = argc > 3 ? std::atoi(argv[3]) : 5;
  const std::uint32_t naive_steps = argc > 4 ? std::atoi(argv[4]) : 2;
  B200::Mode mode = B200::Mode::TF32_FAST;
  if (mode_name == "3xtf32") mode = B200::Mode::FP32_3XTF32;
  else if (mode_name == "fp16") mode = B200::Mode::FP16;
  else if (mode_name == "3xfp16") mode = B200::Mode::FP32_3XFP16;
  else if (mode_name != "tf32") {
    std::cerr << "usage: lstm_steps [tf32|3xtf32|fp16] [steps] [repeats] [naive_steps]" << std::endl;
    return 2;
  }
  try {
    const Inputs in = make_inputs(steps > naive_steps ? steps : naive_steps);
    B200 dev(0, 0, mode);
    Model model(in, dev);
    // parity on a short prefix against the reference's Naive device
    double loss_diff = 0, gwx_diff = 0, gwh_diff = 0, naive_ms_per_step = 0;
    if (naive_steps > 0) {
      Naive naive(0);
      Model ref(in, naive);
      const Result rn = run_loop(ref, in, naive_steps, naive);
      const Result rb = run_loop(model, in, naive_steps, dev);
      loss_diff = std::fabs(rb.loss - rn.loss) / std::fabs(rn.loss);
      gwx_diff = rel_diff(model.wx.gradient().to_vector(), ref.wx.gradient().to_vector());
      gwh_diff = rel_diff(model.wh.gradient().to_vector(), ref.wh.gradient().to_vector());
      naive_ms_per_step = rn.total_ms / naive_steps;
    }
    run_loop(model, in, steps, dev);  // warm-up: fills the memory pool's size classes
    run_loop(model, in, steps, dev);
    double best = 1e30, sum = 0, best_fw = 0;
    for (int r = 0; r < repeats; ++r) {
      const Result res = run_loop(model, in, steps, dev);
      sum += res.total_ms;
      if (res.total_ms < best) { best = res.total_ms; best_fw = res.forward_ms; }
    }
    // one more, untimed loop with per-launch events: device time by kernel kind
    double kind_ms[4] = {0, 0, 0, 0};
    std::uint64_t kind_n[4] = {0, 0, 0, 0};
    b200_profile_read(dev.context(), kind_ms, kind_n);
    b200_profile_enable(dev.context(), 1);
    run_loop(model, in, steps, dev);
    b200_profile_enable(dev.context(), 0);
    b200_profile_read(dev.context(), kind_ms, kind_n);
    std::uint64_t launches = 0;
    b200_launch_count(dev.context(), &launches);
    // 2 forward + 4 backward products per step: 3 x 2 x (4H x E + 4H x H) x batch
    const double flops = 3.0 * 2.0 * (4.0 * kH * kE + 4.0 * kH * kH) * kBatch * steps;
    std::printf("{\"workload\": \"lstm_steps\", \"mode\": \"%s\", \"steps\": %u, \"batch\": %u, \"repeats\": %d, "
                "\"ms_per_loop_mean\": %.4f, \"ms_per_loop_best\": %.4f, \"ms_forward_of_best\": %.4f, "
                "\"matmul_gflops\": %.1f, \"naive_steps\": %u, \"naive_ms_per_step\": %.2f, "
                "\"loss_rel_diff\": %.3e, \"grad_wx_rel_diff\": %.3e, \"grad_wh_rel_diff\": %.3e, "
                "\"device_ms_per_loop\": {\"gemm_tc\": %.3f, \"pack\": %.3f, \"gemm_simt\": %.3f, "
                "\"other\": %.3f}, \"launches_per_loop\": {\"gemm_tc\": %llu, \"pack\": %llu, "
                "\"gemm_simt\": %llu, \"other\": %llu}, \"launches_total\": %llu}\n",
                mode_name.c_str(), steps, kBatch, repeats, sum / repeats, best, best_fw,
                flops / (sum / repeats * 1e-3) / 1e9, naive_steps, naive_ms_per_step, loss_diff, gwx_diff,
                gwh_diff, kind_ms[0], kind_ms[1], kind_ms[2], kind_ms[3],
                static_cast<unsigned long long>(kind_n[0]), static_cast<unsigned long long>(kind_n[1]),
                static_cast<unsigned long long>(kind_n[2]), static_cast<unsigned long long>(kind_n[3]),
                static_cast<unsigned long long>(launches));
  } catch (const std::exception &e) {
    std::cerr << "EXCEPTION: " << e.what() << std::endl;
    return 3;
  }
  return 0;
}
