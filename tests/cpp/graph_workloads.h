// The two graph-level workloads of the measurement programs, written once against primitiv's
// public Graph API so that any primitiv Device can run them: devices::B200 and the reference's
// Naive device (tests/cpp/lstm_steps.cc, mlp_step.cc), and the reference's own devices::CUDA
// (the comparator program beside the checkers).  Only primitiv's core headers are needed.
//
//   lstm:  u_t = Wx . x_t + Wh . h_{t-1} + b          Wx {4H, E}, Wh {4H, H}, b {4H}; x_t {E} x batch
//          i, f, o = sigmoid(u_t[0:H], [H:2H], [2H:3H]);  j = tanh(u_t[3H:4H])
//          c_t = i * j + f * c_{t-1};  h_t = o * tanh(c_t);  loss = sum_t sum_batch sum h_t^2
//          (the structure of the reference's examples/encdec/lstm.h:46-57 and
//          test/graph_test.cc:586-598; E = 512, H = 1024, batch 64)
//
//   mlp:   h1 = relu(W1 . x + b1);  h2 = relu(W2 . h1 + b2);  y = W3 . h2 + b3
//          loss = batch::mean(softmax_cross_entropy(y, labels, 0));  backward;  SGD(0.1) update
//          x {784} x batch, W1 {1024, 784}, W2 {1024, 1024}, W3 {10, 1024}, Xavier-uniform weights
//          (the shape of the reference's examples/mnist/mnist.cc:105-117 with a large minibatch)
//
// Timing is wall clock round graph construction, forward, backward (and update) and a final
// device synchronisation, which the caller supplies: a Device has no public "wait" of its own.
#ifndef PRIMITIV_B200_TESTS_CPP_GRAPH_WORKLOADS_H_
#define PRIMITIV_B200_TESTS_CPP_GRAPH_WORKLOADS_H_

#include <chrono>
#include <cmath>
#include <cstdint>
#include <random>
#include <vector>

#include <primitiv/core/device.h>
#include <primitiv/core/functions.h>
#include <primitiv/core/graph.h>
#include <primitiv/core/initializer_impl.h>
#include <primitiv/core/optimizer_impl.h>
#include <primitiv/core/parameter.h>
#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>

namespace workloads {

// Blocks until everything the device was asked to do has finished (a no-op for a host device).
typedef void (*SyncFn)(primitiv::Device &);

inline double rel_diff(const std::vector<float> &a, const std::vector<float> &b) {
  double num = 0, den = 0;
  for (std::size_t i = 0; i < a.size(); ++i) {
    const double d = static_cast<double>(a[i]) - b[i];
    num += d * d;
    den += static_cast<double>(b[i]) * b[i];
  }
  return std::sqrt(num / (den > 0 ? den : 1));
}

inline double ms_between(std::chrono::steady_clock::time_point a, std::chrono::steady_clock::time_point b) {
  return std::chrono::duration<double, std::milli>(b - a).count();
}

namespace lstm {

const std::uint32_t kE = 512, kH = 1024, kBatch = 64;

struct Inputs {
  std::vector<float> wx, wh;
  std::vector<std::vector<float>> xs;
};

inline Inputs make_inputs(std::uint32_t steps) {
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
  primitiv::Parameter wx, wh, b;
  Model(const Inputs &in, primitiv::Device &dev)
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

// 2 forward + 4 backward products per step: 3 x 2 x (4H x E + 4H x H) x batch
inline double matmul_flops(std::uint32_t steps) {
  return 3.0 * 2.0 * (4.0 * kH * kE + 4.0 * kH * kH) * kBatch * steps;
}

// One forward + backward pass over `steps` time steps.
inline Result run_loop(Model &m, const Inputs &in, std::uint32_t steps, primitiv::Device &dev, SyncFn sync) {
  namespace F = primitiv::functions;
  using primitiv::Node;
  using primitiv::Shape;
  using clock = std::chrono::steady_clock;
  primitiv::Device::set_default(dev);
  m.reset_gradients();
  sync(dev);
  const auto t0 = clock::now();
  primitiv::Graph g;
  primitiv::Graph::set_default(g);
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
  r.forward_ms = ms_between(t0, t1);
  r.total_ms = ms_between(t0, t2);
  return r;
}

}  // namespace lstm

namespace mlp {

const std::uint32_t kIn = 784, kHid = 1024, kOut = 10;

inline std::vector<float> xavier(std::mt19937 &rng, std::uint32_t rows, std::uint32_t cols) {
  const float bound = std::sqrt(6.f / (rows + cols));  // primitiv/core/initializer_impl.cc:34-42
  std::uniform_real_distribution<float> d(-bound, bound);
  std::vector<float> v(static_cast<std::size_t>(rows) * cols);
  for (float &x : v) x = d(rng);
  return v;
}

struct Data {
  std::vector<float> w1, w2, w3, x;
  std::vector<std::uint32_t> labels;
};

inline Data make_data(std::uint32_t batch) {
  std::mt19937 rng(0);
  Data d;
  std::uniform_real_distribution<float> u(0.f, 1.f);
  d.x.resize(static_cast<std::size_t>(kIn) * batch);
  for (float &v : d.x) v = u(rng);
  d.w1 = xavier(rng, kHid, kIn);
  d.w2 = xavier(rng, kHid, kHid);
  d.w3 = xavier(rng, kOut, kHid);
  d.labels.resize(batch);
  for (auto &l : d.labels) l = rng() % kOut;
  return d;
}

struct Model {
  primitiv::Parameter w1, b1, w2, b2, w3, b3;
  primitiv::optimizers::SGD opt;
  Model(const Data &d, primitiv::Device &dev)
      : w1({kHid, kIn}, d.w1, dev), b1({kHid}, primitiv::initializers::Constant(0), dev),
        w2({kHid, kHid}, d.w2, dev), b2({kHid}, primitiv::initializers::Constant(0), dev),
        w3({kOut, kHid}, d.w3, dev), b3({kOut}, primitiv::initializers::Constant(0), dev), opt(0.1f) {
    opt.add(w1, b1, w2, b2, w3, b3);
  }
};

struct Result {
  float loss = 0;
  double ms = 0;                                     // the whole step
  double build_ms = 0, forward_ms = 0, rest_ms = 0;  // graph construction | forward | backward + update
};

// forward + both backward products of the three layers
inline double matmul_flops(std::uint32_t batch) {
  return 3.0 * 2.0 * (static_cast<double>(kHid) * kIn + static_cast<double>(kHid) * kHid +
                      static_cast<double>(kOut) * kHid) * batch;
}

// x and labels may hold more items than `batch`: a prefix is used.
inline Result train_step(Model &m, const Data &d, std::uint32_t batch, primitiv::Device &dev, SyncFn sync) {
  namespace F = primitiv::functions;
  using primitiv::Node;
  using primitiv::Shape;
  using clock = std::chrono::steady_clock;
  primitiv::Device::set_default(dev);
  const std::vector<float> x(d.x.begin(), d.x.begin() + static_cast<std::size_t>(kIn) * batch);
  const std::vector<std::uint32_t> labels(d.labels.begin(), d.labels.begin() + batch);
  sync(dev);
  const auto t0 = clock::now();
  primitiv::Graph g;
  primitiv::Graph::set_default(g);
  const Node in = F::input<Node>(Shape({kIn}, batch), x, dev);
  const Node h1 = F::relu(F::matmul(F::parameter<Node>(m.w1), in) + F::parameter<Node>(m.b1));
  const Node h2 = F::relu(F::matmul(F::parameter<Node>(m.w2), h1) + F::parameter<Node>(m.b2));
  const Node y = F::matmul(F::parameter<Node>(m.w3), h2) + F::parameter<Node>(m.b3);
  const Node loss = F::batch::mean(F::softmax_cross_entropy(y, labels, 0));
  const auto t1 = clock::now();  // the graph holds its own copy of the 784 x batch input by now
  Result r;
  r.loss = loss.to_float();      // uploads the input, runs the forward pass, reads the scalar back
  const auto t2 = clock::now();
  m.opt.reset_gradients();
  loss.backward();
  m.opt.update();
  sync(dev);
  const auto t3 = clock::now();
  r.build_ms = ms_between(t0, t1);
  r.forward_ms = ms_between(t1, t2);
  r.rest_ms = ms_between(t2, t3);
  r.ms = ms_between(t0, t3);
  return r;
}

}  // namespace mlp
}  // namespace workloads

#endif  // PRIMITIV_B200_TESTS_CPP_GRAPH_WORKLOADS_H_
