// One training step of a three-layer perceptron through primitiv's Graph, SGD included, on the
// B200 device: the shape of the reference's examples/mnist/mnist.cc:105-117 with a large
// minibatch, i.e. broadcast weights against tens of thousands of batch items.
//
//   h1 = relu(W1 . x + b1);  h2 = relu(W2 . h1 + b2);  y = W3 . h2 + b3
//   loss = batch::mean(softmax_cross_entropy(y, labels, 0));  backward;  SGD(0.1) update
//   x {784} x batch, W1 {1024, 784}, W2 {1024, 1024}, W3 {10, 1024}, Xavier-uniform weights
//
// The step is timed on the B200 device (wall clock around graph construction, forward,
// backward, update and a final device synchronisation).  The same step is run at a small
// batch on the reference's Naive device from the same weights and inputs: losses and updated
// weights must agree.
//
//   mlp_step [3xtf32|tf32|fp16|3xfp16] [batch] [repeats] [check_batch] [gpus]
// With gpus > 1 the device is a B200Group over GPUs 0 .. gpus-1: the same program, unchanged,
// with the minibatch cut over the GPUs and the weight gradients summed between them.
// Prints one JSON object.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <memory>
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

#include <primitiv_b200.h>

#include "b200_device.h"
#include "b200_group.h"

using primitiv::Device;
using primitiv::Graph;
using primitiv::Node;
using primitiv::Parameter;
using primitiv::Shape;
using primitiv::devices::B200;
using primitiv::devices::B200Group;
using primitiv::devices::Naive;
using std::vector;
namespace F = primitiv::functions;

namespace {

const std::uint32_t kIn = 784, kHid = 1024, kOut = 10;

vector<float> xavier(std::mt19937 &rng, std::uint32_t rows, std::uint32_t cols) {
  const float bound = std::sqrt(6.f / (rows + cols));  // primitiv/core/initializer_impl.cc:34-42
  std::uniform_real_distribution<float> d(-bound, bound);
  vector<float> v(static_cast<std::size_t>(rows) * cols);
  for (float &x : v) x = d(rng);
  return v;
}

struct Data {
  vector<float> w1, w2, w3, x;
  vector<std::uint32_t> labels;
};

Data make_data(std::uint32_t batch) {
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
  Parameter w1, b1, w2, b2, w3, b3;
  primitiv::optimizers::SGD opt;
  Model(const Data &d, Device &dev)
      : w1({kHid, kIn}, d.w1, dev), b1({kHid}, primitiv::initializers::Constant(0), dev),
        w2({kHid, kHid}, d.w2, dev), b2({kHid}, primitiv::initializers::Constant(0), dev),
        w3({kOut, kHid}, d.w3, dev), b3({kOut}, primitiv::initializers::Constant(0), dev), opt(0.1f) {
    opt.add(w1, b1, w2, b2, w3, b3);
  }
};

void sync(Device &dev) {
  if (B200Group *grp = dynamic_cast<B200Group *>(&dev)) {
    grp->synchronize();
    return;
  }
  B200 *b = dynamic_cast<B200 *>(&dev);
  if (!b) return;
  int code = 0;
  b200_status_poll(b->context(), nullptr, &code);
  if (code != 0) throw std::runtime_error("a kernel reported a bounded-wait timeout");
}

struct Result {
  float loss = 0;
  double ms = 0;                                   // the whole step
  double build_ms = 0, forward_ms = 0, rest_ms = 0;  // graph construction | forward | backward + update
};

// x and labels may hold more items than `batch`: a prefix is used.
Result train_step(Model &m, const Data &d, std::uint32_t batch, Device &dev) {
  using clock = std::chrono::steady_clock;
  Device::set_default(dev);
  const vector<float> x(d.x.begin(), d.x.begin() + static_cast<std::size_t>(kIn) * batch);
  const vector<std::uint32_t> labels(d.labels.begin(), d.labels.begin() + batch);
  sync(dev);
  const auto t0 = clock::now();
  Graph g;
  Graph::set_default(g);
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
  r.build_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
  r.forward_ms = std::chrono::duration<double, std::milli>(t2 - t1).count();
  r.rest_ms = std::chrono::duration<double, std::milli>(t3 - t2).count();
  r.ms = std::chrono::duration<double, std::milli>(t3 - t0).count();
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
  const std::string mode_name = argc > 1 ? argv[1] : "3xtf32";
  const std::uint32_t batch = argc > 2 ? std::atoi(argv[2]) : 65536;
  const int repeats = argc > 3 ? std::atoi(argv[3]) : 5;
  const std::uint32_t check_batch = argc > 4 ? std::atoi(argv[4]) : 256;
  const std::uint32_t gpus = argc > 5 ? std::atoi(argv[5]) : 1;
  B200::Mode mode = B200::Mode::FP32_3XTF32;
  if (mode_name == "tf32") mode = B200::Mode::TF32_FAST;
  else if (mode_name == "fp16") mode = B200::Mode::FP16;
  else if (mode_name == "3xfp16") mode = B200::Mode::FP32_3XFP16;
  else if (mode_name != "3xtf32") {
    std::cerr << "usage: mlp_step [3xtf32|tf32|fp16|3xfp16] [batch] [repeats] [check_batch] [gpus]" << std::endl;
    return 2;
  }
  try {
    const Data data = make_data(batch > check_batch ? batch : check_batch);
    std::unique_ptr<Device> owned;
    if (gpus > 1) {
      std::vector<std::uint32_t> ids;
      for (std::uint32_t i = 0; i < gpus; ++i) ids.push_back(i);
      owned.reset(new B200Group(ids, 0, mode));
    } else {
      owned.reset(new B200(0, 0, mode));
    }
    Device &dev = *owned;
    B200 &first = gpus > 1 ? static_cast<B200Group &>(dev).shard(0) : static_cast<B200 &>(dev);
    // parity at a small batch: two steps on both devices from the same weights
    double loss_diff = 0, w1_diff = 0, w3_diff = 0, naive_ms = 0;
    if (check_batch > 0) {
      Naive naive(0);
      Model ref(data, naive), got(data, dev);
      Result rn, rb;
      for (int step = 0; step < 2; ++step) {
        rn = train_step(ref, data, check_batch, naive);
        rb = train_step(got, data, check_batch, dev);
      }
      loss_diff = std::fabs(rb.loss - rn.loss) / std::fabs(rn.loss);
      w1_diff = rel_diff(got.w1.value().to_vector(), ref.w1.value().to_vector());
      w3_diff = rel_diff(got.w3.value().to_vector(), ref.w3.value().to_vector());
      naive_ms = rn.ms;
    }
    Model model(data, dev);
    train_step(model, data, batch, dev);  // warm-up: fills the memory pool's size classes
    train_step(model, data, batch, dev);
    double best = 1e30, sum = 0;
    float last_loss = 0;
    Result fastest;
    for (int r = 0; r < repeats; ++r) {
      const Result res = train_step(model, data, batch, dev);
      sum += res.ms;
      if (res.ms < best) { best = res.ms; fastest = res; }
      last_loss = res.loss;
    }
    double kind_ms[4] = {0, 0, 0, 0};
    std::uint64_t kind_n[4] = {0, 0, 0, 0};
    b200_profile_read(first.context(), kind_ms, kind_n);
    b200_profile_enable(first.context(), 1);
    train_step(model, data, batch, dev);
    b200_profile_enable(first.context(), 0);
    b200_profile_read(first.context(), kind_ms, kind_n);
    // forward + both backward products of the three layers
    const double flops = 3.0 * 2.0 * (static_cast<double>(kHid) * kIn + static_cast<double>(kHid) * kHid +
                                      static_cast<double>(kOut) * kHid) * batch;
    std::printf("{\"workload\": \"mlp_step\", \"mode\": \"%s\", \"gpus\": %u, \"batch\": %u, \"repeats\": %d, "
                "\"ms_per_step_mean\": %.4f, \"ms_per_step_best\": %.4f, \"ms_of_best\": {\"graph_build\": %.3f, "
                "\"upload_forward\": %.3f, \"backward_update\": %.3f}, \"matmul_gflops\": %.1f, \"loss\": %.5f, "
                "\"check_batch\": %u, \"naive_ms_per_step\": %.2f, \"loss_rel_diff\": %.3e, "
                "\"w1_rel_diff\": %.3e, \"w3_rel_diff\": %.3e, "
                "\"device_ms_per_step\": {\"gemm_tc\": %.3f, \"pack\": %.3f, \"gemm_simt\": %.3f, \"other\": %.3f}, "
                "\"launches_per_step\": {\"gemm_tc\": %llu, \"pack\": %llu, \"gemm_simt\": %llu, \"other\": %llu}}\n",
                mode_name.c_str(), gpus, batch, repeats, sum / repeats, best, fastest.build_ms, fastest.forward_ms,
                fastest.rest_ms, flops / (sum / repeats * 1e-3) / 1e9,
                last_loss, check_batch, naive_ms, loss_diff, w1_diff, w3_diff, kind_ms[0], kind_ms[1], kind_ms[2],
                kind_ms[3], static_cast<unsigned long long>(kind_n[0]), static_cast<unsigned long long>(kind_n[1]),
                static_cast<unsigned long long>(kind_n[2]), static_cast<unsigned long long>(kind_n[3]));
  } catch (const std::exception &e) {
    std::cerr << "EXCEPTION: " << e.what() << std::endl;
    return 3;
  }
  return 0;
}
