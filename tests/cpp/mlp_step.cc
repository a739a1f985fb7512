// One training step of a three-layer perceptron through primitiv's Graph, SGD included, on the
// B200 device: the shape of the reference's examples/mnist/mnist.cc:105-117 with a large
// minibatch, i.e. broadcast weights against tens of thousands of batch items.
//
// The model is workloads::mlp of graph_workloads.h (784-1024-1024-10, Xavier-uniform weights).
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
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <primitiv/core/error.h>
#include <primitiv/devices/naive/device.h>

#include <primitiv_b200.h>

#include "b200_device.h"
#include "b200_group.h"
#include "graph_workloads.h"

using primitiv::Device;
using primitiv::devices::B200;
using primitiv::devices::B200Group;
using primitiv::devices::Naive;
using workloads::rel_diff;
using namespace workloads::mlp;

namespace {

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
        rn = train_step(ref, data, check_batch, naive, sync);
        rb = train_step(got, data, check_batch, dev, sync);
      }
      loss_diff = std::fabs(rb.loss - rn.loss) / std::fabs(rn.loss);
      w1_diff = rel_diff(got.w1.value().to_vector(), ref.w1.value().to_vector());
      w3_diff = rel_diff(got.w3.value().to_vector(), ref.w3.value().to_vector());
      naive_ms = rn.ms;
    }
    Model model(data, dev);
    train_step(model, data, batch, dev, sync);  // warm-up: fills the memory pool's size classes
    train_step(model, data, batch, dev, sync);
    double best = 1e30, sum = 0;
    float last_loss = 0;
    Result fastest;
    for (int r = 0; r < repeats; ++r) {
      const Result res = train_step(model, data, batch, dev, sync);
      sum += res.ms;
      if (res.ms < best) { best = res.ms; fastest = res; }
      last_loss = res.loss;
    }
    double kind_ms[4] = {0, 0, 0, 0};
    std::uint64_t kind_n[4] = {0, 0, 0, 0};
    b200_profile_read(first.context(), kind_ms, kind_n);
    b200_profile_enable(first.context(), 1);
    train_step(model, data, batch, dev, sync);
    b200_profile_enable(first.context(), 0);
    b200_profile_read(first.context(), kind_ms, kind_n);
    const double flops = matmul_flops(batch);
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
