// The recurrent step loop of an LSTM encoder through primitiv's Graph on the B200 device:
// many small broadcast matrix products with elementwise work between them, the
// latency-bound counterpart of the large batched products.
//
// The model is workloads::lstm of graph_workloads.h (E = 512, H = 1024, batch 64), 50 steps by default.  Forward and backward through time
// are timed on the B200 device (wall clock around graph construction, forward, backward and a
// final device synchronisation); a short prefix of the same loop is run on the reference's
// Naive device from the same inputs to check the loss and the weight gradients and to give
// a CPU time per step.
//
//   lstm_steps [tf32|3xtf32|fp16] [steps] [repeats] [naive_steps]
// Prints one JSON object.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include <primitiv/core/error.h>
#include <primitiv/devices/naive/device.h>

#include <primitiv_b200.h>

#include "b200_device.h"
#include "graph_workloads.h"

using primitiv::Device;
using primitiv::devices::B200;
using primitiv::devices::Naive;
using workloads::rel_diff;
using namespace workloads::lstm;

namespace {

void sync(Device &dev) {
  B200 *b = dynamic_cast<B200 *>(&dev);
  if (!b) return;
  int code = 0;
  b200_status_poll(b->context(), nullptr, &code);  // waits for the stream, reads the status word
  if (code != 0) throw std::runtime_error("a kernel reported a bounded-wait timeout");
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
      const Result rn = run_loop(ref, in, naive_steps, naive, sync);
      const Result rb = run_loop(model, in, naive_steps, dev, sync);
      loss_diff = std::fabs(rb.loss - rn.loss) / std::fabs(rn.loss);
      gwx_diff = rel_diff(model.wx.gradient().to_vector(), ref.wx.gradient().to_vector());
      gwh_diff = rel_diff(model.wh.gradient().to_vector(), ref.wh.gradient().to_vector());
      naive_ms_per_step = rn.total_ms / naive_steps;
    }
    run_loop(model, in, steps, dev, sync);  // warm-up: fills the memory pool's size classes
    run_loop(model, in, steps, dev, sync);
    double best = 1e30, sum = 0, best_fw = 0;
    float loss = 0;
    for (int r = 0; r < repeats; ++r) {
      const Result res = run_loop(model, in, steps, dev, sync);
      sum += res.total_ms;
      loss = res.loss;
      if (res.total_ms < best) { best = res.total_ms; best_fw = res.forward_ms; }
    }
    // one more, untimed loop with per-launch events: device time by kernel kind
    double kind_ms[4] = {0, 0, 0, 0};
    std::uint64_t kind_n[4] = {0, 0, 0, 0};
    b200_profile_read(dev.context(), kind_ms, kind_n);
    b200_profile_enable(dev.context(), 1);
    run_loop(model, in, steps, dev, sync);
    b200_profile_enable(dev.context(), 0);
    b200_profile_read(dev.context(), kind_ms, kind_n);
    std::uint64_t launches = 0;
    b200_launch_count(dev.context(), &launches);
    const double flops = matmul_flops(steps);
    std::printf("{\"workload\": \"lstm_steps\", \"mode\": \"%s\", \"steps\": %u, \"batch\": %u, \"repeats\": %d, "
                "\"ms_per_loop_mean\": %.4f, \"ms_per_loop_best\": %.4f, \"ms_forward_of_best\": %.4f, "
                "\"matmul_gflops\": %.1f, \"loss\": %.6e, \"naive_steps\": %u, \"naive_ms_per_step\": %.2f, "
                "\"loss_rel_diff\": %.3e, \"grad_wx_rel_diff\": %.3e, \"grad_wh_rel_diff\": %.3e, "
                "\"device_ms_per_loop\": {\"gemm_tc\": %.3f, \"pack\": %.3f, \"gemm_simt\": %.3f, "
                "\"other\": %.3f}, \"launches_per_loop\": {\"gemm_tc\": %llu, \"pack\": %llu, "
                "\"gemm_simt\": %llu, \"other\": %llu}, \"launches_total\": %llu}\n",
                mode_name.c_str(), steps, kBatch, repeats, sum / repeats, best, best_fw,
                flops / (sum / repeats * 1e-3) / 1e9, loss, naive_steps, naive_ms_per_step, loss_diff, gwx_diff,
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
