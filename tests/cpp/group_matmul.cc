// The matrix product of the hot path, forward and backward, through ONE primitiv Device object
// that spans several GPUs (devices::B200Group), called the way primitiv's operators call it:
//
//   y = dev.matmul_fw(a, b);  dev.matmul_bw(a, b, y, gy, ga, gb);
//
//   square     a, b {4096, 4096} x batch, gy likewise: items are independent, GPUs never meet
//   broadcast  a {8192, 8192} without a batch, b and gy {8192, 2048} x batch: ga is a sum over
//              the whole batch, so the GPUs' partial sums meet over NVLink once per step
//
// Operands are drawn on the devices (no host data).  The step is timed on the host clock around
// `steps` iterations between two synchronisations of every GPU: everything is asynchronous, so
// this is the device time of the slowest GPU plus whatever the host thread fails to hide.
//
//   group_matmul <3xtf32|tf32|fp16|3xfp16> <gpus> <square|broadcast> <batch> [steps] [warmup]
// Prints one JSON object.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <vector>

#include <primitiv/core/error.h>
#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>

#include "b200_group.h"

using primitiv::Shape;
using primitiv::Tensor;
using primitiv::devices::B200;
using primitiv::devices::B200Group;

int main(int argc, char **argv) {
  if (argc < 5) {
    std::cerr << "usage: group_matmul <mode> <gpus> <square|broadcast> <batch> [steps] [warmup]" << std::endl;
    return 2;
  }
  const std::string mode_name = argv[1], workload = argv[3];
  const std::uint32_t gpus = std::atoi(argv[2]), batch = std::atoi(argv[4]);
  const int steps = argc > 5 ? std::atoi(argv[5]) : 10, warmup = argc > 6 ? std::atoi(argv[6]) : 3;
  B200::Mode mode = B200::Mode::FP32_3XTF32;
  if (mode_name == "tf32") mode = B200::Mode::TF32_FAST;
  else if (mode_name == "fp16") mode = B200::Mode::FP16;
  else if (mode_name == "3xfp16") mode = B200::Mode::FP32_3XFP16;
  else if (mode_name != "3xtf32") return 2;
  try {
    std::vector<std::uint32_t> ids;
    for (std::uint32_t i = 0; i < gpus; ++i) ids.push_back(i);
    B200Group dev(ids, 0, mode);
    std::uint32_t m, k, n, ba;
    if (workload == "square") { m = k = n = 4096; ba = batch; }
    else if (workload == "broadcast") { m = k = 8192; n = 2048; ba = 1; }
    else return 2;
    const Tensor a = dev.random_normal(Shape({m, k}, ba), 0.f, workload == "square" ? 0.02f : 0.05f);
    const Tensor b = dev.random_normal(Shape({k, n}, batch), 0.f, workload == "square" ? 0.02f : 0.05f);
    const Tensor gy = dev.random_normal(Shape({m, n}, batch), 0.f, 1.f);
    Tensor ga = dev.new_tensor_by_constant(a.shape(), 0.f), gb = dev.new_tensor_by_constant(b.shape(), 0.f);
    using clock = std::chrono::steady_clock;
    double ms = 0;
    for (int it = 0; it < warmup + steps; ++it) {
      if (it == warmup) dev.synchronize();
      const auto t0 = clock::now();
      const Tensor y = dev.matmul_fw(a, b);
      dev.matmul_bw(a, b, y, gy, ga, gb);
      if (it == warmup + steps - 1) dev.synchronize();
      if (it >= warmup) ms += std::chrono::duration<double, std::milli>(clock::now() - t0).count();
    }
    const double flops = 3.0 * 2.0 * m * static_cast<double>(n) * k * batch;
    std::printf("{\"workload\": \"group_matmul_%s\", \"mode\": \"%s\", \"gpus\": %u, \"batch\": %u, \"steps\": %d, "
                "\"ms_per_step\": %.4f, \"tflops\": %.1f, \"cross_gpu_sums\": %llu}\n",
                workload.c_str(), mode_name.c_str(), gpus, batch, steps, ms / steps, flops / (ms / steps * 1e-3) / 1e12,
                static_cast<unsigned long long>(dev.cross_gpu_sums()));
  } catch (const std::exception &e) {
    std::cerr << "EXCEPTION: " << e.what() << std::endl;
    return 3;
  }
  return 0;
}
