// GPU comparator for the graph-level workloads: the recurrent step loop and the perceptron
// training step of tests/cpp/graph_workloads.h on the reference's own devices::CUDA.
//
// Test and measurement infrastructure, not product: this program links the reference library
// built with its CUDA backend (`make -C oracle ref_cuda`) and drives it through primitiv's
// Graph, exactly as tests/cpp/lstm_steps.cc and mlp_step.cc drive devices::B200: the same model
// code, the same seeded inputs, the same wall-clock bracket (graph construction, forward,
// backward, update, device synchronisation).  devices::CUDA multiplies with cublasSgemm in the
// default math mode (fp32 FMA; primitiv/devices/cuda/ops/matmul.cu:26-138) and launches every
// other operation as one kernel on the legacy default stream.  It runs in a process of its own.
//
//   ref_cuda_graphs lstm_steps [steps] [repeats]
//   ref_cuda_graphs mlp_step   [batch] [repeats]
//
// Prints one JSON line.
#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include <primitiv/core/error.h>
#include <primitiv/devices/cuda/device.h>

#include "graph_workloads.h"

namespace {

void sync(primitiv::Device &) {
  const cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(e));
}

const char *kKind = "reference GPU device: devices::CUDA (cublasSgemm, fp32 FMA) under primitiv's Graph";

int run_lstm(std::uint32_t steps, int repeats) {
  using namespace workloads::lstm;
  const Inputs in = make_inputs(steps);
  primitiv::devices::CUDA dev(0, 0);
  Model model(in, dev);
  run_loop(model, in, steps, dev, sync);  // warm-up: fills the device's memory pool
  run_loop(model, in, steps, dev, sync);
  double best = 1e30, sum = 0, best_fw = 0;
  float loss = 0;
  for (int r = 0; r < repeats; ++r) {
    const Result res = run_loop(model, in, steps, dev, sync);
    sum += res.total_ms;
    loss = res.loss;
    if (res.total_ms < best) { best = res.total_ms; best_fw = res.forward_ms; }
  }
  std::printf("{\"kind\": \"%s\", \"workload\": \"lstm_steps\", \"steps\": %u, \"batch\": %u, \"repeats\": %d, "
              "\"ms_per_loop_mean\": %.4f, \"ms_per_loop_best\": %.4f, \"ms_forward_of_best\": %.4f, "
              "\"matmul_gflops\": %.1f, \"loss\": %.6e}\n",
              kKind, steps, kBatch, repeats, sum / repeats, best, best_fw,
              matmul_flops(steps) / (sum / repeats * 1e-3) / 1e9, loss);
  return 0;
}

int run_mlp(std::uint32_t batch, int repeats) {
  using namespace workloads::mlp;
  const Data data = make_data(batch);
  primitiv::devices::CUDA dev(0, 0);
  Model model(data, dev);
  train_step(model, data, batch, dev, sync);  // warm-up
  train_step(model, data, batch, dev, sync);
  double best = 1e30, sum = 0;
  Result fastest;
  float loss = 0;
  for (int r = 0; r < repeats; ++r) {
    const Result res = train_step(model, data, batch, dev, sync);
    sum += res.ms;
    loss = res.loss;
    if (res.ms < best) { best = res.ms; fastest = res; }
  }
  std::printf("{\"kind\": \"%s\", \"workload\": \"mlp_step\", \"batch\": %u, \"repeats\": %d, "
              "\"ms_per_step_mean\": %.4f, \"ms_per_step_best\": %.4f, \"ms_of_best\": {\"graph_build\": %.3f, "
              "\"upload_forward\": %.3f, \"backward_update\": %.3f}, \"matmul_gflops\": %.1f, \"loss\": %.5f}\n",
              kKind, batch, repeats, sum / repeats, best, fastest.build_ms, fastest.forward_ms, fastest.rest_ms,
              matmul_flops(batch) / (sum / repeats * 1e-3) / 1e9, loss);
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  const std::string name = argc > 1 ? argv[1] : "";
  const int size = argc > 2 ? std::atoi(argv[2]) : 0;
  const int repeats = argc > 3 ? std::atoi(argv[3]) : 5;
  try {
    if (name == "lstm_steps" && repeats > 0) return run_lstm(size > 0 ? size : 50, repeats);
    if (name == "mlp_step" && repeats > 0) return run_mlp(size > 0 ? size : 65536, repeats);
  } catch (const std::exception &e) {
    std::fprintf(stderr, "EXCEPTION: %s\n", e.what());
    return 3;
  }
  std::fprintf(stderr, "usage: ref_cuda_graphs <lstm_steps [steps] | mlp_step [batch]> [repeats]\n");
  return 2;
}
