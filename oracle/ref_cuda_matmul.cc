// GPU comparator: times the reference's own CUDA devices on the benchmark workloads.
//
// Test and measurement infrastructure, not product: this program links the reference library
// built with its CUDA backend (`make -C oracle ref_cuda`; devices::CUDA calls cublasSgemm /
// cublasSgemmBatched, primitiv/devices/cuda/ops/matmul.cu:26-138; devices::CUDA16 calls
// cublasHgemm, primitiv/devices/cuda16/ops/matmul.cu:46-266) and drives it through the
// reference's public Device API exactly as primitiv's operators do: Device::matmul_fw then
// Device::matmul_bw with gradients that start from zeros.  It runs in a process of its own; the
// B200 library never links or loads it.
//
//   ref_cuda_matmul <batched_square|fp16_broadcast|plumbing> [steps] [warmup]
//
// Prints one JSON line: algorithmic GFLOP/s (3 products of 2 di dj dk batch FLOP per step),
// CUDA-event time on the legacy default stream the reference device launches on.
#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include <primitiv/core/device.h>
#include <primitiv/core/error.h>
#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>
#include <primitiv/devices/cuda/device.h>
#include <primitiv/devices/cuda16/device.h>

using primitiv::Device;
using primitiv::Shape;
using primitiv::Tensor;

namespace {

struct Workload {
  const char *name;
  std::uint32_t di, dj, dk, ba, bb;
  float sa, sb;
  bool half;
  const char *calls;
};

const Workload kWorkloads[] = {
    {"batched_square", 4096, 4096, 4096, 8, 8, 0.02f, 0.02f, false,
     "devices::CUDA: cublasSgemmBatched x3 (default math mode: fp32 FMA, no TF32)"},
    {"fp16_broadcast", 8192, 8192, 2048, 1, 32, 0.05f, 0.05f, true,
     "devices::CUDA16: cublasHgemm x3 over the combined {dj, dk*batch} matrix"},
    {"plumbing", 256, 256, 64, 1, 16, 1.f, 1.f, false, "devices::CUDA: cublasSgemm x3"},
};

// Seeded N(0, sd) values: a block of 1 Mi draws tiled over the tensor (the arithmetic units see
// random operand bits, which matters for a GEMM that runs against the power limit; drawing
// half a billion normals on the host would only slow the harness).
std::vector<float> values(std::size_t n, float sd, std::uint32_t seed) {
  std::mt19937 rng(seed);
  std::normal_distribution<float> dist(0.f, sd);
  const std::size_t block = n < (1u << 20) ? n : (1u << 20);
  std::vector<float> head(block);
  for (float &x : head) x = dist(rng);
  std::vector<float> v(n);
  for (std::size_t i = 0; i < n; i += block) std::memcpy(&v[i], head.data(), sizeof(float) * (n - i < block ? n - i : block));
  return v;
}

Tensor upload(Device &dev, const Shape &s, float sd, std::uint32_t seed) {
  const std::vector<float> v = values(s.size(), sd, seed);
  return dev.new_tensor_by_array(s, v.data());
}

void check(cudaError_t e, const char *what) {
  if (e != cudaSuccess) {
    std::fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(e));
    std::exit(4);
  }
}

}  // namespace

int main(int argc, char **argv) {
  const std::string name = argc > 1 ? argv[1] : "batched_square";
  const int steps = argc > 2 ? std::atoi(argv[2]) : 5;
  const int warmup = argc > 3 ? std::atoi(argv[3]) : 2;
  const Workload *w = nullptr;
  for (const Workload &c : kWorkloads) if (name == c.name) w = &c;
  if (!w || steps < 1 || warmup < 0) {
    std::fprintf(stderr, "usage: ref_cuda_matmul <batched_square|fp16_broadcast|plumbing> [steps] [warmup]\n");
    return 2;
  }
  try {
    std::unique_ptr<Device> dev;
    if (w->half) dev.reset(new primitiv::devices::CUDA16(0, 0));
    else dev.reset(new primitiv::devices::CUDA(0, 0));
    const std::uint32_t bs = w->ba > w->bb ? w->ba : w->bb;
    const Shape sa({w->di, w->dj}, w->ba), sb({w->dj, w->dk}, w->bb), sy({w->di, w->dk}, bs);
    const Tensor a = upload(*dev, sa, w->sa, 1), b = upload(*dev, sb, w->sb, 2), gy = upload(*dev, sy, 1.f, 3);
    Tensor ga = dev->new_tensor_by_constant(sa, 0.f), gb = dev->new_tensor_by_constant(sb, 0.f);
    cudaEvent_t e0, e1;
    check(cudaEventCreate(&e0), "cudaEventCreate");
    check(cudaEventCreate(&e1), "cudaEventCreate");
    auto step = [&]() {
      const Tensor y = dev->matmul_fw(a, b);
      dev->matmul_bw(a, b, y, gy, ga, gb);
    };
    for (int i = 0; i < warmup; ++i) step();
    check(cudaDeviceSynchronize(), "warm-up");
    check(cudaEventRecord(e0, 0), "cudaEventRecord");
    for (int i = 0; i < steps; ++i) step();
    check(cudaEventRecord(e1, 0), "cudaEventRecord");
    check(cudaEventSynchronize(e1), "timed steps");
    float ms = 0.f;
    check(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
    const double flops = 3.0 * 2.0 * w->di * w->dj * w->dk * bs;
    const double per = ms / steps;
    // a value of the result, so that the products cannot be skipped
    const float probe = ga.to_vector()[0];
    std::printf("{\"kind\": \"reference GPU device: %s\", \"workload\": \"%s\", \"value\": %.1f, \"unit\": \"GFLOP/s\", "
                "\"ms_per_step\": %.4f, \"steps\": %d, \"warmup\": %d, \"probe\": %g}\n",
                w->calls, w->name, flops / (per * 1e-3) / 1e9, per, steps, warmup, probe);
  } catch (const std::exception &e) {
    std::fprintf(stderr, "EXCEPTION: %s\n", e.what());
    return 3;
  }
  return 0;
}
