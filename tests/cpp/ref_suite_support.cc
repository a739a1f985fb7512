// Runs primitiv's OWN tensor / device tests (the reference's test/*.cc, compiled from where
// they lie, unmodified) with devices::B200 in the device list every test loops over.
//
// The reference's tests obtain their devices from test_utils::add_available_devices()
// (declared in its test/test_utils.h, defined in test/test_utils.cc, which is NOT compiled
// here): this file supplies those functions instead.  The list is one Naive device (the tests
// copy tensors between every pair of devices, so the reference's CPU device stays in) plus two
// B200 objects on GPU 0, as the reference adds two objects of each kind, in the numeric mode
// named by the first command-line argument (3xtf32 | tf32 | fp16).  The ULP bound per device
// follows the reference's rule: 4 for fp32 storage, half of the fp32/half mantissa gap for
// half storage.
//
// With PRIMITIV_B200_GROUP=<ordinal,ordinal,...> the first of the two is a devices::B200Group
// with one shard per listed ordinal instead ("0,0,0": three shards on GPU 0, which exercises the
// whole sharding logic, uneven cuts and minibatches smaller than the group included, on one GPU).
//
//   ref_tensor_tests [3xtf32|tf32|fp16|3xfp16] [--filter=<substring of Suite.Name>]
#define MINITEST_MAIN
#include <gtest/gtest.h>

#include <cstdint>
#include <cstdlib>
#include <string>
#include <vector>

#include <primitiv/core/device.h>
#include <primitiv/devices/naive/device.h>

#include "b200_device.h"
#include "b200_group.h"

namespace {
primitiv::devices::B200::Mode g_mode = primitiv::devices::B200::Mode::FP32_3XTF32;
}

namespace test_utils {

std::uint32_t get_default_ulps(const primitiv::Device &dev) {
  return dev.type() == primitiv::DeviceType::CUDA16 ? (1u << 12) : 4u;
}

void add_available_naive_devices(std::vector<primitiv::Device *> &devices) {
  devices.emplace_back(new primitiv::devices::Naive());
}
void add_available_eigen_devices(std::vector<primitiv::Device *> &) {}
void add_available_cuda_devices(std::vector<primitiv::Device *> &devices) {
  // devices::B200 stands where devices::CUDA / CUDA16 would
  // PRIMITIV_B200_PATH_POLICY=2 sends even the tests' tiny products through the tensor-core kernel
  const char *policy = std::getenv("PRIMITIV_B200_PATH_POLICY");
  const char *group = std::getenv("PRIMITIV_B200_GROUP");
  if (group) {
    std::vector<std::uint32_t> ids;
    for (const char *p = group; *p; ++p)
      if (*p >= '0' && *p <= '9') ids.push_back(static_cast<std::uint32_t>(*p - '0'));
    primitiv::devices::B200Group *dev = new primitiv::devices::B200Group(ids, 1, g_mode);
    if (policy)
      for (std::uint32_t i = 0; i < dev->num_shards(); ++i) dev->shard(i).set_matmul_path_policy(std::atoi(policy));
    devices.emplace_back(dev);
    dev->dump_description();
  }
  for (std::uint32_t seed : {1u, 2u}) {
    if (group && seed == 1u) continue;
    primitiv::devices::B200 *dev = new primitiv::devices::B200(0, seed, g_mode);
    if (policy) dev->set_matmul_path_policy(std::atoi(policy));
    devices.emplace_back(dev);
    dev->dump_description();
  }
}
void add_available_cuda16_devices(std::vector<primitiv::Device *> &) {}
void add_available_opencl_devices(std::vector<primitiv::Device *> &) {}

void add_available_devices(std::vector<primitiv::Device *> &devices) {
  add_available_naive_devices(devices);
  add_available_cuda_devices(devices);
}

}  // namespace test_utils

int main(int argc, char **argv) {
  if (argc > 1 && argv[1][0] != '-') {
    const std::string m = argv[1];
    if (m == "tf32") g_mode = primitiv::devices::B200::Mode::TF32_FAST;
    else if (m == "fp16") g_mode = primitiv::devices::B200::Mode::FP16;
    else if (m == "3xfp16") g_mode = primitiv::devices::B200::Mode::FP32_3XFP16;
    else if (m != "3xtf32") {
      std::fprintf(stderr, "usage: ref_tensor_tests [3xtf32|tf32|fp16] [--filter=...]\n");
      return 2;
    }
  }
  const int failed = minitest_run_all(argc, argv);
  return failed == 0 ? 0 : 1;
}
