// Flat C entry points onto the REFERENCE's own Naive device, for the checker.
//
// TEST INFRASTRUCTURE ONLY.  This file is compiled together with the reference's
// unmodified sources (see Makefile, target `ref`) into oracle/_ref/libref_shim.so.
// It contains no arithmetic of its own: it wraps host arrays into
// primitiv::Tensor objects on a primitiv::devices::Naive, calls the public
// Device::matmul_fw / Device::matmul_bw (primitiv/core/device.cc:268-301) and
// copies the results back.  `seconds`, when not null, receives the wall time of
// the device call alone (array wrapping and read-back excluded).
#include <chrono>
#include <cstdint>
#include <cstring>
#include <exception>
#include <vector>

#include <primitiv/core/shape.h>
#include <primitiv/core/tensor.h>
#include <primitiv/devices/naive/device.h>

namespace {

primitiv::Tensor wrap(primitiv::Device &dev, const float *p,
                      std::uint32_t r, std::uint32_t c, std::uint32_t bs) {
  const primitiv::Shape s({r, c}, bs);
  return dev.new_tensor_by_array(s, p);
}

void read_back(const primitiv::Tensor &t, float *out) {
  const std::vector<float> v = t.to_vector();
  std::memcpy(out, v.data(), sizeof(float) * v.size());
}

}  // namespace

extern "C" {

// y = matmul(a, b).  Returns 0, or -1 if the reference threw.
int ref_naive_matmul_fw(const float *a, const float *b, float *y,
                        std::uint32_t di, std::uint32_t dj, std::uint32_t dk,
                        std::uint32_t ba, std::uint32_t bb, double *seconds) {
  try {
    primitiv::devices::Naive dev;
    const primitiv::Tensor ta = wrap(dev, a, di, dj, ba);
    const primitiv::Tensor tb = wrap(dev, b, dj, dk, bb);
    const auto t0 = std::chrono::steady_clock::now();
    const primitiv::Tensor ty = dev.matmul_fw(ta, tb);
    const auto t1 = std::chrono::steady_clock::now();
    if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
    read_back(ty, y);
    return 0;
  } catch (const std::exception &) {
    return -1;
  }
}

// ga += gy . b^T, gb += a^T . gy.  ga / gb hold the pre-fill on entry.
int ref_naive_matmul_bw(const float *a, const float *b, const float *gy,
                        float *ga, float *gb,
                        std::uint32_t di, std::uint32_t dj, std::uint32_t dk,
                        std::uint32_t ba, std::uint32_t bb, double *seconds) {
  try {
    primitiv::devices::Naive dev;
    const std::uint32_t bs = ba > bb ? ba : bb;
    const primitiv::Tensor ta = wrap(dev, a, di, dj, ba);
    const primitiv::Tensor tb = wrap(dev, b, dj, dk, bb);
    const primitiv::Tensor tgy = wrap(dev, gy, di, dk, bs);
    const primitiv::Tensor ty = dev.matmul_fw(ta, tb);
    primitiv::Tensor tga = wrap(dev, ga, di, dj, ba);
    primitiv::Tensor tgb = wrap(dev, gb, dj, dk, bb);
    const auto t0 = std::chrono::steady_clock::now();
    dev.matmul_bw(ta, tb, ty, tgy, tga, tgb);
    const auto t1 = std::chrono::steady_clock::now();
    if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
    read_back(tga, ga);
    read_back(tgb, gb);
    return 0;
  } catch (const std::exception &) {
    return -1;
  }
}

}  // extern "C"
