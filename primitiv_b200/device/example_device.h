// Forced include (-include) for building the reference's examples, unmodified, on the B200
// device: the examples construct their device as `devices::Naive dev;` and tell the reader to
// swap that line for another device.  This header performs the swap from outside the source:
// after primitiv.h and the B200 device are declared, the name Naive denotes a default-constructible
// B200 on GPU 0 (numeric mode from PRIMITIV_B200_MODE, default 3xTF32).  Compiled with
// -DPRIMITIV_B200_EXAMPLE_GROUP it denotes a B200Group instead: one shard per ordinal listed in
// PRIMITIV_B200_GROUP (default "0,0": two shards on GPU 0).
#ifndef PRIMITIV_B200_EXAMPLE_DEVICE_H_
#define PRIMITIV_B200_EXAMPLE_DEVICE_H_

#include <primitiv/primitiv.h>

#include <cstdlib>
#include <vector>

#include "b200_device.h"
#include "b200_group.h"

namespace primitiv {
namespace devices {

class B200OnGpu0 : public B200 {
public:
  B200OnGpu0() : B200(0) {}
};

class B200GroupFromEnvironment : public B200Group {
public:
  B200GroupFromEnvironment() : B200Group(ids()) {}

private:
  static std::vector<std::uint32_t> ids() {
    const char *list = std::getenv("PRIMITIV_B200_GROUP");
    std::vector<std::uint32_t> v;
    for (const char *p = list ? list : "0,0"; *p; ++p)
      if (*p >= '0' && *p <= '9') v.push_back(static_cast<std::uint32_t>(*p - '0'));
    return v;
  }
};

}  // namespace devices
}  // namespace primitiv

#ifdef PRIMITIV_B200_EXAMPLE_GROUP
#define Naive B200GroupFromEnvironment
#else
#define Naive B200OnGpu0
#endif

#endif  // PRIMITIV_B200_EXAMPLE_DEVICE_H_
