// Forced include (-include) for building the reference's examples, unmodified, on the B200
// device: the examples construct their device as `devices::Naive dev;` and tell the reader to
// swap that line for another device.  This header performs the swap from outside the source:
// after primitiv.h and the B200 device are declared, the name Naive denotes a default-constructible
// B200 on GPU 0 (numeric mode from PRIMITIV_B200_MODE, default 3xTF32).
#ifndef PRIMITIV_B200_EXAMPLE_DEVICE_H_
#define PRIMITIV_B200_EXAMPLE_DEVICE_H_

#include <primitiv/primitiv.h>

#include "b200_device.h"

namespace primitiv {
namespace devices {

class B200OnGpu0 : public B200 {
public:
  B200OnGpu0() : B200(0) {}
};

}  // namespace devices
}  // namespace primitiv

#define Naive B200OnGpu0

#endif  // PRIMITIV_B200_EXAMPLE_DEVICE_H_
