/* C API constructors for primitiv::devices::B200, next to primitiv's own
 * primitivCreateCudaDevice (primitiv/c/devices/cuda/device.h:15-34): the returned handle is
 * an ordinary primitivDevice_t and works with every other function of primitiv's C API. */
#ifndef PRIMITIV_C_DEVICES_B200_DEVICE_H_
#define PRIMITIV_C_DEVICES_B200_DEVICE_H_

#include <primitiv/c/define.h>
#include <primitiv/c/device.h>

/* mode: 0 = fp32 (3xTF32), 1 = TF32 single pass, 2 = fp16, 3 = fp32 (3xFP16) */
PRIMITIV_C_API PRIMITIV_C_STATUS primitivCreateB200Device(
    uint32_t device_id, primitivDevice_t **newobj);
PRIMITIV_C_API PRIMITIV_C_STATUS primitivCreateB200DeviceWithSeed(
    uint32_t device_id, uint32_t rng_seed, primitivDevice_t **newobj);
PRIMITIV_C_API PRIMITIV_C_STATUS primitivCreateB200DeviceWithSeedAndMode(
    uint32_t device_id, uint32_t rng_seed, uint32_t mode, primitivDevice_t **newobj);
PRIMITIV_C_API PRIMITIV_C_STATUS primitivGetNumB200Devices(uint32_t *retval);

/* primitiv::devices::B200Group: one device over the n listed GPUs (minibatches cut along the
 * batch axis, everything else replicated). */
PRIMITIV_C_API PRIMITIV_C_STATUS primitivCreateB200GroupDevice(
    const uint32_t *device_ids, size_t n, primitivDevice_t **newobj);
PRIMITIV_C_API PRIMITIV_C_STATUS primitivCreateB200GroupDeviceWithSeedAndMode(
    const uint32_t *device_ids, size_t n, uint32_t rng_seed, uint32_t mode, primitivDevice_t **newobj);

#endif  /* PRIMITIV_C_DEVICES_B200_DEVICE_H_ */
