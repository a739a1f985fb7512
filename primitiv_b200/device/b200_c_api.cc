// C API constructors for primitiv::devices::B200.
#include "b200_c_api.h"

#include <primitiv/c/internal/internal.h>

#include <vector>

#include "b200_device.h"
#include "b200_group.h"

using primitiv::devices::B200;
using primitiv::devices::B200Group;
using primitiv::c::internal::to_c_ptr;

PRIMITIV_C_STATUS primitivCreateB200Device(uint32_t device_id, primitivDevice_t **newobj) try {
  PRIMITIV_C_CHECK_NOT_NULL(newobj);
  *newobj = to_c_ptr(new B200(device_id));
  return PRIMITIV_C_OK;
} PRIMITIV_C_HANDLE_EXCEPTIONS

PRIMITIV_C_STATUS primitivCreateB200DeviceWithSeed(
    uint32_t device_id, uint32_t rng_seed, primitivDevice_t **newobj) try {
  PRIMITIV_C_CHECK_NOT_NULL(newobj);
  *newobj = to_c_ptr(new B200(device_id, rng_seed));
  return PRIMITIV_C_OK;
} PRIMITIV_C_HANDLE_EXCEPTIONS

PRIMITIV_C_STATUS primitivCreateB200DeviceWithSeedAndMode(
    uint32_t device_id, uint32_t rng_seed, uint32_t mode, primitivDevice_t **newobj) try {
  PRIMITIV_C_CHECK_NOT_NULL(newobj);
  if (mode > 3) PRIMITIV_THROW_ERROR("Invalid B200 mode: " << mode);
  *newobj = to_c_ptr(new B200(device_id, rng_seed, static_cast<B200::Mode>(mode)));
  return PRIMITIV_C_OK;
} PRIMITIV_C_HANDLE_EXCEPTIONS

PRIMITIV_C_STATUS primitivGetNumB200Devices(uint32_t *retval) try {
  PRIMITIV_C_CHECK_NOT_NULL(retval);
  *retval = B200::num_devices();
  return PRIMITIV_C_OK;
} PRIMITIV_C_HANDLE_EXCEPTIONS

PRIMITIV_C_STATUS primitivCreateB200GroupDevice(
    const uint32_t *device_ids, size_t n, primitivDevice_t **newobj) try {
  PRIMITIV_C_CHECK_NOT_NULL(device_ids);
  PRIMITIV_C_CHECK_NOT_NULL(newobj);
  *newobj = to_c_ptr(new B200Group(std::vector<std::uint32_t>(device_ids, device_ids + n)));
  return PRIMITIV_C_OK;
} PRIMITIV_C_HANDLE_EXCEPTIONS

PRIMITIV_C_STATUS primitivCreateB200GroupDeviceWithSeedAndMode(
    const uint32_t *device_ids, size_t n, uint32_t rng_seed, uint32_t mode, primitivDevice_t **newobj) try {
  PRIMITIV_C_CHECK_NOT_NULL(device_ids);
  PRIMITIV_C_CHECK_NOT_NULL(newobj);
  if (mode > 3) PRIMITIV_THROW_ERROR("Invalid B200 mode: " << mode);
  *newobj = to_c_ptr(new B200Group(std::vector<std::uint32_t>(device_ids, device_ids + n), rng_seed,
                                   static_cast<B200::Mode>(mode)));
  return PRIMITIV_C_OK;
} PRIMITIV_C_HANDLE_EXCEPTIONS
