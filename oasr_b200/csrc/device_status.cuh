// Device-side status word shared by kernels that contain bounded waits.
#pragma once
#include <stdint.h>

namespace ob {

// Device address of the per-device status word (nullptr if it cannot be resolved).
uint32_t* device_status_ptr();

// Bits OR-ed into the status word by the pipelines when a wait gives up.
enum : uint32_t {
  kStatusGemmProducer = 1u << 0,
  kStatusGemmMma = 1u << 1,
  kStatusGemmEpilogue = 1u << 2,
  kStatusFmhaLoad = 1u << 4,
  kStatusFmhaMma = 1u << 5,
  kStatusFmhaSoftmax = 1u << 6,
  kStatusSelfTest = 1u << 8,
};

}  // namespace ob
