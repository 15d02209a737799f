// Host-side helpers shared by every launcher: TMA tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda) and the per-device status buffer.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace mdb {

// Returns the device-global DeviceStatus of the current device (allocated on first use).
DeviceStatus* status_buffer();

// Encodes a tiled bf16 tensor map with 128-byte swizzle. dims/strides are innermost first;
// strides_bytes has rank-1 entries (the stride of dim i+1). Returns 0 on success.
int encode_tmap_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box);

// Same, for 1-byte elements (fp8 operands), 128-byte swizzle.
int encode_tmap_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box);

// Same, for 4-byte elements (fp32), no swizzle unless box[0]*4 == 128.
int encode_tmap_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int swizzle128);

int sm_count();

}  // namespace mdb

#define MDB_CHECK_CUDA(expr)                      \
  do {                                            \
    cudaError_t _e = (expr);                      \
    if (_e != cudaSuccess) return static_cast<int>(_e); \
  } while (0)
