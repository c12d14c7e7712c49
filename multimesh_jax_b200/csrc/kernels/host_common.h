// Host-side helpers shared by the kernel launchers: per-device status word,
// SM count, TMA tensor-map encoding through the driver entry point.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace mm {

#define MM_CUDA_TRY(expr)                                                        \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess) {                                                     \
      fprintf(stderr, "[mm_kernels] %s failed: %s (%s:%d)\n", #expr,             \
              cudaGetErrorString(_e), __FILE__, __LINE__);                       \
      return static_cast<int>(_e);                                               \
    }                                                                            \
  } while (0)

constexpr int kMaxDevices = 32;

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int* status = nullptr;  // device word: 0 = ok, else the first error code a kernel recorded
};

// Returns the state of the current device, creating it on first use.
DeviceState* device_state();

// Encodes a 2-D bf16 tensor map with 128-byte swizzle. `inner` is the
// contiguous dimension. Returns 0 on success.
int encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

// Encodes a tensor map of rank 2..5 for bf16 data with the given swizzle
// (0 = none, 3 = 128 B). dims/strides are innermost first; strides[0] is unused.
int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle128);

}  // namespace mm
