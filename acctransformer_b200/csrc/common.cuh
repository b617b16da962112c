// Host-side helpers shared by the C-ABI entry points: error reporting, the per-device status
// word, and TMA tensor-map construction (through the driver entry point, so the library does not
// link libcuda directly).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/acct_b200.h"

namespace acct {

// thread-local message buffer behind acct_last_error()
char* last_error_buf();
int fail(int code, const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);

// Device status word (one per device that loads the library); kernels atomicMax into it.
unsigned int* device_status_ptr();   // device address on the current device, or nullptr on failure

struct TensorDesc4 {
  const void* ptr;
  int dtype;              // ACCT_F16 / ACCT_BF16
  int64_t dims[4];        // innermost first: D, S, N, B
  int64_t strides[3];     // element strides of S, N, B
};
// Tiled map with a {64, box_rows, 1, 1} box and 128-byte swizzle (64 two-byte elements per row).
int make_tmap_4d(CUtensorMap* out, const TensorDesc4& t, int box_rows);

inline int64_t packed_or(int64_t given, int64_t packed) { return given == 0 ? packed : given; }

struct DeviceInfo {
  int sm_count;
  int cc_major, cc_minor;
  int max_smem_optin;
};
// Cached per device; fails (non-zero) if the current device is not sm_100.
int device_info(DeviceInfo* out);

}  // namespace acct
