// Shared host-side helpers of libmacko_b200: status reporting and per-device caches.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "macko_b200.h"

namespace macko {

constexpr int kMaxDevices = 64;

// Thread-local text of the last failure (returned by macko_last_error()).
char *last_error_buffer();
int fail(int status, const char *fmt, ...);

struct DeviceInfo {
    int sm_count = 0;
    int max_smem_optin = 0;  // bytes of dynamic shared memory a CTA may opt in to
    bool valid = false;
};

// Attributes of the current device, queried once per device.
int current_device_info(const DeviceInfo **out);

// In-place inclusive prefix sum over counts[1..rows] with counts[0] = 0 (one CTA; defined in compress.cu,
// shared by the compressor and the plan builder).
int launch_row_scan(int *counts, int rows, cudaStream_t stream);

inline bool aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace macko
