// Host-side helpers shared by the C-ABI translation units: error reporting, device info cache,
// tensor-map encoding, conversion of the public hyper-parameter struct to the device one.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/forge_b200.h"
#include "forge_update.cuh"

namespace forge {

// records the message for forge_last_error_string() and returns `code`
int fail(int code, const char* fmt, ...);

struct DeviceInfo {
  int device;
  int sm_count;
  int cc_major;
  int cc_minor;
};

// info of the current device (cached after the first query); nullptr + error recorded on failure
const DeviceInfo* current_device_info();

// 2-D tiled tensor map over a row-major (rows, cols) array with `ld` elements between rows.
//   elem_bytes: 1, 2 (bf16) or 4 (fp32); box = (box_cols, box_rows); swizzle_bytes: 64 or 128
int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, bool is_float_type,
                   int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows,
                   int swizzle_bytes);

// narrows the public hyper-parameters exactly as the reference's kernel arguments are narrowed
Hyper make_hyper(const ForgeHyper& h);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace forge
