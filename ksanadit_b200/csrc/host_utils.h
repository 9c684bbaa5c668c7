// Host-side helpers shared by the C-ABI translation units: error reporting, tensor-map encoding,
// device properties.  Nothing here allocates device memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KSB_OK_RC 0
#define KSB_ERR_INVALID (-1)
#define KSB_ERR_CUDA (-2)
#define KSB_ERR_UNSUPPORTED (-3)

namespace ksb {

// Stores a printf-style message retrievable with ksb_last_error() and returns `rc`.
int fail(int rc, const char* fmt, ...);

// Checks the launch error state after a kernel launch; returns 0 or KSB_ERR_CUDA.
int check_launch(const char* what);

// Encodes a 2-D tiled tensor map (row-major tensor: `inner` contiguous elements, `outer` rows,
// `row_stride_bytes` between rows).  The 128-byte swizzle is used when box_inner bytes == 128.
int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

int sm_count();

// Device address of the status words of the current device (resolved once per device).
int* status_words();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace ksb
