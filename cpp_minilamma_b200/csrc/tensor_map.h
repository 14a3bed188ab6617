// Cached CUtensorMap construction shared by the TMA kernels.
#pragma once
#include <cuda.h>

namespace mll {
// A [rows, cols] bfloat16 row-major matrix read in boxes of [box_rows x 64 columns] with the
// 128-byte swizzle; rows or columns outside the matrix read as zero.  Returns 0 on success.
int tensor_map_bf16(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out);
}  // namespace mll
