// Host helpers shared by the GEMM translation units: cached TMA descriptors.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace mb {

// 2-D row-major [rows, cols] tensor of `elt_bytes`-byte elements, box = [box_rows, 128 bytes],
// 128-byte swizzle, zero fill outside the tensor. Descriptors are cached by (pointer, shape, box).
int cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                uint32_t box_rows, int elt_bytes);

// Unswizzled byte tiles: `box_bytes` bytes (a multiple of 16) x `box_rows` rows of a [rows, cols] byte matrix with row
// pitch `ld` bytes.
int cached_tmap_raw(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_bytes);

}  // namespace mb
