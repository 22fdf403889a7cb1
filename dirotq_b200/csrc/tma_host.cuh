// Host-side construction of TMA tensor maps (driver entry point resolved through the runtime, so
// the library does not link against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "layout.cuh"

namespace dq {
int make_tmap_2d(CUtensorMap* tm, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t cols, uint64_t rows,
                 uint64_t pitch_bytes, uint32_t box_rows);
int make_tmap_2d_ex(CUtensorMap* tm, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t cols, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, bool swizzle128);
int make_tmap_2d_sw(CUtensorMap* tm, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t cols, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, int swizzle_bytes);
}  // namespace dq
