#include "tma_host.cuh"

namespace dq {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `esize`-byte elements; box = box_cols x box_rows elements.
int make_tmap_2d_ex(CUtensorMap* tm, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t cols, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
  return make_tmap_2d_sw(tm, dt, esize, ptr, cols, rows, pitch_bytes, box_cols, box_rows, swizzle128 ? 128 : 0);
}

// swizzle_bytes: 0 (none), 64 or 128 (the inner box extent must not exceed it)
int make_tmap_2d_sw(CUtensorMap* tm, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t cols, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, int swizzle_bytes) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return DIROTQ_E_CUDA;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (pitch_bytes & 15)) return DIROTQ_E_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DIROTQ_OK : DIROTQ_E_CUDA;
}

// box = 128 bytes x box_rows, 128-byte swizzle (the K-major UMMA operand layout).
int make_tmap_2d(CUtensorMap* tm, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t cols, uint64_t rows,
                 uint64_t pitch_bytes, uint32_t box_rows) {
  return make_tmap_2d_ex(tm, dt, esize, ptr, cols, rows, pitch_bytes, (uint32_t)(128 / esize), box_rows, true);
}

}  // namespace dq
