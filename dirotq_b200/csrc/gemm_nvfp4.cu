// Kernel 2 (NVFP4): W4A4 GEMM on the block-scaled FP4 tensor-core path.
//
//   y = out_scale * ( sum over 16-wide blocks  sfx[m,b] sfw[n,b] (e2m1 . e2m1)  +  x_tail . w_tail' ) + bias
//
// tcgen05.mma kind::mxf4nvf4.block_scale: E2M1 codes are read packed (two per byte) from
// 128-byte-swizzled shared memory filled by TMA; the UE4M3 scale factors travel as 512-byte tiles
// (bulk copy global -> smem, tcgen05.cp smem -> TMEM) and are applied by the hardware.  The
// high-precision branch (bf16 top-k coefficients) runs as kind::f16 UMMAs into the SAME fp32
// accumulator (its weights are pre-divided by out_scale), so the epilogue is one multiply-add,
// a bias add and a bf16 store.  Persistent CTAs, two TMEM accumulators: the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Replaces `self.module(x)` of the fused forward (DiRotQ dirotq_fused_unrotation_fast.py:141) for
// quant_dtype == "nvfp4"; the reference's speed path uses nunchaku's FP4 gemm_w4a4 here.
#include <cstdlib>
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace dq {

constexpr int GF_STAGES = 5;
constexpr int GF_TILE_BYTES = 128 * 128;     // 128 rows x 128 bytes (256 E2M1 or 64 bf16 per row)
constexpr int GF_SF_BYTES = 4 * 512;         // four 64-element k-blocks of scale factors for 128 rows
constexpr int GF_STAGE_BYTES = 2 * GF_TILE_BYTES + 2 * GF_SF_BYTES;   // 36864
constexpr int GF_EPI_WARPS = 8;              // two per TMEM lane quarter, 64 output columns each
constexpr int GF_THREADS = (2 + GF_EPI_WARPS) * 32;
constexpr int GF_STG_BYTES = GF_EPI_WARPS * 2048;   // per epilogue warp: 32 rows x 32 bf16 output staging patch
constexpr int GF_SMEM_BYTES = GF_STAGES * GF_STAGE_BYTES + GF_STG_BYTES + 1024 + 256;
constexpr uint32_t GF_TMEM_COLS = 512;
constexpr uint32_t GF_SFA_COL = 256;         // two alternating slots of 16 columns each
constexpr uint32_t GF_SFB_COL = 320;

struct GfRing {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() { if (++s == GF_STAGES) { s = 0; ph ^= 1; } }
};

__global__ void __launch_bounds__(GF_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tm_xq, const __grid_constant__ CUtensorMap tm_wq,
                  const __grid_constant__ CUtensorMap tm_xt, const __grid_constant__ CUtensorMap tm_wt,
                  const __grid_constant__ CUtensorMap tm_y, const GemmFp4Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stg_area = smem + GF_STAGES * GF_STAGE_BYTES;                 // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg_area + GF_STG_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GF_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (GF_STAGES + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * GF_STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * GF_STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < GF_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), GF_EPI_WARPS); }
    abort_flag[0] = 0;
    abort_flag[1] = a.wait_limit_k;
    fence_mbar_init();
    prefetch_tmap(&tm_xq);
    prefetch_tmap(&tm_wq);
    if (a.kt > 0) { prefetch_tmap(&tm_xt); prefetch_tmap(&tm_wt); }
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), GF_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();
  pdl_wait();                       // the kernel that produced the codes has completed
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);

  const int m_tiles = (int)((a.M + 127) / 128), n_tiles = (int)((a.N + 127) / 128);
  const int total_tiles = m_tiles * n_tiles;
  const int n_main = (a.n_chunks + 3) >> 2;      // stages of 256 K-elements
  const int n_tail = (a.kt + 63) >> 6;           // stages of 64 bf16
  const int nkb_pad = n_main * 4;                // 64-element k-blocks per row tile in the SF buffers

  if (warp == 0) {
    if (lane == 0) {
      GfRing r;
      uint32_t issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int mb = t / n_tiles, nb = t - mb * n_tiles;
        for (int st = 0; st < n_main + n_tail; ++st) {
          if (!mbar_wait(empty_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + r.s * GF_STAGE_BYTES;
          const uint32_t sB = sA + GF_TILE_BYTES;
          if (st < n_main) {
            mbar_expect_tx(full_bar(r.s), 2 * GF_TILE_BYTES + 2 * GF_SF_BYTES);
            tma_load_2d(sA, &tm_xq, full_bar(r.s), st * 128, mb * 128);
            tma_load_2d(sB, &tm_wq, full_bar(r.s), st * 128, nb * 128);
            bulk_load(sB + GF_TILE_BYTES, a.xsf + ((int64_t)mb * nkb_pad + st * 4) * 512, GF_SF_BYTES, full_bar(r.s));
            bulk_load(sB + GF_TILE_BYTES + GF_SF_BYTES, a.wsf + ((int64_t)nb * nkb_pad + st * 4) * 512, GF_SF_BYTES,
                      full_bar(r.s));
          } else {
            mbar_expect_tx(full_bar(r.s), 2 * GF_TILE_BYTES);
            tma_load_2d(sA, &tm_xt, full_bar(r.s), (st - n_main) * 64, mb * 128);
            tma_load_2d(sB, &tm_wt, full_bar(r.s), (st - n_main) * 64, nb * 128);
          }
          issued |= 1u << r.s;
          r.next();
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        for (int i = 0; i < GF_STAGES; ++i) {
          if (!(issued & (1u << i))) continue;
          const uint32_t last_ph = (i < r.s) ? r.ph : (r.ph ^ 1);
          while (!mbar_try(full_bar(i), last_ph)) {
            if (clock64() - t0 > kWaitLimitCycles / 8) { if (a.status) atomicCAS(a.status, 0, ERR_WAIT_DRAIN); break; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_f4 = idesc_nvf4(128, 128);
      const uint32_t idesc_bf = idesc_dense(ACC_F32, FMT_BF16, FMT_BF16, 128, 128);
      GfRing r;
      int buf = 0;
      uint32_t aph = 0;
      uint32_t sf_slot = 0;
      const uint64_t op_d0 = smem_desc_sw128(smem_base), sf_d0 = smem_desc_rows16(smem_base);
      const uint32_t op_lo0 = (uint32_t)op_d0, op_hi = (uint32_t)(op_d0 >> 32);
      const uint32_t sf_lo0 = (uint32_t)sf_d0, sf_hi = (uint32_t)(sf_d0 >> 32);
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(acce_bar(buf), aph ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * 128;
        for (int st = 0; st < n_main + n_tail; ++st) {
          if (!mbar_wait(full_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + r.s * GF_STAGE_BYTES;
          const uint64_t adesc = smem_desc_sw128(sA), bdesc = smem_desc_sw128(sA + GF_TILE_BYTES);
          if (st < n_main) {
            const uint32_t sfa_s = sA + 2 * GF_TILE_BYTES, sfb_s = sfa_s + GF_SF_BYTES;
            const uint32_t sfa_t = tmem_base + GF_SFA_COL + sf_slot * 16, sfb_t = tmem_base + GF_SFB_COL + sf_slot * 16;
            const int nkb = min(4, a.n_chunks - st * 4);
            if (nkb == 4) {
              // a whole stage: descriptors from loop-invariant words, eight copies + four UMMAs in one block
              const uint32_t a_lo = op_lo0 + (uint32_t)r.s * (GF_STAGE_BYTES >> 4);
              const uint32_t sf_lo = sf_lo0 + (uint32_t)r.s * (GF_STAGE_BYTES >> 4);
              umma_nvf4_stage4(d, a_lo, a_lo + (GF_TILE_BYTES >> 4), op_hi, idesc_f4, st > 0 ? 1u : 0u, sfa_t, sfb_t,
                               sf_lo + (2 * GF_TILE_BYTES >> 4), sf_lo + ((2 * GF_TILE_BYTES + GF_SF_BYTES) >> 4), sf_hi);
            } else {
            for (int kb = 0; kb < nkb; ++kb) {
              tmem_cp_32x128b_x4(sfa_t + kb * 4, smem_desc_rows16(sfa_s + kb * 512));
              tmem_cp_32x128b_x4(sfb_t + kb * 4, smem_desc_rows16(sfb_s + kb * 512));
            }
            for (int kb = 0; kb < nkb; ++kb)
              umma_nvf4(d, adesc + 2 * kb, bdesc + 2 * kb, idesc_f4, (st > 0 || kb > 0) ? 1u : 0u, sfa_t + kb * 4,
                        sfb_t + kb * 4);
            }
            sf_slot ^= 1;
          } else {
            const uint32_t a_lo = op_lo0 + (uint32_t)r.s * (GF_STAGE_BYTES >> 4);
            umma_f16_ss_x4(d, a_lo, a_lo + (GF_TILE_BYTES >> 4), op_hi, idesc_bf, 1u);
          }
          umma_commit(empty_bar(r.s));
          r.next();
        }
        if (!ok) break;
        umma_commit(accf_bar(buf));
        buf ^= 1;
        if (buf == 0) aph ^= 1;
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const uint32_t stg = smem_u32(stg_area) + (warp - 2) * 2048;
    int buf = 0;
    uint32_t aph = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int mb = t / n_tiles, nb = t - mb * n_tiles;
      if (!mbar_wait(accf_bar(buf), aph, abort_flag, a.status, ERR_WAIT_ACC_FULL)) break;
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 128 + half * 64;
      const int64_t row = (int64_t)mb * 128 + q * 32 + lane;
      const int64_t n0 = (int64_t)nb * 128 + half * 64;
      uint32_t v[64];
      tmem_ld32(taddr, v);
      tmem_ld32(taddr + 32, v + 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acce_bar(buf));      // accumulator is in registers: hand it back early
      // bf16 results leave through 32 x 32 staging patches (64-byte rows, 64-byte swizzle) and TMA stores,
      // which clip at the edges of y; a row-per-thread store would issue 32 separate 16-byte segments per
      // instruction.
      (void)row;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int64_t pcol = n0 + 32 * p;
        if (pcol >= a.N) continue;                       // warp-uniform
        if (lane == 0) bulk_wait_read0();                // the previous patch has left the staging buffer
        __syncwarp();
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
          const int i = 4 * p + i4;
          const int64_t col = n0 + 8 * i;
          uint32_t w[4] = {0u, 0u, 0u, 0u};
          if (col + 8 <= a.N) {
            float b[8];
            if (a.bias) {
              const uint4 bb = __ldg(reinterpret_cast<const uint4*>(a.bias + col));
              const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
              for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(bh[e]); b[2 * e] = f.x; b[2 * e + 1] = f.y; }
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) b[e] = 0.f;
            }
            float sc[8];
            if (a.col_scale) {
              const float4 c0 = __ldg(reinterpret_cast<const float4*>(a.col_scale + col));
              const float4 c1 = __ldg(reinterpret_cast<const float4*>(a.col_scale + col + 4));
              sc[0] = c0.x * a.out_scale; sc[1] = c0.y * a.out_scale; sc[2] = c0.z * a.out_scale; sc[3] = c0.w * a.out_scale;
              sc[4] = c1.x * a.out_scale; sc[5] = c1.y * a.out_scale; sc[6] = c1.z * a.out_scale; sc[7] = c1.w * a.out_scale;
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) sc[e] = a.out_scale;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float f0 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e]), sc[2 * e], b[2 * e]);
              float f1 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e + 1]), sc[2 * e + 1], b[2 * e + 1]);
              if (a.act == 1) { f0 = gelu_tanh_bf16(f0); f1 = gelu_tanh_bf16(f1); }
              __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
              w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};"
                       ::"r"(stg + lane * 64 + (uint32_t)((i4 ^ ((lane >> 1) & 3)) << 4)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tm_y, stg, (int)pcol, mb * 128 + q * 32);
          bulk_commit_group();
        }
      }
      buf ^= 1;
      if (buf == 0) aph ^= 1;
    }
    if (lane == 0) bulk_wait_all0();                     // the output is in global memory before the CTA retires
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, GF_TMEM_COLS);
  }
}

// Tile choice.  CTA pairs (gemm_nvfp4_pair.cu) halve the weight bytes each SM pulls through L2 per flop: 256 x 256 pair
// tiles for long reductions (one accumulator, its hand-over to the epilogue is amortised over many stages), 256 x 128
// with two accumulators for short ones; up to 128 rows a pair would idle half of itself, so the single-CTA 128 x 128
// kernel of this file keeps those.  Measured (M = 16384 .. 32768): K = 3072 -> 1.5 .. 1.7 x the single-CTA kernel with
// 256 x 256, K = 1152 -> 1.15 .. 1.2 x with 256 x 128.  DIROTQ_NVFP4_TILE = single | pair128 | pair256 forces one form
// (measurements, tests).
static int pick_nvfp4_tile(const GemmFp4Args& a) {
  if (const char* e = getenv("DIROTQ_NVFP4_TILE")) {
    if (!strcmp(e, "single")) return 0;
    if (!strcmp(e, "pair128")) return 128;
    if (!strcmp(e, "pair256")) return 256;
  }
  if (a.M <= 128) return 0;
  const int64_t K = (int64_t)a.n_chunks * 64 + a.kt;
  return K >= 2048 ? 256 : 128;
}

int launch_gemm_nvfp4(const GemmFp4Args& a, cudaStream_t st) {
  if (a.M <= 0 || a.N <= 0) return DIROTQ_OK;
  if (a.n_chunks <= 0) return DIROTQ_E_ARG;
  if (const int bn = pick_nvfp4_tile(a)) return launch_gemm_nvfp4_pair(a, bn, st);
  if (a.q_codes) return launch_gemm_nvfp4_pair(a, 128, st);          // quantise-out lives in the CTA-pair kernels
  if (!a.y) return DIROTQ_E_ARG;
  CUtensorMap txq, twq, txt, twt, ty;
  if (a.N % 8) return DIROTQ_E_UNSUPPORTED;
  const uint64_t row_bytes = (uint64_t)a.n_chunks * 32;
  int rc = make_tmap_2d(&txq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, row_bytes, (uint64_t)a.M, row_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&twq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.wq, row_bytes, (uint64_t)a.N, row_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_2d_sw(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, (uint64_t)a.N, (uint64_t)a.M, (uint64_t)a.N * 2, 32, 32, 64);
  if (rc) return rc;
  if (a.kt > 0) {
    rc = make_tmap_2d(&txt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.xt, (uint64_t)a.kt, (uint64_t)a.M, (uint64_t)a.kt_pitch * 2, 128);
    if (rc) return rc;
    rc = make_tmap_2d(&twt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.wt, (uint64_t)a.kt, (uint64_t)a.N, (uint64_t)a.kt_pitch * 2, 128);
    if (rc) return rc;
  } else {
    txt = txq;
    twt = twq;
  }
  static PerDeviceOnce attr_once;
  if (int rc = set_max_dynamic_smem(attr_once, gemm_nvfp4_kernel, GF_SMEM_BYTES)) return rc;
  const int tiles = (int)((a.M + 127) / 128) * (int)((a.N + 127) / 128);
  const int grid = min(tiles, num_sms());
  return launch_pdl(gemm_nvfp4_kernel, dim3(grid), dim3(GF_THREADS), GF_SMEM_BYTES, st, txq, twq, txt, twt, ty, a) == cudaSuccess
             ? DIROTQ_OK : DIROTQ_E_CUDA;
}

}  // namespace dq
