// Kernel 2 (INT): W4A4 / W4A8 GEMM with exact int32 accumulation per 64-wide chunk, the bf16
// high-precision branch, per-chunk dequantisation and bias -- one kernel, one pass over the operands.
//
//   y[m,n] = sum_c xs[c,m] ws[c,n] ( sum_k qx[m,c,k] qw[n,c,k]  -  xz[c,m] wsum[c,n] )
//            + x_tail[m,:] . w_tail[n,:] + bias[n]
//
// Data flow per persistent CTA (128 x 128 output tiles, K walked in stages of two 64-wide chunks):
//   TMA            packed 4-bit codes (64 B per row per stage) and the per-chunk scale rows
//                  -> "raw" shared-memory ring (deep: hides L2 / HBM latency with no registers held)
//   converter warps  raw ring -> "expanded" ring: every nibble widened to a byte (nibble << 4 is the
//                  sign-extended value times 16: two logic ops per 8 codes, the power-of-two factor is
//                  folded into the activation scale), written in the 128-byte-swizzled K-major layout
//   UMMA issuer    tcgen05.mma kind::i8, two K=32 instructions per chunk -> 128 x 128 int32 in TMEM;
//                  two PAIRS of accumulators alternate, one hand-off per stage (two chunks)
//   16 epilogue warps tcgen05.ld, exact int -> float, * ws[c,n] * xs[c,m], fp32 accumulate in registers
//   tail           bf16 TMA tiles straight into the expanded ring, kind::f16 UMMAs, added last
//
// Replaces the inner `self.module(x)` of the fused forward (DiRotQ
// dirotq_fused_unrotation_fast.py:141), which the reference's speed path hands to the third-party
// nunchaku gemm_w4a4.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "ptx.cuh"
#include "quant_math.cuh"
#include "tma_host.cuh"

namespace dq {

constexpr int GI_RAW_STAGES = 4;
constexpr int GI_EXP_STAGES = 3;
constexpr int GI_TILE_BYTES = 128 * 128;                 // one expanded operand tile
constexpr int GI_AUX_BYTES = 4 * 2 * 128 * 4;            // sw, sx, wsum, xz : [2 chunks][128] fp32
constexpr int GI_EXP_STAGE_BYTES = 2 * GI_TILE_BYTES + GI_AUX_BYTES;   // 36864
constexpr int GI_RAW_B_BYTES = 128 * 64;
constexpr int GI_RAW_AUX_BYTES = 1024 + 1024 + 512 + 512;   // ws, wsum (fp32 [2][128]); xs, xz (bf16 [2][128])
constexpr int GI_EPI_WARPS = 16;                       // 4 lane quarters x 4 column quarters
constexpr int GI_NACC = 4;                             // TMEM accumulators of 128 columns in flight
constexpr int GI_CONV_WARPS = 2;
constexpr int GI_THREADS = (GI_EPI_WARPS + 2 + GI_CONV_WARPS) * 32;     // 384
constexpr int GI_CONV_THREADS = GI_CONV_WARPS * 32;

template <int A_MODE> struct GiCfg {
  static constexpr int RAW_A_BYTES = (A_MODE == MODE_INT8_ASYM) ? 128 * 128 : 128 * 64;
  static constexpr int RAW_STAGE_BYTES = RAW_A_BYTES + GI_RAW_B_BYTES + GI_RAW_AUX_BYTES;
  static constexpr int SMEM_BYTES = GI_EXP_STAGES * GI_EXP_STAGE_BYTES + GI_RAW_STAGES * RAW_STAGE_BYTES + 1024 + 256;
};

struct GiMaps {
  CUtensorMap xq, wq, ws, wsum, xs, xz, xt, wt;
};

template <int N> struct RingN {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() { if (++s == N) { s = 0; ph ^= 1; } }
};

__device__ __forceinline__ uint32_t swz(uint32_t tile, int r, int c) {
  return tile + r * 128 + ((c ^ (r & 7)) << 4);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

template <int A_MODE, bool DUMP>
__global__ void __launch_bounds__(GI_THREADS, 1)
gemm_int_kernel(const __grid_constant__ GiMaps tm, const GemmIntArgs a) {
  using Cfg = GiCfg<A_MODE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_area = smem + GI_EXP_STAGES * GI_EXP_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw_area + GI_RAW_STAGES * Cfg::RAW_STAGE_BYTES);
  // barriers: raw_full[R], raw_empty[R], exp_full[E], exp_empty[E], acc_full[NACC], acc_empty[NACC]
  constexpr int NB = 2 * GI_RAW_STAGES + 2 * GI_EXP_STAGES + 2 * GI_NACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto rawf_bar = [&](int s) { return bar0 + 8u * s; };
  auto rawe_bar = [&](int s) { return bar0 + 8u * (GI_RAW_STAGES + s); };
  auto expf_bar = [&](int s) { return bar0 + 8u * (2 * GI_RAW_STAGES + s); };
  auto expe_bar = [&](int s) { return bar0 + 8u * (2 * GI_RAW_STAGES + GI_EXP_STAGES + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * GI_RAW_STAGES + 2 * GI_EXP_STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * GI_RAW_STAGES + 2 * GI_EXP_STAGES + GI_NACC + b); };

  constexpr int W_MMA = GI_EPI_WARPS, W_TMA = GI_EPI_WARPS + 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < GI_RAW_STAGES; ++s) { mbar_init(rawf_bar(s), 1); mbar_init(rawe_bar(s), GI_CONV_WARPS); }
    for (int s = 0; s < GI_EXP_STAGES; ++s) { mbar_init(expf_bar(s), GI_CONV_WARPS); mbar_init(expe_bar(s), 1 + GI_EPI_WARPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), GI_EPI_WARPS); }
    abort_flag[0] = 0;
    abort_flag[1] = a.wait_limit_k;
    fence_mbar_init();
    prefetch_tmap(&tm.xq);
    prefetch_tmap(&tm.wq);
  }
  if (warp == W_MMA) tmem_alloc(smem_u32(tmem_slot), 128 * GI_NACC);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t exp_base = smem_u32(smem);
  const uint32_t raw_base = smem_u32(raw_area);

  const int n_main = (a.n_chunks + 1) >> 1;               // stages of two chunks
  const int n_tail = (a.kt + 63) >> 6;                    // stages of 64 bf16
  const int n_tiles_n = (int)((a.N + 127) / 128);
  const int total_tiles = n_tiles_n * (int)((a.M + 127) / 128);
  constexpr bool ASYM = (A_MODE != MODE_INT4_SYM);
  constexpr float INV_F = ASYM ? (1.f / 16.f) : (1.f / 256.f);
  constexpr float F_ = ASYM ? 16.f : 256.f;
  constexpr uint32_t RAW_TX = Cfg::RAW_A_BYTES + GI_RAW_B_BYTES + 1024 + 512 + (ASYM ? 1024 + 512 : 0);
  // raw stage layout: A | B | ws | wsum | xs | xz
  constexpr int OFF_B = Cfg::RAW_A_BYTES, OFF_WS = OFF_B + GI_RAW_B_BYTES, OFF_WSUM = OFF_WS + 1024,
                OFF_XS = OFF_WSUM + 1024, OFF_XZ = OFF_XS + 512;
  // Persistent CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ...; consecutive tiles share the
  // activation row block (n fastest), so concurrently running CTAs hit the same rows in L2.  All
  // rings and the accumulator counter run on across tiles, so the loads and UMMAs of tile i+1
  // overlap the drain of tile i.

  if (warp == W_TMA) {
    // ------------------------------ TMA producer ---------------------------------------------
    if (lane == 0) {
      RingN<GI_RAW_STAGES> r;
      uint32_t issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = (t / n_tiles_n) * 128, n0 = (t % n_tiles_n) * 128;
        for (int st = 0; st < n_main; ++st) {
          if (!mbar_wait(rawe_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sb = raw_base + r.s * Cfg::RAW_STAGE_BYTES;
          const uint32_t bar = rawf_bar(r.s);
          mbar_expect_tx(bar, RAW_TX);
          tma_load_2d(sb, &tm.xq, bar, st * (A_MODE == MODE_INT8_ASYM ? 128 : 64), m0);
          tma_load_2d(sb + OFF_B, &tm.wq, bar, st * 64, n0);
          tma_load_2d(sb + OFF_WS, &tm.ws, bar, n0, st * 2);
          tma_load_2d(sb + OFF_XS, &tm.xs, bar, m0, st * 2);
          if constexpr (ASYM) {
            tma_load_2d(sb + OFF_WSUM, &tm.wsum, bar, n0, st * 2);
            tma_load_2d(sb + OFF_XZ, &tm.xz, bar, m0, st * 2);
          }
          issued |= 1u << r.s;
          r.next();
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        for (int i = 0; i < GI_RAW_STAGES; ++i) {
          if (!(issued & (1u << i))) continue;
          const uint32_t last_ph = (i < r.s) ? r.ph : (r.ph ^ 1);
          while (!mbar_try(rawf_bar(i), last_ph))
            if (clock64() - t0 > kWaitLimitCycles / 8) { if (a.status) atomicCAS(a.status, 0, ERR_WAIT_DRAIN); break; }
        }
      }
    }
  } else if (warp > W_TMA) {
    // ------------------------------ converters: raw ring -> expanded ring --------------------
    const int ct = threadIdx.x - (W_TMA + 1) * 32;        // 0..63
    RingN<GI_RAW_STAGES> r;
    RingN<GI_EXP_STAGES> e;
    uint32_t issued_e = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int m0 = (t / n_tiles_n) * 128, n0 = (t % n_tiles_n) * 128;
      for (int st = 0; st < n_main; ++st) {
        if (!mbar_wait(rawf_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
        if (!mbar_wait(expe_bar(e.s), e.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
        const uint32_t sraw = raw_base + r.s * Cfg::RAW_STAGE_BYTES;
        const uint32_t sA = exp_base + e.s * GI_EXP_STAGE_BYTES;
        const uint32_t sB = sA + GI_TILE_BYTES;
        // B (weights): 128 rows x 4 granules of 32 codes; all loads first, then widen + store
        {
          uint4 p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) p[i] = lds128(sraw + OFF_B + (ct + i * GI_CONV_THREADS) * 16);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int id = ct + i * GI_CONV_THREADS;
            const int row = id >> 2, gi = id & 3;
            sts128(swz(sB, row, 2 * gi), make_uint4((p[i].x << 4) & 0xF0F0F0F0u, (p[i].y << 4) & 0xF0F0F0F0u,
                                                    (p[i].z << 4) & 0xF0F0F0F0u, (p[i].w << 4) & 0xF0F0F0F0u));
            sts128(swz(sB, row, 2 * gi + 1), make_uint4(p[i].x & 0xF0F0F0F0u, p[i].y & 0xF0F0F0F0u,
                                                        p[i].z & 0xF0F0F0F0u, p[i].w & 0xF0F0F0F0u));
          }
        }
        if constexpr (A_MODE == MODE_INT8_ASYM) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4 p[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) p[i] = lds128(sraw + (ct + (h * 8 + i) * GI_CONV_THREADS) * 16);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int id = ct + (h * 8 + i) * GI_CONV_THREADS;
              sts128(swz(sA, id >> 3, id & 7), p[i]);
            }
          }
        } else {
          uint4 p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) p[i] = lds128(sraw + (ct + i * GI_CONV_THREADS) * 16);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int id = ct + i * GI_CONV_THREADS;
            const int row = id >> 2, gi = id & 3;
            if constexpr (A_MODE == MODE_INT4_SYM) {
              sts128(swz(sA, row, 2 * gi), make_uint4((p[i].x << 4) & 0xF0F0F0F0u, (p[i].y << 4) & 0xF0F0F0F0u,
                                                      (p[i].z << 4) & 0xF0F0F0F0u, (p[i].w << 4) & 0xF0F0F0F0u));
              sts128(swz(sA, row, 2 * gi + 1), make_uint4(p[i].x & 0xF0F0F0F0u, p[i].y & 0xF0F0F0F0u,
                                                          p[i].z & 0xF0F0F0F0u, p[i].w & 0xF0F0F0F0u));
            } else {
              sts128(swz(sA, row, 2 * gi), make_uint4(p[i].x & 0x0F0F0F0Fu, p[i].y & 0x0F0F0F0Fu,
                                                      p[i].z & 0x0F0F0F0Fu, p[i].w & 0x0F0F0F0Fu));
              sts128(swz(sA, row, 2 * gi + 1), make_uint4((p[i].x >> 4) & 0x0F0F0F0Fu, (p[i].y >> 4) & 0x0F0F0F0Fu,
                                                          (p[i].z >> 4) & 0x0F0F0F0Fu, (p[i].w >> 4) & 0x0F0F0F0Fu));
            }
          }
        }
        // per-chunk scales / zero points / code sums of the tile's 128 rows and 128 columns
        {
          const uint8_t* rs = raw_area + r.s * Cfg::RAW_STAGE_BYTES;
          float* aux = reinterpret_cast<float*>(smem + e.s * GI_EXP_STAGE_BYTES + 2 * GI_TILE_BYTES);
          const float* rws = reinterpret_cast<const float*>(rs + OFF_WS);
          const float* rwsum = reinterpret_cast<const float*>(rs + OFF_WSUM);
          const __nv_bfloat16* rxs = reinterpret_cast<const __nv_bfloat16*>(rs + OFF_XS);
          const __nv_bfloat16* rxz = reinterpret_cast<const __nv_bfloat16*>(rs + OFF_XZ);
#pragma unroll
          for (int i = ct; i < 256; i += GI_CONV_THREADS) {
            aux[i] = rws[i];
            aux[256 + i] = __bfloat162float(rxs[i]) * INV_F;
            if constexpr (ASYM) {
              aux[512 + i] = rwsum[i];
              aux[768 + i] = __bfloat162float(rxz[i]) * F_;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(expf_bar(e.s));
          mbar_arrive(rawe_bar(r.s));
        }
        r.next();
        e.next();
      }
      // tail: bf16 tiles go by TMA straight into the expanded ring.  Issued from a converter thread
      // (not from the TMA warp) because the converters walk the expanded ring in order; both
      // converter warps poll every slot so that no waiter is ever more than one phase away from
      // the barrier it polls.
      for (int st = 0; st < n_tail && ok; ++st) {
        if (!mbar_wait(expe_bar(e.s), e.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
        if (ct == 0) {
          const uint32_t sA = exp_base + e.s * GI_EXP_STAGE_BYTES;
          const uint32_t bar = expf_bar(e.s);
          mbar_expect_tx(bar, 2 * GI_TILE_BYTES);           // first of the two expected arrivals
          mbar_arrive(bar);                                  // second (the other converter warp's slot)
          tma_load_2d(sA, &tm.xt, bar, st * 64, m0);
          tma_load_2d(sA + GI_TILE_BYTES, &tm.wt, bar, st * 64, n0);
          issued_e |= 1u << e.s;
        }
        e.next();
      }
    }
    if (!ok && ct == 0) {
      const long long t0 = clock64();
      for (int i = 0; i < GI_EXP_STAGES; ++i) {
        if (!(issued_e & (1u << i))) continue;
        const uint32_t last_ph = (i < e.s) ? e.ph : (e.ph ^ 1);
        while (!mbar_try(expf_bar(i), last_ph))
          if (clock64() - t0 > kWaitLimitCycles / 8) { if (a.status) atomicCAS(a.status, 0, ERR_WAIT_DRAIN); break; }
      }
    }
  } else if (warp == W_MMA) {
    // ------------------------------ UMMA issuer ----------------------------------------------
    if (lane == 0) {
      const uint32_t idesc_i8 = idesc_dense(ACC_S32, ASYM ? FMT_U8 : FMT_S8, FMT_S8, 128, 128);
      const uint32_t idesc_bf = idesc_dense(ACC_F32, FMT_BF16, FMT_BF16, 128, 128);
      RingN<GI_EXP_STAGES> e;
      int use = 0;   // hand-offs so far: accumulator pair = use & 1, phase = (use >> 1) & 1
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int st = 0; st < n_main && ok; ++st) {
          if (!mbar_wait(expf_bar(e.s), e.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = exp_base + e.s * GI_EXP_STAGE_BYTES;
          const uint64_t adesc = smem_desc_sw128(sA), bdesc = smem_desc_sw128(sA + GI_TILE_BYTES);
          // one hand-off per stage: the stage's two chunks go to the two accumulators of a pair
          const int pair = use & 1;
          if (!mbar_wait(acce_bar(pair), ((use >> 1) & 1) ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) { ok = false; break; }
          tc_fence_after();
          for (int c = 0; c < 2; ++c) {
            if (st * 2 + c >= a.n_chunks) break;
            const uint32_t d = tmem_base + (2 * pair + c) * 128;
            umma_i8(d, adesc + 4 * c, bdesc + 4 * c, idesc_i8, 0u);
            umma_i8(d, adesc + 4 * c + 2, bdesc + 4 * c + 2, idesc_i8, 1u);
          }
          umma_commit(accf_bar(pair));
          ++use;
          umma_commit(expe_bar(e.s));
          e.next();
        }
        if (ok && n_tail > 0) {
          const int pair = use & 1;
          if (!mbar_wait(acce_bar(pair), ((use >> 1) & 1) ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + (2 * pair) * 128;
          for (int st = 0; st < n_tail; ++st) {
            if (!mbar_wait(expf_bar(e.s), e.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sA = exp_base + e.s * GI_EXP_STAGE_BYTES;
            const uint64_t adesc = smem_desc_sw128(sA), bdesc = smem_desc_sw128(sA + GI_TILE_BYTES);
#pragma unroll
            for (int j = 0; j < 4; ++j) umma_f16(d, adesc + 2 * j, bdesc + 2 * j, idesc_bf, (st > 0 || j > 0) ? 1u : 0u);
            umma_commit(expe_bar(e.s));
            e.next();
          }
          if (ok) { umma_commit(accf_bar(pair)); ++use; }
        }
      }
    }
  } else {
    // ------------------------------ epilogue: 16 warps ---------------------------------------
    // warp w: TMEM lane quarter w & 3 (rows), column quarter w >> 2 (32 of the tile's 128 columns).
    // The drain is the kernel's critical resource (CUDA-core issue slots), so it runs on the packed
    // fp32x2 pipe: per PAIR of values two integer adds (exact int32 -> fp32), one packed subtract,
    // one packed multiply by ws[c,n], one packed fused multiply-add by xs[c,m].
    const int q = warp & 3, cq = warp >> 2;
    const int trow = q * 32 + lane;                       // row inside the tile
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16) + cq * 32;
    RingN<GI_EXP_STAGES> e;
    int use = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int m0 = (t / n_tiles_n) * 128, n0 = (t % n_tiles_n) * 128;
      const int64_t row = (int64_t)m0 + trow;
      float2 acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = make_float2(0.f, 0.f);
      for (int st = 0; st < n_main && ok; ++st) {
        if (!mbar_wait(expf_bar(e.s), e.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
        const float* aux = reinterpret_cast<const float*>(smem + e.s * GI_EXP_STAGE_BYTES + 2 * GI_TILE_BYTES);
        const int pair = use & 1;
        if (!mbar_wait(accf_bar(pair), (use >> 1) & 1, abort_flag, a.status, ERR_WAIT_ACC_FULL)) { ok = false; break; }
        __syncwarp();
        tc_fence_after();
        ++use;
        const int nc = min(2, a.n_chunks - st * 2);
        for (int c = 0; c < nc; ++c) {
          uint32_t v[32];
          tmem_ld32(tlane + (2 * pair + c) * 128, v);
          tmem_wait_ld();
          if (c == nc - 1) {                       // both chunks are out of TMEM: hand the pair back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(pair));
          }
          const float sx = aux[256 + c * 128 + trow];
          const float2 sx2 = make_float2(sx, sx);
          const float4* sw4 = reinterpret_cast<const float4*>(aux + c * 128 + cq * 32);
          const float4* ws4 = reinterpret_cast<const float4*>(aux + 512 + c * 128 + cq * 32);
          float zf = 0.f;
          if constexpr (ASYM) zf = aux[768 + c * 128 + trow];
          const float2 nz2 = make_float2(-zf, -zf);
          const float2 nmagic = make_float2(-12582912.f, -12582912.f);
          if constexpr (DUMP) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float f = __int_as_float((int)v[j] + 0x4B400000) - 12582912.f;
              if constexpr (ASYM) f = __fmaf_rn(-zf, aux[512 + c * 128 + cq * 32 + j], f);
              if (row < a.M && n0 + cq * 32 + j < a.N)
                a.acc_dump[((int64_t)(st * 2 + c) * a.M + row) * a.N + n0 + cq * 32 + j] = (int)(f * INV_F);
            }
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 s4 = sw4[j4];
            float4 w4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if constexpr (ASYM) w4 = ws4[j4];
            const float2 sp[2] = {make_float2(s4.x, s4.y), make_float2(s4.z, s4.w)};
            const float2 wp[2] = {make_float2(w4.x, w4.y), make_float2(w4.z, w4.w)};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int j = 4 * j4 + 2 * u;
              // exact int32 -> fp32 for |v| < 2^22: add 1.5 * 2^23 as integer, subtract as float
              float2 f = make_float2(__int_as_float((int)v[j] + 0x4B400000), __int_as_float((int)v[j + 1] + 0x4B400000));
              f = __fadd2_rn(f, nmagic);
              if constexpr (ASYM) f = __ffma2_rn(nz2, wp[u], f);
              acc[j >> 1] = __ffma2_rn(__fmul2_rn(f, sp[u]), sx2, acc[j >> 1]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(expe_bar(e.s));
        e.next();
      }
      if (ok && n_tail > 0) {
        for (int st = 0; st < n_tail; ++st) {
          if (!mbar_wait(expf_bar(e.s), e.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
          __syncwarp();
          if (lane == 0) mbar_arrive(expe_bar(e.s));
          e.next();
        }
        const int pair = use & 1;
        if (ok && mbar_wait(accf_bar(pair), (use >> 1) & 1, abort_flag, a.status, ERR_WAIT_ACC_FULL)) {
          __syncwarp();
          tc_fence_after();
          uint32_t v[32];
          tmem_ld32(tlane + (2 * pair) * 128, v);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acce_bar(pair));
          ++use;
#pragma unroll
          for (int j = 0; j < 16; ++j) { acc[j].x += __uint_as_float(v[2 * j]); acc[j].y += __uint_as_float(v[2 * j + 1]); }
        } else {
          ok = false;
        }
      }
      if (ok && row < a.M) {
        const int64_t col0 = (int64_t)n0 + cq * 32;
        __nv_bfloat16* yr = a.y + row * a.N + col0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (col0 + 8 * i + 8 <= a.N) {
            float b[8];
            if (a.bias) {
              const uint4 bb = __ldg(reinterpret_cast<const uint4*>(a.bias + col0 + 8 * i));
              const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
              for (int e2 = 0; e2 < 4; ++e2) { float2 f = __bfloat1622float2(bh[e2]); b[2 * e2] = f.x; b[2 * e2 + 1] = f.y; }
            } else {
#pragma unroll
              for (int e2 = 0; e2 < 8; ++e2) b[e2] = 0.f;
            }
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              __nv_bfloat162 h = __floats2bfloat162_rn(acc[4 * i + e2].x + b[2 * e2], acc[4 * i + e2].y + b[2 * e2 + 1]);
              w[e2] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(yr + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 128 * GI_NACC);
  }
}

template <int A_MODE, bool DUMP>
static int launch_gi(const GiMaps& tm, const GemmIntArgs& a, cudaStream_t st) {
  auto k = gemm_int_kernel<A_MODE, DUMP>;
  static PerDeviceOnce attr_once;
  if (int rc = set_max_dynamic_smem(attr_once, k, GiCfg<A_MODE>::SMEM_BYTES)) return rc;
  const int tiles = (int)((a.N + 127) / 128) * (int)((a.M + 127) / 128);
  const int grid = min(tiles, num_sms());
  k<<<grid, GI_THREADS, GiCfg<A_MODE>::SMEM_BYTES, st>>>(tm, a);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int launch_gemm_int(const GemmIntArgs& a, cudaStream_t st) {
  if (a.M <= 0 || a.N <= 0) return DIROTQ_OK;
  if (reinterpret_cast<uintptr_t>(a.bias) & 15) return DIROTQ_E_ALIGN;
  GiMaps tm;
  const bool a8 = a.a_mode == DIROTQ_INT8_ASYM;
  const bool asym = a.a_mode != DIROTQ_INT4_SYM;
  int rc = make_tmap_2d_ex(&tm.xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, (uint64_t)a.x_row_bytes, (uint64_t)a.M,
                           (uint64_t)a.x_row_bytes, a8 ? 128 : 64, 128, false);
  if (rc) return rc;
  rc = make_tmap_2d_ex(&tm.wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.wq, (uint64_t)a.w_row_bytes, (uint64_t)a.N,
                       (uint64_t)a.w_row_bytes, 64, 128, false);
  if (rc) return rc;
  rc = make_tmap_2d_ex(&tm.ws, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.ws, (uint64_t)a.N, (uint64_t)a.n_chunks,
                       (uint64_t)a.ldn * 4, 128, 2, false);
  if (rc) return rc;
  rc = make_tmap_2d_ex(&tm.xs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.xs, (uint64_t)a.M, (uint64_t)a.n_chunks,
                       (uint64_t)a.ldm * 2, 128, 2, false);
  if (rc) return rc;
  if (asym) {
    rc = make_tmap_2d_ex(&tm.wsum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.wsum, (uint64_t)a.N, (uint64_t)a.n_chunks,
                         (uint64_t)a.ldn * 4, 128, 2, false);
    if (rc) return rc;
    rc = make_tmap_2d_ex(&tm.xz, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.xz, (uint64_t)a.M, (uint64_t)a.n_chunks,
                         (uint64_t)a.ldm * 2, 128, 2, false);
    if (rc) return rc;
  } else {
    tm.wsum = tm.ws;
    tm.xz = tm.xs;
  }
  if (a.kt > 0) {
    rc = make_tmap_2d(&tm.xt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.xt, (uint64_t)a.kt, (uint64_t)a.M, (uint64_t)a.kt_pitch * 2, 128);
    if (rc) return rc;
    rc = make_tmap_2d(&tm.wt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.wt, (uint64_t)a.kt, (uint64_t)a.N, (uint64_t)a.kt_pitch * 2, 128);
    if (rc) return rc;
  } else {
    tm.xt = tm.xq;
    tm.wt = tm.wq;
  }
  switch (a.a_mode) {
    // the per-chunk int32 dump (tests) is a separate instantiation: the production kernel carries none of its code
    case DIROTQ_INT4_SYM: return a.acc_dump ? launch_gi<MODE_INT4_SYM, true>(tm, a, st) : launch_gi<MODE_INT4_SYM, false>(tm, a, st);
    case DIROTQ_INT4_ASYM: return a.acc_dump ? launch_gi<MODE_INT4_ASYM, true>(tm, a, st) : launch_gi<MODE_INT4_ASYM, false>(tm, a, st);
    case DIROTQ_INT8_ASYM: return a.acc_dump ? launch_gi<MODE_INT8_ASYM, true>(tm, a, st) : launch_gi<MODE_INT8_ASYM, false>(tm, a, st);
  }
  return DIROTQ_E_UNSUPPORTED;
}

}  // namespace dq
