// Kernel 2 (INT4, tensor-rate variant): W4A4 GEMM whose 4-bit operands are dequantised to fp16 on their
// way to the tensor core, so that ONE fp32 accumulator runs over the whole K and the per-chunk
// CUDA-core drain of the exact-integer kernel (gemm_int.cu) disappears.
//
//   y[m,n] = rs[m] cs[n] ( sum_k a'[m,k] b'[n,k] + xt'[m,:] . wt'[n,:] ) + bias[n]
//   a'[m,k] = (qx[m,k] - zx[m,c]) * sx[m,c] / rs[m]      exact in fp16 for symmetric codes
//   b'[n,k] =  qw[n,k]            * sw[n,c] / cs[n]      rounded once to fp16 (11 bits; the reference
//                                                         keeps bf16(qw * sw), 8 bits)
//   rs[m], cs[n] = powers of two that bring a row's / a column's largest scale to [2^-10, 2^-9)
//
// This is the arithmetic of the reference's own linear on the fake-quantised tensor
// (DiRotQ dirotq_fused_unrotation_fast.py:141: a 16-bit GEMM with fp32 accumulation over
// s*(q-z) and the stored weight), with operands that stay 4-bit in HBM, L2 and the TMA ring.
//
// Nibble -> fp16 without integer-to-float conversion: a nibble m left in the low mantissa bits of an
// otherwise zero half is the subnormal m * 2^-24; one fused multiply-add with the pre-scaled group
// scale (s * 2^24) and the addend -(z * s) gives (m - z) * s with a single rounding.  Two nibbles
// of a byte are taken in place (bits 0-3 and 4-7, the latter with the multiplier s * 2^20), so a
// 32-bit word of eight codes costs one shift, four logic ops and four packed FMAs.
// The order in which a chunk's 64 values land along K is a fixed permutation, the same for both
// operands, which a dot product does not see.
//
// Conversion work (issue slots, shared-memory stores), not tensor arithmetic, bounds a kernel that expands
// operands on chip, and every CTA that expands a weight tile repeats what M / 128 other CTAs do.  So:
//   * the weight operand is expanded ONCE per call by a small pre-pass (expand_weight_panel_kernel: codes
//     + records -> an fp16 [N, K] panel in scratch, 2 bytes per weight, L2-resident for DiT layer sizes;
//     the stored weights stay 4-bit) and reaches the operand ring by TMA, already swizzled;
//   * the activation operand never touches shared memory in expanded form: its converter threads (one
//     per row = one TMEM lane) store the fp16 values straight into tensor memory, and the UMMA takes A
//     from TMEM, B from smem.
//
// Data flow per persistent CTA (128 x BN output tiles, K walked in 64-wide chunks):
//   TMA (A)        4-bit codes (four chunks = 128 B per row per stage, 128-byte swizzle) + per-row records of
//                  the chunk's multipliers (bulk copies) -> "raw" ring
//   TMA (B)        one BN x 64 fp16 tile of the panel (or of the bf16 tail weights) per operand stage, straight
//                  into the stage's 128-byte-swizzled K-major slot as soon as the UMMAs that read it retire
//   converter warps  two groups of four taking alternate chunks; a warp expands 32 activation rows into TMEM
//                  (tcgen05.st); for a tail stage it copies the bf16 rows from the raw ring instead
//   UMMA issuer    tcgen05.mma kind::f16 (A from TMEM, B from smem descriptor), 4 x K=16 per chunk, fp32
//                  128 x BN accumulator in TMEM; the bf16 tail accumulates into the same tile
//   8 epilogue warps  tcgen05.ld, * rs[m] * cs[n], + bias, bf16 -> 32 x 32 staging patches -> TMA stores; two
//                  accumulators alternate so the next tile's UMMAs overlap the epilogue
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"
#include "quant_math.cuh"

namespace dq {

#ifndef GF_CPS_DEF
#define GF_CPS_DEF 4
#endif
#ifndef GF_RAW_DEF
#define GF_RAW_DEF 2
#endif
#ifndef GF_EXP_MAX
#define GF_EXP_MAX 8
#endif
#ifndef GF_GROUPS
#define GF_GROUPS 2
#endif
constexpr int GF_CPS = GF_CPS_DEF;   // chunks per raw stage: 128 bytes of codes per row and stage
constexpr int GF_EPI_WARPS = 8;

// A chunk of a 128-row tile is four conversion units of 32 rows (a thread per row = TMEM lane); a group is
// the four warps that cover the four lane quarters.
template <int BN, bool A8 = false> struct GfCfg {
  static constexpr int GROUP_WARPS = 4;
  static constexpr int GROUPS = GF_GROUPS;
  static constexpr int CONV_WARPS = GROUPS * GROUP_WARPS;
  static constexpr int THREADS = (GF_EPI_WARPS + 3 + CONV_WARPS) * 32;
  static constexpr int B_EXP = BN * 128;                   // BN rows x 64 halves
  static constexpr int EXP_STAGE = B_EXP;                  // only the weight operand is staged in shared memory
  static constexpr int RAW_A = 128 * 32 * GF_CPS * (A8 ? 2 : 1);   // 8-bit activation codes: two 128-byte boxes per row
  static constexpr int OFF_C = RAW_A;                      // [chunk][128] 8-byte records
  static constexpr int RAW_STAGE = OFF_C + GF_CPS * 128 * 8;
  // Accumulators: two (the next tile's UMMAs overlap the epilogue) up to 192 columns; a 256-wide tile has one, and its
  // UMMAs wait until the epilogue has read the previous tile out of tensor memory.
  static constexpr int NACC = BN > 192 ? 1 : 2;
  // Operand stages in flight: every tensor-memory column the accumulators leave free holds activations
  // (32 columns per 64-wide chunk), as far as shared memory holds the weight tiles beside them.
  static constexpr int RAW_STAGES = GF_RAW_DEF;
  static constexpr int STG_BYTES = GF_EPI_WARPS * 2048;     // per epilogue warp: 32 rows x 32 bf16 output staging
  static constexpr int EXP_TMEM = (512 - NACC * BN) / 32;
  static constexpr int EXP_SMEM = (232448 - 1024 - 256 - STG_BYTES - RAW_STAGES * RAW_STAGE) / EXP_STAGE;
  static constexpr int EXP_CAP = EXP_TMEM < GF_EXP_MAX ? EXP_TMEM : GF_EXP_MAX;
  static constexpr int EXP_STAGES = EXP_CAP < EXP_SMEM ? EXP_CAP : EXP_SMEM;
  static constexpr int SMEM_BYTES = EXP_STAGES * EXP_STAGE + RAW_STAGES * RAW_STAGE + STG_BYTES + 1024 + 256;
  static constexpr int TMEM_A0 = NACC * BN;                 // first column of the activation operand slots
  static constexpr int TMEM_COLS = 512;                     // accumulators + EXP_STAGES x 32 columns of A
  static_assert(NACC * BN + EXP_STAGES * 32 <= 512 && EXP_STAGES >= 2, "tensor memory");
  static_assert(SMEM_BYTES <= 232448, "shared memory");
  static_assert(RAW_A >= 128 * 128 && GF_CPS == 4, "a raw stage must hold one 128 x 64 bf16 tail tile of the activations");
};

struct GfMaps {
  CUtensorMap xq, wp, xt, wt, y;
};

template <int N> struct GfRing {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() { if (++s == N) { s = 0; ph ^= 1; } }
};

__device__ __forceinline__ void gf_sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ uint2 gf_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 gf_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// (a & b) ^ c in one logic op
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// One 32-bit word of eight planar nibbles -> four fp16 pairs.
//   xr : per-nibble XOR (0x8 turns a two's-complement nibble into offset binary; 0 for unsigned codes)
//   mlo = (s * 2^24) twice, mhi = (s * 2^20) twice, add = -(z * s) twice (z = 8 for signed codes)
__device__ __forceinline__ void expand_word(uint32_t w, uint32_t xr, uint32_t mlo, uint32_t mhi, uint32_t add, uint32_t* y) {
  const uint32_t t = w >> 8;
  y[0] = hfma2_u(and_xor(w, 0x000F000Fu, xr), mlo, add);
  y[1] = hfma2_u(and_xor(w, 0x00F000F0u, xr << 4), mhi, add);
  y[2] = hfma2_u(and_xor(t, 0x000F000Fu, xr), mlo, add);
  y[3] = hfma2_u(and_xor(t, 0x00F000F0u, xr << 4), mhi, add);
}
__device__ __forceinline__ uint32_t hmul2_2m4(uint32_t m) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(0x2C002C00u));     // * 2^-4
  return r;
}

// AMODE: 0 = signed 4-bit activation codes, 1 = unsigned 4-bit with zero points, 2 = unsigned 8-bit with zero points
template <int BN, int AMODE>
__global__ void __launch_bounds__(GfCfg<BN, AMODE == 2>::THREADS, 1)
gemm_int_f16_kernel(const __grid_constant__ GfMaps tm, const GemmIntF16Args a) {
  constexpr bool ASYM = AMODE != 0, A8 = AMODE == 2;
  using Cfg = GfCfg<BN, A8>;
  constexpr int GF_EXP_STAGES = Cfg::EXP_STAGES, GF_RAW_STAGES = Cfg::RAW_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_area = smem + GF_EXP_STAGES * Cfg::EXP_STAGE;
  uint8_t* stg_area = raw_area + GF_RAW_STAGES * Cfg::RAW_STAGE;       // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg_area + Cfg::STG_BYTES);
  constexpr int NB = 2 * GF_RAW_STAGES + 3 * GF_EXP_STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto rawf_bar = [&](int s) { return bar0 + 8u * s; };
  auto rawe_bar = [&](int s) { return bar0 + 8u * (GF_RAW_STAGES + s); };
  auto expf_bar = [&](int s) { return bar0 + 8u * (2 * GF_RAW_STAGES + s); };
  auto expe_bar = [&](int s) { return bar0 + 8u * (2 * GF_RAW_STAGES + GF_EXP_STAGES + s); };
  auto expw_bar = [&](int s) { return bar0 + 8u * (2 * GF_RAW_STAGES + 2 * GF_EXP_STAGES + s); };   // weight tile landed
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * GF_RAW_STAGES + 3 * GF_EXP_STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * GF_RAW_STAGES + 3 * GF_EXP_STAGES + 2 + b); };

  constexpr int W_MMA = GF_EPI_WARPS, W_TMA = GF_EPI_WARPS + 1, W_TMB = GF_EPI_WARPS + 2;
  if (threadIdx.x == 0) {
    for (int s = 0; s < GF_RAW_STAGES; ++s) { mbar_init(rawf_bar(s), 1); mbar_init(rawe_bar(s), Cfg::CONV_WARPS); }
    for (int s = 0; s < GF_EXP_STAGES; ++s) { mbar_init(expf_bar(s), Cfg::GROUP_WARPS); mbar_init(expe_bar(s), 1); mbar_init(expw_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), GF_EPI_WARPS); }
    abort_flag[0] = 0;
    abort_flag[1] = a.wait_limit_k;
    fence_mbar_init();
    prefetch_tmap(&tm.xq);
    prefetch_tmap(&tm.wp);
  }
  if (warp == W_MMA) tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();
  pdl_wait();                       // the kernels that produced the codes / records have completed
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t exp_base = smem_u32(smem);
  const uint32_t raw_base = smem_u32(raw_area);

  const int n_raw = a.n_chunks;                                    // chunks of codes in the raw stream
  const bool hc = a.half_chunks != 0;                              // two half-padded chunks per operand stage
  const int n_main = hc ? (a.n_chunks + 1) >> 1 : a.n_chunks;      // operand stages of codes
  const int n_tail = (a.kt + 63) >> 6;
  const int n_tiles_n = (int)((a.N + BN - 1) / BN);
  const int n_tiles_m = (int)((a.M + 127) / 128);
  const int total_tiles = n_tiles_n * n_tiles_m;
  // Tile order: column tiles in groups of `a.raster` (n fastest inside a group, then m, then the next group), so the
  // tiles in flight at one time share a bounded set of weight columns and activation rows in L2.
  const int rast = a.raster > 0 && a.raster < n_tiles_n ? a.raster : n_tiles_n;
  auto tile_mn = [&](int t, int& tm_, int& tn_) {
    const int per_group = rast * n_tiles_m;
    const int grp = t / per_group, r = t - grp * per_group;
    const int width = min(rast, n_tiles_n - grp * rast);
    tm_ = r / width;
    tn_ = grp * rast + (r - tm_ * width);
  };
  // Persistent CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ... with n fastest, so CTAs running at
  // the same time read the same activation rows through L2.  Rings and the accumulator counter run on
  // across tiles.  Operand stage q of the kernel-wide sequence (chunks and tail stages of all tiles)
  // lives in slot q % EXP_STAGES; its barrier phase is (q / EXP_STAGES) & 1.

  if (warp == W_TMA) {
    // ------------------------------ TMA producer ---------------------------------------------
    if (lane == 0) {
      GfRing<GF_RAW_STAGES> r;
      uint32_t issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tm_, tn_;
        tile_mn(t, tm_, tn_);
        const int m0 = tm_ * 128;
        for (int c = 0; c < n_raw; c += GF_CPS) {
          if (!mbar_wait_hot(rawe_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sb = raw_base + r.s * Cfg::RAW_STAGE;
          const uint32_t bar = rawf_bar(r.s);
          const int nv = min(GF_CPS, n_raw - c);
          // 8-bit codes: the second 128-byte box is issued only when it holds a chunk (a box that lies
          // wholly outside the tensor is never requested; its bytes are not part of the count either)
          const bool second_box = A8 && nv > 2;
          mbar_expect_tx(bar, (uint32_t)(Cfg::RAW_A - ((A8 && !second_box) ? 128 * 128 : 0) + nv * 128 * 8));
          if constexpr (A8) {
            tma_load_2d(sb, &tm.xq, bar, c * 64, m0);
            if (second_box) tma_load_2d(sb + 128 * 128, &tm.xq, bar, c * 64 + 128, m0);
          } else {
            tma_load_2d(sb, &tm.xq, bar, c * 32, m0);
          }
          for (int j = 0; j < nv; ++j)
            bulk_load(sb + Cfg::OFF_C + j * 128 * 8, a.a_const + ((int64_t)(c + j) * a.ldm + m0), 128 * 8, bar);
          issued |= 1u << r.s;
          r.next();
        }
        // tail: the activations' bf16 tile travels through the raw ring like a chunk (its rows go on to TMEM)
        for (int st = 0; st < n_tail && ok; ++st) {
          if (!mbar_wait_hot(rawe_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t bar = rawf_bar(r.s);
          mbar_expect_tx(bar, 128u * 128u);                    // one 128 x 64 bf16 tile
          tma_load_2d(raw_base + r.s * Cfg::RAW_STAGE, &tm.xt, bar, st * 64, m0);
          issued |= 1u << r.s;
          r.next();
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        for (int i = 0; i < GF_RAW_STAGES; ++i) {
          if (!(issued & (1u << i))) continue;
          const uint32_t last_ph = (i < r.s) ? r.ph : (r.ph ^ 1);
          while (!mbar_try(rawf_bar(i), last_ph))
            if (clock64() - t0 > kWaitLimitCycles / 8) { if (a.status) atomicCAS(a.status, 0, ERR_WAIT_DRAIN); break; }
        }
      }
    }
  } else if (warp == W_TMB) {
    // ------------------------------ weight-tile producer ---------------------------------------
    // Operand stage q's weight tile goes straight into slot q % EXP_STAGES as soon as the slot is free.
    if (lane == 0) {
      int q = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tm_, tn_;
        tile_mn(t, tm_, tn_);
        const int n0 = tn_ * BN;
        for (int st = 0; st < n_main + n_tail; ++st, ++q) {
          const int es = q % GF_EXP_STAGES;
          if (!mbar_wait_hot(expe_bar(es), (uint32_t)(((q / GF_EXP_STAGES) & 1) ^ 1), abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t bar = expw_bar(es);
          mbar_expect_tx(bar, Cfg::B_EXP);                     // the box is counted whole, zero fill included
          if (st < n_main) tma_load_2d(exp_base + es * Cfg::EXP_STAGE, &tm.wp, bar, st * 64, n0);
          else tma_load_2d(exp_base + es * Cfg::EXP_STAGE, &tm.wt, bar, (st - n_main) * 64, n0);
        }
      }
      if (!ok) {
        // the copies of the last EXP_STAGES stages issued may still be in flight
        const long long t0 = clock64();
        for (int qq = max(0, q - GF_EXP_STAGES); qq < q; ++qq)
          while (!mbar_try(expw_bar(qq % GF_EXP_STAGES), (uint32_t)((qq / GF_EXP_STAGES) & 1)))
            if (clock64() - t0 > kWaitLimitCycles / 8) { if (a.status) atomicCAS(a.status, 0, ERR_WAIT_DRAIN); break; }
      }
    }
  } else if (warp > W_TMB) {
    // ------------------------------ converters ------------------------------------------------
    // Two groups take alternate operand stages (stage q goes to group q % GROUPS), so one group's barrier
    // waits, shared-memory latencies and fences overlap the other group's arithmetic.  A warp owns the 32
    // activation rows of its own TMEM lane quarter (warp index mod 4).
    const int cw = warp - (W_TMB + 1);
    constexpr int GW = Cfg::GROUP_WARPS;
    const int grp = cw / GW;
    const int quarter = warp & 3;
    const int rowA = quarter * 32 + lane;
    GfRing<GF_RAW_STAGES> r;
    int q = 0;
    bool ok = true;
    auto exp_slot = [](int qq) { return qq % Cfg::EXP_STAGES; };
    auto exp_phase = [](int qq) { return (uint32_t)((qq / Cfg::EXP_STAGES) & 1); };
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      for (int c = 0; c < n_raw && ok; c += GF_CPS) {
        if (!mbar_wait_hot(rawf_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
        const uint32_t sraw = raw_base + r.s * Cfg::RAW_STAGE;
        const int nv = min(GF_CPS, n_raw - c);
        const int njc = hc ? (nv + 1) >> 1 : nv;               // operand stages this raw stage feeds
        for (int jc = 0; jc < njc; ++jc, ++q) {
          if (q % Cfg::GROUPS != grp) continue;
          // The row is expanded into registers before the slot is known to be free, so that only the
          // tensor-memory store remains on the path between "slot free" and "stage ready".
          uint32_t y1[32];
          if (hc) {
            // half chunks: the first 32 slots of chunks 2 jc and 2 jc + 1, each with its own record, side by side
            const int c0 = 2 * jc, c1 = 2 * jc + 1;
            const bool has1 = c1 < nv;
            const uint2 ka0 = gf_lds64(sraw + Cfg::OFF_C + c0 * 128 * 8 + rowA * 8);
            const uint2 ka1 = has1 ? gf_lds64(sraw + Cfg::OFF_C + c1 * 128 * 8 + rowA * 8) : make_uint2(0u, 0u);
            const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
            if constexpr (A8) {
              const uint32_t rb0 = sraw + (c0 >> 1) * (128 * 128) + rowA * 128, rb1 = sraw + (c1 >> 1) * (128 * 128) + rowA * 128;
              uint4 pq[4];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                pq[u] = gf_lds128(rb0 + ((((c0 & 1) * 4 + u) ^ (rowA & 7)) << 4));
                pq[2 + u] = has1 ? gf_lds128(rb1 + ((((c1 & 1) * 4 + u) ^ (rowA & 7)) << 4)) : z4;
              }
              const uint32_t w16[16] = {pq[0].x, pq[0].y, pq[0].z, pq[0].w, pq[1].x, pq[1].y, pq[1].z, pq[1].w,
                                        pq[2].x, pq[2].y, pq[2].z, pq[2].w, pq[3].x, pq[3].y, pq[3].z, pq[3].w};
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint2 ka = h ? ka1 : ka0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const uint32_t wl = w16[8 * h + i], wh = w16[8 * h + 4 + i];
                  uint32_t* y = y1 + 16 * h + 4 * i;
                  y[0] = hfma2_u(__byte_perm(wl, 0u, 0x4240), ka.x, ka.y);
                  y[1] = hfma2_u(__byte_perm(wh, 0u, 0x4240), ka.x, ka.y);
                  y[2] = hfma2_u(__byte_perm(wl, 0u, 0x4341), ka.x, ka.y);
                  y[3] = hfma2_u(__byte_perm(wh, 0u, 0x4341), ka.x, ka.y);
                }
              }
            } else {
              const uint32_t rb = sraw + rowA * 128;
              const int sw = rowA & 7;
              const uint4 pa0 = gf_lds128(rb + (((2 * c0) ^ sw) << 4));
              const uint4 pa1 = has1 ? gf_lds128(rb + (((2 * c1) ^ sw) << 4)) : z4;
              const uint32_t w8[8] = {pa0.x, pa0.y, pa0.z, pa0.w, pa1.x, pa1.y, pa1.z, pa1.w};
              const uint32_t xr1 = ASYM ? 0u : 0x00080008u;
              const uint32_t mhi0 = hmul2_2m4(ka0.x), mhi1 = hmul2_2m4(ka1.x);
#pragma unroll
              for (int i = 0; i < 4; ++i) expand_word(w8[i], xr1, ka0.x, mhi0, ka0.y, y1 + 4 * i);
#pragma unroll
              for (int i = 4; i < 8; ++i) expand_word(w8[i], xr1, ka1.x, mhi1, ka1.y, y1 + 4 * i);
            }
          } else {
          const uint2 ka = gf_lds64(sraw + Cfg::OFF_C + jc * 128 * 8 + rowA * 8);
          if constexpr (A8) {
            // 8-bit codes: 64 bytes of this row = four 16-byte pieces of box jc >> 1.  A byte alone in a zero
            // half is the subnormal q * 2^-24, so (q - z) * s is one packed FMA again; the values are emitted
            // in the K order the 4-bit weight expansion produces (see expand_word).
            const uint32_t rb = sraw + (jc >> 1) * (128 * 128) + rowA * 128;
            uint4 pq[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) pq[u] = gf_lds128(rb + ((((jc & 1) * 4 + u) ^ (rowA & 7)) << 4));
            const uint32_t w16[16] = {pq[0].x, pq[0].y, pq[0].z, pq[0].w, pq[1].x, pq[1].y, pq[1].z, pq[1].w,
                                      pq[2].x, pq[2].y, pq[2].z, pq[2].w, pq[3].x, pq[3].y, pq[3].z, pq[3].w};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t wl = w16[8 * h + i], wh = w16[8 * h + 4 + i];
                uint32_t* y = y1 + 16 * h + 4 * i;
                y[0] = hfma2_u(__byte_perm(wl, 0u, 0x4240), ka.x, ka.y);
                y[1] = hfma2_u(__byte_perm(wh, 0u, 0x4240), ka.x, ka.y);
                y[2] = hfma2_u(__byte_perm(wl, 0u, 0x4341), ka.x, ka.y);
                y[3] = hfma2_u(__byte_perm(wh, 0u, 0x4341), ka.x, ka.y);
              }
          } else {
            // two 16-byte pieces of the swizzled 128-byte raw row
            const uint32_t rb = sraw + rowA * 128;
            const int sw = rowA & 7;
            const uint4 pa0 = gf_lds128(rb + (((2 * jc) ^ sw) << 4));
            const uint4 pa1 = gf_lds128(rb + (((2 * jc + 1) ^ sw) << 4));
            const uint32_t w8[8] = {pa0.x, pa0.y, pa0.z, pa0.w, pa1.x, pa1.y, pa1.z, pa1.w};
            const uint32_t mhi = hmul2_2m4(ka.x);
            const uint32_t xr1 = ASYM ? 0u : 0x00080008u;
#pragma unroll
            for (int i = 0; i < 8; ++i) expand_word(w8[i], xr1, ka.x, mhi, ka.y, y1 + 4 * i);
          }
          }
          const int es = exp_slot(q);
          if (!mbar_wait_hot(expe_bar(es), exp_phase(q) ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          tc_fence_after();
          tmem_st32(tmem_base + ((uint32_t)(quarter * 32) << 16) + Cfg::TMEM_A0 + es * 32, y1);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(expf_bar(es));
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(rawe_bar(r.s));
        r.next();
      }
      // tail: the activations' bf16 tile (already divided by rs) arrives in the raw ring and its rows are
      // copied to TMEM like an expanded chunk
      for (int st = 0; st < n_tail && ok; ++st, ++q) {
        if (!mbar_wait_hot(rawf_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
        if (q % Cfg::GROUPS == grp) {
          const int es = exp_slot(q);
          const uint32_t rb = raw_base + r.s * Cfg::RAW_STAGE + rowA * 128;
          uint32_t y[32];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 v = gf_lds128(rb + (uint32_t)((i ^ (rowA & 7)) << 4));
            y[4 * i] = v.x; y[4 * i + 1] = v.y; y[4 * i + 2] = v.z; y[4 * i + 3] = v.w;
          }
          if (!mbar_wait_hot(expe_bar(es), exp_phase(q) ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          tc_fence_after();
          tmem_st32(tmem_base + ((uint32_t)(quarter * 32) << 16) + Cfg::TMEM_A0 + es * 32, y);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(expf_bar(es));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(rawe_bar(r.s));
        r.next();
      }
    }
  } else if (warp == W_MMA) {
    // ------------------------------ UMMA issuer ----------------------------------------------
    if (lane == 0) {
      const uint32_t idesc_h = idesc_dense(ACC_F32, FMT_F16, FMT_F16, 128, BN);
      const uint32_t idesc_bf = idesc_dense(ACC_F32, FMT_BF16, FMT_BF16, 128, BN);
      int use = 0;
      bool ok = true;
      // loop-invariant pieces of the per-stage operands: barrier addresses are 8 bytes per slot apart, the weight
      // descriptor's low word holds the slot address >> 4, the activation slots are 32 tensor-memory columns apart
      int es0 = 0;
      uint32_t ph0 = 0;
      const uint32_t expw0 = expw_bar(0);
      constexpr uint32_t kFullOff = 8u * 2 * GF_EXP_STAGES;      // expw_bar(s) - expf_bar(s)
      constexpr uint32_t kEmptyOff = 8u * GF_EXP_STAGES;         // expw_bar(s) - expe_bar(s)
      const uint64_t bdesc0 = smem_desc_sw128(exp_base);
      const uint32_t bdesc_lo0 = (uint32_t)bdesc0, bdesc_hi = (uint32_t)(bdesc0 >> 32);
      constexpr uint32_t kDescStep = Cfg::EXP_STAGE >> 4;
      const uint32_t a_tmem0 = tmem_base + Cfg::TMEM_A0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int buf = Cfg::NACC == 2 ? (use & 1) : 0;
        const uint32_t acc_ph = (uint32_t)(Cfg::NACC == 2 ? (use >> 1) & 1 : use & 1);
        if (!mbar_wait_hot(acce_bar(buf), acc_ph ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + buf * BN;
        // A UMMA occupies the issuing thread until the tensor pipe has taken it, so whatever else this thread
        // does between UMMAs is time the pipe idles; a barrier test costs about a hundred cycles, hit or miss.
        // So stages go two at a time: the four tests of a pair are issued back to back (their latencies
        // overlap) and eight UMMAs follow without a break.
        const int ns = n_main + n_tail;
        for (int st = 0; st < ns && ok;) {
          const bool two = st + 1 < ns;
          // slot / phase of the pair's second stage (the first stage's again when the tile ends on a single one)
          int es1 = es0;
          uint32_t ph1 = ph0;
          if (two && ++es1 == GF_EXP_STAGES) { es1 = 0; ph1 ^= 1u; }
          const uint32_t w0 = expw0 + 8u * es0, w1 = expw0 + 8u * es1;       // expf / expe lie at fixed offsets from expw
          const uint32_t rdy = mbar_test4(w0, ph0, w0 - kFullOff, ph0, w1, ph1, w1 - kFullOff, ph1);
          if (rdy != 15u) {
            if (!(rdy & 1u)) ok = mbar_wait_hot(w0, ph0, abort_flag, a.status, ERR_WAIT_FULL);
            if (ok && !(rdy & 2u)) ok = mbar_wait_hot(w0 - kFullOff, ph0, abort_flag, a.status, ERR_WAIT_FULL);
            if (ok && !(rdy & 4u)) ok = mbar_wait_hot(w1, ph1, abort_flag, a.status, ERR_WAIT_FULL);
            if (ok && !(rdy & 8u)) ok = mbar_wait_hot(w1 - kFullOff, ph1, abort_flag, a.status, ERR_WAIT_FULL);
            if (!ok) break;
          }
          tc_fence_after();
          umma_f16_ts_x4(d, a_tmem0 + 32u * es0, bdesc_lo0 + kDescStep * es0, bdesc_hi, st < n_main ? idesc_h : idesc_bf,
                         st > 0 ? 1u : 0u);
          umma_commit(w0 - kEmptyOff);
          if (two) {
            umma_f16_ts_x4(d, a_tmem0 + 32u * es1, bdesc_lo0 + kDescStep * es1, bdesc_hi, st + 1 < n_main ? idesc_h : idesc_bf, 1u);
            umma_commit(w1 - kEmptyOff);
            st += 2;
          } else {
            st += 1;
          }
          es0 = es1;
          ph0 = ph1;
          if (++es0 == GF_EXP_STAGES) { es0 = 0; ph0 ^= 1u; }
        }
        if (ok) { umma_commit(accf_bar(buf)); ++use; }
      }
    }
  } else {
    // ------------------------------ epilogue: 8 warps -----------------------------------------
    // warp w: TMEM lane quarter w & 3 (32 rows), column half w >> 2 (BN / 2 columns), 32 columns at a time:
    // tcgen05.ld -> * rs[m] * cs[n] + bias -> bf16 -> the warp's 32 x 32 staging patch in shared memory
    // (64-byte rows, 64-byte swizzle: conflict-free) -> one TMA store, which clips the patch at the edges
    // of y.  A row-per-thread store straight to global memory would put 32 separate 16-byte segments per
    // instruction through the load/store unit that the converter warps depend on.
    const int q = warp & 3, ch = warp >> 2;
    const int trow = q * 32 + lane;
    constexpr int CW = BN / 2;
    const uint32_t stg = smem_u32(stg_area) + warp * 2048;
    const uint32_t stg_row = stg + lane * 64;
    const int stg_sw = (lane >> 1) & 3;
    int use = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int tm_, tn_;
      tile_mn(t, tm_, tn_);
      const int m0 = tm_ * 128, n0 = tn_ * BN;
      const int64_t row = (int64_t)m0 + trow;
      const float rs = (row < a.M) ? __ldg(a.rs + row) : 0.f;
      const int buf = Cfg::NACC == 2 ? (use & 1) : 0;
      if (!mbar_wait(accf_bar(buf), (uint32_t)(Cfg::NACC == 2 ? (use >> 1) & 1 : use & 1), abort_flag, a.status, ERR_WAIT_ACC_FULL)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      ++use;
      const uint32_t tl = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + ch * CW;
      if (a.q_codes) {
        // ---- quantise-out: every 64 columns of the tile are one group of the following layer; the two warps of a
        // lane quarter take them alternately (a 192-wide tile: groups 0 and 2 here, group 1 there) ----
#pragma unroll 1
        for (int gi = ch; gi < BN / 64; gi += 2) {
          uint32_t v[64];
          const uint32_t tg = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + gi * 64;
          tmem_ld32(tg, v);
          tmem_ld32(tg + 32, v + 32);
          tmem_wait_ld();
          if (gi + 2 >= BN / 64) {                      // the accumulator is out of TMEM: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(buf));
          }
          const int64_t col0 = (int64_t)n0 + gi * 64;
          if (col0 + 64 > a.N) continue;               // padding of the last tile (N is a multiple of 64 here)
          uint32_t w[32];                               // the activated output, bf16 pairs: what the next quantiser sees
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 c0 = __ldg(reinterpret_cast<const float4*>(a.cs + col0 + 8 * i));
            const float4 c1 = __ldg(reinterpret_cast<const float4*>(a.cs + col0 + 8 * i + 4));
            const float cs8[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
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
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              float f0 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e2]), rs * cs8[2 * e2], b[2 * e2]);
              float f1 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e2 + 1]), rs * cs8[2 * e2 + 1], b[2 * e2 + 1]);
              if (a.act == 1) { f0 = gelu_tanh_bf16(f0); f1 = gelu_tanh_bf16(f1); }
              __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
              w[4 * i + e2] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          if (a.y) {                                    // the bf16 tensor as well, when the caller wants it
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              if (lane == 0) bulk_wait_read0();
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i)
                gf_sts128(stg_row + (uint32_t)((i ^ stg_sw) << 4), w[16 * g + 4 * i], w[16 * g + 4 * i + 1], w[16 * g + 4 * i + 2],
                          w[16 * g + 4 * i + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tm.y, stg, (int)col0 + 32 * g, m0 + q * 32);
                bulk_commit_group();
              }
            }
          }
          if (col0 >= a.q_len) {                        // the following layer's 16-bit channels
            if (row < a.M) {
              uint4* t = reinterpret_cast<uint4*>(a.q_tail + row * a.q_tail_pitch + (col0 - a.q_len));
#pragma unroll
              for (int i = 0; i < 8; ++i) t[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            }
            continue;
          }
          if (row < a.M) {
            const int chunk = (int)(col0 >> 6);
            uint4* dst = reinterpret_cast<uint4*>(a.q_codes + row * a.q_row_bytes + (int64_t)chunk * 32);
            GroupParams p;
            if (a.q_mode == DIROTQ_INT4_SYM) {
              const float amax = fmaxf(fmaxf(amax_bf16x16(w), amax_bf16x16(w + 8)), fmaxf(amax_bf16x16(w + 16), amax_bf16x16(w + 24)));
              p = int_sym_params<true>(amax, -amax, a.q_clip, 7.f);
              const float rcp = __frcp_rn(p.scale);
              dst[0] = int_sym_planar32_packed(w, rcp, a.q_clip < 1.f);
              dst[1] = int_sym_planar32_packed(w + 16, rcp, a.q_clip < 1.f);
            } else {
              float mx = -INFINITY, mn = INFINITY;
              minmax_bf16x16(w, mx, mn);
              minmax_bf16x16(w + 8, mx, mn);
              minmax_bf16x16(w + 16, mx, mn);
              minmax_bf16x16(w + 24, mx, mn);
              p = int_asym_params<true>(mx, mn, a.q_clip, 15.f);
              const float rcp = __frcp_rn(p.scale);
              dst[0] = int_asym_planar32_packed(w, rcp, p.zero);
              dst[1] = int_asym_planar32_packed(w + 16, rcp, p.zero);
              a.q_zeros[(int64_t)chunk * a.q_ldm + row] = __float2bfloat16_rn(p.zero);
            }
            a.q_scales[(int64_t)chunk * a.q_ldm + row] = __float2bfloat16_rn(p.scale);
          }
        }
        continue;
      }
#pragma unroll 1
      for (int g = 0; g < CW / 32; ++g) {
        uint32_t v[32];
        tmem_ld32(tl + g * 32, v);
        tmem_wait_ld();
        if (g == CW / 32 - 1) {                      // the accumulator is out of TMEM: hand it back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acce_bar(buf));
        }
        const int64_t col0 = (int64_t)n0 + ch * CW + g * 32;
        if (col0 >= a.N) continue;                     // warp-uniform: nothing of this patch lies inside y
        if (lane == 0) bulk_wait_read0();              // the previous patch has left the staging buffer
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t w[4] = {0u, 0u, 0u, 0u};
          if (col0 + 8 * i + 8 <= a.N) {
            const float4 c0 = __ldg(reinterpret_cast<const float4*>(a.cs + col0 + 8 * i));
            const float4 c1 = __ldg(reinterpret_cast<const float4*>(a.cs + col0 + 8 * i + 4));
            const float cs8[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
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
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              float f0 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e2]), rs * cs8[2 * e2], b[2 * e2]);
              float f1 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e2 + 1]), rs * cs8[2 * e2 + 1], b[2 * e2 + 1]);
              if (a.act == 1) { f0 = gelu_tanh_bf16(f0); f1 = gelu_tanh_bf16(f1); }
              __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
              w[e2] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          gf_sts128(stg_row + (uint32_t)((i ^ stg_sw) << 4), w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tm.y, stg, (int)col0, m0 + q * 32);
          bulk_commit_group();
        }
      }
    }
    if (lane == 0) bulk_wait_all0();                   // the output is in global memory before the CTA retires
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------
// Scale preparation, per row (activations: token; weights: output channel): the largest
// chunk scale picks the row's power of two; every chunk scale becomes one 8-byte record
// { (s * 2^24 / rs) twice, -(z * s / rs) twice } of fp16 pairs, ready to be used as packed-FMA operands; the row's 16-bit tail is divided by rs (exact) into its own buffer.
// ---------------------------------------------------------------------------------------------------
template <typename ST> __device__ __forceinline__ float scale_to_float(ST v);
template <> __device__ __forceinline__ float scale_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float scale_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ uint32_t half_twice(float v) {
  const uint32_t h = __half_as_ushort(__float2half_rn(v));
  return h | (h << 16);
}

// Block = 64 rows x 4 chunk phases (thread tid: row tid & 63, chunks c = tid >> 6 (mod 4)).
template <typename ST>
__device__ __forceinline__ void fold_scales_block(int block, const ST* __restrict__ s, const __nv_bfloat16* __restrict__ z,
                                                  int n_chunks, int64_t rows, int64_t ld_in, uint2* __restrict__ rec,
                                                  int64_t ld_rec, float* __restrict__ rs, const __nv_bfloat16* __restrict__ tail,
                                                  __nv_bfloat16* __restrict__ tail_out, int kt_pitch) {
  __shared__ float part_max[4][64];
  __shared__ float inv_s[64];
  const int lr = threadIdx.x & 63, part = threadIdx.x >> 6;
  const int64_t r0 = (int64_t)block * 64;
  const int64_t r = r0 + lr;
  // the tail tile's loads go out first: they do not depend on the scales
  const int units = tail ? kt_pitch / 8 : 0;             // 16-byte units per row
  constexpr int TAIL_IT = 4;
  uint4 tv[TAIL_IT];
  int n_it = 0;
  if (tail) {
#pragma unroll
    for (int it = 0; it < TAIL_IT; ++it) {
      const int i = threadIdx.x + it * 256;
      const int rr = i / units;
      if (i < 64 * units && r0 + rr < rows) {
        tv[it] = __ldg(reinterpret_cast<const uint4*>(tail + (r0 + rr) * kt_pitch) + (i % units));
        n_it = it + 1;
      }
    }
  }
  float smax = 0.f;
  if (r < rows)
    for (int c = part; c < n_chunks; c += 4) smax = fmaxf(smax, fabsf(scale_to_float<ST>(s[(int64_t)c * ld_in + r])));
  part_max[part][lr] = smax;
  __syncthreads();
  smax = fmaxf(fmaxf(part_max[0][lr], part_max[1][lr]), fmaxf(part_max[2][lr], part_max[3][lr]));
  int E = (int)((__float_as_uint(smax) >> 23) & 0xFF) - 127;          // smax = 1.f * 2^E
  E = max(-100, min(100, E));
  const float inv = __uint_as_float((uint32_t)(127 - 10 - E) << 23);  // 2^(-10 - E): smax * inv in [2^-10, 2^-9)
  if (part == 0) {
    inv_s[lr] = inv;
    if (r < rows) rs[r] = __uint_as_float((uint32_t)(127 + 10 + E) << 23);
  }
  const float up = inv * 16777216.f;                                    // * 2^24 (E >= -100 keeps this finite)
  if (r < rows) {
    for (int c = part; c < n_chunks; c += 4) {
      const float sc = scale_to_float<ST>(s[(int64_t)c * ld_in + r]);
      const float zp = z ? __bfloat162float(z[(int64_t)c * ld_in + r]) : 8.f;
      rec[(int64_t)c * ld_rec + r] = make_uint2(half_twice(sc * up), half_twice(-zp * sc * inv));
    }
  } else if (r < ld_rec) {
    for (int c = part; c < n_chunks; c += 4) rec[(int64_t)c * ld_rec + r] = make_uint2(0u, 0u);
  }
  if (tail == nullptr) return;
  __syncthreads();
  auto scale_store = [&](int i, uint4 v) {
    const int rr = i / units, u = i % units;
    const float f = inv_s[rr];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = __bfloat1622float2(h[j]);
      h[j] = __floats2bfloat162_rn(x.x * f, x.y * f);
    }
    *(reinterpret_cast<uint4*>(tail_out + (r0 + rr) * kt_pitch) + u) = v;
  };
#pragma unroll
  for (int it = 0; it < TAIL_IT; ++it)
    if (it < n_it) scale_store(threadIdx.x + it * 256, tv[it]);
  // wide tails (more than 4 x 256 units per 64 rows): the rest, load and store in turn
  for (int i = threadIdx.x + TAIL_IT * 256; i < 64 * units; i += 256) {
    const int rr = i / units;
    if (r0 + rr >= rows) break;
    scale_store(i, __ldg(reinterpret_cast<const uint4*>(tail + (r0 + rr) * kt_pitch) + (i % units)));
  }
}

template <typename ST>
__global__ void __launch_bounds__(256)
fold_scales_kernel(const ST* __restrict__ s, const __nv_bfloat16* __restrict__ z, int n_chunks, int64_t rows, int64_t ld_in,
                   uint2* __restrict__ rec, int64_t ld_rec, float* __restrict__ rs,
                   const __nv_bfloat16* __restrict__ tail, __nv_bfloat16* __restrict__ tail_out, int kt_pitch) {
  pdl_launch_dependents();
  pdl_wait();
  fold_scales_block<ST>((int)blockIdx.x, s, z, n_chunks, rows, ld_in, rec, ld_rec, rs, tail, tail_out, kt_pitch);
}

// Weight pre-pass: codes + records -> the fp16 panel [N, n_chunks * 64] the GEMM's weight-tile TMA reads.
// One thread = one row x one chunk: 32 bytes of codes in, 128 bytes out, with the arithmetic and the K
// order of the activation converters (expand_word), so a dot product pairs the right values.
// hc != 0 (half chunks: per-head groups of at most 32 channels, whose chunks are half padding): only the first 32 code slots of
// a chunk are expanded and two chunks share one 64-wide stage of the panel, [N, ceil(n_chunks / 2) * 64].
__device__ __forceinline__ void expand_weight_panel_block(int block, const uint8_t* __restrict__ wq, int64_t w_row_bytes,
                                                          const uint2* __restrict__ rec, int64_t ld_rec, int64_t N, int n_chunks,
                                                          uint4* __restrict__ panel, int hc) {
  const int64_t tid = (int64_t)block * blockDim.x + threadIdx.x;
  if (tid >= N * n_chunks) return;
  const int64_t n = tid / n_chunks;
  const int c = (int)(tid - n * n_chunks);
  const uint4* src = reinterpret_cast<const uint4*>(wq + n * w_row_bytes + (int64_t)c * 32);
  const uint4 p0 = __ldg(src), p1 = __ldg(src + 1);
  const uint2 k = __ldg(rec + (int64_t)c * ld_rec + n);
  const uint32_t w8[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
  const uint32_t mhi = hmul2_2m4(k.x);
  if (hc) {
    const int n_stage = (n_chunks + 1) >> 1;
    uint4* dst = panel + (n * n_stage + (c >> 1)) * 8 + (c & 1) * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t y[4];
      expand_word(w8[i], 0x00080008u, k.x, mhi, k.y, y);
      dst[i] = make_uint4(y[0], y[1], y[2], y[3]);
    }
    if (c == n_chunks - 1 && !(c & 1)) {              // odd chunk count: the last stage's second half is empty
#pragma unroll
      for (int i = 4; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }
  uint4* dst = panel + tid * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t y[4];
    expand_word(w8[i], 0x00080008u, k.x, mhi, k.y, y);
    dst[i] = make_uint4(y[0], y[1], y[2], y[3]);
  }
}

__global__ void __launch_bounds__(256)
expand_weight_panel_kernel(const uint8_t* __restrict__ wq, int64_t w_row_bytes, const uint2* __restrict__ rec, int64_t ld_rec,
                           int64_t N, int n_chunks, uint4* __restrict__ panel, int hc) {
  pdl_launch_dependents();
  pdl_wait();
  expand_weight_panel_block((int)blockIdx.x, wq, w_row_bytes, rec, ld_rec, N, n_chunks, panel, hc);
}

// Both per-call preparations of one GEMM in one launch (each alone is a few microseconds of launch and latency):
// blocks [0, fold_blocks) fold the activation scales, the rest expand the weight panel.
struct FoldExpandArgs {
  const __nv_bfloat16* s; const __nv_bfloat16* z; int n_chunks; int64_t rows; int64_t ld_in; uint2* rec; int64_t ld_rec; float* rs;
  const __nv_bfloat16* tail; __nv_bfloat16* tail_out; int kt_pitch;
  const uint8_t* wq; int64_t w_row_bytes; const uint2* w_rec; int64_t ld_wrec; int64_t N; uint4* panel;
  int fold_blocks;
  int hc;
};
__global__ void __launch_bounds__(256) fold_expand_kernel(const FoldExpandArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x < a.fold_blocks)
    fold_scales_block<__nv_bfloat16>((int)blockIdx.x, a.s, a.z, a.n_chunks, a.rows, a.ld_in, a.rec, a.ld_rec, a.rs, a.tail,
                                     a.tail_out, a.kt_pitch);
  else
    expand_weight_panel_block((int)blockIdx.x - a.fold_blocks, a.wq, a.w_row_bytes, a.w_rec, a.ld_wrec, a.N, a.n_chunks, a.panel,
                              a.hc);
}

int launch_expand_weight_panel(const uint8_t* wq, int n_chunks, int64_t N, const void* rec, void* panel, cudaStream_t st, int hc) {
  if (N <= 0 || n_chunks <= 0) return DIROTQ_OK;
  const int64_t total = N * n_chunks;
  return launch_pdl(expand_weight_panel_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, wq,
                    (int64_t)n_chunks * 32, reinterpret_cast<const uint2*>(rec), f16_ld_weight(N), N, n_chunks,
                    reinterpret_cast<uint4*>(panel), hc) == cudaSuccess
             ? DIROTQ_OK : DIROTQ_E_CUDA;
}

// Records are read in whole tiles of rows (bulk copies, no bounds handling), so the record arrays are
// padded: activations to 128 rows, weights to 768 (a multiple of every column-tile width).
int64_t f16_ld_act(int64_t M) { return round_up64(M, 128); }
int64_t f16_ld_weight(int64_t N) { return round_up64(N, 768); }

int launch_fold_act_scales(const __nv_bfloat16* s, const __nv_bfloat16* z, int n_chunks, int64_t M, int64_t ldm,
                           void* rec, float* rs, const __nv_bfloat16* tail, __nv_bfloat16* tail_out,
                           int kt_pitch, cudaStream_t st) {
  if (M <= 0) return DIROTQ_OK;
  const int64_t ld_rec = f16_ld_act(M);
  return launch_pdl(fold_scales_kernel<__nv_bfloat16>, dim3((unsigned)(ld_rec / 64)), dim3(256), 0, st, s, z, n_chunks, M,
                    ldm, reinterpret_cast<uint2*>(rec), ld_rec, rs, tail, tail_out, kt_pitch) == cudaSuccess
             ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int launch_fold_act_and_expand(const __nv_bfloat16* s, const __nv_bfloat16* z, int n_chunks, int64_t M, int64_t ldm, void* rec,
                               float* rs, const __nv_bfloat16* tail, __nv_bfloat16* tail_out, int kt_pitch, const uint8_t* wq,
                               int64_t N, const void* w_rec, void* panel, cudaStream_t st, int hc) {
  if (M <= 0 || N <= 0) return DIROTQ_OK;
  FoldExpandArgs a;
  a.hc = hc;
  a.s = s; a.z = z; a.n_chunks = n_chunks; a.rows = M; a.ld_in = ldm; a.rec = reinterpret_cast<uint2*>(rec);
  a.ld_rec = f16_ld_act(M); a.rs = rs; a.tail = tail; a.tail_out = tail_out; a.kt_pitch = kt_pitch;
  a.wq = wq; a.w_row_bytes = (int64_t)n_chunks * 32; a.w_rec = reinterpret_cast<const uint2*>(w_rec);
  a.ld_wrec = f16_ld_weight(N); a.N = N; a.panel = reinterpret_cast<uint4*>(panel);
  a.fold_blocks = (int)(a.ld_rec / 64);
  const unsigned blocks = (unsigned)a.fold_blocks + (unsigned)((N * n_chunks + 255) / 256);
  return launch_pdl(fold_expand_kernel, dim3(blocks), dim3(256), 0, st, a) == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int launch_fold_weight_scales(const float* s, int n_chunks, int64_t N, int64_t ldn, void* rec, float* cs,
                              const __nv_bfloat16* tail, __nv_bfloat16* tail_out, int kt_pitch, cudaStream_t st) {
  if (N <= 0) return DIROTQ_OK;
  const int64_t ld_rec = f16_ld_weight(N);
  fold_scales_kernel<float><<<(unsigned)(ld_rec / 64), 256, 0, st>>>(
      s, nullptr, n_chunks, N, ldn, reinterpret_cast<uint2*>(rec), ld_rec, cs, tail, tail_out, kt_pitch);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

template <int BN, int AMODE>
static int launch_gf(const GfMaps& tm, const GemmIntF16Args& a, cudaStream_t st) {
  using Cfg = GfCfg<BN, AMODE == 2>;
  auto k = gemm_int_f16_kernel<BN, AMODE>;
  static PerDeviceOnce attr_once;
  if (int rc = set_max_dynamic_smem(attr_once, k, Cfg::SMEM_BYTES)) return rc;
  const int tiles = (int)((a.N + BN - 1) / BN) * (int)((a.M + 127) / 128);
  const int grid = min(tiles, num_sms());
  return launch_pdl(k, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, tm, a) == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

// Column-tile width.  The persistent grid runs ceil(tiles / SMs) rounds; a round costs, per 64-wide K stage, a part
// proportional to the tile width (the UMMAs) and a part that is the same for every width (the issuer's per-stage barrier
// protocol): 6.84 us for 128 columns and 7.81 us for 192 at K = 1152, i.e. the fixed part is worth about 320 columns.  A
// 256-wide tile has a single accumulator (tensor memory: 256 + 8 x 32 activation columns), so the part of its epilogue
// that reads the accumulator is not hidden behind the next tile's UMMAs: about 2300 column-stages per round more.  The
// choice minimises rounds x ((width + 320) x stages [+ 2300]) -- padded columns and a nearly empty last round both count:
// 256 for long K and widths that divide (3072 -> 12288 at 18432 rows: 1050 us against 1151 with 192; 12288 -> 3072: 968
// against 1112; 2240 x 2240: 143 against 152), 192 for K = 1152 (1152 x 1152 at 16384 rows: 48 us against 59 with 128 or
// 256), 128 where 192 would leave the last of two rounds a third full (1152 x 1152 at 4096 rows: 19.7 us against 21.6).
// DIROTQ_GF_BN overrides.
static int pick_bn_f16(int64_t M, int64_t N, int64_t stages) {
  if (const char* e = getenv("DIROTQ_GF_BN")) return atoi(e);
  const int cand[3] = {256, 192, 128};
  const int64_t m_tiles = (M + 127) / 128, sms = num_sms();
  int best = 128;
  int64_t best_cost = -1;
  for (int i = 0; i < 3; ++i) {
    const int64_t tiles = m_tiles * ((N + cand[i] - 1) / cand[i]);
    const int64_t cost = ((tiles + sms - 1) / sms) * ((cand[i] + 320) * stages + (cand[i] > 192 ? 2300 : 0));
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = cand[i]; }
  }
  return best;
}

// Column tiles per rasterisation group.  With n fastest over the whole width, the CTAs of one round read every weight
// column tile of the layer; once the fp16 panel no longer sits in L2 next to the activation and output streams (3072 ->
// 12288: 75 MB) those reads go to HBM again on every round.  Groups bound the weight tiles in flight to about 24 MB
// (3072 -> 12288 at 18432 rows: 1325 -> 1169 us, 3072 -> 9216: 927 -> 880, 12288 -> 3072: 1172 -> 1126); layers whose
// panel fits (under 32 MB) keep the plain order, which was 1-2 % faster for them.  DIROTQ_GF_RASTER overrides.
static int pick_raster_f16(int BN, int64_t N, int64_t k_total) {
  if (const char* e = getenv("DIROTQ_GF_RASTER")) return atoi(e);
  const int64_t tile_bytes = (int64_t)BN * k_total * 2, panel_bytes = N * k_total * 2;
  if (panel_bytes <= (32ll << 20) || tile_bytes <= 0) return 0;
  const int64_t g = ((24ll << 20) + tile_bytes / 2) / tile_bytes;
  return (int)(g < 4 ? 4 : g > 16 ? 16 : g);
}

int launch_gemm_int_f16(const GemmIntF16Args& a_in, cudaStream_t st) {
  GemmIntF16Args a = a_in;
  if (a.M <= 0 || a.N <= 0) return DIROTQ_OK;
  if (a.a_mode != DIROTQ_INT4_SYM && a.a_mode != DIROTQ_INT4_ASYM && a.a_mode != DIROTQ_INT8_ASYM) return DIROTQ_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a.bias) & 15) || (reinterpret_cast<uintptr_t>(a.cs) & 15) || (a.N & 7) ||
      (reinterpret_cast<uintptr_t>(a.a_const) & 15) || (reinterpret_cast<uintptr_t>(a.w_panel) & 15) || !a.w_panel)
    return DIROTQ_E_ALIGN;
  const int64_t k_stages = (a.half_chunks ? (a.n_chunks + 1) / 2 : a.n_chunks) + (a.kt + 63) / 64;
  int BN = a.force_bn ? a.force_bn : pick_bn_f16(a.M, a.N, k_stages);
  if (a.q_codes) {
    if (a.N % 64 || a.q_len % 64 || a.q_len <= 0 || a.q_len > a.N || a.q_row_bytes < a.q_len / 2 || (a.q_row_bytes & 15) ||
        (a.q_len < a.N && (!a.q_tail || a.q_tail_pitch < a.N - a.q_len || (a.q_tail_pitch & 7) ||
                           (reinterpret_cast<uintptr_t>(a.q_tail) & 15))) ||
        !a.q_scales || (a.q_mode != DIROTQ_INT4_SYM && a.q_mode != DIROTQ_INT4_ASYM) ||
        (a.q_mode == DIROTQ_INT4_ASYM && !a.q_zeros) || (reinterpret_cast<uintptr_t>(a.q_codes) & 15))
      return DIROTQ_E_ARG;
  } else if (!a.y) {
    return DIROTQ_E_ARG;
  }
#ifdef GF_FORCE_BN
  BN = GF_FORCE_BN;
#endif
  GfMaps tm;
  int rc = make_tmap_2d_sw(&tm.xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, (uint64_t)a.x_row_bytes, (uint64_t)a.M,
                           (uint64_t)a.x_row_bytes, 32 * GF_CPS, 128, 32 * GF_CPS);
  if (rc) return rc;
  const uint64_t n_stage = a.half_chunks ? (uint64_t)((a.n_chunks + 1) / 2) : (uint64_t)a.n_chunks;
  if (a.raster == 0) a.raster = pick_raster_f16(BN, a.N, (int64_t)n_stage * 64 + ((a.kt + 63) / 64) * 64);
  rc = make_tmap_2d(&tm.wp, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.w_panel, n_stage * 64, (uint64_t)a.N, n_stage * 128, BN);
  if (rc) return rc;
  // without an output tensor (quantise-out only) the map is never used: any valid address will do
  rc = make_tmap_2d_sw(&tm.y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y ? (const void*)a.y : a.w_panel, (uint64_t)a.N, (uint64_t)a.M, (uint64_t)a.N * 2,
                       32, 32, 64);
  if (rc) return rc;
  if (a.kt > 0) {
    rc = make_tmap_2d(&tm.xt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.xt, (uint64_t)a.kt, (uint64_t)a.M, (uint64_t)a.kt_pitch * 2, 128);
    if (rc) return rc;
    rc = make_tmap_2d(&tm.wt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.wt, (uint64_t)a.kt, (uint64_t)a.N, (uint64_t)a.kt_pitch * 2, BN);
    if (rc) return rc;
  } else {
    tm.xt = tm.xq;
    tm.wt = tm.wp;
  }
  const int amode = a.a_mode == DIROTQ_INT4_SYM ? 0 : a.a_mode == DIROTQ_INT4_ASYM ? 1 : 2;
  switch (BN * 4 + amode) {
    case 256 * 4 + 0: return launch_gf<256, 0>(tm, a, st);
    case 256 * 4 + 1: return launch_gf<256, 1>(tm, a, st);
    case 256 * 4 + 2: return launch_gf<256, 2>(tm, a, st);
    case 192 * 4 + 0: return launch_gf<192, 0>(tm, a, st);
    case 192 * 4 + 1: return launch_gf<192, 1>(tm, a, st);
    case 192 * 4 + 2: return launch_gf<192, 2>(tm, a, st);
    case 128 * 4 + 0: return launch_gf<128, 0>(tm, a, st);
    case 128 * 4 + 1: return launch_gf<128, 1>(tm, a, st);
    case 128 * 4 + 2: return launch_gf<128, 2>(tm, a, st);
  }
  return DIROTQ_E_ARG;
}

}  // namespace dq
