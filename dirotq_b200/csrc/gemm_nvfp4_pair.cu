// Kernel 2 (NVFP4), CTA-pair form: the same product as gemm_nvfp4.cu,
//
//   y = out_scale * c[n] * ( sum over 16-wide blocks  sfx[m,b] sfw[n,b] (e2m1 . e2m1)  +  x_tail . w_tail' ) + bias
//
// computed by clusters of two CTAs that drive ONE tcgen05.mma.cta_group::2 per k-block: a 256 x BN output tile per
// pair, each CTA holding 128 of its rows.  Per 256 K-elements a CTA fetches its own 128 activation rows and only
// HALF of the weight tile (BN/2 rows; the tensor core reads the other half from the peer's shared memory), so a
// 256 x 256 pair tile moves half the operand bytes per flop of the 128 x 128 single-CTA kernel -- which is bound by
// L2 -> SM operand delivery, not by the FP4 pipe.  No load is shared through the cluster: every CTA fetches exactly
// what it keeps.
//
// Roles per CTA: warp 0 = TMA producer (codes and the 512-byte scale-factor tiles by tiled TMA), warp 1 = UMMA issuer
// (leader only; allocates TMEM in both), warps 2..5 = scale-factor movers, warps 6..13 = epilogue.
// Scale factors reach tensor memory through REGISTERS: each mover warp reads the stage's tiles from shared memory
// (16 bytes per lane and k-block) and writes them into its own TMEM lane quarter with tcgen05.st -- the layout
// tcgen05.cp.32x128b.warpx4 would produce, four identical copies.  Measured on this kernel, the twelve tcgen05.cp per
// stage held the UMMA issuer's queue for about as long as the stage's four UMMAs (573 us against 386 us without
// them on a 16384 x 3072 x 12288 layer); the movers run beside the issuer instead of inside its instruction stream.
// Barriers: full[s] lives in the leader: one expect-tx arrival for the operand bytes of both CTAs plus one arrival per
// mover warp of the pair, made once its tcgen05.st have completed (arrivals from the peer carry no memory ordering:
// their payload is tensor memory, and a cluster-scope release costs about a microsecond each); sf_full[s] in each CTA
// (its own scale-factor bytes); empty[s] and accumulator-full in each CTA (the leader commits to both);
// accumulator-empty in the leader (epilogue warps of both CTAs arrive on it).
//
// BN = 256: one 256-column accumulator (TMEM: 256 + scale-factor slots); the epilogue pulls its 128 x 256 fp32 half
// into registers first and hands the accumulator back before converting and storing, so the next tile's main loop
// waits only for that pull.  BN = 128: two 128-column accumulators, epilogue fully overlapped.
//
// Replaces `self.module(x)` of the fused forward (DiRotQ dirotq_fused_unrotation_fast.py:141) for
// quant_dtype == "nvfp4"; the reference's speed path uses nunchaku's FP4 gemm_w4a4 here.
#include <cstring>
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "ptx.cuh"
#include "ptx_pair.cuh"
#include "tma_host.cuh"
#include "quant_math.cuh"

namespace dq {

template <int BN>
struct GpCfg {
  static constexpr int A_BYTES = 128 * 128;                 // 128 rows x 256 E2M1 (or 64 bf16)
  static constexpr int B_BYTES = (BN / 2) * 128;            // this CTA's half of the weight tile
  static constexpr int SFA_BYTES = 4 * 512;                 // four k-blocks of scale factors for 128 rows
  static constexpr int SFB_BYTES = (BN / 128) * 4 * 512;    // all BN weight rows: each CTA needs every column's factors
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = BN == 256 ? 5 : 6;
  static constexpr int NACC = BN == 256 ? 1 : 2;
  static constexpr int EPI_WARPS = 8;                       // two per TMEM lane quarter, BN/2 output columns each
  static constexpr int SF_WARPS = 4;                        // one per TMEM lane quarter
  static constexpr int EPI_WARP0 = 2 + SF_WARPS;
  static constexpr int THREADS = (2 + SF_WARPS + EPI_WARPS) * 32;
  static constexpr int STG_BYTES = EPI_WARPS * 2 * 2048;    // per epilogue warp: two 32 rows x 32 bf16 staging patches
  static constexpr int TAB_BYTES = BN * 8;                  // per output column of the tile: {scale, bias} as floats
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_BYTES + TAB_BYTES + 1024 + 256;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t SF_COL = 256;                   // one slot per shared-memory stage:
  static constexpr uint32_t SF_SLOT = 16 + 16 * (BN / 128); //   16 columns for the activations' factors + 16 per 128 weight rows
  static constexpr uint32_t OP_TX = 2u * (A_BYTES + B_BYTES);   // operand bytes of both CTAs, counted in the leader
  static constexpr uint32_t SF_TX = SFA_BYTES + SFB_BYTES;      // scale-factor bytes, counted in each CTA
  static constexpr int NBARS = 3 * STAGES + 8;
  static_assert(SF_COL + STAGES * SF_SLOT <= TMEM_COLS, "tensor memory");
  static_assert(STAGE_BYTES % 1024 == 0, "operand tiles need 1024-byte alignment");
  static_assert(SMEM_BYTES <= 232448, "shared memory");
};

template <int STAGES>
struct GfRingT {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() { if (++s == STAGES) { s = 0; ph ^= 1; } }
};

// QOUT: the epilogue also quantises its output for a following NVFP4 layer (GemmFp4Args::q_codes).  A separate
// instantiation, so that the registers this costs do not weigh on the plain kernel.
template <int BN, bool QOUT>
__global__ void __launch_bounds__(GpCfg<BN>::THREADS, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tm_xq, const __grid_constant__ CUtensorMap tm_wq,
                       const __grid_constant__ CUtensorMap tm_xsf, const __grid_constant__ CUtensorMap tm_wsf,
                       const __grid_constant__ CUtensorMap tm_xt, const __grid_constant__ CUtensorMap tm_wt,
                       const __grid_constant__ CUtensorMap tm_y, const GemmFp4Args a) {
  using Cfg = GpCfg<BN>;
  constexpr int STAGES = Cfg::STAGES, NACC = Cfg::NACC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stg_area = smem + STAGES * Cfg::STAGE_BYTES;                 // 1024-byte aligned
  float2* col_tab = reinterpret_cast<float2*>(stg_area + Cfg::STG_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg_area + Cfg::STG_BYTES + Cfg::TAB_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 = leader (issues the UMMAs), 1 = peer
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto sffull_bar = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (3 * STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (3 * STAGES + 2 + b); };
  auto tab_bar = [&](int half, int which) { return bar0 + 8u * (3 * STAGES + 4 + 2 * half + which); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1 + 2 * Cfg::SF_WARPS);     // producer's expect-tx arrival + the pair's eight mover warps
      mbar_init(empty_bar(s), 1);
      mbar_init(sffull_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accf_bar(b), 1);
      mbar_init(acce_bar(b), 2 * Cfg::EPI_WARPS);
      mbar_init(tab_bar(b, 0), 4);
      mbar_init(tab_bar(b, 1), 4);
    }
    abort_flag[0] = 0;
    abort_flag[1] = a.wait_limit_k;
    fence_mbar_init();
    prefetch_tmap(&tm_xq);
    prefetch_tmap(&tm_wq);
    prefetch_tmap(&tm_xsf);
    prefetch_tmap(&tm_wsf);
    if (a.kt > 0) { prefetch_tmap(&tm_xt); prefetch_tmap(&tm_wt); }
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();               // both CTAs' barriers are initialised before anything arrives on them remotely
  tc_fence_after();
  pdl_launch_dependents();
  pdl_wait();                       // the kernel that produced the codes has completed
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);

  const int m_pairs = (int)((a.M + 255) / 256), n_tiles = (int)((a.N + BN - 1) / BN);
  const int total_tiles = m_pairs * n_tiles;
  const int n_main = (a.n_chunks + 3) >> 2;      // stages of 256 K-elements
  const int n_tail = (a.kt + 63) >> 6;           // stages of 64 bf16
  const int nkb_pad = n_main * 4;                // 64-element k-blocks per row tile in the scale-factor arrays
  const int first = (int)cluster_id_x(), step = (int)cluster_count_x();

  if (warp == 0) {
    if (lane == 0) {
      GfRingT<STAGES> r;
      bool ok = true;
      for (int t = first; t < total_tiles && ok; t += step) {
        const int mp = t / n_tiles, nb = t - mp * n_tiles;
        const int row_a = mp * 256 + (int)rank * 128;            // this CTA's activation rows
        const int row_b = nb * BN + (int)rank * (BN / 2);        // this CTA's half of the weight rows
        for (int st = 0; st < n_main + n_tail; ++st) {
          if (!mbar_wait(empty_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + r.s * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint32_t fb = map_to_rank(full_bar(r.s), 0);     // completions are counted in the leader
          if (rank == 0) mbar_expect_tx(full_bar(r.s), Cfg::OP_TX);
          if (st < n_main) {
            // scale-factor tiles first (the movers need them before the UMMAs need the codes): "rows" of 512 bytes,
            // tile (row block, k-block) at row  row_block * nkb_pad + k-block
            const uint32_t sSF = sB + Cfg::B_BYTES;
            mbar_expect_tx(sffull_bar(r.s), Cfg::SF_TX);
            tma_load_2d(sSF, &tm_xsf, sffull_bar(r.s), 0, (row_a >> 7) * nkb_pad + st * 4);
#pragma unroll
            for (int h = 0; h < BN / 128; ++h)
              tma_load_2d(sSF + Cfg::SFA_BYTES + h * 2048, &tm_wsf, sffull_bar(r.s), 0, (nb * (BN / 128) + h) * nkb_pad + st * 4);
            tma_load_2d_pair(sA, &tm_xq, fb, st * 128, row_a);
            tma_load_2d_pair(sB, &tm_wq, fb, st * 128, row_b);
          } else {
            mbar_arrive(sffull_bar(r.s));                          // no scale factors in a 16-bit stage: phases stay in step
            tma_load_2d_pair(sA, &tm_xt, fb, (st - n_main) * 64, row_a);
            tma_load_2d_pair(sB, &tm_wt, fb, (st - n_main) * 64, row_b);
          }
          r.next();
        }
      }
      if (!ok) {
        // copies of this CTA may still be in flight towards its shared memory; their completion is counted in the
        // leader, so the peer cannot test it: give them a bounded time before the CTA may retire
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_f4 = idesc_nvf4(256, BN);
      const uint32_t idesc_bf = idesc_dense(ACC_F32, FMT_BF16, FMT_BF16, 256, BN);
      GfRingT<STAGES> r;
      int buf = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = first; t < total_tiles && ok; t += step) {
        if (!mbar_wait(acce_bar(buf), aph ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * BN;
        for (int st = 0; st < n_main + n_tail; ++st) {
          // one wait covers the operand bytes of both CTAs and the scale factors in both CTAs' tensor memory
          if (!mbar_wait(full_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + r.s * Cfg::STAGE_BYTES;
          const uint64_t adesc = smem_desc_sw128(sA), bdesc = smem_desc_sw128(sA + Cfg::A_BYTES);
          if (st < n_main) {
            const uint32_t sfa_t = tmem_base + Cfg::SF_COL + r.s * Cfg::SF_SLOT, sfb_t = sfa_t + 16;
            const int nkb = min(4, a.n_chunks - st * 4);
            for (int kb = 0; kb < nkb; ++kb)
              umma_nvf4_pair(d, adesc + 2 * kb, bdesc + 2 * kb, idesc_f4, (st > 0 || kb > 0) ? 1u : 0u, sfa_t + kb * 4,
                             sfb_t + kb * (BN / 32));
          } else {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) umma_f16_pair(d, adesc + 2 * kb, bdesc + 2 * kb, idesc_bf, 1u);
          }
          // the stage is free in BOTH CTAs once these UMMAs have read it
          umma_commit_pair(empty_bar(r.s));
          umma_commit_pair(map_to_rank(empty_bar(r.s), 1));
          r.next();
        }
        if (!ok) break;
        umma_commit_pair(accf_bar(buf));
        umma_commit_pair(map_to_rank(accf_bar(buf), 1));
        if (NACC == 2) {
          buf ^= 1;
          if (buf == 0) aph ^= 1;
        } else {
          aph ^= 1;
        }
      }
    }
  } else if (warp < Cfg::EPI_WARP0) {
    // ---- scale-factor movers: shared memory -> registers -> this warp's TMEM lane quarter ----
    const uint32_t q = warp & 3;
    const uint32_t ready_leader = map_to_rank(full_bar(0), 0);
    GfRingT<STAGES> r;
    bool ok = true;
    for (int t = first; t < total_tiles && ok; t += step) {
      for (int st = 0; st < n_main + n_tail; ++st) {
        // one lane polls (thirty-two pollers per warp would load the shared-memory pipe the UMMAs read through)
        int got = 1;
        if (lane == 0) got = mbar_wait_hot(sffull_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_SF) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, got, 0)) { ok = false; break; }
        if (st < n_main) {
          const uint32_t sSF = smem_base + r.s * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::B_BYTES + lane * 16;
          const uint32_t tdst = tmem_base + ((q * 32u) << 16) + Cfg::SF_COL + r.s * Cfg::SF_SLOT;
          uint32_t v[16];
          // activations: k-block kb -> columns 4 kb .. 4 kb + 3 (word j = rows 32 j + lane of the 128-row tile)
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[4 * kb]), "=r"(v[4 * kb + 1]), "=r"(v[4 * kb + 2]), "=r"(v[4 * kb + 3]) : "r"(sSF + kb * 512));
          tmem_st16(tdst, v);
          // weights: BN / 128 row blocks side by side per k-block (columns (BN / 32) kb + 4 h ..)
#pragma unroll
          for (int c = 0; c < BN / 128; ++c) {            // 16 columns per store
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = 16 * c + 4 * j;              // first of four columns inside the weights' slot
              const int kb = col / (BN / 32), h = (col % (BN / 32)) / 4;
              asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(v[4 * j]), "=r"(v[4 * j + 1]), "=r"(v[4 * j + 2]), "=r"(v[4 * j + 3])
                           : "r"(sSF + Cfg::SFA_BYTES + h * 2048 + kb * 512));
            }
            tmem_st16(tdst + 16 + 16 * c, v);
          }
          tmem_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(full_bar(r.s));
          else mbar_arrive_cluster_relaxed(ready_leader + 8u * r.s);
        }
        r.next();
      }
    }
  } else {
    constexpr int WCOLS = BN / 2;                       // output columns per epilogue warp
    const int ew = warp - Cfg::EPI_WARP0;
    const int q = warp & 3, half = ew >> 2;
    const uint32_t stg = smem_u32(stg_area) + ew * 4096;
    const uint32_t acce_leader = map_to_rank(acce_bar(0), 0);
    float2* tab = col_tab + half * WCOLS;               // this half's {scale, bias} per column, shared by its four warps
    constexpr int CPW = WCOLS / 4;                      // table columns filled by each of the half's four warps
    const int tcol = (ew & 3) * CPW + lane;             // this thread's column of the table (lanes below CPW)
    int buf = 0;
    uint32_t aph = 0, patch = 0, tph = 0;
    for (int t = first; t < total_tiles; t += step) {
      const int mp = t / n_tiles, nb = t - mp * n_tiles;
      const int row0 = mp * 256 + (int)rank * 128 + q * 32;
      const int64_t n0 = (int64_t)nb * BN + half * WCOLS;
      // per-column factors of this tile, fetched while the UMMAs of the tile still run: y = acc * scale + bias
      // (hand-offs between the half's four warps go through mbarriers: their waits are bounded like all others)
      __syncwarp();
      if (lane == 0) mbar_arrive(tab_bar(half, 0));
      if (!mbar_wait(tab_bar(half, 0), tph, abort_flag, a.status, ERR_WAIT_ACC_FULL)) break;   // all four are done with the last table
      if (lane < CPW) {
        const int64_t col = n0 + tcol;
        float2 e = make_float2(0.f, 0.f);
        if (col < a.N) {
          e.x = a.col_scale ? __ldg(a.col_scale + col) * a.out_scale : a.out_scale;
          e.y = a.bias ? __bfloat162float(a.bias[col]) : 0.f;
        }
        tab[tcol] = e;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(tab_bar(half, 1));
      if (!mbar_wait(tab_bar(half, 1), tph, abort_flag, a.status, ERR_WAIT_ACC_FULL)) break;   // table complete
      tph ^= 1;
      // a single accumulator keeps the UMMA issuer waiting for this pull: poll instead of sleeping
      if (!(NACC == 1 ? mbar_wait_hot(accf_bar(buf), aph, abort_flag, a.status, ERR_WAIT_ACC_FULL)
                      : mbar_wait(accf_bar(buf), aph, abort_flag, a.status, ERR_WAIT_ACC_FULL))) break;
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * WCOLS;
      uint32_t v[WCOLS];
#pragma unroll
      for (int c = 0; c < WCOLS; c += 32) tmem_ld32(taddr + c, v + c);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {                                   // accumulator is in registers: hand it back early
        if (rank == 0) mbar_arrive(acce_bar(buf));
        else mbar_arrive_cluster_relaxed(acce_leader + 8u * buf);
      }
      // bf16 results leave through 32 x 32 staging patches (64-byte rows, 64-byte swizzle; two per warp, used in turn)
      // and TMA stores, which clip at the edges of y
      if constexpr (QOUT) {
        // ---- quantise-out: every 64 columns are one scale-factor word (four blocks of 16) of the following layer ----
        const int64_t row = (int64_t)row0 + lane;
#pragma unroll
        for (int c = 0; c < WCOLS / 64; ++c) {
          const int64_t col0 = n0 + 64 * c;
          if (col0 + 64 > a.N || row0 >= a.M) continue;  // warp-uniform
          uint32_t w[32];                                // the activated output as bf16 pairs: what that layer's quantiser reads
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float4 sb = *reinterpret_cast<const float4*>(tab + 64 * c + 2 * i);
            float f0 = __fmaf_rn(__uint_as_float(v[64 * c + 2 * i]), sb.x, sb.y);
            float f1 = __fmaf_rn(__uint_as_float(v[64 * c + 2 * i + 1]), sb.z, sb.w);
            if (a.act == 1) { f0 = gelu_tanh_bf16(f0); f1 = gelu_tanh_bf16(f1); }
            __nv_bfloat162 h2 = __floats2bfloat162_rn(f0, f1);
            w[i] = *reinterpret_cast<uint32_t*>(&h2);
          }
          if (a.y != nullptr) {                          // the bf16 tensor as well, when the caller wants it
#pragma unroll
            for (int p = 0; p < 2; ++p) {
              const uint32_t sp = stg + (patch & 1u) * 2048;
              ++patch;
              if (lane == 0) bulk_wait_read1();
              __syncwarp();
#pragma unroll
              for (int i4 = 0; i4 < 4; ++i4)
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};"
                             ::"r"(sp + lane * 64 + (uint32_t)((i4 ^ ((lane >> 1) & 3)) << 4)), "r"(w[16 * p + 4 * i4]),
                               "r"(w[16 * p + 4 * i4 + 1]), "r"(w[16 * p + 4 * i4 + 2]), "r"(w[16 * p + 4 * i4 + 3])
                             : "memory");
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tm_y, sp, (int)col0 + 32 * p, row0);
                bulk_commit_group();
              }
            }
          }
          if (row >= a.M) continue;
          if (col0 >= a.q_len) {                         // that layer's 16-bit channels
            uint4* t = reinterpret_cast<uint4*>(a.q_tail + row * a.q_tail_pitch + (col0 - a.q_len));
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            continue;
          }
          uint32_t packed[8];
          uint32_t sfw = 0;
#pragma unroll
          for (int gi = 0; gi < 4; ++gi) {
            float eff;
            const uint8_t sbyte = nvfp4_hw_scale(amax_bf16x16(w + 8 * gi), a.q_clip, a.q_T, &eff);
            uint2 cc = make_uint2(0u, 0u);
            if (eff > 0.f) cc = nvfp4_hw_group_packed(w + 8 * gi, eff);
            packed[2 * gi] = cc.x;
            packed[2 * gi + 1] = cc.y;
            sfw |= (uint32_t)sbyte << (8 * gi);
          }
          const int chunk = (int)(col0 >> 6);
          uint4* dst = reinterpret_cast<uint4*>(a.q_codes + row * a.q_row_bytes + (int64_t)chunk * 32);
          dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          *reinterpret_cast<uint32_t*>(a.q_sf + sf_offset(row, chunk * 4, a.q_n_kb64_pad)) = sfw;
        }
      }
      if constexpr (!QOUT) {
#pragma unroll
      for (int p = 0; p < WCOLS / 32; ++p) {
        const int64_t pcol = n0 + 32 * p;
        if (pcol >= a.N || row0 >= a.M) continue;        // warp-uniform: nothing of this patch lies inside y
        const uint32_t sp = stg + (patch & 1u) * 2048;
        ++patch;
        if (lane == 0) bulk_wait_read1();                // the store issued from this patch two turns ago has read it
        __syncwarp();
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
          const int i = 4 * p + i4;
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float4 sb = *reinterpret_cast<const float4*>(tab + 8 * i + 2 * e);    // {s0, b0, s1, b1}, same address in all lanes
            float f0 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e]), sb.x, sb.y);
            float f1 = __fmaf_rn(__uint_as_float(v[8 * i + 2 * e + 1]), sb.z, sb.w);
            if (a.act == 1) { f0 = gelu_tanh_bf16(f0); f1 = gelu_tanh_bf16(f1); }
            __nv_bfloat162 h2 = __floats2bfloat162_rn(f0, f1);
            w[e] = *reinterpret_cast<uint32_t*>(&h2);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};"
                       ::"r"(sp + lane * 64 + (uint32_t)((i4 ^ ((lane >> 1) & 3)) << 4)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tm_y, sp, (int)pcol, row0);
          bulk_commit_group();
        }
      }
      }
      if (NACC == 2) {
        buf ^= 1;
        if (buf == 0) aph ^= 1;
      } else {
        aph ^= 1;
      }
    }
    if (lane == 0) bulk_wait_all0();                     // the output is in global memory before the CTA retires
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // neither CTA retires (or frees TMEM) while the other may still read its shared memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

static bool nvfp4_pow2_tensor_scale_host(float T) {
  uint32_t u;
  memcpy(&u, &T, 4);
  return T > 0.f && (u & 0x7FFFFFu) == 0u;
}

template <int BN, bool QOUT>
static int launch_pair(const GemmFp4Args& a, cudaStream_t st) {
  using Cfg = GpCfg<BN>;
  CUtensorMap txq, twq, txsf, twsf, txt, twt, ty;
  const uint64_t row_bytes = (uint64_t)a.n_chunks * 32;
  int rc = make_tmap_2d(&txq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, row_bytes, (uint64_t)a.M, row_bytes, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&twq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.wq, row_bytes, (uint64_t)a.N, row_bytes, BN / 2);
  if (rc) return rc;
  // scale-factor tile arrays as [row blocks * k-blocks, 128 words]: a stage's four k-blocks are four consecutive rows
  const uint64_t nkb_pad = (uint64_t)((a.n_chunks + 3) / 4 * 4);
  rc = make_tmap_2d_sw(&txsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.xsf, 128, (uint64_t)((a.M + 127) / 128) * nkb_pad, 512, 128, 4, 0);
  if (rc) return rc;
  rc = make_tmap_2d_sw(&twsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.wsf, 128, (uint64_t)((a.N + 127) / 128) * nkb_pad, 512, 128, 4, 0);
  if (rc) return rc;
  // without an output tensor (quantise-out only) the map is never used: any valid address will do
  rc = make_tmap_2d_sw(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y ? (const void*)a.y : (const void*)a.wq, (uint64_t)a.N,
                       (uint64_t)a.M, (uint64_t)a.N * 2, 32, 32, 64);
  if (rc) return rc;
  if (a.kt > 0) {
    rc = make_tmap_2d(&txt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.xt, (uint64_t)a.kt, (uint64_t)a.M, (uint64_t)a.kt_pitch * 2, 128);
    if (rc) return rc;
    rc = make_tmap_2d(&twt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.wt, (uint64_t)a.kt, (uint64_t)a.N, (uint64_t)a.kt_pitch * 2, BN / 2);
    if (rc) return rc;
  } else {
    txt = txq;
    twt = twq;
  }
  auto k = gemm_nvfp4_pair_kernel<BN, QOUT>;
  static PerDeviceOnce attr_once;
  if (int rc2 = set_max_dynamic_smem(attr_once, k, Cfg::SMEM_BYTES)) return rc2;
  const int tiles = (int)((a.M + 255) / 256) * (int)((a.N + BN - 1) / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // persistent grid: as many pairs as can be resident at once (SM pairs must share a processing cluster, so this can
  // be fewer than half the SM count), remembered per device
  static std::atomic<int> resident[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DIROTQ_E_CUDA;
  int max_pairs = resident[dev].load(std::memory_order_relaxed);
  if (max_pairs <= 0) {
    cfg.gridDim = dim3(2 * (num_sms() / 2));
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&max_pairs, k, &cfg) != cudaSuccess || max_pairs <= 0) max_pairs = num_sms() / 2;
    resident[dev].store(max_pairs, std::memory_order_relaxed);
  }
  cfg.gridDim = dim3(2 * min(tiles, max_pairs));
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, k, txq, twq, txsf, twsf, txt, twt, ty, a) == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

// bn: 128 or 256
int launch_gemm_nvfp4_pair(const GemmFp4Args& a, int bn, cudaStream_t st) {
  if (a.M <= 0 || a.N <= 0) return DIROTQ_OK;
  if (a.n_chunks <= 0) return DIROTQ_E_ARG;
  if (a.N % 8) return DIROTQ_E_UNSUPPORTED;
  if (a.q_codes) {
    if (a.N % 64 || a.q_len % 64 || a.q_len <= 0 || a.q_len > a.N || a.q_row_bytes < a.q_len / 2 || (a.q_row_bytes & 15) ||
        !a.q_sf || (reinterpret_cast<uintptr_t>(a.q_codes) & 15) || (reinterpret_cast<uintptr_t>(a.q_sf) & 15) ||
        a.q_n_kb64_pad * 64 < a.q_len || (a.q_n_kb64_pad & 3) || !nvfp4_pow2_tensor_scale_host(a.q_T) ||
        (a.q_len < a.N && (!a.q_tail || a.q_tail_pitch < a.N - a.q_len || (a.q_tail_pitch & 7) ||
                           (reinterpret_cast<uintptr_t>(a.q_tail) & 15))))
      return DIROTQ_E_ARG;
  } else if (!a.y) {
    return DIROTQ_E_ARG;
  }
  if (a.q_codes) {
    // DIROTQ_NVFP4_QOUT_TILE=128 forces the narrower tile (measurements)
    const char* e = getenv("DIROTQ_NVFP4_QOUT_TILE");
    if (e && !strcmp(e, "128")) bn = 128;
    return bn == 256 ? launch_pair<256, true>(a, st) : launch_pair<128, true>(a, st);
  }
  return bn == 256 ? launch_pair<256, false>(a, st) : launch_pair<128, false>(a, st);
}

}  // namespace dq
