// Kernel 1: fused rotate + split + quantise.
//
//   x [M, D] bf16  --TMA-->  smem (128-byte swizzle)  --tcgen05.mma kind::f16-->  TMEM fp32
//   TMEM --tcgen05.ld--> registers: round to bf16 (this IS x_rot of the reference's bf16 path),
//   split into the quantised region and the passthrough tail, per-group extrema, scale / zero
//   point, 4-bit (or 8-bit) codes, packed 16-byte stores.  The rotated tensor never touches HBM.
//
// Persistent, warp-specialised: warp 0 = TMA producer, warp 1 = UMMA issuer (owns TMEM),
// warps 2..9 = epilogue (two per TMEM lane quarter, alternating over the 64-column groups).  Two TMEM accumulators of 256 columns let
// the epilogue of tile i overlap the main loop of tile i+1.  Tiles are 128 rows x BN columns of
// the rotated tensor; consecutive tiles share the x row-block, so x and the rotation stay in L2.
//
// Replaces: `x_flat @ self.rotation` + find_params + quantizer (DiRotQ
// dirotq_fused_unrotation_fast.py:69-74), the per-head branch (:76-104) and the stand-alone
// rotation kernels speedup/kernels/{int8,fp8,bf16}_rotation.py.
#include <cstdlib>
#include <cstring>
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

constexpr int RQ_A_BYTES = 128 * 128;           // 128 rows x 64 bf16
// One CTA per tile: the whole rotation tile (up to 256 rows x 64 bf16) per stage, four stages.  CTA pairs
// (tcgen05 cta_group::2, 256 token rows per pair): each CTA fetches only HALF of the rotation tile -- the tensor core
// reads the other half from the peer's shared memory -- so a stage is 32 KB instead of 48 and six fit.
template <bool PAIR> struct RqStage {
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int B_BYTES = (PAIR ? 128 : 256) * 128;
  static constexpr int STAGE_BYTES = RQ_A_BYTES + B_BYTES;
};
// Epilogue warps per TMEM lane quarter: they take the 64-column chunks (per-head layouts: the heads) of their rows in
// turns.  The NVFP4 epilogue is the longest (seven threshold compares per value) and latency-bound, and the per-head
// epilogues wait on several tensor-memory reads per head, so those get more warps.
#ifndef RQ_WPQ_NVFP4
#define RQ_WPQ_NVFP4 4
#endif
#ifndef RQ_WPQ_PERHEAD
#define RQ_WPQ_PERHEAD 4
#endif
template <int EPI, bool PAIR = false> struct RqCfg {
  static constexpr int WPQ = (EPI == 2 /* EPI_NVFP4_HIDDEN */) ? RQ_WPQ_NVFP4 : (EPI == 3 || EPI == 4 /* per-head */) ? RQ_WPQ_PERHEAD : 2;
  static constexpr int EPI_WARPS = 4 * WPQ;
  static constexpr int THREADS = (2 + EPI_WARPS) * 32;
  // plain-GEMM epilogue (EPI_ROT_ONLY = 0): a 32 x 32 bf16 staging patch per epilogue warp for its TMA stores
  static constexpr int STG_BYTES = (EPI == 0) ? EPI_WARPS * 2048 : 0;
  static constexpr int SMEM_BYTES = RqStage<PAIR>::STAGES * RqStage<PAIR>::STAGE_BYTES + STG_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

enum : int { EPI_ROT_ONLY = 0, EPI_INT_HIDDEN = 1, EPI_NVFP4_HIDDEN = 2, EPI_INT_PERHEAD = 3, EPI_NVFP4_PERHEAD = 4 };


__device__ __forceinline__ void tile_k_range(const RotArgs& a, int nb, int& kb, int& ke) {
  const int kchunks = (a.K + 63) / 64;
  if (a.band == 0) { kb = 0; ke = kchunks; return; }
  const int n0 = nb * a.BN;
  const int n1 = min(n0 + a.BN, a.g.D);
  const int h0 = n0 / a.band, h1 = (n1 - 1) / a.band;
  kb = (h0 * a.band) / 64;
  ke = min(kchunks, ((h1 + 1) * a.band + 63) / 64);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// 32 code slots -> 16 bytes; byte j = slot j | slot 16+j << 4
__device__ __forceinline__ uint4 pack_planar32(const uint32_t* q) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t x = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) x |= ((q[4 * i + j] & 0xF) | ((q[16 + 4 * i + j] & 0xF) << 4)) << (8 * j);
    w[i] = x;
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- epilogues: thread = one row of the tile; `taddr` already points at this warp's lanes.
// Several warps (wpq) share a lane quarter; `turn` counts work items (64-column chunks, heads) across tiles
// and a warp takes the items whose index modulo wpq equals its `half`, which balances odd counts per tile.
template <int MODE>
__device__ __forceinline__ void epi_int_hidden(const RotArgs& a, uint32_t taddr, int64_t row, int n0, int half, uint32_t& turn, int wpq = 2) {
  const ActGeom& g = a.g;
  const bool row_ok = row < a.M;
  constexpr float maxq = (MODE == MODE_INT4_SYM) ? 7.f : (MODE == MODE_INT4_ASYM ? 15.f : 255.f);
  for (int c0 = 0; c0 < a.BN; c0 += 64) {
    const int col = n0 + c0;
    if (col >= g.D) break;
    if (((turn++) % (uint32_t)wpq) != (uint32_t)half) continue;
    uint32_t r[64];
    tmem_ld32(taddr + c0, r);
    tmem_ld32(taddr + c0 + 32, r + 32);
    tmem_wait_ld();
    // round the fp32 accumulators to bf16: this IS x_rot of the reference's bf16 forward
    uint32_t xb[32];     // bf16x2 pairs
    float v[64];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      xb[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
      v[2 * j] = __uint_as_float(xb[j] << 16);
      v[2 * j + 1] = __uint_as_float(xb[j] & 0xFFFF0000u);
    }
    if (a.x_rot && row_ok) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (col + 8 * i + 8 <= g.D)
          *reinterpret_cast<uint4*>(a.x_rot + row * g.D + col + 8 * i) = make_uint4(xb[4 * i], xb[4 * i + 1], xb[4 * i + 2], xb[4 * i + 3]);
    }
    if (!a.codes) continue;
    const int nq = max(0, min(64, g.q_len - col));
    if (nq < 64 && row_ok && a.tail) {
      __nv_bfloat16* tr = a.tail + row * g.tail_pitch;
      const int t0 = col - g.q_len;               // tail index of v[0] (may be negative)
      if (nq == 0 && (t0 & 7) == 0 && col + 64 <= g.D) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(tr + t0 + 8 * i) = make_uint4(xb[4 * i], xb[4 * i + 1], xb[4 * i + 2], xb[4 * i + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j >= nq && col + j < g.D) tr[t0 + j] = __float2bfloat16_rn(v[j]);
      }
    }
    if (nq > 0) {
      const int chunk = col >> 6;
      float mx = -INFINITY, mn = INFINITY;
      if (nq == 64) {
#pragma unroll
        for (int j = 0; j < 64; ++j) { mx = fmaxf(mx, v[j]); mn = fminf(mn, v[j]); }
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j < nq) { mx = fmaxf(mx, v[j]); mn = fminf(mn, v[j]); }
        mx = fmaxf(mx, 0.f);                                     // zero padding of the last group
        mn = fminf(mn, 0.f);
      }
      GroupParams p;
      if constexpr (MODE == MODE_INT4_SYM) p = int_sym_params<true>(mx, mn, g.clip, maxq);
      else p = int_asym_params<true>(mx, mn, g.clip, maxq);
      const float rcp = __frcp_rn(p.scale);
      if (nq < 64) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j >= nq) v[j] = 0.f;            // padding slots: symmetric code 0; asymmetric slots meet zero weights
      }
      if (row_ok) {
        if constexpr (MODE == MODE_INT4_SYM) {
          uint32_t n8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) n8[i] = int_sym_nib8_fast(v + 8 * i, p.scale, rcp);
          uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32);
          dst[0] = planar32_from_nib8(n8[0], n8[1], n8[2], n8[3]);
          dst[1] = planar32_from_nib8(n8[4], n8[5], n8[6], n8[7]);
        } else if constexpr (MODE == MODE_INT4_ASYM) {
          uint32_t n8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint2 b = int_asym_byte8_fast(v + 8 * i, p.scale, rcp, p.zero, maxq);
            n8[i] = squeeze_nibbles(b.x) | (squeeze_nibbles(b.y) << 16);
          }
          uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32);
          dst[0] = planar32_from_nib8(n8[0], n8[1], n8[2], n8[3]);
          dst[1] = planar32_from_nib8(n8[4], n8[5], n8[6], n8[7]);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 64);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint2 b0 = int_asym_byte8_fast(v + 16 * i, p.scale, rcp, p.zero, maxq);
            const uint2 b1 = int_asym_byte8_fast(v + 16 * i + 8, p.scale, rcp, p.zero, maxq);
            dst[i] = make_uint4(b0.x, b0.y, b1.x, b1.y);
          }
        }
        a.scales[(int64_t)chunk * a.ldm + row] = __float2bfloat16_rn(p.scale);
        if constexpr (MODE != MODE_INT4_SYM) a.zeros[(int64_t)chunk * a.ldm + row] = __float2bfloat16_rn(p.zero);
      }
    }
  }
}

// One 16-column quantisation group at a time (tcgen05.ld x16, a rolled loop over the chunk's four groups):
// the longest epilogue of the kernel stays small in registers and in code, so more warps can share a lane
// quarter and hide each other's latencies.
template <int MODE>
__device__ __forceinline__ void epi_nvfp4_hidden(const RotArgs& a, uint32_t taddr, int64_t row, int n0, int half, uint32_t& turn, int wpq = 2) {
  const ActGeom& g = a.g;
  const bool row_ok = row < a.M;
  const int n_kb64_pad = (g.n_chunks + 3) & ~3;
  const bool short_T = nvfp4_short_tensor_scale(g.T);
  const bool pow2_T = nvfp4_pow2_tensor_scale(g.T);
  for (int c0 = 0; c0 < a.BN; c0 += 64) {
    const int col = n0 + c0;
    if (col >= g.D) break;
    if (((turn++) % (uint32_t)wpq) != (uint32_t)half) continue;
    const int nq = max(0, min(64, g.q_len - col));
    const int chunk = col >> 6;
    uint32_t sfw = 0;
#pragma unroll 1
    for (int gi = 0; gi < 4; ++gi) {
      const int gcol = col + 16 * gi;
      if (gcol >= g.D) break;
      uint32_t r[16];
      tmem_ld16(taddr + c0 + 16 * gi, r);
      tmem_wait_ld();
      // the rotated values, rounded to bf16 and packed in pairs: what the quantiser is defined on
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      if (a.x_rot && row_ok) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
          if (gcol + 8 * i + 8 <= g.D)
            *reinterpret_cast<uint4*>(a.x_rot + row * g.D + gcol + 8 * i) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
      if (!a.codes) continue;
      const int nvalid = max(0, min(16, nq - 16 * gi));
      if constexpr (MODE == MODE_NVFP4_HW) {
        if (nvalid == 16 && pow2_T) {
          // whole group, power-of-two tensor scale: decided on the packed pairs (nvfp4_hw_group_packed)
          float eff = 0.f;
          const uint8_t sb = nvfp4_hw_scale(amax_bf16x16(w), g.clip, g.T, &eff);
          uint2 c = make_uint2(0u, 0u);
          if (eff > 0.f) c = nvfp4_hw_group_packed(w, eff);
          sfw |= (uint32_t)sb << (8 * gi);
          if (row_ok) *reinterpret_cast<uint2*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32 + gi * 8) = c;
          continue;
        }
      }
      float v[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      }
      if (nvalid > 0) {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < nvalid) amax = fmaxf(amax, fabsf(v[j]));
        uint32_t lo = 0, hi = 0;
        if constexpr (MODE == MODE_NVFP4_REF) {
          const float sc = nvfp4_ref_scale<true>(amax, g.clip);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            lo |= (j < nvalid ? nvfp4_ref_code<true>(v[j], sc) : 0u) << (4 * j);
            hi |= (8 + j < nvalid ? nvfp4_ref_code<true>(v[8 + j], sc) : 0u) << (4 * j);
          }
          if (row_ok) a.scales[(int64_t)(chunk * 4 + gi) * a.ldm + row] = __float2bfloat16_rn(sc);
        } else {
          float eff = 0.f;
          const uint8_t sb = nvfp4_hw_scale(amax, g.clip, g.T, &eff);
          uint2 c;
          if (nvalid == 16 && eff > 0.f && short_T)
            c = nvfp4_hw_group_fast(v, eff);
          else
            c = nvfp4_hw_group_partial(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12],
                                       v[13], v[14], v[15], nvalid, eff);
          lo = c.x;
          hi = c.y;
          sfw |= (uint32_t)sb << (8 * gi);
        }
        if (row_ok)
          *reinterpret_cast<uint2*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32 + gi * 8) = make_uint2(lo, hi);
      } else if (nq > 0 && row_ok) {
        // a group of the chunk that lies wholly in the tail region: its code slots stay zero
        *reinterpret_cast<uint2*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32 + gi * 8) = make_uint2(0u, 0u);
      }
      if (nvalid < 16 && row_ok && a.tail) {
        __nv_bfloat16* tr = a.tail + row * g.tail_pitch;
        const int t0 = gcol - g.q_len;
        if (nvalid == 0 && gcol + 16 <= g.D && ((t0 | g.tail_pitch) & 7) == 0) {
          // a group that lies wholly in the 16-bit tail: two 16-byte stores instead of sixteen 2-byte ones
#pragma unroll
          for (int i = 0; i < 2; ++i)
            *reinterpret_cast<uint4*>(tr + t0 + 8 * i) =
                make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                           pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j >= nvalid && gcol + j < g.D) tr[t0 + j] = __float2bfloat16_rn(v[j]);
        }
      }
    }
    if constexpr (MODE == MODE_NVFP4_HW)
      if (a.codes && nq > 0 && row_ok) *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, chunk * 4, n_kb64_pad)) = sfw;
  }
}

// 32 columns starting at a column that is only 8-aligned (heads of 72 channels): four
// naturally aligned 8-column reads, one wait.
__device__ __forceinline__ void ld32_by8(uint32_t taddr, uint32_t* r) {
  tmem_ld8(taddr, r);
  tmem_ld8(taddr + 8, r + 8);
  tmem_ld8(taddr + 16, r + 16);
  tmem_ld8(taddr + 24, r + 24);
  tmem_wait_ld();
}

// Planar-32 codes (byte j = slots j and 16 + j): the nibbles of the first nv slots.
__device__ __forceinline__ uint4 planar32_valid_mask(int nv) {
  const int nlo = min(nv, 16), nhi = max(nv - 16, 0);
  uint32_t w[4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const int lc = min(max(nlo - 4 * wd, 0), 4), hc = min(max(nhi - 4 * wd, 0), 4);
    const uint32_t lm = lc == 4 ? 0xFFFFFFFFu : ((1u << (8 * lc)) - 1u), hm = hc == 4 ? 0xFFFFFFFFu : ((1u << (8 * hc)) - 1u);
    w[wd] = (0x0F0F0F0Fu & lm) | (0xF0F0F0F0u & hm);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Per-head layout: head h = tile columns [hh*d, hh*d + d): first d_q quantised as ONE group,
// last hlen passthrough.  Two passes over TMEM (extrema, then codes) keep registers small.
template <int MODE>
__device__ __forceinline__ void epi_int_perhead(const RotArgs& a, uint32_t taddr, int64_t row, int n0, int half, uint32_t& turn, int wpq = 2) {
  const ActGeom& g = a.g;
  const bool row_ok = row < a.M;
  constexpr float maxq = (MODE == MODE_INT4_SYM) ? 7.f : (MODE == MODE_INT4_ASYM ? 15.f : 255.f);
  const int d = g.d, d_q = g.group;
  const int nblk = (d_q + 31) >> 5;
  for (int cb = 0; cb < a.BN; cb += d) {
    const int h = (n0 + cb) / d;
    if (h >= g.H) break;
    if (((turn++) % (uint32_t)wpq) != (uint32_t)half) continue;
    if (a.x_rot) {
      for (int c8 = 0; c8 < d; c8 += 8) {
        uint32_t r[8];
        tmem_ld8(taddr + cb + c8, r);
        tmem_wait_ld();
        if (row_ok)
          *reinterpret_cast<uint4*>(a.x_rot + row * g.D + n0 + cb + c8) =
              make_uint4(pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])),
                         pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
                         pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])),
                         pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
      }
    }
    if (!a.codes) continue;
    float mx = -INFINITY, mn = INFINITY;
    GroupParams p;
    if constexpr (MODE != MODE_INT8_ASYM) {
      // 4-bit modes, on packed bf16 pairs: a block of 32 columns becomes 16 words (one conversion per pair = the bf16
      // rounding of x_rot), the extrema are packed min / max, the codes come out in the planar layout directly
      // (quant_math.cuh).  A ragged last block takes part with its invalid slots replaced (extrema) or cleared (codes).
      // A head of one block (SANA: 28 of 32 columns) keeps its words between the two passes.
      uint32_t pw[16];
      for (int b = 0; b < nblk; ++b) {
        uint32_t r[32];
        ld32_by8(taddr + cb + 32 * b, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) pw[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        const int nv = min(32, d_q - 32 * b);
        if (nv == 32) {
          minmax_bf16x16(pw, mx, mn);
          minmax_bf16x16(pw + 8, mx, mn);
        } else {
          const uint32_t fill = (pw[0] << 16) | (pw[0] & 0xFFFFu);      // slot 0 of the block (always valid) twice
          uint32_t pm[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint32_t vm = (2 * i + 1 < nv) ? 0xFFFFFFFFu : ((2 * i < nv) ? 0x0000FFFFu : 0u);
            pm[i] = (pw[i] & vm) | (fill & ~vm);
          }
          minmax_bf16x16(pm, mx, mn);
          minmax_bf16x16(pm + 8, mx, mn);
        }
      }
      if constexpr (MODE == MODE_INT4_SYM) p = int_sym_params<true>(mx, mn, g.clip, maxq);
      else p = int_asym_params<true>(mx, mn, g.clip, maxq);
      const float rcp = __frcp_rn(p.scale);
      for (int b = 0; b < 2 * g.cpg; ++b) {
        uint4 c4 = make_uint4(0u, 0u, 0u, 0u);
        if (b < nblk) {
          if (nblk > 1) {
            uint32_t r[32];
            ld32_by8(taddr + cb + 32 * b, r);
#pragma unroll
            for (int i = 0; i < 16; ++i) pw[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
          }
          if constexpr (MODE == MODE_INT4_SYM) c4 = int_sym_planar32_packed(pw, rcp, g.clip < 1.f);
          else c4 = int_asym_planar32_packed(pw, rcp, p.zero);
          const int nv = d_q - 32 * b;
          if (nv < 32) {
            const uint4 m4 = planar32_valid_mask(nv);
            c4 = make_uint4(c4.x & m4.x, c4.y & m4.y, c4.z & m4.z, c4.w & m4.w);
          }
        }
        if (row_ok)
          *reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + ((int64_t)h * g.cpg * 64 + 32 * b) / 2) = c4;
      }
    } else {
    for (int b = 0; b < nblk; ++b) {
      uint32_t r[32];
      ld32_by8(taddr + cb + 32 * b, r);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (32 * b + j < d_q) {
          float f = rnd<true>(__uint_as_float(r[j]));
          mx = fmaxf(mx, f);
          mn = fminf(mn, f);
        }
    }
    p = int_asym_params<true>(mx, mn, g.clip, maxq);
    const float rcp = __frcp_rn(p.scale);
    for (int b = 0; b < 2 * g.cpg; ++b) {
      // 8-bit mode: eight codes per pair of words by the division-free exact form (guarded reciprocal, quant_math.cuh);
      // an octet that straddles the end of the group is computed whole and its invalid bytes cleared
      uint2 b8[4] = {make_uint2(0u, 0u), make_uint2(0u, 0u), make_uint2(0u, 0u), make_uint2(0u, 0u)};
      if (b < nblk) {
        uint32_t r[32];
        ld32_by8(taddr + cb + 32 * b, r);
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = rnd<true>(__uint_as_float(r[j]));
#pragma unroll
        for (int o = 0; o < 4; ++o) {
          const int nvo = d_q - (32 * b + 8 * o);                // valid values of this octet
          if (nvo > 0) {
            b8[o] = int_asym_byte8_fast(f + 8 * o, p.scale, rcp, p.zero, maxq);
            if (nvo < 8) {
              const uint32_t lo_m = nvo >= 4 ? 0xFFFFFFFFu : ((1u << (8 * nvo)) - 1u);
              const uint32_t hi_m = nvo > 4 ? ((1u << (8 * (nvo - 4))) - 1u) : 0u;
              b8[o] = make_uint2(b8[o].x & lo_m, b8[o].y & hi_m);
            }
          }
        }
      }
      if (row_ok) {
        uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)h * g.cpg * 64 + 32 * b);
        dst[0] = make_uint4(b8[0].x, b8[0].y, b8[1].x, b8[1].y);
        dst[1] = make_uint4(b8[2].x, b8[2].y, b8[3].x, b8[3].y);
      }
    }
    }
    if (row_ok) {
      for (int c = 0; c < g.cpg; ++c) {
        a.scales[(int64_t)(h * g.cpg + c) * a.ldm + row] = __float2bfloat16_rn(p.scale);
        if constexpr (MODE != MODE_INT4_SYM) a.zeros[(int64_t)(h * g.cpg + c) * a.ldm + row] = __float2bfloat16_rn(p.zero);
      }
    }
    if (a.tail) {
      for (int c8 = d_q & ~7; c8 < d; c8 += 8) {
        uint32_t r[8];
        tmem_ld8(taddr + cb + c8, r);
        tmem_wait_ld();
        if (row_ok) {
          __nv_bfloat16* tr = a.tail + row * g.tail_pitch + h * g.hlen;
          const int t0 = c8 - d_q;                                  // tail index of r[0] within the head (may be negative)
          if (t0 >= 0 && ((t0 | g.hlen | g.tail_pitch) & 7) == 0) {        // a whole, 16-byte aligned octet of tail channels
            *reinterpret_cast<uint4*>(tr + t0) =
                make_uint4(pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])), pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
                           pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])), pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
          } else if (t0 == -4 && ((g.hlen | g.tail_pitch) & 3) == 0) {     // the octet's upper half starts the head's tail
            *reinterpret_cast<uint2*>(tr) = make_uint2(pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])),
                                                       pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c8 + j >= d_q) tr[c8 + j - d_q] = __float2bfloat16_rn(__uint_as_float(r[j]));
          }
        }
      }
    }
  }
}

// Per-head layout, NVFP4 (hardware recipe): head h = tile columns [hh*d, hh*d + d): its first d - hlen coefficients go to
// code slots h * (d - hlen) .. in blocks of 16 (one UE4M3 scale each, byte-addressed: a head's blocks need not fill a
// scale-factor word), its last hlen to the 16-bit tail.  The GEMM then reads the codes as one hidden-layout row.
__device__ __forceinline__ void epi_nvfp4_perhead(const RotArgs& a, uint32_t taddr, int64_t row, int n0, int half, uint32_t& turn, int wpq = 2) {
  const ActGeom& g = a.g;
  const bool row_ok = row < a.M;
  const int d = g.d, d_q = g.d - g.hlen;
  const int n_kb64_pad = (g.n_chunks + 3) & ~3;
  const bool pow2_T = nvfp4_pow2_tensor_scale(g.T);
  for (int cb = 0; cb < a.BN; cb += d) {
    const int h = (n0 + cb) / d;
    if (h >= g.H) break;
    if (((turn++) % (uint32_t)wpq) != (uint32_t)half) continue;
#pragma unroll 1
    for (int c16 = 0; c16 < d; c16 += 16) {
      uint32_t r[16];
      tmem_ld16(taddr + cb + c16, r);
      tmem_wait_ld();
      uint32_t w[8];                       // the rotated values, rounded to bf16 and packed in pairs
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      if (!row_ok) continue;
      if (a.x_rot) {
        uint4* xr = reinterpret_cast<uint4*>(a.x_rot + row * g.D + n0 + cb + c16);
        xr[0] = make_uint4(w[0], w[1], w[2], w[3]);
        xr[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
      if (!a.codes) continue;
      if (c16 < d_q) {
        const int slot = h * d_q + c16;                       // first code slot of this block (a multiple of 16)
        float eff = 0.f;
        uint8_t sb;
        uint2 c = make_uint2(0u, 0u);
        if (pow2_T) {
          sb = nvfp4_hw_scale(amax_bf16x16(w), g.clip, g.T, &eff);
          if (eff > 0.f) c = nvfp4_hw_group_packed(w, eff);
        } else {
          float v[16];
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
          }
          sb = nvfp4_hw_scale(amax, g.clip, g.T, &eff);
          c = nvfp4_hw_group_partial(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[13],
                                     v[14], v[15], 16, eff);
        }
        *reinterpret_cast<uint2*>(a.codes + row * g.code_row_bytes + (slot >> 1)) = c;
        a.sf[sf_offset(row, slot >> 4, n_kb64_pad)] = sb;
      } else {
        __nv_bfloat16* tr = a.tail + row * g.tail_pitch + h * g.hlen + (c16 - d_q);
        const int left = d - c16;                             // 16, or fewer at the end of a head whose tail is no multiple of 16
        if (left >= 16 && (((h * g.hlen + c16 - d_q) | g.tail_pitch) & 7) == 0) {
          reinterpret_cast<uint4*>(tr)[0] = make_uint4(w[0], w[1], w[2], w[3]);
          reinterpret_cast<uint4*>(tr)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < left) tr[j] = __ushort_as_bfloat16((unsigned short)((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xFFFFu)));
        }
      }
    }
    // code slots between the last head's blocks and the end of the last 64-slot chunk: zero codes under zero scales
    if (row_ok && a.codes && h == g.H - 1) {
      for (int slot = g.q_len; slot < g.k_pad; slot += 16)
        *reinterpret_cast<uint2*>(a.codes + row * g.code_row_bytes + (slot >> 1)) = make_uint2(0u, 0u);
    }
  }
}

// Plain GEMM epilogue: y[M, N] = acc (+ bias) as bf16; used for the stand-alone rotation and for
// the bf16 GEMM behind the W4A16 layer.  32 columns at a time: tcgen05.ld -> + bias -> bf16 -> the warp's 32 x 32
// staging patch in shared memory (64-byte rows, 64-byte swizzle) -> one TMA store, which clips the patch at the
// edges of y.  (A row-per-thread store straight to global memory puts 32 separate 16-byte segments per
// instruction through the load/store unit.)
__device__ __forceinline__ void epi_rot_only(const RotArgs& a, const CUtensorMap* tm_y, uint32_t stg, uint32_t taddr, int row0,
                                             int lane, int n0, int half, uint32_t& turn, int wpq = 2) {
  const ActGeom& g = a.g;
  const uint32_t stg_row = stg + lane * 64;
  const int sw = (lane >> 1) & 3;
  for (int c0 = 0; c0 < a.BN; c0 += 32) {
    const int col = n0 + c0;
    if (col >= g.D) break;
    if (((turn++) % (uint32_t)wpq) != (uint32_t)half) continue;
    uint32_t r[32];
    tmem_ld32(taddr + c0, r);
    tmem_wait_ld();
    if (lane == 0) bulk_wait_read0();              // the previous patch has left the staging buffer
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * i + e]);
      if (a.bias && col + 8 * i + 8 <= g.D) {
        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(a.bias + col + 8 * i));
        const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
          const float2 b2 = __bfloat1622float2(bh[e2]);
          f[2 * e2] += b2.x;
          f[2 * e2 + 1] += b2.y;
        }
      }
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(stg_row + (uint32_t)((i ^ sw) << 4)),
                   "r"(pack_bf16x2(f[0], f[1])), "r"(pack_bf16x2(f[2], f[3])), "r"(pack_bf16x2(f[4], f[5])),
                   "r"(pack_bf16x2(f[6], f[7]))
                   : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && row0 < a.M) {
      tma_store_2d(tm_y, stg, col, row0);
      bulk_commit_group();
    }
  }
}

// PAIR: clusters of two CTAs share one 256-row tile through tcgen05.mma.cta_group::2 (each CTA its own 128 token
// rows and half of the rotation tile); completions of both CTAs' loads are counted on the leader's full barrier, the
// leader commits to both CTAs' empty / accumulator-full barriers, epilogue warps of both arrive on the leader's
// accumulator-empty barrier (the peer's arrivals carry no memory ordering: their payload is tensor memory).
template <int EPI, int MODE, bool PAIR>
__global__ void __launch_bounds__(RqCfg<EPI>::THREADS, 1)
rotate_quant_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_u,
                    const __grid_constant__ CUtensorMap tm_y, const RotArgs a) {
  constexpr int RQ_STAGES = RqStage<PAIR>::STAGES, RQ_STAGE_BYTES = RqStage<PAIR>::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stg_area = smem + RQ_STAGES * RQ_STAGE_BYTES;                  // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg_area + RqCfg<EPI>::STG_BYTES);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) acc_full, [2S+2..2S+4) acc_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * RQ_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;      // 0 = leader (issues the UMMAs)
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (RQ_STAGES + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * RQ_STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * RQ_STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < RQ_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), (PAIR ? 2 : 1) * RqCfg<EPI>::EPI_WARPS); }
    abort_flag[0] = 0;
    abort_flag[1] = a.wait_limit_k;
    fence_mbar_init();
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_u);
  }
  if (warp == 1) {
    if constexpr (PAIR) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    else tmem_alloc(smem_u32(tmem_slot), 512);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after();
  pdl_launch_dependents();
  pdl_wait();                       // whatever produced x (and last used the output buffers) has completed
  const uint32_t tmem_base = *tmem_slot;
  // tiles: (128-row block, column block), or (256-row pair block, column block) walked by clusters
  const int total_tiles = (PAIR ? (a.m_tiles + 1) / 2 : a.m_tiles) * a.n_tiles;
  const int first = PAIR ? (int)cluster_id_x() : (int)blockIdx.x, step = PAIR ? (int)cluster_count_x() : (int)gridDim.x;
  const int bn_own = PAIR ? a.BN / 2 : a.BN;                 // rotation-tile rows this CTA fetches
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint32_t issued = 0;   // bit s set: a load into stage s has been issued at least once
      bool ok = true;
      for (int t = first; t < total_tiles && ok; t += step) {
        const int mt = t / a.n_tiles, nb = t - mt * a.n_tiles;
        const int mb = PAIR ? 2 * mt + (int)rank : mt;
        int kb, ke;
        tile_k_range(a, nb, kb, ke);
        for (int kc = kb; kc < ke; ++kc) {
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sa = smem_base + s * RQ_STAGE_BYTES;
          if constexpr (PAIR) {
            const uint32_t fb = map_to_rank(full_bar(s), 0);
            if (rank == 0) mbar_expect_tx(full_bar(s), 2u * (RQ_A_BYTES + bn_own * 128));
            tma_load_2d_pair(sa, &tm_x, fb, kc * 64, mb * 128);
            tma_load_2d_pair(sa + RQ_A_BYTES, &tm_u, fb, kc * 64, nb * a.BN + (int)rank * bn_own);
          } else {
            mbar_expect_tx(full_bar(s), RQ_A_BYTES + a.BN * 128);
            tma_load_2d(sa, &tm_x, full_bar(s), kc * 64, mb * 128);
            tma_load_2d(sa + RQ_A_BYTES, &tm_u, full_bar(s), kc * 64, nb * a.BN);
          }
          issued |= 1u << s;
          if (++s == RQ_STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (PAIR && !ok) {
        // the completions of this CTA's copies are counted in the leader, where the peer cannot test them: give
        // copies in flight a bounded time to land before the CTA may retire
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
      } else if (!ok) {
        // unwind: let copies already in flight land before the CTA exits (bounded)
        const long long t0 = clock64();
        for (int i = 0; i < RQ_STAGES; ++i) {
          if (!(issued & (1u << i))) continue;
          const uint32_t last_ph = (i < s) ? ph : (ph ^ 1);
          while (!mbar_try(full_bar(i), last_ph)) {
            if (clock64() - t0 > kWaitLimitCycles / 8) { if (a.status) atomicCAS(a.status, 0, ERR_WAIT_DRAIN); break; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = idesc_dense(ACC_F32, FMT_BF16, FMT_BF16, PAIR ? 256 : 128, (uint32_t)a.BN);
      int s = 0, buf = 0;
      uint32_t ph = 0, aph = 0;
      bool ok = true;
      const uint64_t op_d0 = smem_desc_sw128(smem_base);
      const uint32_t op_lo0 = (uint32_t)op_d0, op_hi = (uint32_t)(op_d0 >> 32);
      for (int t = first; t < total_tiles && ok; t += step) {
        const int nb = t % a.n_tiles;
        int kb, ke;
        tile_k_range(a, nb, kb, ke);
        if (!mbar_wait(acce_bar(buf), aph ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kc = kb; kc < ke; ++kc) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          // descriptors from loop-invariant words; the stage's four UMMAs in one block (what this thread does between
          // UMMAs is time the tensor pipe idles)
          const uint32_t a_lo = op_lo0 + (uint32_t)s * (RQ_STAGE_BYTES >> 4);
          if constexpr (PAIR) {
            umma_f16_ss_x4_pair(d_tmem, a_lo, a_lo + (RQ_A_BYTES >> 4), op_hi, idesc, kc > kb ? 1u : 0u);
            umma_commit_pair(empty_bar(s));
            umma_commit_pair(map_to_rank(empty_bar(s), 1));
          } else {
            umma_f16_ss_x4(d_tmem, a_lo, a_lo + (RQ_A_BYTES >> 4), op_hi, idesc, kc > kb ? 1u : 0u);
            umma_commit(empty_bar(s));
          }
          if (++s == RQ_STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        if constexpr (PAIR) {
          umma_commit_pair(accf_bar(buf));
          umma_commit_pair(map_to_rank(accf_bar(buf), 1));
        } else {
          umma_commit(accf_bar(buf));
        }
        buf ^= 1;
        if (buf == 0) aph ^= 1;
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    int buf = 0;
    uint32_t aph = 0, turn = 0;
    const uint32_t acce_leader = PAIR ? map_to_rank(acce_bar(0), 0) : 0u;
    for (int t = first; t < total_tiles; t += step) {
      const int mt = t / a.n_tiles, nb = t - mt * a.n_tiles;
      const int mb = PAIR ? 2 * mt + (int)rank : mt;
      if (!mbar_wait(accf_bar(buf), aph, abort_flag, a.status, ERR_WAIT_ACC_FULL)) break;
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256;
      const int64_t row = (int64_t)mb * 128 + q * 32 + lane;
      const int n0 = nb * a.BN;
      if constexpr (EPI == EPI_ROT_ONLY)
        epi_rot_only(a, &tm_y, smem_u32(stg_area) + (warp - 2) * 2048, taddr, mb * 128 + q * 32, lane, n0, half, turn);
      else if constexpr (EPI == EPI_INT_HIDDEN) epi_int_hidden<MODE>(a, taddr, row, n0, half, turn);
      else if constexpr (EPI == EPI_NVFP4_HIDDEN) epi_nvfp4_hidden<MODE>(a, taddr, row, n0, half, turn, RqCfg<EPI>::WPQ);
      else if constexpr (EPI == EPI_NVFP4_PERHEAD) epi_nvfp4_perhead(a, taddr, row, n0, half, turn, RqCfg<EPI>::WPQ);
      else epi_int_perhead<MODE>(a, taddr, row, n0, half, turn, RqCfg<EPI>::WPQ);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && rank != 0) mbar_arrive_cluster_relaxed(acce_leader + 8u * buf);
        else mbar_arrive(acce_bar(buf));
      }
      buf ^= 1;
      if (buf == 0) aph ^= 1;
    }
    if constexpr (EPI == EPI_ROT_ONLY)
      if (lane == 0) bulk_wait_all0();                 // the output is in global memory before the CTA retires
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA retires while the other may still read its shared memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// ---- host side ----------------------------------------------------------------------------------
int num_sms() {
  // per device: a process may drive GPUs of different sizes
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

template <int EPI, int MODE, bool PAIR>
static int launch_rq_impl(const CUtensorMap& tx, const CUtensorMap& tu, const CUtensorMap& ty, const RotArgs& a, cudaStream_t st) {
  using Cfg = RqCfg<EPI, PAIR>;
  auto k = rotate_quant_kernel<EPI, MODE, PAIR>;
  static PerDeviceOnce attr_once;
  if (int rc = set_max_dynamic_smem(attr_once, k, Cfg::SMEM_BYTES)) return rc;
  if constexpr (!PAIR) {
    const int grid = min(a.m_tiles * a.n_tiles, num_sms());
    return launch_pdl(k, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, tx, tu, ty, a) == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
  } else {
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
    // persistent grid: as many pairs as can be resident at once, remembered per device
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
    const int tiles = ((a.m_tiles + 1) / 2) * a.n_tiles;
    cfg.gridDim = dim3(2 * min(tiles, max_pairs));
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, k, tx, tu, ty, a) == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
  }
}

// tu_pair: the rotation's tensor map with a box of BN / 2 rows (what one CTA of a pair fetches); used when the call
// has more than one 128-row block (DIROTQ_ROTATE_TILE = single | pair forces one form: measurements, tests).
template <int EPI, int MODE>
static int launch_rq(const CUtensorMap& tx, const CUtensorMap& tu, const CUtensorMap& tu_pair, const RotArgs& a, cudaStream_t st) {
  CUtensorMap ty = tx;                                 // only the plain-GEMM epilogue stores through a tensor map
  if constexpr (EPI == EPI_ROT_ONLY) {
    if ((a.g.D & 7) || (reinterpret_cast<uintptr_t>(a.x_rot) & 15)) return DIROTQ_E_ALIGN;
    int rc = make_tmap_2d_sw(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.x_rot, (uint64_t)a.g.D, (uint64_t)a.M,
                             (uint64_t)a.g.D * 2, 32, 32, 64);
    if (rc) return rc;
  }
  bool pair = a.m_tiles >= 2 && (a.BN / 2) % 8 == 0;
  if (const char* e = getenv("DIROTQ_ROTATE_TILE")) {
    if (!strcmp(e, "single")) pair = false;
    else if (!strcmp(e, "pair")) pair = (a.BN / 2) % 8 == 0;
  }
  if (pair) return launch_rq_impl<EPI, MODE, true>(tx, tu_pair, ty, a, st);
  return launch_rq_impl<EPI, MODE, false>(tx, tu, ty, a, st);
}

// Picks the N tile.  Per-head layouts: a whole number of heads (and a multiple of 16 for the UMMA shape).  Hidden
// layouts: a multiple of 64; the persistent grid runs ceil(tiles / SMs) rounds, and a round costs a part that grows with
// the tile width (the UMMAs) plus a part that does not (the per-stage barrier protocol of the issuer, the same for every
// width).  Measured at D = 1152, 32768 rows: 6.03 / 6.68 / 7.59 us per round for 128 / 192 / 256 columns, i.e. the fixed
// part is worth about 370 columns; the choice minimises rounds x (width + 370) -- padding of D and a nearly empty last
// round both count (32768 rows of a 1152-wide layer take 256: 68 us against 74 with 192; a 4096-row shard takes 128).
int pick_bn(const ActGeom& g, int64_t M) {
  if (g.H > 0) {
    int best = 0;
    for (int k = 1; k * g.d <= 256; ++k)
      if ((k * g.d) % 16 == 0) best = k * g.d;
    return best;
  }
  const int cand[3] = {256, 192, 128};
  const int64_t m_tiles = (M + 127) / 128, sms = num_sms();
  int best = 256;
  int64_t best_cost = -1;
  for (int i = 0; i < 3; ++i) {
    const int64_t tiles = m_tiles * ceil_div(g.D, cand[i]);
    const int64_t cost = ((tiles + sms - 1) / sms) * (cand[i] + 370);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = cand[i]; }
  }
  return best;
}

int launch_rotate_quantize(const ActGeom& g, const void* x, const void* rot_t, int64_t M, RotArgs a, cudaStream_t st) {
  if (M <= 0) return DIROTQ_OK;
  a.g = g;
  a.M = M;
  a.K = g.D;
  a.bias = nullptr;
  a.ldm = ld_rows(M);
  const bool rot_only = a.codes == nullptr;
  if (rot_only && !a.x_rot) return DIROTQ_E_ARG;
  // The rotation-only epilogue stores whole 32-column patches, so it takes the tile widths of the hidden layouts even
  // under a per-head rotation (whose whole-head widths, 144 for 72-wide heads, are not multiples of 32); the K range of
  // a tile follows the heads its columns touch either way.
  ActGeom g_tile = g;
  if (rot_only) g_tile.H = 0;
  a.BN = pick_bn(g_tile, M);
  if (a.BN <= 0) return DIROTQ_E_UNSUPPORTED;
  a.n_tiles = ceil_div(g.D, a.BN);
  a.m_tiles = (int)((M + 127) / 128);
  a.band = g.H > 0 ? g.d : 0;
  if (!rot_only && g.H > 0) {
    // 32-column TMEM reads of a head's group must stay inside the head
    if (((g.group + 31) / 32) * 32 > g.d) return DIROTQ_E_UNSUPPORTED;
  }
  if (!rot_only && g.H == 0 && !is_nvfp4(g.mode) && g.group != 64) return DIROTQ_E_UNSUPPORTED;
  if (!rot_only && g.per_token) return DIROTQ_E_UNSUPPORTED;     // a row's scale needs the whole rotated row: rotate, then quantise
  CUtensorMap tx, tu;
  int rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)g.D, (uint64_t)M, (uint64_t)g.D * 2, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&tu, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rot_t, (uint64_t)g.D, (uint64_t)g.D, (uint64_t)g.D * 2,
                    (uint32_t)a.BN);
  if (rc) return rc;
  CUtensorMap tu2 = tu;
  if ((a.BN / 2) % 8 == 0) {
    rc = make_tmap_2d(&tu2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rot_t, (uint64_t)g.D, (uint64_t)g.D, (uint64_t)g.D * 2,
                      (uint32_t)(a.BN / 2));
    if (rc) return rc;
  }
  if (rot_only) return launch_rq<EPI_ROT_ONLY, 0>(tx, tu, tu2, a, st);
  if (g.H > 0) {
    switch (g.mode) {
      case DIROTQ_INT4_SYM: return launch_rq<EPI_INT_PERHEAD, MODE_INT4_SYM>(tx, tu, tu2, a, st);
      case DIROTQ_INT4_ASYM: return launch_rq<EPI_INT_PERHEAD, MODE_INT4_ASYM>(tx, tu, tu2, a, st);
      case DIROTQ_INT8_ASYM: return launch_rq<EPI_INT_PERHEAD, MODE_INT8_ASYM>(tx, tu, tu2, a, st);
      case DIROTQ_NVFP4_HW: return launch_rq<EPI_NVFP4_PERHEAD, MODE_NVFP4_HW>(tx, tu, tu2, a, st);
      default: return DIROTQ_E_UNSUPPORTED;
    }
  }
  switch (g.mode) {
    case DIROTQ_INT4_SYM: return launch_rq<EPI_INT_HIDDEN, MODE_INT4_SYM>(tx, tu, tu2, a, st);
    case DIROTQ_INT4_ASYM: return launch_rq<EPI_INT_HIDDEN, MODE_INT4_ASYM>(tx, tu, tu2, a, st);
    case DIROTQ_INT8_ASYM: return launch_rq<EPI_INT_HIDDEN, MODE_INT8_ASYM>(tx, tu, tu2, a, st);
    case DIROTQ_NVFP4_REF: return launch_rq<EPI_NVFP4_HIDDEN, MODE_NVFP4_REF>(tx, tu, tu2, a, st);
    case DIROTQ_NVFP4_HW: return launch_rq<EPI_NVFP4_HIDDEN, MODE_NVFP4_HW>(tx, tu, tu2, a, st);
  }
  return DIROTQ_E_UNSUPPORTED;
}

// y[M, N] = x[M, K] @ w_t[N, K]^T (+ bias), all bf16, fp32 accumulation on tcgen05.
int launch_gemm_bf16(const void* x, const void* w_t, int64_t M, int64_t N, int64_t K, const void* bias, void* y,
                     int* status, cudaStream_t st) {
  if (M <= 0) return DIROTQ_OK;
  if (N % 8 || K % 8) return DIROTQ_E_UNSUPPORTED;
  RotArgs a{};
  a.g = ActGeom{};
  a.g.D = (int)N;
  a.M = M;
  a.K = (int)K;
  a.ldm = ld_rows(M);
  a.BN = pick_bn(a.g, M);
  a.n_tiles = ceil_div((int)N, a.BN);
  a.m_tiles = (int)((M + 127) / 128);
  a.band = 0;
  a.x_rot = static_cast<__nv_bfloat16*>(y);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.status = status;
  a.wait_limit_k = wait_limit_k();
  CUtensorMap tx, tu;
  int rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&tu, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_t, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, (uint32_t)a.BN);
  if (rc) return rc;
  CUtensorMap tu2;
  rc = make_tmap_2d(&tu2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_t, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, (uint32_t)(a.BN / 2));
  if (rc) return rc;
  return launch_rq<EPI_ROT_ONLY, 0>(tx, tu, tu2, a, st);
}

}  // namespace dq
