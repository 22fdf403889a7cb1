// Kernel 1a: split + quantise of an already rotated / permuted activation tensor.  HBM-bound:
// every input element is read once (16-byte loads where alignment allows), group extrema are
// combined with warp shuffles, and codes leave as packed 16/32-byte stores.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "quant_math.cuh"

namespace dq {


// Source column of element e of group grp.
__device__ __forceinline__ int src_col(const ActGeom& g, int grp, int e) {
  return g.H > 0 ? grp * g.d + e : grp * g.group + e;
}

// Partial blocks (the end of a group that is not a multiple of 32): the plain exact forms, padding slots get code 0.
template <int MODE>
static __device__ __noinline__ void quant_int_block_slow(const __nv_bfloat16* x, int64_t x_pitch, const int64_t* perm,
                                                         uint8_t* codes, int code_row_bytes, float scale, float zero,
                                                         int nvalid, int c0, int64_t row, int b) {
  constexpr float maxq = (MODE == MODE_INT4_SYM) ? 7.f : (MODE == MODE_INT4_ASYM ? 15.f : 255.f);
  GroupParams p;
  p.scale = scale;
  p.zero = zero;
  float v[32];                      // re-read here: a pointer to the caller's values would push them to local memory
  const __nv_bfloat16* xr = x + row * x_pitch;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float f = 0.f;
    if (j < nvalid) {
      int64_t c = c0 + j;
      if (perm) c = perm[c];
      f = __bfloat162float(xr[c]);
    }
    v[j] = f;
  }
  uint32_t q[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    int c = 0;
    if (j < nvalid) {
      if constexpr (MODE == MODE_INT4_SYM) c = int_sym_code<true>(v[j], p.scale, maxq);
      else c = int_asym_code<true>(v[j], p.scale, p.zero, maxq);
    }
    q[j] = (uint32_t)c;
  }
  if constexpr (MODE == MODE_INT8_ASYM) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      w[i] = (q[4 * i] & 0xFF) | ((q[4 * i + 1] & 0xFF) << 8) | ((q[4 * i + 2] & 0xFF) << 16) | ((q[4 * i + 3] & 0xFF) << 24);
    uint4* dst = reinterpret_cast<uint4*>(codes + row * code_row_bytes + (int64_t)b * 32);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t x = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t byte = (q[4 * i + j] & 0xF) | ((q[16 + 4 * i + j] & 0xF) << 4);
        x |= byte << (8 * j);
      }
      w[i] = x;
    }
    *reinterpret_cast<uint4*>(codes + row * code_row_bytes + (int64_t)b * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// One thread = one block of 32 code slots of one row.  The 2*cpg threads that share a group sit
// on consecutive lanes (aligned), so the group extrema need log2(2*cpg) shuffles.
template <int MODE>
__global__ void __launch_bounds__(256) quant_int_kernel(const QuantArgs a) {
  const ActGeom& g = a.g;
  const int bpr = g.n_chunks * 2;                      // 32-slot blocks per row
  const int64_t total = a.M * bpr;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = tid < total;
  const int64_t t = live ? tid : total - 1;
  int64_t row;
  int b;
  if (total <= 0x7fffffffLL) {                         // the usual case: a 32-bit divide instead of the 64-bit routine
    const uint32_t r32 = (uint32_t)t / (uint32_t)bpr;
    row = r32;
    b = (int)((uint32_t)t - r32 * (uint32_t)bpr);
  } else {
    row = t / bpr;
    b = (int)(t - row * bpr);
  }
  const int chunk = b >> 1, half = b & 1;
  const int grp = chunk / g.cpg;
  const int e0 = (chunk % g.cpg) * 64 + half * 32;     // first element of the group this block covers
  int glen = g.group;
  if (g.H == 0) glen = min(g.group, g.q_len - grp * g.group);
  const int nvalid = max(0, min(32, glen - e0));
  const bool padded = glen < g.group;                  // zero padding takes part in min / max

  float v[32];
  const __nv_bfloat16* xr = a.x + row * a.x_pitch;
  const int c0 = src_col(g, grp, e0);
  const bool vec_ok = (a.perm == nullptr) && ((c0 & 7) == 0) && ((a.x_pitch & 7) == 0) &&
                      ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) && (c0 + 32 <= g.D);
  // Whole groups of a 4-bit layer (the common case) stay on the packed bf16 pairs as loaded: extrema by packed max / min,
  // codes by int_sym_planar32_packed / int_asym_planar32_packed, no conversion to fp32 beyond the multiply.  The choice is the same for
  // every thread of a group; the shuffles below run outside it, on all lanes of the warp.
  const bool packed_path = (MODE == MODE_INT4_SYM || MODE == MODE_INT4_ASYM) && vec_ok && glen == 64 * g.cpg;
  uint32_t w[16];
  float mx = -INFINITY, mn = INFINITY;
  if (packed_path) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(xr + c0) + i);
      w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
    }
    if constexpr (MODE == MODE_INT4_SYM) {
      mx = fmaxf(amax_bf16x16(w), amax_bf16x16(w + 8));
      mn = -mx;
    } else {
      minmax_bf16x16(w, mx, mn);
      minmax_bf16x16(w + 8, mx, mn);
    }
  } else
  if (vec_ok) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q = __ldg(reinterpret_cast<const uint4*>(xr + c0) + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        v[i * 8 + j * 2] = f.x;
        v[i * 8 + j * 2 + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float f = 0.f;
      if (j < nvalid) {
        int64_t c = c0 + j;
        if (a.perm) c = a.perm[c];
        f = __bfloat162float(xr[c]);
      }
      v[j] = f;
    }
  }
  if (!packed_path) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < nvalid) { mx = fmaxf(mx, v[j]); mn = fminf(mn, v[j]); }
    }
    // an all-padding block of a real group, or zero padding inside the group
    if (padded) { mx = fmaxf(mx, 0.f); mn = fminf(mn, 0.f); }
  }
  const int nb = 2 * g.cpg;
  for (int o = 1; o < nb; o <<= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  constexpr float maxq = (MODE == MODE_INT4_SYM) ? 7.f : (MODE == MODE_INT4_ASYM ? 15.f : 255.f);
  GroupParams p;
  if constexpr (MODE == MODE_INT4_SYM) p = int_sym_params<true>(mx, mn, g.clip, maxq);
  else p = int_asym_params<true>(mx, mn, g.clip, maxq);

  if (!live) return;
  if (packed_path) {
    const float rcp = __frcp_rn(p.scale);
    *reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)b * 16) =
        (MODE == MODE_INT4_SYM) ? int_sym_planar32_packed(w, rcp, g.clip < 1.f) : int_asym_planar32_packed(w, rcp, p.zero);
  } else if (nvalid == 32) {
    // full block: the division-free exact forms (reciprocal multiply, see quant_math.cuh)
    const float rcp = __frcp_rn(p.scale);
    if constexpr (MODE == MODE_INT4_SYM) {
      uint32_t n8[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) n8[i] = int_sym_nib8_fast(v + 8 * i, p.scale, rcp);
      *reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)b * 16) = planar32_from_nib8(n8[0], n8[1], n8[2], n8[3]);
    } else if constexpr (MODE == MODE_INT4_ASYM) {
      uint32_t n8[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint2 bb = int_asym_byte8_fast(v + 8 * i, p.scale, rcp, p.zero, maxq);
        n8[i] = squeeze_nibbles(bb.x) | (squeeze_nibbles(bb.y) << 16);
      }
      *reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)b * 16) = planar32_from_nib8(n8[0], n8[1], n8[2], n8[3]);
    } else {
      uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)b * 32);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint2 b0 = int_asym_byte8_fast(v + 16 * i, p.scale, rcp, p.zero, maxq);
        const uint2 b1 = int_asym_byte8_fast(v + 16 * i + 8, p.scale, rcp, p.zero, maxq);
        dst[i] = make_uint4(b0.x, b0.y, b1.x, b1.y);
      }
    }
  } else {
    quant_int_block_slow<MODE>(a.x, a.x_pitch, a.perm, a.codes, g.code_row_bytes, p.scale, p.zero, nvalid, c0, row, b);
  }
  if (half == 0) {
    a.scales[(int64_t)chunk * a.ldm + row] = __float2bfloat16_rn(p.scale);
    if constexpr (MODE != MODE_INT4_SYM) a.zeros[(int64_t)chunk * a.ldm + row] = __float2bfloat16_rn(p.zero);
  }
}

// Per-token scales: one CTA per row.  Pass 1: extrema of the quantised channels, zero included
// (utils/quant_utils.py:246-249 starts the reduction from a zero tensor); pass 2: codes in the chunk layout, the row's
// scale and zero point repeated for every chunk.  The row (a few KB) is read twice; the second read hits L1 / L2.
template <int MODE>
__global__ void __launch_bounds__(256) quant_int_token_kernel(const QuantArgs a) {
  const ActGeom& g = a.g;
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = a.x + row * a.x_pitch;
  float mx = 0.f, mn = 0.f;
  for (int c = threadIdx.x; c < g.q_len; c += blockDim.x) {
    const float f = __bfloat162float(xr[a.perm ? a.perm[c] : c]);
    mx = fmaxf(mx, f);
    mn = fminf(mn, f);
  }
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  __shared__ float s_mx[8], s_mn[8];
  if ((threadIdx.x & 31) == 0) { s_mx[threadIdx.x >> 5] = mx; s_mn[threadIdx.x >> 5] = mn; }
  __syncthreads();
  mx = s_mx[0];
  mn = s_mn[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) { mx = fmaxf(mx, s_mx[i]); mn = fminf(mn, s_mn[i]); }
  constexpr float maxq = (MODE == MODE_INT4_SYM) ? 7.f : (MODE == MODE_INT4_ASYM ? 15.f : 255.f);
  GroupParams p;
  if constexpr (MODE == MODE_INT4_SYM) p = int_sym_params<true>(mx, mn, g.clip, maxq);
  else p = int_asym_params<true>(mx, mn, g.clip, maxq);
  for (int b = threadIdx.x; b < g.n_chunks * 2; b += blockDim.x) {
    const int nvalid = max(0, min(32, g.q_len - b * 32));
    quant_int_block_slow<MODE>(a.x, a.x_pitch, a.perm, a.codes, g.code_row_bytes, p.scale, p.zero, nvalid, b * 32, row, b);
  }
  for (int chunk = threadIdx.x; chunk < g.n_chunks; chunk += blockDim.x) {
    a.scales[(int64_t)chunk * a.ldm + row] = __float2bfloat16_rn(p.scale);
    if constexpr (MODE != MODE_INT4_SYM) a.zeros[(int64_t)chunk * a.ldm + row] = __float2bfloat16_rn(p.zero);
  }
}

// One thread = one 64-slot chunk (4 groups of 16) of one row; hidden layout only.
template <int MODE>
__global__ void __launch_bounds__(256) quant_nvfp4_kernel(const QuantArgs a) {
  const ActGeom& g = a.g;
  const int64_t total = a.M * g.n_chunks;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  int64_t row;
  int chunk;
  if (total <= 0x7fffffffLL) {                         // 32-bit divide in the usual case
    const uint32_t r32 = (uint32_t)tid / (uint32_t)g.n_chunks;
    row = r32;
    chunk = (int)((uint32_t)tid - r32 * (uint32_t)g.n_chunks);
  } else {
    row = tid / g.n_chunks;
    chunk = (int)(tid - row * g.n_chunks);
  }
  const __nv_bfloat16* xr = a.x + row * a.x_pitch;
  const int c0 = chunk * 64;
  const int n_kb64_pad = (g.n_chunks + 3) & ~3;
  const bool short_T = nvfp4_short_tensor_scale(g.T);
  uint32_t packed[8];
  uint32_t sfw = 0;
  if constexpr (MODE == MODE_NVFP4_HW) {
    // whole chunk inside the quantised region, 16-byte aligned, power-of-two tensor scale: everything on packed bf16
    // pairs as loaded, no conversion to fp32 (see nvfp4_hw_group_packed)
    if (a.perm == nullptr && (a.x_pitch & 7) == 0 && c0 + 64 <= g.q_len && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
        nvfp4_pow2_tensor_scale(g.T)) {
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(xr + c0) + i);
        w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
      }
#pragma unroll
      for (int gi = 0; gi < 4; ++gi) {
        float eff;
        const uint8_t sb = nvfp4_hw_scale(amax_bf16x16(w + 8 * gi), g.clip, g.T, &eff);
        uint2 c = make_uint2(0u, 0u);
        if (eff > 0.f) c = nvfp4_hw_group_packed(w + 8 * gi, eff);
        packed[2 * gi] = c.x;
        packed[2 * gi + 1] = c.y;
        sfw |= (uint32_t)sb << (8 * gi);
      }
      uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32);
      dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, chunk * 4, n_kb64_pad)) = sfw;
      return;
    }
  }
  // whole chunk in range and 16-byte aligned: eight 16-byte loads instead of 64 scalar ones
  const bool vec_ok = (a.perm == nullptr) && ((a.x_pitch & 7) == 0) && (c0 + 64 <= g.D) &&
                      ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
  uint4 raw[8];
  if (vec_ok) {
#pragma unroll
    for (int i = 0; i < 8; ++i) raw[i] = __ldg(reinterpret_cast<const uint4*>(xr + c0) + i);
  }
#pragma unroll
  for (int gi = 0; gi < 4; ++gi) {
    float v[16];
    const int cg = c0 + gi * 16;
    const int nvalid = max(0, min(16, g.q_len - cg));
    if (vec_ok) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[2 * gi]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = (2 * j < nvalid) ? f.x : 0.f;
        v[2 * j + 1] = (2 * j + 1 < nvalid) ? f.y : 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float f = 0.f;
        if (j < nvalid) {
          int64_t c = cg + j;
          if (a.perm) c = a.perm[c];
          f = __bfloat162float(xr[c]);
        }
        v[j] = f;
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    uint32_t lo = 0, hi = 0;
    if constexpr (MODE == MODE_NVFP4_REF) {
      float s = nvfp4_ref_scale<true>(amax, g.clip);
#pragma unroll
      for (int j = 0; j < 8; ++j) lo |= (j < nvalid ? nvfp4_ref_code<true>(v[j], s) : 0u) << (4 * j);
#pragma unroll
      for (int j = 0; j < 8; ++j) hi |= (8 + j < nvalid ? nvfp4_ref_code<true>(v[8 + j], s) : 0u) << (4 * j);
      if (nvalid > 0) a.scales[(int64_t)(chunk * 4 + gi) * a.ldm + row] = __float2bfloat16_rn(s);
    } else {
      float eff;
      uint8_t sb = nvfp4_hw_scale(amax, g.clip, g.T, &eff);
      if (nvalid == 0) { sb = 0; eff = 0.f; }
      if (nvalid == 16 && eff > 0.f && short_T) {
        const uint2 c = nvfp4_hw_group_fast(v, eff);
        lo = c.x;
        hi = c.y;
      } else {
        const uint2 c = nvfp4_hw_group_partial(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11],
                                               v[12], v[13], v[14], v[15], nvalid, eff);
        lo = c.x;
        hi = c.y;
      }
      sfw |= (uint32_t)sb << (8 * gi);
    }
    packed[gi * 2] = lo;
    packed[gi * 2 + 1] = hi;
  }
  uint4* dst = reinterpret_cast<uint4*>(a.codes + row * g.code_row_bytes + (int64_t)chunk * 32);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  if constexpr (MODE == MODE_NVFP4_HW)
    *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, chunk * 4, n_kb64_pad)) = sfw;
}

// Passthrough channels -> tail buffer [M, tail_pitch] (pad columns zero).
__global__ void __launch_bounds__(256) copy_tail_kernel(const QuantArgs a) {
  const ActGeom& g = a.g;
  const int64_t total = a.M * g.tail_pitch;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int64_t row = tid / g.tail_pitch;
  const int t = (int)(tid - row * g.tail_pitch);
  __nv_bfloat16 val = __float2bfloat16_rn(0.f);
  if (t < g.tail_total) {
    int64_t c;
    if (g.H > 0) { int h = t / g.hlen; c = (int64_t)h * g.d + g.group + (t - h * g.hlen); }
    else c = g.q_len + t;
    if (a.perm) c = a.perm[c];
    val = a.x[row * a.x_pitch + c];
  }
  a.tail[tid] = val;
}


// Passthrough channels of the hidden layout, eight per thread (16-byte loads and stores).
__global__ void __launch_bounds__(256) copy_tail_vec_kernel(const QuantArgs a) {
  const ActGeom& g = a.g;
  const int per_row = g.tail_pitch >> 3;
  const int64_t total = a.M * per_row;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int64_t row = tid / per_row;
  const int t = (int)(tid - row * per_row) * 8;
  uint4 val = make_uint4(0u, 0u, 0u, 0u);
  if (t < g.tail_total) val = __ldg(reinterpret_cast<const uint4*>(a.x + row * a.x_pitch + g.q_len + t));
  *reinterpret_cast<uint4*>(a.tail + row * g.tail_pitch + t) = val;
}

int launch_quantize(const QuantArgs& a, cudaStream_t st) {
  const ActGeom& g = a.g;
  if (a.M <= 0) return DIROTQ_OK;
  const int threads = 256;
  if (is_nvfp4(g.mode) && g.H > 0) return DIROTQ_E_UNSUPPORTED;   // per-head NVFP4 exists only fused with its rotation
  if (is_nvfp4(g.mode)) {
    int64_t total = a.M * g.n_chunks;
    unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (g.mode == DIROTQ_NVFP4_REF) quant_nvfp4_kernel<MODE_NVFP4_REF><<<blocks, threads, 0, st>>>(a);
    else quant_nvfp4_kernel<MODE_NVFP4_HW><<<blocks, threads, 0, st>>>(a);
  } else if (g.per_token) {
    if (a.M > 0x7fffffff) return DIROTQ_E_TOO_LARGE;
    if (g.mode == DIROTQ_INT4_SYM) quant_int_token_kernel<MODE_INT4_SYM><<<(unsigned)a.M, threads, 0, st>>>(a);
    else if (g.mode == DIROTQ_INT4_ASYM) quant_int_token_kernel<MODE_INT4_ASYM><<<(unsigned)a.M, threads, 0, st>>>(a);
    else quant_int_token_kernel<MODE_INT8_ASYM><<<(unsigned)a.M, threads, 0, st>>>(a);
  } else {
    int64_t total = a.M * g.n_chunks * 2;
    unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (g.mode == DIROTQ_INT4_SYM) quant_int_kernel<MODE_INT4_SYM><<<blocks, threads, 0, st>>>(a);
    else if (g.mode == DIROTQ_INT4_ASYM) quant_int_kernel<MODE_INT4_ASYM><<<blocks, threads, 0, st>>>(a);
    else quant_int_kernel<MODE_INT8_ASYM><<<blocks, threads, 0, st>>>(a);
  }
  if (g.tail_total > 0 && a.tail) {
    const bool vec = g.H == 0 && !a.perm && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.x_pitch & 7) == 0 &&
                     (reinterpret_cast<uintptr_t>(a.tail) & 15) == 0 && g.q_len % 8 == 0 && g.tail_total % 8 == 0 &&
                     g.tail_pitch % 8 == 0;
    if (vec) {
      int64_t total = a.M * (g.tail_pitch / 8);
      copy_tail_vec_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, st>>>(a);
    } else {
      int64_t total = a.M * g.tail_pitch;
      copy_tail_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, st>>>(a);
    }
  }
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

}  // namespace dq
