// Kernel 3: weight quantiser + packer (offline, bandwidth-bound).  Arithmetic follows
// _quant_group_int / _quant_group_nvfp4 (DiRotQ utils/quant_utils.py:714-767) in fp32 and the
// two-level NVFP4 recipe of speedup/weight_only_nvfp4.py:42-72; the byte layouts are the
// tensor-core-friendly ones declared in include/dirotq_b200.h (K-major rows, 64-slot chunks,
// group-major scale planes, 512-byte scale-factor tiles), not an mma.sync fragment order.
#include <cuda_runtime.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "quant_math.cuh"

namespace dq {


// One thread = one block of 32 code slots of one output row (same slot layout as activations).
__global__ void __launch_bounds__(256) pack_int4_kernel(const PackIntArgs a) {
  const int bpr = a.n_chunks * 2;
  const int64_t total = a.N * bpr;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = tid < total;
  const int64_t t = live ? tid : total - 1;
  const int64_t n = t / bpr;
  const int b = (int)(t - n * bpr);
  const int chunk = b >> 1, half = b & 1;
  const int grp = chunk / a.cpg;
  const int e0 = (chunk % a.cpg) * 64 + half * 32;
  const int glen = (int)min((int64_t)a.group, a.n_low - (int64_t)grp * a.group);
  const int nvalid = max(0, min(32, glen - e0));
  const float* wr = a.w + n * a.n_low + (int64_t)grp * a.group + e0;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = (j < nvalid) ? __ldg(wr + j) : 0.f;
  float scale;
  if (a.scale_in) {
    scale = a.scale_in[n * a.n_groups + grp];
  } else {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
    for (int o = 1; o < 2 * a.cpg; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    scale = __fdiv_rn(fmaxf(amax, 1e-5f), 7.f);
  }
  int q[32];
  int sum = 0;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    int c = 0;
    if (j < nvalid) {
      float r = a.w_is_codes ? v[j] : rintf(__fdiv_rn(v[j], scale));
      c = (int)fminf(fmaxf(r, -8.f), 7.f);
    }
    q[j] = c;
    sum += c;
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);   // both halves of the chunk
  if (!live) return;
  uint32_t w4[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t x = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t byte = ((uint32_t)q[4 * i + j] & 0xF) | (((uint32_t)q[16 + 4 * i + j] & 0xF) << 4);
      x |= byte << (8 * j);
    }
    w4[i] = x;
  }
  *reinterpret_cast<uint4*>(a.codes + n * (int64_t)(a.n_chunks * 32) + (int64_t)b * 16) =
      make_uint4(w4[0], w4[1], w4[2], w4[3]);
  if (half == 0) {
    a.scales[(int64_t)chunk * a.ldn + n] = scale;
    a.wsum[(int64_t)chunk * a.ldn + n] = (float)sum;
  }
}


// One thread = one 64-slot chunk (4 groups of 16) of one output row.
__global__ void __launch_bounds__(256) pack_nvfp4_kernel(const PackFp4Args a) {
  const int64_t total = a.N * a.n_chunks;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int64_t n = tid / a.n_chunks;
  const int chunk = (int)(tid - n * a.n_chunks);
  const int n_kb64_pad = (a.n_chunks + 3) & ~3;
  const int ngrp_row = (int)((a.n_low + 15) / 16);
  uint32_t packed[8];
  uint32_t sfw = 0;
#pragma unroll
  for (int gi = 0; gi < 4; ++gi) {
    const int64_t cg = (int64_t)chunk * 64 + gi * 16;
    const int nvalid = (int)max((int64_t)0, min((int64_t)16, a.n_low - cg));
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (j < nvalid) ? __ldg(a.w + n * a.n_low + cg + j) : 0.f;
    uint8_t sb = 0;
    float eff = 0.f;
    if (nvalid > 0) {
      if (a.scale_in) {
        sb = a.scale_in[n * ngrp_row + chunk * 4 + gi];
        eff = __fmul_rn(e4m3_to_float(sb), a.T);
      } else {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
        sb = nvfp4_hw_scale(amax, 1.f, a.T, &eff);
      }
    }
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t c0 = 0, c1 = 0;
      if (j < nvalid) c0 = a.w_is_codes ? ((uint32_t)v[j] & 0xF) : nvfp4_hw_code(v[j], eff);
      if (8 + j < nvalid) c1 = a.w_is_codes ? ((uint32_t)v[8 + j] & 0xF) : nvfp4_hw_code(v[8 + j], eff);
      lo |= c0 << (4 * j);
      hi |= c1 << (4 * j);
    }
    packed[gi * 2] = lo;
    packed[gi * 2 + 1] = hi;
    sfw |= (uint32_t)sb << (8 * gi);
  }
  uint4* dst = reinterpret_cast<uint4*>(a.codes + n * (int64_t)(a.n_chunks * 32) + (int64_t)chunk * 32);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  *reinterpret_cast<uint32_t*>(a.sf + sf_offset(n, chunk * 4, n_kb64_pad)) = sfw;
}

// ---- the reference's own two-level NVFP4 weight recipe (speedup/weight_only_nvfp4.py:42-72) ----------------------
//   group_scale_g = max(amax_g / 6, 1e-12)            gscale[n] = max(max_g(group_scale_g) / 448, 1e-12)   (fp32)
//   micro_g = e4m3_rn(group_scale_g / gscale[n])      eff_g = float(micro_g) * gscale[n]
//   code = first argmin_i |w / eff_g - codebook[i]| over [0 .5 1 1.5 2 3 4 6 -0 -.5 ... -6]
// The first-argmin rule sends an exact midpoint to the value of smaller magnitude and never yields -0; a group whose
// micro-scale rounds to zero (w / 0 = inf or nan, every distance inf or nan) gets index 0 throughout.  The stored
// per-channel scale is gscale rounded to bf16 (what the reference's dequantiser multiplies by); codes are taken
// against the unrounded fp32 value, as there.
// One warp per output row: row maximum, then the per-channel scale in both forms.
__global__ void __launch_bounds__(256) nvfp4_row_scale_kernel(const float* __restrict__ w, int64_t N, int64_t n_low,
                                                              float* __restrict__ g_exact, float* __restrict__ g_stored) {
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const int lane = threadIdx.x & 31;
  float amax = 0.f;
  for (int64_t k = lane; k < n_low; k += 32) amax = fmaxf(amax, fabsf(__ldg(w + n * n_low + k)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) {
    // max over groups of fl(amax_g / 6) = fl(row amax / 6): the division is monotone
    const float gs = fmaxf(__fdiv_rn(amax, 6.f), 1e-12f);
    const float g = fmaxf(__fdiv_rn(gs, 448.f), 1e-12f);
    g_exact[n] = g;
    g_stored[n] = __bfloat162float(__float2bfloat16_rn(g));
  }
}

__device__ __forceinline__ uint32_t e2m1_nibble_argmin(float v) {
  const float a = fabsf(v);
  if (!(a <= 3.0e38f)) return 0u;                    // inf / nan: index 0, as the first argmin over inf / nan distances
  const uint32_t m = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.f);
  return (m && v < 0.f) ? (8u | m) : m;
}

// One thread = one 64-slot chunk (4 groups of 16) of one output row; same outputs as pack_nvfp4_kernel.
__global__ void __launch_bounds__(256) pack_nvfp4_rowscale_kernel(const PackFp4Args a, const float* __restrict__ g_exact) {
  const int64_t total = a.N * a.n_chunks;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int64_t n = tid / a.n_chunks;
  const int chunk = (int)(tid - n * a.n_chunks);
  const int n_kb64_pad = (a.n_chunks + 3) & ~3;
  const float g = g_exact[n];
  uint32_t packed[8];
  uint32_t sfw = 0;
#pragma unroll
  for (int gi = 0; gi < 4; ++gi) {
    const int64_t cg = (int64_t)chunk * 64 + gi * 16;
    const int nvalid = (int)max((int64_t)0, min((int64_t)16, a.n_low - cg));
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (j < nvalid) ? __ldg(a.w + n * a.n_low + cg + j) : 0.f;
    uint8_t sb = 0;
    float eff = 0.f;
    if (nvalid > 0) {
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
      const float gs = fmaxf(__fdiv_rn(amax, 6.f), 1e-12f);
      sb = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(gs, g), __NV_SATFINITE, __NV_E4M3);
      eff = __fmul_rn(e4m3_to_float(sb), g);
    }
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t c0 = (j < nvalid) ? e2m1_nibble_argmin(__fdiv_rn(v[j], eff)) : 0u;
      const uint32_t c1 = (8 + j < nvalid) ? e2m1_nibble_argmin(__fdiv_rn(v[8 + j], eff)) : 0u;
      lo |= c0 << (4 * j);
      hi |= c1 << (4 * j);
    }
    packed[gi * 2] = lo;
    packed[gi * 2 + 1] = hi;
    sfw |= (uint32_t)sb << (8 * gi);
  }
  uint4* dst = reinterpret_cast<uint4*>(a.codes + n * (int64_t)(a.n_chunks * 32) + (int64_t)chunk * 32);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  *reinterpret_cast<uint32_t*>(a.sf + sf_offset(n, chunk * 4, n_kb64_pad)) = sfw;
}

int launch_pack_nvfp4_rowscale(const PackFp4Args& a, float* g_exact, float* g_stored, cudaStream_t st) {
  if (a.N <= 0 || a.n_chunks <= 0) return DIROTQ_OK;
  nvfp4_row_scale_kernel<<<(unsigned)((a.N + 7) / 8), 256, 0, st>>>(a.w, a.N, a.n_low, g_exact, g_stored);
  const int64_t total = a.N * a.n_chunks;
  pack_nvfp4_rowscale_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a, g_exact);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int launch_pack_int4(const PackIntArgs& a, cudaStream_t st) {
  int64_t total = a.N * a.n_chunks * 2;
  if (total <= 0) return DIROTQ_OK;
  pack_int4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}
int launch_pack_nvfp4(const PackFp4Args& a, cudaStream_t st) {
  int64_t total = a.N * a.n_chunks;
  if (total <= 0) return DIROTQ_OK;
  pack_nvfp4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

// Packed INT4 weight -> bf16 [N, n_chunks*64] (q * scale rounded once), the operand of the W4A16 GEMM.
// One thread = one block of 32 code slots.
__global__ void __launch_bounds__(256) dequant_int4_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales,
                                                           int64_t N, int n_chunks, int64_t ldn, __nv_bfloat16* __restrict__ w) {
  const int bpr = n_chunks * 2;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= N * bpr) return;
  const int64_t n = tid / bpr;
  const int b = (int)(tid - n * bpr);
  const uint4 p = __ldg(reinterpret_cast<const uint4*>(codes + n * (int64_t)(n_chunks * 32) + (int64_t)b * 16));
  const float s = __ldg(scales + (int64_t)(b >> 1) * ldn + n);
  const uint32_t pw[4] = {p.x, p.y, p.z, p.w};
  __nv_bfloat16 out[32];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = (pw[i] >> (8 * j)) & 0xFF;
      const int lo = (int)((byte & 0xF) ^ 8) - 8, hi = (int)((byte >> 4) ^ 8) - 8;
      out[4 * i + j] = __float2bfloat16_rn((float)lo * s);
      out[16 + 4 * i + j] = __float2bfloat16_rn((float)hi * s);
    }
  uint4* dst = reinterpret_cast<uint4*>(w + n * (int64_t)(n_chunks * 64) + (int64_t)b * 32);
  const uint4* src = reinterpret_cast<const uint4*>(out);
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[i] = src[i];
}

// Packed NVFP4 weight (sequential E2M1 nibbles, tiled UE4M3 group scales, fp32 tensor scale or per-channel scales)
// -> bf16 [N, n_chunks*64]: value * (micro * scale) rounded once, the arithmetic of the reference's dequantiser
// (speedup/weight_only_nvfp4.py:96-112).  One thread = one group of 16.
__global__ void __launch_bounds__(256) dequant_nvfp4_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                                            float T, const float* __restrict__ row_scale, int64_t N,
                                                            int n_chunks, __nv_bfloat16* __restrict__ w) {
  const int gpr = n_chunks * 4;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= N * gpr) return;
  const int64_t n = tid / gpr;
  const int gi = (int)(tid - n * gpr);
  const int n_kb64_pad = (n_chunks + 3) & ~3;
  const float s = __fmul_rn(e4m3_to_float(__ldg(sf + sf_offset(n, gi, n_kb64_pad))), row_scale ? __ldg(row_scale + n) : T);
  const uint2 p = __ldg(reinterpret_cast<const uint2*>(codes + n * (int64_t)(n_chunks * 32) + (int64_t)gi * 8));
  const uint32_t pw[2] = {p.x, p.y};
  __nv_bfloat16 out[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t nib = (pw[j >> 3] >> (4 * (j & 7))) & 0xF;
    const uint32_t m = nib & 7;
    // E2M1 magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6
    const float mag = m < 2 ? 0.5f * (float)m : (m < 4 ? 0.5f * (float)m : (m < 6 ? (float)(m - 2) : (m == 6 ? 4.f : 6.f)));
    out[j] = __float2bfloat16_rn((nib & 8) ? -mag * s : mag * s);
  }
  uint4* dst = reinterpret_cast<uint4*>(w + n * (int64_t)(n_chunks * 64) + (int64_t)gi * 16);
  const uint4* src = reinterpret_cast<const uint4*>(out);
  dst[0] = src[0];
  dst[1] = src[1];
}

int launch_dequant_nvfp4(const uint8_t* codes, const uint8_t* sf, float T, const float* row_scale, int64_t N, int n_chunks,
                         __nv_bfloat16* w, cudaStream_t st) {
  const int64_t total = N * n_chunks * 4;
  if (total <= 0) return DIROTQ_OK;
  dequant_nvfp4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(codes, sf, T, row_scale, N, n_chunks, w);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int launch_dequant_int4(const uint8_t* codes, const float* scales, int64_t N, int n_chunks, int64_t ldn,
                        __nv_bfloat16* w, cudaStream_t st) {
  const int64_t total = N * n_chunks * 2;
  if (total <= 0) return DIROTQ_OK;
  dequant_int4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(codes, scales, N, n_chunks, ldn, w);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

}  // namespace dq
