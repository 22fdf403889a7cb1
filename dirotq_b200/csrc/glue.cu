// Block glue around the quantised linears of a DiT block: the row-wise, HBM-bound passes that sit between two wrapped
// linears in the reference's model forwards (speedup/report_flux_w4a4_no_rot_ffdown.py:199-228, :240-252: AdaLayerNorm +
// modulation in front of the rotation, gate * branch + residual behind the out-projections; :261-276: nunchaku's
// fused_qkv_norm_rottary on the q / k / v projections).  PyTorch runs each of them as three to six elementwise kernels
// with a bf16 round trip through HBM per step; here every pass reads its inputs once, works in fp32 and rounds once.
//
//   layernorm_modulate : y = LayerNorm(x) * (1 + scale[b]) + shift[b]          (no affine, biased variance, fp32)
//   gated_residual     : out = h + gate[b] * (y + y2)                           (gate, y2 optional)
//   qkv_norm_rope      : per head: q, k -> RMSNorm * w -> rotary embedding; v copied; all three written token-major
//                        ([B, T_total, H, d], at a token offset) so that text and image streams land in one buffer
//                        without a concatenation and the attention output needs no transpose.
//
// One warp per row (layernorm_modulate), one thread per 8 values (the other two); 16-byte loads and stores.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"

namespace dq {

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

// NV = 16-byte vectors per lane (D <= 256 * NV)
template <int NV>
__global__ void __launch_bounds__(256) layernorm_modulate_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int D,
                                                                 int64_t rows_per_sample, const __nv_bfloat16* __restrict__ scale,
                                                                 const __nv_bfloat16* __restrict__ shift, int64_t mod_pitch,
                                                                 float eps, __nv_bfloat16* __restrict__ y) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int nvec = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  uint4 v[NV];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + 32 * i;
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (idx < nvec) {
      v[i] = __ldg(xr + idx);
      float f[8];
      unpack8(v[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += f[e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / (float)D;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < nvec) {
      float f[8];
      unpack8(v[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) { const float c = f[e] - mean; sq = fmaf(c, c, sq); }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq / (float)D + eps);
  const int64_t b = row / rows_per_sample;
  const uint4* sc = scale ? reinterpret_cast<const uint4*>(scale + b * mod_pitch) : nullptr;
  const uint4* sh = shift ? reinterpret_cast<const uint4*>(shift + b * mod_pitch) : nullptr;
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + 32 * i;
    if (idx < nvec) {
      float f[8], s[8], t[8];
      unpack8(v[i], f);
      if (sc) unpack8(__ldg(sc + idx), s);
      if (sh) unpack8(__ldg(sh + idx), t);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float r = (f[e] - mean) * rstd;
        if (sc) r *= 1.f + s[e];
        if (sh) r += t[e];
        f[e] = r;
      }
      yr[idx] = pack8(f);
    }
  }
}

__global__ void __launch_bounds__(256) gated_residual_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ y,
                                                             const __nv_bfloat16* __restrict__ y2,
                                                             const __nv_bfloat16* __restrict__ gate, int64_t mod_pitch, int64_t M,
                                                             int D, int64_t rows_per_sample, __nv_bfloat16* __restrict__ out) {
  const int nvec = D >> 3;
  const int64_t total = M * nvec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / nvec;
    const int c = (int)(i - row * nvec);
    float a[8], b[8], g[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(h) + i), a);
    unpack8(__ldg(reinterpret_cast<const uint4*>(y) + i), b);
    if (y2) {
      float b2[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(y2) + i), b2);
#pragma unroll
      for (int e = 0; e < 8; ++e) b[e] += b2[e];
    }
    if (gate) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(gate + (row / rows_per_sample) * mod_pitch) + c), g);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = fmaf(g[e], b[e], a[e]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += b[e];
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(a);
  }
}

struct QkvArgs {
  const __nv_bfloat16* in[3];     // q, k, v: [B * T, H * d] with row pitch `pitch` (elements)
  __nv_bfloat16* out[3];          // [B, T_total, H, d]
  const __nv_bfloat16* w[2];      // RMSNorm weights of q and k, [d] (null: no normalisation)
  const __nv_bfloat16* cos;       // [T_total, d] (null: no rotary embedding)
  const __nv_bfloat16* sin;
  int64_t pitch;
  int64_t B, T, T_total, t0;
  int H, d;
  float eps;
};

// LPH = lanes per head (d / 8): 8 or 16; a head's lanes are consecutive and aligned inside a warp
template <int LPH>
__global__ void __launch_bounds__(256) qkv_norm_rope_kernel(const QkvArgs a) {
  const int vec_per_row = a.H * LPH;
  const int64_t total = a.B * a.T * 3 * vec_per_row;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = i < total;
  const int64_t ii = live ? i : total - 1;               // keep whole warps in the shuffles
  const int64_t rp = ii / vec_per_row;                   // (row, part)
  const int c = (int)(ii - rp * vec_per_row);            // vector inside the row
  const int part = (int)(rp % 3);
  const int64_t row = rp / 3;
  const int64_t b = row / a.T, t = row - b * a.T;
  float f[8];
  const __nv_bfloat16* in = part == 0 ? a.in[0] : (part == 1 ? a.in[1] : a.in[2]);
  unpack8(__ldg(reinterpret_cast<const uint4*>(in + row * a.pitch) + c), f);
  const int64_t pos = a.t0 + t;
  // sum of squares over the head: every lane takes part in the shuffles (a warp may hold lanes of two parts)
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (part < 2) {
    const __nv_bfloat16* wp = part == 0 ? a.w[0] : a.w[1];
    if (wp) {
      const float r = rsqrtf(ss / (float)a.d + a.eps);
      float w[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(wp) + (c % LPH)), w);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = f[e] * r * w[e];
    }
    if (a.cos) {
      float cs[8], sn[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(a.cos + pos * a.d) + (c % LPH)), cs);
      unpack8(__ldg(reinterpret_cast<const uint4*>(a.sin + pos * a.d) + (c % LPH)), sn);
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const float x0 = f[e], x1 = f[e + 1];
        f[e] = x0 * cs[e] - x1 * sn[e];
        f[e + 1] = x1 * cs[e + 1] + x0 * sn[e + 1];
      }
    }
  }
  __nv_bfloat16* outp = part == 0 ? a.out[0] : (part == 1 ? a.out[1] : a.out[2]);
  if (live) reinterpret_cast<uint4*>(outp + (b * a.T_total + pos) * (int64_t)(a.H * a.d))[c] = pack8(f);
}

}  // namespace dq

using namespace dq;

extern "C" {

int dirotq_layernorm_modulate(const void* x, int64_t M, int32_t D, int64_t rows_per_sample, const void* scale,
                              const void* shift, int64_t mod_pitch, float eps, void* y, void* stream) {
  if (!x || !y || M < 0 || D <= 0 || rows_per_sample <= 0) return DIROTQ_E_ARG;
  if (D % 8 || D > 4096 || ((scale || shift) && mod_pitch % 8)) return DIROTQ_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(scale) |
       reinterpret_cast<uintptr_t>(shift)) & 15)
    return DIROTQ_E_ALIGN;
  if (M == 0) return DIROTQ_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((M + 7) / 8);
  const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16*>(x), *sc = static_cast<const __nv_bfloat16*>(scale),
                      *sh = static_cast<const __nv_bfloat16*>(shift);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  const int nv = (D / 8 + 31) / 32;
  if (nv <= 4) layernorm_modulate_kernel<4><<<blocks, 256, 0, st>>>(xp, M, D, rows_per_sample, sc, sh, mod_pitch, eps, yp);
  else if (nv <= 8) layernorm_modulate_kernel<8><<<blocks, 256, 0, st>>>(xp, M, D, rows_per_sample, sc, sh, mod_pitch, eps, yp);
  else if (nv <= 12) layernorm_modulate_kernel<12><<<blocks, 256, 0, st>>>(xp, M, D, rows_per_sample, sc, sh, mod_pitch, eps, yp);
  else layernorm_modulate_kernel<16><<<blocks, 256, 0, st>>>(xp, M, D, rows_per_sample, sc, sh, mod_pitch, eps, yp);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int dirotq_gated_residual(const void* h, const void* y, const void* y2, const void* gate, int64_t mod_pitch, int64_t M,
                          int32_t D, int64_t rows_per_sample, void* out, void* stream) {
  if (!h || !y || !out || M < 0 || D <= 0 || rows_per_sample <= 0) return DIROTQ_E_ARG;
  if (D % 8 || (gate && mod_pitch % 8)) return DIROTQ_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(y2) |
       reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(out)) & 15)
    return DIROTQ_E_ALIGN;
  if (M == 0) return DIROTQ_OK;
  const int64_t total = M * (D / 8);
  const int64_t want = (total + 255) / 256, cap = (int64_t)num_sms() * 16;
  const unsigned blocks = (unsigned)(want < cap ? want : cap);
  gated_residual_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(y2),
      static_cast<const __nv_bfloat16*>(gate), mod_pitch, M, D, rows_per_sample, static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int dirotq_qkv_norm_rope(const void* q, const void* k, const void* v, int64_t pitch, int64_t B, int64_t T, int32_t H,
                         int32_t d, const void* w_q, const void* w_k, const void* cos, const void* sin, int64_t T_total,
                         int64_t t0, float eps, void* out_q, void* out_k, void* out_v, void* stream) {
  if (!q || !k || !v || !out_q || !out_k || !out_v || B < 0 || T < 0 || H <= 0) return DIROTQ_E_ARG;
  if ((d != 64 && d != 128) || pitch % 8 || pitch < (int64_t)H * d) return DIROTQ_E_UNSUPPORTED;
  if (t0 < 0 || t0 + T > T_total || (!cos != !sin)) return DIROTQ_E_ARG;
  const uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                       reinterpret_cast<uintptr_t>(out_q) | reinterpret_cast<uintptr_t>(out_k) |
                       reinterpret_cast<uintptr_t>(out_v) | reinterpret_cast<uintptr_t>(w_q) |
                       reinterpret_cast<uintptr_t>(w_k) | reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin);
  if (al & 15) return DIROTQ_E_ALIGN;
  if (B == 0 || T == 0) return DIROTQ_OK;
  QkvArgs a;
  a.in[0] = static_cast<const __nv_bfloat16*>(q);
  a.in[1] = static_cast<const __nv_bfloat16*>(k);
  a.in[2] = static_cast<const __nv_bfloat16*>(v);
  a.out[0] = static_cast<__nv_bfloat16*>(out_q);
  a.out[1] = static_cast<__nv_bfloat16*>(out_k);
  a.out[2] = static_cast<__nv_bfloat16*>(out_v);
  a.w[0] = static_cast<const __nv_bfloat16*>(w_q);
  a.w[1] = static_cast<const __nv_bfloat16*>(w_k);
  a.cos = static_cast<const __nv_bfloat16*>(cos);
  a.sin = static_cast<const __nv_bfloat16*>(sin);
  a.pitch = pitch;
  a.B = B; a.T = T; a.T_total = T_total; a.t0 = t0;
  a.H = H; a.d = d;
  a.eps = eps;
  const int64_t total = B * T * 3 * H * (d / 8);
  if ((total + 255) / 256 > 0x7fffffff) return DIROTQ_E_TOO_LARGE;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d == 128) qkv_norm_rope_kernel<16><<<blocks, 256, 0, st>>>(a);
  else qkv_norm_rope_kernel<8><<<blocks, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

}  // extern "C"
