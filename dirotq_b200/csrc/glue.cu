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
// Four warps per row (layernorm_modulate), one thread per 8 values (the other two); 16-byte loads and stores, 32-bit
// index arithmetic.
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

// WPR warps per row (1: short rows, no shared memory; 4: long rows, more loads in flight per row), 8 / WPR rows per CTA;
// NV = 16-byte vectors per thread (D <= 256 * WPR * NV).  The row stays in registers between the two reductions (mean,
// then centred sum of squares) and the output pass.
template <int NV, int WPR>
__global__ void __launch_bounds__(256) layernorm_modulate_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int D,
                                                                 int64_t rows_per_sample, const __nv_bfloat16* __restrict__ scale,
                                                                 const __nv_bfloat16* __restrict__ shift, int64_t mod_pitch,
                                                                 float eps, __nv_bfloat16* __restrict__ y) {
  constexpr int TPR = 32 * WPR, RPC = 8 / WPR;                                               // threads per row, rows per CTA
  __shared__ float red[2][RPC][WPR];
  const int lane = threadIdx.x & 31, wr = (threadIdx.x >> 5) % WPR, rr = threadIdx.x / TPR;  // warp in row, row in CTA
  const int tr = threadIdx.x % TPR;                                                          // thread in row
  const int64_t row = (int64_t)blockIdx.x * RPC + rr;
  const bool live = row < M;
  const int nvec = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (live ? row : 0) * D);
  float f[NV][8];                         // the row, unpacked once
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = tr + TPR * i;
#pragma unroll
    for (int e = 0; e < 8; ++e) f[i][e] = 0.f;
    if (live && idx < nvec) {
      unpack8(__ldg(xr + idx), f[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += f[i][e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if constexpr (WPR > 1) {
    if (lane == 0) red[0][rr][wr] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) sum += red[0][rr][w];
  }
  const float mean = sum / (float)D;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (tr + TPR * i < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { const float c = f[i][e] - mean; sq = fmaf(c, c, sq); }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if constexpr (WPR > 1) {
    if (lane == 0) red[1][rr][wr] = sq;
    __syncthreads();
    sq = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) sq += red[1][rr][w];
  }
  if (!live) return;
  const float rstd = rsqrtf(sq / (float)D + eps);
  const int64_t b = row / rows_per_sample;
  const uint4* sc = scale ? reinterpret_cast<const uint4*>(scale + b * mod_pitch) : nullptr;
  const uint4* sh = shift ? reinterpret_cast<const uint4*>(shift + b * mod_pitch) : nullptr;
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = tr + TPR * i;
    if (idx < nvec) {
      // y = (x - mean) * rstd * (1 + scale) + shift = x * a + c with a = rstd * (1 + scale), c = shift - mean * a
      float s[8], t[8], r[8];
      if (sc) unpack8(__ldg(sc + idx), s);
      if (sh) unpack8(__ldg(sh + idx), t);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a = sc ? fmaf(rstd, s[e], rstd) : rstd;
        const float c = fmaf(-mean, a, sh ? t[e] : 0.f);
        r[e] = fmaf(f[i][e], a, c);
      }
      yr[idx] = pack8(r);
    }
  }
}

__global__ void __launch_bounds__(256) gated_residual_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ y,
                                                             const __nv_bfloat16* __restrict__ y2,
                                                             const __nv_bfloat16* __restrict__ gate, int64_t mod_pitch, int64_t M,
                                                             int D, int64_t rows_per_sample, __nv_bfloat16* __restrict__ out) {
  const int nvec = D >> 3;
  const int64_t total = M * nvec;
  const bool small = total <= 0x7fffffffLL && rows_per_sample <= 0x7fffffffLL;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t row, smp = 0;
    int c;
    if (small) {                                   // 32-bit divides in the usual case
      const uint32_t r32 = (uint32_t)i / (uint32_t)nvec;
      row = r32;
      c = (int)((uint32_t)i - r32 * (uint32_t)nvec);
      if (gate) smp = r32 / (uint32_t)rows_per_sample;
    } else {
      row = i / nvec;
      c = (int)(i - row * nvec);
      if (gate) smp = row / rows_per_sample;
    }
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
      unpack8(__ldg(reinterpret_cast<const uint4*>(gate + smp * mod_pitch) + c), g);
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
  const uint32_t vec_per_row = (uint32_t)(a.H * LPH);
  const uint32_t total = (uint32_t)(a.B * a.T) * vec_per_row;      // per part; the launcher keeps it below 2^32
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = i < total;
  const uint32_t ii = live ? i : total - 1;              // keep whole warps in the shuffles
  const int part = blockIdx.y;                           // 0 = q, 1 = k, 2 = v
  const uint32_t row32 = ii / vec_per_row;
  const int c = (int)(ii - row32 * vec_per_row);         // vector inside the row
  const uint32_t b32 = row32 / (uint32_t)a.T;
  const int64_t row = row32, b = b32, t = row32 - b32 * (uint32_t)a.T;
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
      unpack8(__ldg(reinterpret_cast<const uint4*>(wp) + (c & (LPH - 1))), w);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = f[e] * r * w[e];
    }
    if (a.cos) {
      float cs[8], sn[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(a.cos + pos * a.d) + (c & (LPH - 1))), cs);
      unpack8(__ldg(reinterpret_cast<const uint4*>(a.sin + pos * a.d) + (c & (LPH - 1))), sn);
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
  if ((M + 1) / 2 > 0x7fffffff) return DIROTQ_E_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16*>(x), *sc = static_cast<const __nv_bfloat16*>(scale),
                      *sh = static_cast<const __nv_bfloat16*>(shift);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  const int nvec = D / 8;
#define DQ_LN(NV, WPR)                                                                                            \
  layernorm_modulate_kernel<NV, WPR><<<(unsigned)((M + 8 / WPR - 1) / (8 / WPR)), 256, 0, st>>>(xp, M, D, rows_per_sample, sc, \
                                                                                                 sh, mod_pitch, eps, yp)
  if (nvec <= 64) DQ_LN(2, 1);
  else if (nvec <= 160) DQ_LN(5, 1);           // PixArt's 1152: a warp per row
  else if (nvec <= 256) DQ_LN(2, 4);
  else if (nvec <= 384) DQ_LN(3, 4);           // SANA's 2240, FLUX's 3072: four warps per row
  else DQ_LN(4, 4);
#undef DQ_LN
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
  const int64_t total = B * T * H * (d / 8);             // 16-byte vectors per part
  if (total > 0xffffff00LL) return DIROTQ_E_TOO_LARGE;
  const dim3 blocks((unsigned)((total + 255) / 256), 3);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d == 128) qkv_norm_rope_kernel<16><<<blocks, 256, 0, st>>>(a);
  else qkv_norm_rope_kernel<8><<<blocks, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

}  // extern "C"
