// Activation-quantiser arithmetic, one operation at a time with explicit rounding, so that codes,
// scales and zero points are bit-identical to what torch computes for the reference expressions
// (DiRotQ utils/quant_utils.py:63-85, :148-180, :201-216) on a bf16 (or fp32) tensor.
// Every step is an IEEE round-to-nearest operation followed, in bf16 mode, by a round to bf16 --
// exactly the sequence of eager tensor ops.  The "fast" forms further down replace the per-element
// divide by a guarded reciprocal multiply that is proven bit-identical (see div_round_bf16).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cstdint>

namespace dq {

enum QuantMode : int {
  MODE_INT4_SYM = 0,   // codes in [-8, 7]
  MODE_INT4_ASYM = 1,  // codes in [0, 15] + zero point
  MODE_INT8_ASYM = 2,  // codes in [0, 255] + zero point (W4A8)
  MODE_NVFP4_REF = 3,  // E2M1 codes, bf16 group scale exactly as the reference (not GEMM-consumable)
  MODE_NVFP4_HW = 4,   // E2M1 codes, UE4M3 group scale relative to an fp32 tensor scale
};

template <bool BF16>
__device__ __forceinline__ float rnd(float v) {
  if constexpr (BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

struct GroupParams {
  float scale;
  float zero;
};

// quant_utils.py:202-209 (symmetric branch).  mx/mn: max and min over the group.
template <bool BF16>
__device__ __forceinline__ GroupParams int_sym_params(float mx, float mn, float clip, float maxq) {
  float xmax = rnd<BF16>(__fmul_rn(mx, clip));
  float xmin = rnd<BF16>(__fmul_rn(mn, clip));
  float a = fmaxf(fabsf(xmin), xmax);
  GroupParams p;
  p.scale = (a == 0.f) ? 1.f : rnd<BF16>(__fdiv_rn(a, maxq));
  p.zero = 0.f;
  return p;
}
// quant_utils.py:67
template <bool BF16>
__device__ __forceinline__ int int_sym_code(float x, float scale, float maxq) {
  float q = rintf(rnd<BF16>(__fdiv_rn(x, scale)));
  q = fminf(fmaxf(q, -maxq - 1.f), maxq);
  return (int)q;
}
// ---- fast exact forms used by the fused kernel's epilogue ---------------------------------------
// bf16_rn(fl32(x / s)) without a divide per element: multiply by the correctly rounded reciprocal
// (one per group) and fall back to the IEEE divide only when the approximate quotient lies within
// 3 fp32 ulps of a bf16 rounding boundary (low half in [0x7FFD, 0x8003], probability ~1e-4), where
// the <= 2 ulp error of the product could change the bf16 result.  Bit-identical to the slow form.
__device__ __forceinline__ float div_round_bf16(float x, float s, float rcp_s) {
  float qa = __fmul_rn(x, rcp_s);
  const uint32_t b = __float_as_uint(qa);
  if (((b + 0x8003u) & 0xFFFFu) <= 6u) qa = __fdiv_rn(x, s);
  return __bfloat162float(__float2bfloat16_rn(qa));
}
// round-half-even of a bf16-valued float: the 1.5 * 2^23 trick below 2^22, identity above (bf16
// values >= 256 are integers already)
__device__ __forceinline__ float rint_small(float r) { return (r + 12582912.f) - 12582912.f; }
__device__ __forceinline__ float rint_bf16(float r) { return fabsf(r) < 4194304.f ? rint_small(r) : r; }
// two's-complement nibble of an integer-valued float in [-8, 7] (or the byte of one in [0, 255])
__device__ __forceinline__ uint32_t int_bits(float c) { return __float_as_uint(c + 12582912.f); }

__device__ __forceinline__ uint32_t int_sym_nibble_fast(float x, float s, float rcp_s) {
  float r = div_round_bf16(x, s, rcp_s);
  r = fminf(fmaxf(r, -8.f), 7.f);          // clamp commutes with round-half-even for integer bounds
  return int_bits(r) & 0xFu;               // the add rounds half-even, the low mantissa bits are the code
}
__device__ __forceinline__ uint32_t int_asym_code_fast(float x, float s, float rcp_s, float zero, float maxq) {
  float r = rint_bf16(div_round_bf16(x, s, rcp_s));
  float q = __bfloat162float(__float2bfloat16_rn(__fadd_rn(r, zero)));
  q = fminf(fmaxf(q, 0.f), maxq);
  return int_bits(q) & 0xFFu;
}

// quant_utils.py:211-215
template <bool BF16>
__device__ __forceinline__ GroupParams int_asym_params(float mx, float mn, float clip, float maxq) {
  float xmax = rnd<BF16>(__fmul_rn(mx, clip));
  float xmin = rnd<BF16>(__fmul_rn(mn, clip));
  if (xmin == 0.f && xmax == 0.f) { xmin = -1.f; xmax = 1.f; }
  float d = rnd<BF16>(__fsub_rn(xmax, xmin));
  d = fmaxf(d, rnd<BF16>(1e-5f));
  GroupParams p;
  p.scale = rnd<BF16>(__fdiv_rn(d, maxq));
  p.zero = rnd<BF16>(rintf(rnd<BF16>(__fdiv_rn(-xmin, p.scale))));
  return p;
}
// quant_utils.py:80
template <bool BF16>
__device__ __forceinline__ int int_asym_code(float x, float scale, float zero, float maxq) {
  float q = rnd<BF16>(__fadd_rn(rintf(rnd<BF16>(__fdiv_rn(x, scale))), zero));
  q = fminf(fmaxf(q, 0.f), maxq);
  return (int)q;
}

// Eight consecutive values -> eight codes (nibble i = value i; bytes for the 8-bit mode).  The guard
// of div_round_bf16 is evaluated for all eight and OR-ed; only if one of them is close to a rounding
// boundary are the eight redone with the IEEE divide, in an out-of-line function so that the compiler
// cannot if-convert the expensive path into the common one.
static __device__ __noinline__ uint32_t int_sym_nib8_exact(float v0, float v1, float v2, float v3, float v4, float v5,
                                                           float v6, float v7, float s) {
  const float v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) w |= ((uint32_t)int_sym_code<true>(v[j], s, 7.f) & 0xFu) << (4 * j);
  return w;
}
__device__ __forceinline__ uint32_t int_sym_nib8_fast(const float* v, float s, float rcp_s) {
  // Two values per packed bf16 instruction: round the quotients to bf16, clamp to [-8, 7], add 192 (bf16 spacing 1 in
  // [128, 256): the add rounds half-even to the integer, whose two's-complement nibble is the low mantissa bits).
  const __nv_bfloat162 lo2 = __floats2bfloat162_rn(-8.f, -8.f), hi2 = __floats2bfloat162_rn(7.f, 7.f),
                       magic = __floats2bfloat162_rn(192.f, 192.f);
  uint32_t w = 0, near = 0;
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float q0 = __fmul_rn(v[j], rcp_s), q1 = __fmul_rn(v[j + 1], rcp_s);
    near |= (uint32_t)(((__float_as_uint(q0) + 0x8003u) & 0xFFFFu) <= 6u) |
            (uint32_t)(((__float_as_uint(q1) + 0x8003u) & 0xFFFFu) <= 6u);
    __nv_bfloat162 r = __floats2bfloat162_rn(q0, q1);          // .x (low half) = q0
    r = __hadd2(__hmin2(__hmax2(r, lo2), hi2), magic);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(&r) & 0x000F000Fu;
    w |= ((b & 0xFu) | (b >> 12)) << (4 * j);
  }
  if (near) w = int_sym_nib8_exact(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], s);
  return w;
}
// asymmetric: codes in [0, maxq]; returned as eight bytes in two words
static __device__ __noinline__ uint2 int_asym_byte8_exact(float v0, float v1, float v2, float v3, float v4, float v5,
                                                          float v6, float v7, float s, float zero, float maxq) {
  const float v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j >> 2] |= ((uint32_t)int_asym_code<true>(v[j], s, zero, maxq) & 0xFFu) << (8 * (j & 3));
  return make_uint2(w[0], w[1]);
}
__device__ __forceinline__ uint2 int_asym_byte8_fast(const float* v, float s, float rcp_s, float zero, float maxq) {
  uint32_t w[2] = {0u, 0u};
  uint32_t near = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float qa = __fmul_rn(v[j], rcp_s);
    near |= (uint32_t)(((__float_as_uint(qa) + 0x8003u) & 0xFFFFu) <= 6u);
    const float r = rint_bf16(__bfloat162float(__float2bfloat16_rn(qa)));
    float q = __bfloat162float(__float2bfloat16_rn(__fadd_rn(r, zero)));
    q = fminf(fmaxf(q, 0.f), maxq);
    w[j >> 2] |= (int_bits(q) & 0xFFu) << (8 * (j & 3));
  }
  if (near) return int_asym_byte8_exact(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], s, zero, maxq);
  return make_uint2(w[0], w[1]);
}
// four bytes holding 4-bit values -> four nibbles in the low 16 bits
__device__ __forceinline__ uint32_t squeeze_nibbles(uint32_t b) {
  b = (b | (b >> 4)) & 0x00FF00FFu;
  return (b | (b >> 8)) & 0xFFFFu;
}
// four nibbles (low 16 bits) -> four bytes
__device__ __forceinline__ uint32_t spread_nibbles(uint32_t x) {
  x = (x | (x << 8)) & 0x00FF00FFu;
  return (x | (x << 4)) & 0x0F0F0F0Fu;
}
// 32 codes given as four words of eight sequential nibbles -> the planar-32 layout
// (byte j = code j | code 16+j << 4)
__device__ __forceinline__ uint4 planar32_from_nib8(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
  return make_uint4(spread_nibbles(a0 & 0xFFFFu) | (spread_nibbles(a2 & 0xFFFFu) << 4),
                    spread_nibbles(a0 >> 16) | (spread_nibbles(a2 >> 16) << 4),
                    spread_nibbles(a1 & 0xFFFFu) | (spread_nibbles(a3 & 0xFFFFu) << 4),
                    spread_nibbles(a1 >> 16) | (spread_nibbles(a3 >> 16) << 4));
}

// E2M1 nibble of a normalised value with the reference's bucketize rule (quant_utils.py:30-35):
// an exact midpoint goes to the LOWER codebook value (toward -inf); there is no negative zero.
__device__ __forceinline__ uint32_t e2m1_nibble(float v) {
  float a = fabsf(v);
  uint32_t m;
  if (v >= 0.f) {
    m = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.f);
    return m;
  }
  m = (a >= 0.25f) + (a >= 0.75f) + (a >= 1.25f) + (a >= 1.75f) + (a >= 2.5f) + (a >= 3.5f) + (a >= 5.f);
  return m ? (8u | m) : 0u;
}

// quant_utils.py:172-173
template <bool BF16>
__device__ __forceinline__ float nvfp4_ref_scale(float amax, float clip) {
  float s = rnd<BF16>(__fmul_rn(amax, clip));
  s = rnd<BF16>(__fdiv_rn(s, 6.f));
  return fmaxf(s, rnd<BF16>(1e-5f));
}
template <bool BF16>
__device__ __forceinline__ uint32_t nvfp4_ref_code(float x, float scale) {
  return e2m1_nibble(rnd<BF16>(__fdiv_rn(x, scale)));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}
// Two-level scale: micro = e4m3_rn(clamp(amax*clip/6/T, 2^-9, 448)), 0 for an all-zero group.
// Returns the e4m3 byte and the effective fp32 scale micro*T.
__device__ __forceinline__ uint8_t nvfp4_hw_scale(float amax, float clip, float T, float* eff) {
  if (amax == 0.f) { *eff = 0.f; return 0; }
  float s = __fdiv_rn(__fmul_rn(amax, clip), 6.f);
  float r = fmaxf(__fdiv_rn(s, T), 0.001953125f);
  r = fminf(r, 448.f);
  uint8_t b = (uint8_t)__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
  *eff = __fmul_rn(e4m3_to_float(b), T);
  return b;
}
__device__ __forceinline__ uint32_t nvfp4_hw_code(float x, float eff) {
  return eff > 0.f ? e2m1_nibble(__fdiv_rn(x, eff)) : 0u;
}
// ---- fast exact form of the two-level NVFP4 quantiser -------------------------------------------
// The reference decides  fl32(x / eff) > thr  (thr = 0.25 ... 5, '>=' for negative x).  x is a bf16
// value (8 significant bits), eff = micro * T with micro a UE4M3 value (4 bits).  When T has at most 12
// significant bits, thr * eff is exact in fp32 and is either equal to |x| or differs from it by more
// than 2^-19 relative, far more than the 2^-24 the fp32 quotient can move; hence
//      fl32(|x| / eff) > thr   <=>   |x| > thr * eff
// and no division is needed at all: seven exact threshold products per group, seven integer compares
// per value (adding the sign bit to the magnitude bits turns '>=' into '>').  The guarded-reciprocal
// trick used for INT codes does not work here: with so few bits in eff, x * (1/eff) lands on or next to
// a decision threshold for a quarter of all values.
__device__ __forceinline__ bool nvfp4_short_tensor_scale(float T) { return (__float_as_uint(T) & 0xFFFu) == 0u; }
static __device__ __noinline__ uint2 nvfp4_hw_group_exact(float v0, float v1, float v2, float v3, float v4, float v5, float v6, float v7, float v8, float v9, float v10, float v11, float v12, float v13, float v14, float v15, float eff) {
  const float v[16] = {v0, v1, v2, v3, v4, v5, v6, v7, v8, v9, v10, v11, v12, v13, v14, v15};
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    lo |= nvfp4_hw_code(v[j], eff) << (4 * j);
    hi |= nvfp4_hw_code(v[8 + j], eff) << (4 * j);
  }
  return make_uint2(lo, hi);
}
// Any group (partial, all-zero scale): exact per-element path, out of line for the same reason.
static __device__ __noinline__ uint2 nvfp4_hw_group_partial(float v0, float v1, float v2, float v3, float v4, float v5, float v6, float v7, float v8, float v9, float v10, float v11, float v12, float v13, float v14, float v15, int nvalid, float eff) {
  const float v[16] = {v0, v1, v2, v3, v4, v5, v6, v7, v8, v9, v10, v11, v12, v13, v14, v15};
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    lo |= (j < nvalid ? nvfp4_hw_code(v[j], eff) : 0u) << (4 * j);
    hi |= (8 + j < nvalid ? nvfp4_hw_code(v[8 + j], eff) : 0u) << (4 * j);
  }
  return make_uint2(lo, hi);
}
__device__ __forceinline__ uint2 nvfp4_hw_group_fast(const float* v, float eff) {
  const uint32_t t0 = __float_as_uint(__fmul_rn(0.25f, eff)), t1 = __float_as_uint(__fmul_rn(0.75f, eff)),
                 t2 = __float_as_uint(__fmul_rn(1.25f, eff)), t3 = __float_as_uint(__fmul_rn(1.75f, eff)),
                 t4 = __float_as_uint(__fmul_rn(2.5f, eff)), t5 = __float_as_uint(__fmul_rn(3.5f, eff)),
                 t6 = __float_as_uint(__fmul_rn(5.f, eff));
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t bits = __float_as_uint(v[j]);
    const uint32_t neg = bits >> 31;
    const uint32_t a = (bits & 0x7FFFFFFFu) + neg;
    const uint32_t m = (a > t0) + (a > t1) + (a > t2) + (a > t3) + (a > t4) + (a > t5) + (a > t6);
    w[j >> 3] |= (m | ((m != 0u ? neg : 0u) << 3)) << (4 * (j & 7));
  }
  return make_uint2(w[0], w[1]);
}

}  // namespace dq
