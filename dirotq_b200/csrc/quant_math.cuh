// Activation-quantiser arithmetic, one operation at a time with explicit rounding, so that codes,
// scales and zero points are bit-identical to what torch computes for the reference expressions
// (DiRotQ utils/quant_utils.py:63-85, :148-180, :201-216) on a bf16 (or fp32) tensor.
// Every step is an IEEE round-to-nearest operation followed, in bf16 mode, by a round to bf16 --
// exactly the sequence of eager tensor ops.  The "fast" forms further down replace the per-element
// divide by a reciprocal multiply that is bit-identical for bf16 operands (see div_round_bf16).
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
  // a and maxq (7, 15, 255) are bf16 values: the reciprocal multiply rounds to the same bf16 as the divide (see
  // div_round_bf16 below); the fp32 forms of the slow path keep the divide
  if constexpr (BF16) p.scale = (a == 0.f) ? 1.f : rnd<true>(__fmul_rn(a, __frcp_rn(maxq)));
  else p.scale = (a == 0.f) ? 1.f : __fdiv_rn(a, maxq);
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
// bf16_rn(fl32(x / s)) without a divide: multiply by the correctly rounded reciprocal of s (one per group).
// Bit-identical to the divide whenever x and s are bf16 values (they always are here: x is the bf16-rounded rotated
// tensor, s a scale already cast to bf16).  Reason: x = a 2^e and s = b 2^f with integer significands a <= 255,
// 128 <= b <= 255, so the exact quotient a / b is either dyadic with at most 8 significant bits (then both forms
// give it exactly) or at least 1 / (512 b) >= 2^-17 (relative) away from every bf16 rounding boundary -- two orders
// of magnitude more than the 2^-23 the product x * fl32(1 / s) can be off.  Checked exhaustively over all
// significand pairs and exponent differences: the product never comes closer than 129 fp32 ulps to a boundary.
__device__ __forceinline__ float div_round_bf16(float x, float s, float rcp_s) {
  (void)s;
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(x, rcp_s)));
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
  if constexpr (BF16) {
    // d, maxq, xmin and the scale are bf16 values: reciprocal multiplies round to the same bf16 as the divides
    p.scale = rnd<true>(__fmul_rn(d, __frcp_rn(maxq)));
    p.zero = rnd<true>(rintf(rnd<true>(__fmul_rn(-xmin, __frcp_rn(p.scale)))));
  } else {
    p.scale = __fdiv_rn(d, maxq);
    p.zero = rintf(__fdiv_rn(-xmin, p.scale));
  }
  return p;
}
// quant_utils.py:80
template <bool BF16>
__device__ __forceinline__ int int_asym_code(float x, float scale, float zero, float maxq) {
  float q = rnd<BF16>(__fadd_rn(rintf(rnd<BF16>(__fdiv_rn(x, scale))), zero));
  q = fminf(fmaxf(q, 0.f), maxq);
  return (int)q;
}

// Eight consecutive values -> eight codes (nibble i = value i; bytes for the 8-bit mode), by the reciprocal multiply
// of div_round_bf16 (no divide, no guard: see there).
__device__ __forceinline__ uint32_t int_sym_nib8_fast(const float* v, float s, float rcp_s) {
  // Two values per packed bf16 instruction: round the quotients to bf16, clamp to [-8, 7], add 192 (bf16 spacing 1 in
  // [128, 256): the add rounds half-even to the integer, whose two's-complement nibble is the low mantissa bits).
  (void)s;
  const __nv_bfloat162 lo2 = __floats2bfloat162_rn(-8.f, -8.f), hi2 = __floats2bfloat162_rn(7.f, 7.f),
                       magic = __floats2bfloat162_rn(192.f, 192.f);
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    __nv_bfloat162 r = __floats2bfloat162_rn(__fmul_rn(v[j], rcp_s), __fmul_rn(v[j + 1], rcp_s));   // .x (low half) = value j
    r = __hadd2(__hmin2(__hmax2(r, lo2), hi2), magic);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(&r) & 0x000F000Fu;
    w |= ((b & 0xFu) | (b >> 12)) << (4 * j);
  }
  return w;
}
// The same from four words of packed bf16 pairs (as loaded): value 2 i in the low half of word i.
__device__ __forceinline__ uint32_t int_sym_nib8_packed(const uint32_t* p, float rcp_s) {
  const __nv_bfloat162 lo2 = __floats2bfloat162_rn(-8.f, -8.f), hi2 = __floats2bfloat162_rn(7.f, 7.f),
                       magic = __floats2bfloat162_rn(192.f, 192.f);
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float f0 = __uint_as_float(p[i] << 16), f1 = __uint_as_float(p[i] & 0xFFFF0000u);
    __nv_bfloat162 r = __floats2bfloat162_rn(__fmul_rn(f0, rcp_s), __fmul_rn(f1, rcp_s));
    r = __hadd2(__hmin2(__hmax2(r, lo2), hi2), magic);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(&r) & 0x000F000Fu;
    w |= ((b & 0xFu) | (b >> 12)) << (8 * i);
  }
  return w;
}
// Thirty-two values as sixteen words of packed pairs -> the sixteen bytes of the planar-32 layout directly: value j is
// paired with value 16 + j BEFORE the packed rounding, so that the two nibbles of byte j come out of one register
// (no re-ordering of nibbles afterwards).  The two quotients of a pair are one packed fp32 multiply.  `clamp` is
// needed only when the scale was clipped (clip_ratio < 1): with scale = bf16(amax / 7) no quotient exceeds 7.03.
__device__ __forceinline__ uint4 int_sym_planar32_packed(const uint32_t* p, float rcp_s, bool clamp) {
  const __nv_bfloat162 lo2 = __floats2bfloat162_rn(-8.f, -8.f), hi2 = __floats2bfloat162_rn(7.f, 7.f),
                       magic = __floats2bfloat162_rn(192.f, 192.f);
  const uint64_t rr = ((uint64_t)__float_as_uint(rcp_s) << 32) | __float_as_uint(rcp_s);
  uint32_t out[4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = 4 * wd + k;                          // byte j: slots j and 16 + j
      const uint32_t a = p[j >> 1], b = p[8 + (j >> 1)];
      const uint32_t fa = (j & 1) ? (a & 0xFFFF0000u) : (a << 16), fb = (j & 1) ? (b & 0xFFFF0000u) : (b << 16);
      uint64_t q;
      asm("{\n\t.reg .b64 x;\n\tmov.b64 x, {%1, %2};\n\tmul.rn.f32x2 %0, x, %3;\n\t}" : "=l"(q) : "r"(fa), "r"(fb), "l"(rr));
      __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float((uint32_t)q), __uint_as_float((uint32_t)(q >> 32)));
      if (clamp) r = __hmin2(__hmax2(r, lo2), hi2);
      r = __hadd2(r, magic);
      const uint32_t c = *reinterpret_cast<const uint32_t*>(&r) & 0x000F000Fu;
      acc |= ((c & 0xFu) | (c >> 12)) << (8 * k);
    }
    out[wd] = acc;
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}
// The asymmetric 4-bit form of the same: code = clamp(rint(bf16(x / s)) + zero, 0, 15).  On packed bf16 pairs: adding
// 192 rounds the quotient (|q| <= 15.1) half-even to an integer (bf16 spacing is 1 in [128, 256)); adding (zero - 192)
// gives rint(q) + zero exactly (both are integers below 2^8); clamp; adding 128 leaves the code in the low mantissa bits.
__device__ __forceinline__ uint4 int_asym_planar32_packed(const uint32_t* p, float rcp_s, float zero) {
  const __nv_bfloat162 c192 = __floats2bfloat162_rn(192.f, 192.f), c0 = __floats2bfloat162_rn(0.f, 0.f),
                       c15 = __floats2bfloat162_rn(15.f, 15.f), c128 = __floats2bfloat162_rn(128.f, 128.f),
                       zm = __floats2bfloat162_rn(zero - 192.f, zero - 192.f);
  const uint64_t rr = ((uint64_t)__float_as_uint(rcp_s) << 32) | __float_as_uint(rcp_s);
  uint32_t out[4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = 4 * wd + k;
      const uint32_t a = p[j >> 1], b = p[8 + (j >> 1)];
      const uint32_t fa = (j & 1) ? (a & 0xFFFF0000u) : (a << 16), fb = (j & 1) ? (b & 0xFFFF0000u) : (b << 16);
      uint64_t q;
      asm("{\n\t.reg .b64 x;\n\tmov.b64 x, {%1, %2};\n\tmul.rn.f32x2 %0, x, %3;\n\t}" : "=l"(q) : "r"(fa), "r"(fb), "l"(rr));
      __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float((uint32_t)q), __uint_as_float((uint32_t)(q >> 32)));
      r = __hadd2(__hadd2(r, c192), zm);
      r = __hadd2(__hmin2(__hmax2(r, c0), c15), c128);
      const uint32_t c = *reinterpret_cast<const uint32_t*>(&r) & 0x000F000Fu;
      acc |= ((c & 0xFu) | (c >> 12)) << (8 * k);
    }
    out[wd] = acc;
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}
// largest and smallest of sixteen packed bf16 values
__device__ __forceinline__ void minmax_bf16x16(const uint32_t* w, float& mx, float& mn) {
  __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&w[0]), lo = hi;
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    hi = __hmax2(hi, x);
    lo = __hmin2(lo, x);
  }
  const uint32_t h = *reinterpret_cast<const uint32_t*>(&hi), l = *reinterpret_cast<const uint32_t*>(&lo);
  mx = fmaxf(mx, fmaxf(__uint_as_float(h << 16), __uint_as_float(h & 0xFFFF0000u)));
  mn = fminf(mn, fminf(__uint_as_float(l << 16), __uint_as_float(l & 0xFFFF0000u)));
}
// asymmetric: codes in [0, maxq]; returned as eight bytes in two words
__device__ __forceinline__ uint2 int_asym_byte8_fast(const float* v, float s, float rcp_s, float zero, float maxq) {
  (void)s;
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float r = rint_bf16(__bfloat162float(__float2bfloat16_rn(__fmul_rn(v[j], rcp_s))));
    float q = __bfloat162float(__float2bfloat16_rn(__fadd_rn(r, zero)));
    q = fminf(fmaxf(q, 0.f), maxq);
    w[j >> 2] |= (int_bits(q) & 0xFFu) << (8 * (j & 3));
  }
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

// The same decision on PACKED bf16 pairs, two values per instruction and no conversion to fp32.  For a power-of-two
// tensor scale the seven threshold products thr * eff have at most 3 + 4 significant bits, so they are exact in bf16
// too, and  |x| > thr * eff  can be taken on the bf16 values themselves (positive floats order like their bit
// patterns; adding the sign bit to the magnitude bits turns '>=' into '>' for negative x).  Per pair: seven packed
// compares that yield 1.0 / 0.0, six packed adds (the count, exact), one add of 128 that leaves the count in the low
// mantissa bits, and a handful of logic operations for the sign (no negative zero) and the nibble packing.
// w[i] holds values 2 i (low half) and 2 i + 1; returns the sixteen nibbles in sequential order.
__device__ __forceinline__ bool nvfp4_pow2_tensor_scale(float T) { return (__float_as_uint(T) & 0x7FFFFFu) == 0u; }
__device__ __forceinline__ uint2 nvfp4_hw_group_packed(const uint32_t* w, float eff) {
  __nv_bfloat162 t[7];
  const float thr[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.f};
#pragma unroll
  for (int i = 0; i < 7; ++i) {
    const float p = __fmul_rn(thr[i], eff);
    t[i] = __floats2bfloat162_rn(p, p);
  }
  const __nv_bfloat162 c128 = __floats2bfloat162_rn(128.f, 128.f);
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t neg2 = (w[i] >> 15) & 0x00010001u;
    const uint32_t a2 = (w[i] & 0x7FFF7FFFu) + neg2;
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&a2);
    __nv_bfloat162 m = __hadd2(__hadd2(__hadd2(__hgt2(a, t[0]), __hgt2(a, t[1])), __hadd2(__hgt2(a, t[2]), __hgt2(a, t[3]))),
                               __hadd2(__hadd2(__hgt2(a, t[4]), __hgt2(a, t[5])), __hgt2(a, t[6])));
    m = __hadd2(m, c128);
    const uint32_t mi = *reinterpret_cast<const uint32_t*>(&m) & 0x00070007u;
    const uint32_t nz2 = ((mi + 0x00070007u) >> 3) & 0x00010001u;           // 1 where the magnitude index is not zero
    const uint32_t c2 = mi | ((neg2 & nz2) << 3);
    out[i >> 2] |= ((c2 & 0xFu) | (c2 >> 12)) << (8 * (i & 3));
  }
  return make_uint2(out[0], out[1]);
}
// largest magnitude of sixteen packed bf16 values
__device__ __forceinline__ float amax_bf16x16(const uint32_t* w) {
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t a = w[i] & 0x7FFF7FFFu;
    const __nv_bfloat162 x = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&m));
    m = *reinterpret_cast<const uint32_t*>(&x);
  }
  return fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xFFFF0000u));
}

}  // namespace dq
