// Kernel 2 (INT): W4A4 / W4A8 GEMM with exact int32 accumulation per 64-wide chunk, the bf16
// high-precision branch, per-chunk dequantisation and bias -- one kernel, one pass over the operands.
//
//   y[m,n] = sum_c xs[c,m] ws[c,n] ( sum_k qx[m,c,k] qw[n,c,k]  -  xz[c,m] wsum[c,n] )
//            + x_tail[m,:] . w_tail[n,:] + bias[n]
//
// 4-bit codes stay packed in HBM / L2.  Producer warps load them with 16-byte loads, widen every
// nibble to a byte *in registers* (nibble << 4 is already the sign-extended value times 16, so two
// logic ops per 8 codes; the factor is a power of two folded into the activation scale) and store
// the bytes into shared memory in the 128-byte-swizzled K-major layout tcgen05.mma kind::i8 reads.
// One UMMA pair (K = 2 x 32) fills a 128 x 128 int32 accumulator in TMEM per chunk; two accumulators
// alternate, so the tensor pipe computes chunk c+1 while eight epilogue warps drain chunk c:
// tcgen05.ld, exact int -> float, scale by ws[c,n] and xs[c,m], add into fp32 registers.
// The tail branch runs as kind::f16 UMMAs into the same TMEM and is added last.
//
// Replaces the inner `self.module(x)` of the fused forward (DiRotQ
// dirotq_fused_unrotation_fast.py:141), which the reference's speed path hands to the third-party
// nunchaku gemm_w4a4.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace dq {

constexpr int GI_STAGES = 5;
constexpr int GI_TILE_BYTES = 128 * 128;                 // one operand tile: 128 rows x 128 bytes
constexpr int GI_AUX_FLOATS = 4 * 2 * 128;               // sw, sx, wsum, xz : [2 chunks][128]
constexpr int GI_STAGE_BYTES = 2 * GI_TILE_BYTES + GI_AUX_FLOATS * 4;   // 36864
constexpr int GI_EPI_WARPS = 8;
constexpr int GI_PROD_WARPS = 2;
constexpr int GI_THREADS = (GI_EPI_WARPS + 1 + GI_PROD_WARPS) * 32;     // 352
constexpr int GI_PROD_THREADS = GI_PROD_WARPS * 32;
constexpr int GI_SMEM_BYTES = GI_STAGES * GI_STAGE_BYTES + 1024 + 256;

struct Ring {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() { if (++s == GI_STAGES) { s = 0; ph ^= 1; } }
};

// 16-byte chunk c of row r inside a 128-byte-swizzled tile
__device__ __forceinline__ uint32_t swz(uint32_t tile, int r, int c) {
  return tile + r * 128 + ((c ^ (r & 7)) << 4);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int A_MODE>
__global__ void __launch_bounds__(GI_THREADS, 1) gemm_int_kernel(const GemmIntArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GI_STAGES * GI_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GI_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (GI_STAGES + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * GI_STAGES + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * GI_STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < GI_STAGES; ++s) { mbar_init(full_bar(s), GI_PROD_THREADS); mbar_init(empty_bar(s), 1 + GI_EPI_WARPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), GI_EPI_WARPS); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == GI_EPI_WARPS) tmem_alloc(smem_u32(tmem_slot), 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);

  const int64_t m0 = (int64_t)blockIdx.y * 128;
  const int64_t n0 = (int64_t)blockIdx.x * 128;
  const int n_main = (a.n_chunks + 1) >> 1;               // stages of two chunks
  const int n_tail = (a.kt + 63) >> 6;                    // stages of 64 bf16
  constexpr bool ASYM = (A_MODE != MODE_INT4_SYM);
  constexpr float INV_F = ASYM ? (1.f / 16.f) : (1.f / 256.f);
  constexpr float F_ = ASYM ? 16.f : 256.f;

  if (warp > GI_EPI_WARPS) {
    // ------------------------------ producers ------------------------------------------------
    const int pt = threadIdx.x - (GI_EPI_WARPS + 1) * 32;  // 0..63
    Ring r;
    bool ok = true;
    for (int st = 0; st < n_main && ok; ++st) {
      if (!mbar_wait(empty_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
      const uint32_t sA = smem_base + r.s * GI_STAGE_BYTES;
      const uint32_t sB = sA + GI_TILE_BYTES;
      float* aux = reinterpret_cast<float*>(smem + r.s * GI_STAGE_BYTES + 2 * GI_TILE_BYTES);
      const int c0 = st * 2;
      // B (weights): 128 rows x 4 granules of 32 codes
#pragma unroll 4
      for (int id = pt; id < 512; id += GI_PROD_THREADS) {
        const int row = id >> 2, gi = id & 3;
        uint4 p = make_uint4(0, 0, 0, 0);
        if (n0 + row < a.N && c0 + (gi >> 1) < a.n_chunks)
          p = __ldg(reinterpret_cast<const uint4*>(a.wq + (n0 + row) * a.w_row_bytes + (int64_t)c0 * 32 + gi * 16));
        uint4 lo = make_uint4((p.x << 4) & 0xF0F0F0F0u, (p.y << 4) & 0xF0F0F0F0u, (p.z << 4) & 0xF0F0F0F0u, (p.w << 4) & 0xF0F0F0F0u);
        uint4 hi = make_uint4(p.x & 0xF0F0F0F0u, p.y & 0xF0F0F0F0u, p.z & 0xF0F0F0F0u, p.w & 0xF0F0F0F0u);
        sts128(swz(sB, row, 2 * gi), lo);
        sts128(swz(sB, row, 2 * gi + 1), hi);
      }
      // A (activations)
      if constexpr (A_MODE == MODE_INT8_ASYM) {
#pragma unroll 4
        for (int id = pt; id < 1024; id += GI_PROD_THREADS) {
          const int row = id >> 3, gi = id & 7;
          uint4 p = make_uint4(0, 0, 0, 0);
          if (m0 + row < a.M && c0 + (gi >> 2) < a.n_chunks)
            p = __ldg(reinterpret_cast<const uint4*>(a.xq + (m0 + row) * a.x_row_bytes + (int64_t)c0 * 64 + gi * 16));
          sts128(swz(sA, row, gi), p);
        }
      } else {
#pragma unroll 4
        for (int id = pt; id < 512; id += GI_PROD_THREADS) {
          const int row = id >> 2, gi = id & 3;
          uint4 p = make_uint4(0, 0, 0, 0);
          if (m0 + row < a.M && c0 + (gi >> 1) < a.n_chunks)
            p = __ldg(reinterpret_cast<const uint4*>(a.xq + (m0 + row) * a.x_row_bytes + (int64_t)c0 * 32 + gi * 16));
          uint4 lo, hi;
          if constexpr (A_MODE == MODE_INT4_SYM) {
            lo = make_uint4((p.x << 4) & 0xF0F0F0F0u, (p.y << 4) & 0xF0F0F0F0u, (p.z << 4) & 0xF0F0F0F0u, (p.w << 4) & 0xF0F0F0F0u);
            hi = make_uint4(p.x & 0xF0F0F0F0u, p.y & 0xF0F0F0F0u, p.z & 0xF0F0F0F0u, p.w & 0xF0F0F0F0u);
          } else {
            lo = make_uint4(p.x & 0x0F0F0F0Fu, p.y & 0x0F0F0F0Fu, p.z & 0x0F0F0F0Fu, p.w & 0x0F0F0F0Fu);
            hi = make_uint4((p.x >> 4) & 0x0F0F0F0Fu, (p.y >> 4) & 0x0F0F0F0Fu, (p.z >> 4) & 0x0F0F0F0Fu, (p.w >> 4) & 0x0F0F0F0Fu);
          }
          sts128(swz(sA, row, 2 * gi), lo);
          sts128(swz(sA, row, 2 * gi + 1), hi);
        }
      }
      // per-chunk scales (and zero points / code sums) of the tile's 128 rows and 128 columns
      for (int i = pt; i < 256; i += GI_PROD_THREADS) {
        const int c = i >> 7, j = i & 127;
        const bool cok = c0 + c < a.n_chunks;
        const bool nok = cok && (n0 + j < a.N), mok = cok && (m0 + j < a.M);
        aux[i] = nok ? __ldg(a.ws + (int64_t)(c0 + c) * a.ldn + n0 + j) : 0.f;
        aux[256 + i] = mok ? __bfloat162float(a.xs[(int64_t)(c0 + c) * a.ldm + m0 + j]) * INV_F : 0.f;
        if constexpr (ASYM) {
          aux[512 + i] = nok ? __ldg(a.wsum + (int64_t)(c0 + c) * a.ldn + n0 + j) : 0.f;
          aux[768 + i] = mok ? __bfloat162float(a.xz[(int64_t)(c0 + c) * a.ldm + m0 + j]) * F_ : 0.f;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(full_bar(r.s));
      r.next();
    }
    for (int st = 0; st < n_tail && ok; ++st) {
      if (!mbar_wait(empty_bar(r.s), r.ph ^ 1, abort_flag, a.status, ERR_WAIT_EMPTY)) { ok = false; break; }
      const uint32_t sA = smem_base + r.s * GI_STAGE_BYTES;
      const uint32_t sB = sA + GI_TILE_BYTES;
      const int k0 = st * 64;
#pragma unroll 4
      for (int id = pt; id < 2048; id += GI_PROD_THREADS) {
        const int op = id >> 10, row = (id & 1023) >> 3, gi = id & 7;
        const int k = k0 + gi * 8;
        uint4 p = make_uint4(0, 0, 0, 0);
        const __nv_bfloat16* src = nullptr;
        if (op == 0) { if (m0 + row < a.M) src = a.xt + (m0 + row) * a.kt_pitch + k; }
        else { if (n0 + row < a.N) src = a.wt + (n0 + row) * a.kt_pitch + k; }
        if (src) {
          if (k + 8 <= a.kt) {
            p = __ldg(reinterpret_cast<const uint4*>(src));
          } else if (k < a.kt) {
            __nv_bfloat16 tmp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = (k + e < a.kt) ? src[e] : __float2bfloat16_rn(0.f);
            p = *reinterpret_cast<uint4*>(tmp);
          }
        }
        sts128(swz(op == 0 ? sA : sB, row, gi), p);
      }
      fence_proxy_async_smem();
      mbar_arrive(full_bar(r.s));
      r.next();
    }
  } else if (warp == GI_EPI_WARPS) {
    // ------------------------------ UMMA issuer ----------------------------------------------
    if (lane == 0) {
      const uint32_t idesc_i8 = idesc_dense(ACC_S32, ASYM ? FMT_U8 : FMT_S8, FMT_S8, 128, 128);
      const uint32_t idesc_bf = idesc_dense(ACC_F32, FMT_BF16, FMT_BF16, 128, 128);
      Ring r;
      int use = 0;   // accumulator uses so far: buffer = use & 1, phase = (use >> 1) & 1
      bool ok = true;
      for (int st = 0; st < n_main && ok; ++st) {
        if (!mbar_wait(full_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sA = smem_base + r.s * GI_STAGE_BYTES;
        const uint64_t adesc = smem_desc_sw128(sA), bdesc = smem_desc_sw128(sA + GI_TILE_BYTES);
        for (int c = 0; c < 2; ++c) {
          if (st * 2 + c >= a.n_chunks) break;
          const int buf = use & 1;
          if (!mbar_wait(acce_bar(buf), ((use >> 1) & 1) ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + buf * 128;
          umma_i8(d, adesc + 4 * c, bdesc + 4 * c, idesc_i8, 0u);
          umma_i8(d, adesc + 4 * c + 2, bdesc + 4 * c + 2, idesc_i8, 1u);
          umma_commit(accf_bar(buf));
          ++use;
        }
        umma_commit(empty_bar(r.s));
        r.next();
      }
      if (ok && n_tail > 0) {
        const int buf = use & 1;
        if (mbar_wait(acce_bar(buf), ((use >> 1) & 1) ^ 1, abort_flag, a.status, ERR_WAIT_ACC_EMPTY)) {
          tc_fence_after();
          const uint32_t d = tmem_base + buf * 128;
          for (int st = 0; st < n_tail; ++st) {
            if (!mbar_wait(full_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sA = smem_base + r.s * GI_STAGE_BYTES;
            const uint64_t adesc = smem_desc_sw128(sA), bdesc = smem_desc_sw128(sA + GI_TILE_BYTES);
#pragma unroll
            for (int j = 0; j < 4; ++j) umma_f16(d, adesc + 2 * j, bdesc + 2 * j, idesc_bf, (st > 0 || j > 0) ? 1u : 0u);
            umma_commit(empty_bar(r.s));
            r.next();
          }
          if (ok) umma_commit(accf_bar(buf));
        }
      }
    }
  } else {
    // ------------------------------ epilogue: 8 warps ----------------------------------------
    const int q = warp & 3, half = warp >> 2;
    const int trow = q * 32 + lane;                       // row inside the tile
    const int64_t row = m0 + trow;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16) + half * 64;
    float acc[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) acc[j] = 0.f;
    Ring r;
    int use = 0;
    bool ok = true;
    for (int st = 0; st < n_main && ok; ++st) {
      if (!mbar_wait(full_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
      const float* aux = reinterpret_cast<const float*>(smem + r.s * GI_STAGE_BYTES + 2 * GI_TILE_BYTES);
      for (int c = 0; c < 2; ++c) {
        if (st * 2 + c >= a.n_chunks) break;
        const int buf = use & 1;
        if (!mbar_wait(accf_bar(buf), (use >> 1) & 1, abort_flag, a.status, ERR_WAIT_ACC_FULL)) { ok = false; break; }
        tc_fence_after();
        uint32_t v[64];
        tmem_ld32(tlane + buf * 128, v);
        tmem_ld32(tlane + buf * 128 + 32, v + 32);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acce_bar(buf));
        ++use;
        const float sx = aux[256 + c * 128 + trow];
        const float* sw = aux + c * 128 + half * 64;
        float zf = 0.f;
        const float* wsm = aux + 512 + c * 128 + half * 64;
        if constexpr (ASYM) zf = aux[768 + c * 128 + trow];
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          // exact int32 -> fp32 for |v| < 2^22: add 1.5 * 2^23 as integer, subtract as float
          float f = __int_as_float((int)v[j] + 0x4B400000) - 12582912.f;
          if constexpr (ASYM) f = __fmaf_rn(-zf, wsm[j], f);
          if (a.acc_dump && row < a.M && n0 + half * 64 + j < a.N)
            a.acc_dump[((int64_t)(st * 2 + c) * a.M + row) * a.N + n0 + half * 64 + j] = (int)(f * INV_F);
          acc[j] = __fmaf_rn(f * sw[j], sx, acc[j]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(r.s));
      r.next();
    }
    if (ok && n_tail > 0) {
      for (int st = 0; st < n_tail; ++st) {
        if (!mbar_wait(full_bar(r.s), r.ph, abort_flag, a.status, ERR_WAIT_FULL)) { ok = false; break; }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(r.s));
        r.next();
      }
      const int buf = use & 1;
      if (ok && mbar_wait(accf_bar(buf), (use >> 1) & 1, abort_flag, a.status, ERR_WAIT_ACC_FULL)) {
        tc_fence_after();
        uint32_t v[64];
        tmem_ld32(tlane + buf * 128, v);
        tmem_ld32(tlane + buf * 128 + 32, v + 32);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] += __uint_as_float(v[j]);
      } else {
        ok = false;
      }
    }
    if (ok && row < a.M) {
      const int64_t col0 = n0 + half * 64;
      __nv_bfloat16* yr = a.y + row * a.N + col0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (col0 + 8 * i + 8 <= a.N) {
          float b[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) b[e] = a.bias ? __bfloat162float(a.bias[col0 + 8 * i + e]) : 0.f;
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(acc[8 * i + 2 * e] + b[2 * e], acc[8 * i + 2 * e + 1] + b[2 * e + 1]);
            w[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(yr + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == GI_EPI_WARPS) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int A_MODE>
static int launch_gi(const GemmIntArgs& a, cudaStream_t st) {
  auto k = gemm_int_kernel<A_MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GI_SMEM_BYTES) != cudaSuccess)
      return DIROTQ_E_CUDA;
    attr_set = true;
  }
  dim3 grid((unsigned)((a.N + 127) / 128), (unsigned)((a.M + 127) / 128));
  k<<<grid, GI_THREADS, GI_SMEM_BYTES, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

int launch_gemm_int(const GemmIntArgs& a, cudaStream_t st) {
  if (a.M <= 0 || a.N <= 0) return DIROTQ_OK;
  switch (a.a_mode) {
    case DIROTQ_INT4_SYM: return launch_gi<MODE_INT4_SYM>(a, st);
    case DIROTQ_INT4_ASYM: return launch_gi<MODE_INT4_ASYM>(a, st);
    case DIROTQ_INT8_ASYM: return launch_gi<MODE_INT8_ASYM>(a, st);
  }
  return DIROTQ_E_UNSUPPORTED;
}

}  // namespace dq
