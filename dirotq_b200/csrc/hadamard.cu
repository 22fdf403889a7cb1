// Walsh-Hadamard front end of the layers the reference rotates with a randomised Hadamard transform
// instead of a dense PCA rotation (DiRotQ dirotq_fused_unrotation_fast.py:106-128, utils/hadamard_utils.py:56-80):
//   y[:, :n] = FWHT(x[:, :n] * flips) / sqrt(n)   (fp32 butterflies, stage order h = 1, 2, 4, ...)
//   y[:, n:] = x[:, n:]
// Every output is produced by the same sequence of fp32 additions as the reference's butterfly, so the
// result is bit-identical to it; the quantiser then runs on y.  HBM-bound: 2 D bytes in, 2 D bytes out per
// row.  One CTA per row, 16 contiguous elements per thread: four stages in registers, the rest through
// shared memory.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"

namespace dq {

__global__ void __launch_bounds__(512)
hadamard_low_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int D, int n, const __nv_bfloat16* __restrict__ flips,
                    float inv_norm_is_exact, float norm, __nv_bfloat16* __restrict__ y) {
  extern __shared__ float sh[];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * D;
  __nv_bfloat16* yr = y + row * D;
  const int t = threadIdx.x;
  const int base = 16 * t;
  float v[16];
  {
    const uint4 a = *reinterpret_cast<const uint4*>(xr + base);
    const uint4 b = *reinterpret_cast<const uint4*>(xr + base + 8);
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 p = ha[j], q = hb[j];
      if (flips) {                      // the product with +-1 is taken in bf16, as the reference does
        p = __hmul2(p, *reinterpret_cast<const __nv_bfloat162*>(flips + base + 2 * j));
        q = __hmul2(q, *reinterpret_cast<const __nv_bfloat162*>(flips + base + 8 + 2 * j));
      }
      const float2 fp = __bfloat1622float2(p), fq = __bfloat1622float2(q);
      v[2 * j] = fp.x; v[2 * j + 1] = fp.y; v[8 + 2 * j] = fq.x; v[8 + 2 * j + 1] = fq.y;
    }
  }
  // stages h = 1, 2, 4, 8: pairs (i, i + h) inside blocks of 2h, all inside this thread's 16 elements
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const float p = v[i], q = v[i + h];
        v[i] = __fadd_rn(p, q);
        v[i + h] = __fsub_rn(p, q);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) sh[base + i] = v[i];
  __syncthreads();
  // stages h = 16 ... n/2 in shared memory: n/2 butterflies per stage, 8 per thread
  for (int h = 16; h < n; h <<= 1) {
    float p[8], q[8];
    int idx[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int b = t + k * blockDim.x;                 // butterfly number 0 .. n/2-1
      const int i = ((b / h) * 2 * h) + (b % h);        // lower element of the pair
      idx[k] = i;
      p[k] = sh[i];
      q[k] = sh[i + h];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      sh[idx[k]] = __fadd_rn(p[k], q[k]);
      sh[idx[k] + h] = __fsub_rn(p[k], q[k]);
    }
    __syncthreads();
  }
  // normalise (IEEE division by sqrt(n), exact scaling when n is a power of four) and store
  {
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f0 = inv_norm_is_exact != 0.f ? sh[base + 2 * j] * inv_norm_is_exact : __fdiv_rn(sh[base + 2 * j], norm);
      const float f1 = inv_norm_is_exact != 0.f ? sh[base + 2 * j + 1] * inv_norm_is_exact : __fdiv_rn(sh[base + 2 * j + 1], norm);
      __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
      w[j] = *reinterpret_cast<uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(yr + base) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(yr + base + 8) = make_uint4(w[4], w[5], w[6], w[7]);
  }
  // untouched channels
  for (int c = n + 8 * t; c < D; c += 8 * blockDim.x)
    *reinterpret_cast<uint4*>(yr + c) = *reinterpret_cast<const uint4*>(xr + c);
}

int launch_hadamard_low(const void* x, int64_t M, int D, int n, const void* flips, void* y, cudaStream_t st) {
  if (M <= 0) return DIROTQ_OK;
  if (n < 16 || n > 8192 || (n & (n - 1)) || n > D || D % 8) return DIROTQ_E_UNSUPPORTED;
  int log2n = 0;
  while ((1 << log2n) < n) ++log2n;
  const float norm = sqrtf((float)n);
  const float inv_exact = (log2n % 2 == 0) ? 1.f / norm : 0.f;    // power of four: the division is an exact scaling
  const int threads = n / 16;
  const size_t smem = (size_t)n * sizeof(float);
  hadamard_low_kernel<<<(unsigned)M, threads, smem, st>>>(static_cast<const __nv_bfloat16*>(x), M, D, n,
                                                           static_cast<const __nv_bfloat16*>(flips), inv_exact, norm,
                                                           static_cast<__nv_bfloat16*>(y));
  return cudaGetLastError() == cudaSuccess ? DIROTQ_OK : DIROTQ_E_CUDA;
}

}  // namespace dq
