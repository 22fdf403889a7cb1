// W4A16 entry point: dequantise the packed weight into caller scratch, then the bf16 tcgen05 GEMM.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"

using namespace dq;

extern "C" {

size_t dirotq_gemm_w4a16_workspace_bytes(int64_t N, int64_t K) {
  if (N <= 0 || K <= 0) return 0;
  return pad256((size_t)N * (size_t)round_up64(K, 64) * 2);
}

int dirotq_gemm_w4a16(int64_t M, int64_t N, int64_t K, const void* x, const void* w_codes, const float* w_scales,
                      const void* bias, void* y, void* workspace, size_t workspace_bytes, int32_t* status,
                      void* stream) {
  if (M < 0 || N <= 0 || K <= 0 || !x || !w_codes || !w_scales || !y || !workspace) return DIROTQ_E_ARG;
  if (K % 64 || N % 8) return DIROTQ_E_UNSUPPORTED;
  if (workspace_bytes < dirotq_gemm_w4a16_workspace_bytes(N, K)) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)
    return DIROTQ_E_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = launch_dequant_int4(static_cast<const uint8_t*>(w_codes), w_scales, N, (int)(K / 64), ld_rows(N),
                               static_cast<__nv_bfloat16*>(workspace), st);
  if (rc) return rc;
  return launch_gemm_bf16(x, workspace, M, N, K, bias, y, status, st);
}

int dirotq_gemm_w4a16_nvfp4(int64_t M, int64_t N, int64_t K, const void* x, const void* w_codes, const void* w_sf,
                            float w_tensor_scale, const float* w_rowscale, const void* bias, void* y, void* workspace,
                            size_t workspace_bytes, int32_t* status, void* stream) {
  if (M < 0 || N <= 0 || K <= 0 || !x || !w_codes || !w_sf || !y || !workspace) return DIROTQ_E_ARG;
  if (!w_rowscale && !(w_tensor_scale > 0.f)) return DIROTQ_E_ARG;
  if (K % 64 || N % 8) return DIROTQ_E_UNSUPPORTED;
  if (workspace_bytes < dirotq_gemm_w4a16_workspace_bytes(N, K)) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)
    return DIROTQ_E_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = launch_dequant_nvfp4(static_cast<const uint8_t*>(w_codes), static_cast<const uint8_t*>(w_sf), w_tensor_scale, w_rowscale, N,
                                (int)(K / 64), static_cast<__nv_bfloat16*>(workspace), st);
  if (rc) return rc;
  return launch_gemm_bf16(x, workspace, M, N, K, bias, y, status, st);
}

int dirotq_dequant_weight_int4(int64_t N, int64_t K, const void* w_codes, const float* w_scales, void* w_out, void* stream) {
  if (N <= 0 || K <= 0 || !w_codes || !w_scales || !w_out) return DIROTQ_E_ARG;
  if (K % 64) return DIROTQ_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(w_out) | reinterpret_cast<uintptr_t>(w_codes)) & 15) return DIROTQ_E_ALIGN;
  return launch_dequant_int4(static_cast<const uint8_t*>(w_codes), w_scales, N, (int)(K / 64), ld_rows(N),
                             static_cast<__nv_bfloat16*>(w_out), static_cast<cudaStream_t>(stream));
}

int dirotq_gemm_bf16(int64_t M, int64_t N, int64_t K, const void* x, const void* w, const void* bias, void* y,
                     int32_t* status, void* stream) {
  if (M < 0 || N <= 0 || K <= 0 || !x || !w || !y) return DIROTQ_E_ARG;
  if (K % 64 || N % 8) return DIROTQ_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)
    return DIROTQ_E_ALIGN;
  return launch_gemm_bf16(x, w, M, N, K, bias, y, status, static_cast<cudaStream_t>(stream));
}

int dirotq_dequant_weight_nvfp4(int64_t N, int64_t K, const void* w_codes, const void* w_sf, float w_tensor_scale,
                                const float* w_rowscale, void* w_out, void* stream) {
  if (N <= 0 || K <= 0 || !w_codes || !w_sf || !w_out) return DIROTQ_E_ARG;
  if (!w_rowscale && !(w_tensor_scale > 0.f)) return DIROTQ_E_ARG;
  if (K % 64) return DIROTQ_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(w_out) | reinterpret_cast<uintptr_t>(w_codes)) & 15) return DIROTQ_E_ALIGN;
  return launch_dequant_nvfp4(static_cast<const uint8_t*>(w_codes), static_cast<const uint8_t*>(w_sf), w_tensor_scale,
                              w_rowscale, N, (int)(K / 64), static_cast<__nv_bfloat16*>(w_out),
                              static_cast<cudaStream_t>(stream));
}

}  // extern "C"
