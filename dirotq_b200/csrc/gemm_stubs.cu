// Temporary: entry points whose kernels are not written yet.
#include "layout.cuh"
extern "C" {
int dirotq_gemm_w4a4_int(int32_t, int64_t, int64_t, int32_t, const void*, const void*, const void*, const void*,
                         const float*, const float*, const void*, const void*, int32_t, int32_t, const void*, void*,
                         int32_t*, int32_t*, void*) { return DIROTQ_E_UNSUPPORTED; }
int dirotq_gemm_w4a4_nvfp4(int64_t, int64_t, int32_t, const void*, const void*, const void*, const void*, float,
                           const void*, const void*, int32_t, int32_t, const void*, void*, int32_t*, void*) { return DIROTQ_E_UNSUPPORTED; }
int dirotq_gemm_w4a16(int64_t, int64_t, int64_t, const void*, const void*, const float*, const void*, void*, int32_t*,
                      void*) { return DIROTQ_E_UNSUPPORTED; }
size_t dirotq_linear_workspace_bytes(const dirotq_linear*, int64_t) { return 0; }
int dirotq_linear_forward(const dirotq_linear*, const void*, int64_t, void*, void*, size_t, int32_t*, void*) { return DIROTQ_E_UNSUPPORTED; }
}
