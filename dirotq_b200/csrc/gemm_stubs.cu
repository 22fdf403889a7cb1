// Entry points whose kernels are not written yet.
#include "layout.cuh"
extern "C" {
int dirotq_gemm_w4a16(int64_t, int64_t, int64_t, const void*, const void*, const float*, const void*, void*, int32_t*,
                      void*) { return DIROTQ_E_UNSUPPORTED; }
}
