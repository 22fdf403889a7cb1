// Argument blocks and host launchers shared between the kernels' translation units and api.cu.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"

#include <atomic>
#include <utility>

namespace dq {

// cudaFuncSetAttribute acts on the CURRENT device only, so "done" is remembered per device (bit = device ordinal),
// not per process: a host that drives several GPUs from one process sets it on each of them.
struct PerDeviceOnce {
  std::atomic<unsigned long long> done{0};
};
template <typename K>
inline int set_max_dynamic_smem(PerDeviceOnce& once, K kernel, int bytes) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return DIROTQ_E_CUDA;
  if (dev >= 64) return DIROTQ_E_UNSUPPORTED;
  const unsigned long long bit = 1ull << dev;
  if (!(once.done.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return DIROTQ_E_CUDA;
    once.done.fetch_or(bit, std::memory_order_release);
  }
  return DIROTQ_OK;
}

// Launch with programmatic stream serialization allowed (see pdl_wait() in ptx.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

struct QuantArgs {
  ActGeom g;
  const __nv_bfloat16* x;
  int64_t x_pitch;
  const int64_t* perm;
  int64_t M;
  int64_t ldm;
  uint8_t* codes;
  __nv_bfloat16* scales;   // INT / NVFP4_REF
  uint8_t* sf;             // NVFP4_HW tiled bytes
  __nv_bfloat16* zeros;
  __nv_bfloat16* tail;
};

struct PackIntArgs {
  const float* w;       // [N, n_low]
  int64_t N;
  int64_t n_low;
  int group;
  int n_groups;
  int cpg;
  int n_chunks;
  const float* scale_in;  // [N, n_groups] or null
  int w_is_codes;
  uint8_t* codes;       // [N, n_chunks*32]
  float* scales;        // [n_chunks, ldn]
  float* wsum;          // [n_chunks, ldn]
  int64_t ldn;
};

struct PackFp4Args {
  const float* w;
  int64_t N;
  int64_t n_low;
  int n_chunks;
  float T;
  const uint8_t* scale_in;  // [N, ceil(n_low/16)] e4m3 bytes or null
  int w_is_codes;
  uint8_t* codes;           // [N, n_chunks*32]
  uint8_t* sf;              // tiled
};

struct RotArgs {
  int wait_limit_k = 0;        // bounded device waits give up after this many units of 1024 cycles (0 = default)
  ActGeom g;
  int64_t M;
  int64_t ldm;
  int BN;
  int n_tiles;
  int m_tiles;
  int K;                  // contraction length (== g.D for a rotation)
  int band;               // 0 = dense rotation, else head_dim of a block-diagonal rotation
  const __nv_bfloat16* bias;  // plain-GEMM epilogue only
  __nv_bfloat16* x_rot;   // optional [M, D]
  uint8_t* codes;
  __nv_bfloat16* scales;
  uint8_t* sf;
  __nv_bfloat16* zeros;
  __nv_bfloat16* tail;
  int* status;
};

struct GemmIntArgs {
  int wait_limit_k = 0;        // bounded device waits give up after this many units of 1024 cycles (0 = default)
  int a_mode;
  int64_t M, N;
  int n_chunks;
  const uint8_t* xq;           // activation codes [M, x_row_bytes]
  int64_t x_row_bytes;
  const __nv_bfloat16* xs;     // [n_chunks, ldm]
  const __nv_bfloat16* xz;     // [n_chunks, ldm] or null
  int64_t ldm;
  const uint8_t* wq;           // weight codes [N, n_chunks * 32]
  int64_t w_row_bytes;
  const float* ws;             // [n_chunks, ldn]
  const float* wsum;           // [n_chunks, ldn]
  int64_t ldn;
  const __nv_bfloat16* xt;     // [M, kt_pitch]
  const __nv_bfloat16* wt;     // [N, kt_pitch]
  int kt;
  int kt_pitch;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;            // [M, N]
  int32_t* acc_dump;
  int* status;
};

struct GemmIntF16Args {
  int wait_limit_k = 0;        // bounded device waits give up after this many units of 1024 cycles (0 = default)
  int a_mode;                  // DIROTQ_INT4_SYM or DIROTQ_INT4_ASYM
  int64_t M, N;
  int n_chunks;
  const uint8_t* xq;           // activation codes [M, n_chunks * 32]
  int64_t x_row_bytes;
  const uint2* a_const;        // [n_chunks, ldm] records {s*2^24/rs, -(z*s)/rs}, fp16 pairs
  const float* rs;             // [M] row powers of two
  int64_t ldm;                 // f16_ld_act(M)
  const void* w_panel;         // [N, n_chunks * 64] fp16: (qw - 8) * sw / cs, in the converters' K order
  const float* cs;             // [N] column powers of two
  const __nv_bfloat16* xt;     // [M, kt_pitch] tail / rs
  const __nv_bfloat16* wt;     // [N, kt_pitch] tail / cs
  int kt;
  int kt_pitch;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;            // [M, N]
  int* status;
  int half_chunks = 0;         // per-head groups of at most 32 channels: two chunks' first halves per operand stage (the
                               // weight panel is laid out to match: [N, ceil(n_chunks / 2) * 64])
  int force_bn;                // 0 = pick the column-tile width from N
  int raster = 0;              // column tiles per rasterisation group (0 = all: n fastest over the whole width)
  int act;                     // epilogue activation: 0 none, 1 GELU (tanh form) on the bf16-rounded output
  // Optional: the epilogue ALSO quantises its (activated, bf16-rounded) output rows for a following un-rotated INT4
  // layer of width N with groups of 64 (and, optionally, its last columns kept in 16 bits) -- codes / scales / zero points in that layer's activation
  // layout -- so that the layer's quantise-only kernel and a round trip of the [M, N] tensor disappear; y may then be
  // null.
  uint8_t* q_codes = nullptr;       // [M, N / 2]
  __nv_bfloat16* q_scales = nullptr;  // [N / 64, q_ldm]
  __nv_bfloat16* q_zeros = nullptr;   // asymmetric mode only
  int64_t q_ldm = 0;
  int64_t q_len = 0;                // quantised columns (multiple of 64); columns beyond go to q_tail as bf16
  __nv_bfloat16* q_tail = nullptr;  // [M, q_tail_pitch], (N - q_len) columns used
  int q_tail_pitch = 0;
  int q_row_bytes = 0;              // bytes between code rows
  int q_mode = 0;                   // DIROTQ_INT4_SYM or DIROTQ_INT4_ASYM
  float q_clip = 1.f;
};

struct GemmFp4Args {
  int wait_limit_k = 0;        // bounded device waits give up after this many units of 1024 cycles (0 = default)
  int64_t M, N;
  int n_chunks;
  const uint8_t* xq;           // [M, n_chunks * 32]
  const uint8_t* xsf;          // tiled UE4M3
  const uint8_t* wq;           // [N, n_chunks * 32]
  const uint8_t* wsf;
  float out_scale;
  const float* col_scale;      // optional fp32 [N]: per-channel weight scale (the reference's two-level weight recipe)
  int act;                     // epilogue activation: 0 none, 1 GELU (tanh form)
  const __nv_bfloat16* xt;
  const __nv_bfloat16* wt;
  int kt;
  int kt_pitch;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  int* status;
  // Optional (CTA-pair kernels): the epilogue also quantises its activated, bf16-rounded output rows for a following
  // un-rotated NVFP4 layer of width N (power-of-two tensor scale) -- E2M1 codes, UE4M3 block scales in their tile
  // layout, the layer's trailing 16-bit channels -- so that its quantise kernel and a round trip of the [M, N] tensor
  // disappear; y may then be null.
  uint8_t* q_codes = nullptr;        // [M, q_row_bytes]
  uint8_t* q_sf = nullptr;           // tiled UE4M3 (pad entries stay as the owner zeroed them)
  int64_t q_len = 0;                 // quantised columns (multiple of 64); columns beyond go to q_tail as bf16
  __nv_bfloat16* q_tail = nullptr;   // [M, q_tail_pitch]
  int q_tail_pitch = 0;
  int q_row_bytes = 0;
  int q_n_kb64_pad = 0;              // 64-column blocks per row of the scale-factor tile array (rounded up to 4)
  float q_clip = 1.f;
  float q_T = 1.f;
};

int launch_gemm_int(const GemmIntArgs& a, cudaStream_t st);
int launch_gemm_nvfp4(const GemmFp4Args& a, cudaStream_t st);
int launch_gemm_nvfp4_pair(const GemmFp4Args& a, int bn, cudaStream_t st);
int launch_gemm_int_f16(const GemmIntF16Args& a, cudaStream_t st);
int launch_expand_weight_panel(const uint8_t* wq, int n_chunks, int64_t N, const void* rec, void* panel, cudaStream_t st,
                               int half_chunks = 0);
int launch_fold_act_and_expand(const __nv_bfloat16* s, const __nv_bfloat16* z, int n_chunks, int64_t M, int64_t ldm, void* rec,
                               float* rs, const __nv_bfloat16* tail, __nv_bfloat16* tail_out, int kt_pitch, const uint8_t* wq,
                               int64_t N, const void* w_rec, void* panel, cudaStream_t st, int half_chunks = 0);
int64_t f16_ld_act(int64_t M);
int64_t f16_ld_weight(int64_t N);
int launch_fold_act_scales(const __nv_bfloat16* s, const __nv_bfloat16* z, int n_chunks, int64_t M, int64_t ldm,
                           void* rec, float* rs, const __nv_bfloat16* tail, __nv_bfloat16* tail_out,
                           int kt_pitch, cudaStream_t st);
int launch_fold_weight_scales(const float* s, int n_chunks, int64_t N, int64_t ldn, void* rec, float* cs,
                              const __nv_bfloat16* tail, __nv_bfloat16* tail_out, int kt_pitch, cudaStream_t st);

int launch_quantize(const QuantArgs& a, cudaStream_t st);
int launch_pack_int4(const PackIntArgs& a, cudaStream_t st);
int launch_pack_nvfp4(const PackFp4Args& a, cudaStream_t st);
int launch_rotate_quantize(const ActGeom& g, const void* x, const void* rot_t, int64_t M, RotArgs a, cudaStream_t st);
int launch_hadamard_low(const void* x, int64_t M, int D, int n, const void* flips, void* y, cudaStream_t st);
int num_sms();
int wait_limit_k();   // process-wide setting of dirotq_set_wait_limit_cycles, in units of 1024 cycles
int launch_gemm_bf16(const void* x, const void* w_t, int64_t M, int64_t N, int64_t K, const void* bias, void* y,
                     int* status, cudaStream_t st);
int launch_dequant_nvfp4(const uint8_t* codes, const uint8_t* sf, float T, const float* row_scale, int64_t N, int n_chunks,
                         __nv_bfloat16* w, cudaStream_t st);
int launch_pack_nvfp4_rowscale(const PackFp4Args& a, float* g_exact, float* g_stored, cudaStream_t st);
int launch_dequant_int4(const uint8_t* codes, const float* scales, int64_t N, int n_chunks, int64_t ldn,
                        __nv_bfloat16* w, cudaStream_t st);


}  // namespace dq
