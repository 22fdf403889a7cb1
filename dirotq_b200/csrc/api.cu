// C ABI glue: argument checks on the host, geometry, launches.  See include/dirotq_b200.h.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"

#include <atomic>
#include <cstring>

using namespace dq;

static std::atomic<int> g_wait_limit_k{0};
namespace dq {
int wait_limit_k() { return g_wait_limit_k.load(std::memory_order_relaxed); }
}

extern "C" {

int dirotq_abi_version(void) { return DIROTQ_ABI_VERSION; }

int dirotq_set_wait_limit_cycles(int64_t cycles) {
  if (cycles < 0 || cycles > (int64_t)2000000000 * 1024) return DIROTQ_E_ARG;
  g_wait_limit_k.store(cycles == 0 ? 0 : (int)((cycles + 1023) / 1024), std::memory_order_relaxed);
  return DIROTQ_OK;
}

const char* dirotq_error_string(int code) {
  switch (code) {
    case DIROTQ_OK: return "ok";
    case DIROTQ_E_ARG: return "invalid argument (null pointer, bad size or inconsistent format)";
    case DIROTQ_E_UNSUPPORTED: return "combination not supported by the sm_100a kernels";
    case DIROTQ_E_ALIGN: return "pointer or row pitch not 16-byte aligned";
    case DIROTQ_E_CUDA: return "a CUDA runtime or driver call failed";
    case DIROTQ_E_TOO_LARGE: return "size exceeds a fixed capacity of this entry point";
  }
  return "unknown error";
}

const char* dirotq_status_string(int status) {
  switch (status) {
    case 0: return "ok";
    case 1: return "timeout: UMMA issuer waited for a filled shared-memory stage";
    case 2: return "timeout: producer waited for a free shared-memory stage";
    case 3: return "timeout: epilogue waited for an accumulator";
    case 4: return "timeout: UMMA issuer waited for a drained accumulator";
    case 5: return "timeout: teardown waited for copies in flight";
    case 6: return "timeout: scale factors did not reach tensor memory";
  }
  return "unknown device status";
}

int dirotq_act_layout_of(const dirotq_act_format* fmt, dirotq_act_layout* out) {
  ActGeom g;
  int rc = make_geom(fmt, &g);
  if (rc) return rc;
  if (!out) return DIROTQ_E_ARG;
  out->q_len = g.q_len;
  out->group = g.group;
  out->n_groups = g.n_groups;
  out->chunks_per_group = g.cpg;
  out->n_chunks = g.n_chunks;
  out->k_pad = g.k_pad;
  out->code_row_bytes = g.code_row_bytes;
  out->tail_total = g.tail_total;
  out->tail_pitch = g.tail_pitch;
  out->n_scales = g.n_scales;
  return DIROTQ_OK;
}

size_t dirotq_act_codes_bytes(const dirotq_act_layout* l, int64_t M) {
  return pad256((size_t)M * (size_t)l->code_row_bytes);
}
size_t dirotq_act_scales_bytes(const dirotq_act_format* f, const dirotq_act_layout* l, int64_t M) {
  if (f->mode == DIROTQ_NVFP4_HW) {
    size_t rb = (size_t)((M + 127) / 128), kb = (size_t)((l->n_chunks + 3) / 4 * 4);
    return pad256(rb * kb * 512);
  }
  return pad256((size_t)l->n_scales * (size_t)ld_rows(M) * 2);
}
size_t dirotq_act_zeros_bytes(const dirotq_act_format* f, const dirotq_act_layout* l, int64_t M) {
  if (!is_asym(f->mode)) return 0;
  return pad256((size_t)l->n_scales * (size_t)ld_rows(M) * 2);
}
size_t dirotq_act_tail_bytes(const dirotq_act_layout* l, int64_t M) {
  return pad256((size_t)M * (size_t)l->tail_pitch * 2);
}

static int check_act_outputs(const ActGeom& g, void* codes, void* scales, void* zeros, void* tail) {
  if (!codes || !scales) return DIROTQ_E_ARG;
  if (is_asym(g.mode) && !zeros) return DIROTQ_E_ARG;
  if (g.tail_total > 0 && !tail) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(tail) & 15) ||
      (reinterpret_cast<uintptr_t>(scales) & 15))
    return DIROTQ_E_ALIGN;
  return DIROTQ_OK;
}

int dirotq_quantize_act(const dirotq_act_format* fmt, const void* x, int64_t x_pitch, const int64_t* perm_idx,
                        int64_t M, void* codes, void* scales, void* zeros, void* tail, void* stream) {
  ActGeom g;
  int rc = make_geom(fmt, &g);
  if (rc) return rc;
  if (!x || M < 0 || x_pitch < g.D) return DIROTQ_E_ARG;
  rc = check_act_outputs(g, codes, scales, zeros, tail);
  if (rc) return rc;
  QuantArgs a;
  a.g = g;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.x_pitch = x_pitch;
  a.perm = perm_idx;
  a.M = M;
  a.ldm = ld_rows(M);
  a.codes = static_cast<uint8_t*>(codes);
  a.scales = static_cast<__nv_bfloat16*>(scales);
  a.sf = static_cast<uint8_t*>(scales);
  a.zeros = static_cast<__nv_bfloat16*>(zeros);
  a.tail = static_cast<__nv_bfloat16*>(tail);
  return launch_quantize(a, static_cast<cudaStream_t>(stream));
}

int dirotq_rotate_quantize(const dirotq_act_format* fmt, const void* x, const void* rot_t, int64_t M, void* x_rot,
                           void* codes, void* scales, void* zeros, void* tail, int32_t* status, void* stream) {
  ActGeom g;
  int rc = make_geom(fmt, &g);
  if (rc) return rc;
  if (!x || !rot_t || M < 0) return DIROTQ_E_ARG;
  if (codes) {
    rc = check_act_outputs(g, codes, scales, zeros, tail);
    if (rc) return rc;
  } else if (!x_rot) {
    return DIROTQ_E_ARG;
  }
  if (x_rot && (reinterpret_cast<uintptr_t>(x_rot) & 15)) return DIROTQ_E_ALIGN;
  RotArgs a{};
  a.x_rot = static_cast<__nv_bfloat16*>(x_rot);
  a.codes = static_cast<uint8_t*>(codes);
  a.scales = static_cast<__nv_bfloat16*>(scales);
  a.sf = static_cast<uint8_t*>(scales);
  a.zeros = static_cast<__nv_bfloat16*>(zeros);
  a.tail = static_cast<__nv_bfloat16*>(tail);
  a.status = status;
  a.wait_limit_k = wait_limit_k();
  return launch_rotate_quantize(g, x, rot_t, M, a, static_cast<cudaStream_t>(stream));
}

int dirotq_pack_weight_int4(const float* w_low, int64_t N, int64_t n_low, int32_t group, const float* scale_in,
                            int32_t w_is_codes, void* codes, float* scales, float* wsum, void* stream) {
  if (!w_low || !codes || !scales || !wsum || N <= 0 || n_low <= 0) return DIROTQ_E_ARG;
  if (group <= 0 || group > 128) return DIROTQ_E_UNSUPPORTED;
  if (w_is_codes && !scale_in) return DIROTQ_E_ARG;
  if (reinterpret_cast<uintptr_t>(codes) & 15) return DIROTQ_E_ALIGN;
  PackIntArgs a;
  a.w = w_low;
  a.N = N;
  a.n_low = n_low;
  a.group = group;
  a.n_groups = (int)((n_low + group - 1) / group);
  a.cpg = ceil_div(group, 64);
  a.n_chunks = a.n_groups * a.cpg;
  a.scale_in = scale_in;
  a.w_is_codes = w_is_codes;
  a.codes = static_cast<uint8_t*>(codes);
  a.scales = scales;
  a.wsum = wsum;
  a.ldn = ld_rows(N);
  return launch_pack_int4(a, static_cast<cudaStream_t>(stream));
}

int dirotq_pack_weight_nvfp4(const float* w_low, int64_t N, int64_t n_low, float tensor_scale,
                             const uint8_t* scale_in, int32_t w_is_codes, void* codes, void* sf, void* stream) {
  if (!w_low || !codes || !sf || N <= 0 || n_low <= 0 || !(tensor_scale > 0.f)) return DIROTQ_E_ARG;
  if (w_is_codes && !scale_in) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(sf) & 15)) return DIROTQ_E_ALIGN;
  PackFp4Args a;
  a.w = w_low;
  a.N = N;
  a.n_low = n_low;
  a.n_chunks = (int)((n_low + 63) / 64);
  a.T = tensor_scale;
  a.scale_in = scale_in;
  a.w_is_codes = w_is_codes;
  a.codes = static_cast<uint8_t*>(codes);
  a.sf = static_cast<uint8_t*>(sf);
  return launch_pack_nvfp4(a, static_cast<cudaStream_t>(stream));
}

int dirotq_pack_weight_nvfp4_rowscale(const float* w_low, int64_t N, int64_t n_low, void* codes, void* sf,
                                      float* row_scale, float* row_scale_exact, void* stream) {
  if (!w_low || !codes || !sf || !row_scale || !row_scale_exact || N <= 0 || n_low <= 0) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(sf) & 15)) return DIROTQ_E_ALIGN;
  PackFp4Args a;
  a.w = w_low;
  a.N = N;
  a.n_low = n_low;
  a.n_chunks = (int)((n_low + 63) / 64);
  a.T = 1.f;
  a.scale_in = nullptr;
  a.w_is_codes = 0;
  a.codes = static_cast<uint8_t*>(codes);
  a.sf = static_cast<uint8_t*>(sf);
  return launch_pack_nvfp4_rowscale(a, row_scale_exact, row_scale, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// GEMMs and the whole wrapped linear
// ---------------------------------------------------------------------------------------------
extern "C" {

int dirotq_gemm_w4a4_int(int32_t a_mode, int64_t M, int64_t N, int32_t n_chunks, const void* x_codes,
                         const void* x_scales, const void* x_zeros, const void* w_codes, const float* w_scales,
                         const float* w_sum, const void* x_tail, const void* w_tail, int32_t tail_total,
                         int32_t tail_pitch, const void* bias, void* y, int32_t* acc_dump, int32_t* status,
                         void* stream) {
  if (a_mode != DIROTQ_INT4_SYM && a_mode != DIROTQ_INT4_ASYM && a_mode != DIROTQ_INT8_ASYM) return DIROTQ_E_UNSUPPORTED;
  if (M < 0 || N <= 0 || n_chunks <= 0 || !x_codes || !x_scales || !w_codes || !w_scales || !y) return DIROTQ_E_ARG;
  if (N % 8 != 0) return DIROTQ_E_UNSUPPORTED;
  if (a_mode != DIROTQ_INT4_SYM && (!x_zeros || !w_sum)) return DIROTQ_E_ARG;
  if (tail_total < 0 || (tail_total > 0 && (!x_tail || !w_tail || tail_pitch < tail_total || tail_pitch % 8))) return DIROTQ_E_ARG;
  const uintptr_t al = reinterpret_cast<uintptr_t>(x_codes) | reinterpret_cast<uintptr_t>(w_codes) |
                       reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x_tail) |
                       reinterpret_cast<uintptr_t>(w_tail);
  if (al & 15) return DIROTQ_E_ALIGN;
  GemmIntArgs a;
  a.a_mode = a_mode;
  a.M = M;
  a.N = N;
  a.n_chunks = n_chunks;
  a.xq = static_cast<const uint8_t*>(x_codes);
  a.x_row_bytes = (a_mode == DIROTQ_INT8_ASYM) ? (int64_t)n_chunks * 64 : (int64_t)n_chunks * 32;
  a.xs = static_cast<const __nv_bfloat16*>(x_scales);
  a.xz = static_cast<const __nv_bfloat16*>(x_zeros);
  a.ldm = ld_rows(M);
  a.wq = static_cast<const uint8_t*>(w_codes);
  a.w_row_bytes = (int64_t)n_chunks * 32;
  a.ws = w_scales;
  a.wsum = w_sum;
  a.ldn = ld_rows(N);
  a.xt = static_cast<const __nv_bfloat16*>(x_tail);
  a.wt = static_cast<const __nv_bfloat16*>(w_tail);
  a.kt = tail_total;
  a.kt_pitch = tail_pitch;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.acc_dump = acc_dump;
  a.status = status;
  a.wait_limit_k = wait_limit_k();
  return launch_gemm_int(a, static_cast<cudaStream_t>(stream));
}

int dirotq_hadamard_low(const void* x, int64_t M, int32_t width, int32_t low_dim, const void* sign_flips, void* y,
                        void* stream) {
  if (!x || !y || M < 0 || width <= 0) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(sign_flips)) & 15)
    return DIROTQ_E_ALIGN;
  return launch_hadamard_low(x, M, width, low_dim, sign_flips, y, static_cast<cudaStream_t>(stream));
}

int dirotq_fold_weight_scales_f16(int32_t n_chunks, int64_t N, const float* w_scales, const void* w_tail,
                                  int32_t tail_total, int32_t tail_pitch, void* w_mult, float* w_colscale,
                                  void* w_tail_out, void* stream) {
  if (n_chunks <= 0 || N <= 0 || !w_scales || !w_mult || !w_colscale) return DIROTQ_E_ARG;
  if (tail_total < 0 || (tail_total > 0 && (!w_tail || !w_tail_out || tail_pitch < tail_total || tail_pitch % 8)))
    return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(w_tail) | reinterpret_cast<uintptr_t>(w_tail_out)) & 15) return DIROTQ_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(w_mult) & 15) return DIROTQ_E_ALIGN;
  return launch_fold_weight_scales(w_scales, n_chunks, N, ld_rows(N), w_mult, w_colscale,
                                   tail_total > 0 ? static_cast<const __nv_bfloat16*>(w_tail) : nullptr,
                                   static_cast<__nv_bfloat16*>(w_tail_out), tail_pitch, static_cast<cudaStream_t>(stream));
}

struct F16Carve {
  size_t rec, rs, tail, panel, total;
};
static size_t panel_bytes(int32_t n_chunks, int64_t N) {
  return ((size_t)N * (size_t)n_chunks * 128 + 255) & ~size_t(255);
}
// N_panel > 0: room for the fp16 weight panel of an N_panel-channel layer (callers without a panel of their own)
static F16Carve carve_f16(int64_t M, int32_t n_chunks, int32_t tail_pitch, int64_t N_panel) {
  F16Carve c;
  const size_t ldm = (size_t)f16_ld_act(M);
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  c.rec = 0;
  c.rs = up(c.rec + (size_t)n_chunks * ldm * 8);
  c.tail = up(c.rs + ldm * 4);
  c.panel = up(c.tail + (size_t)M * (size_t)tail_pitch * 2);
  c.total = c.panel + (N_panel > 0 ? panel_bytes(n_chunks, N_panel) : 0);
  return c;
}

size_t dirotq_fold_weight_records_bytes(int32_t n_chunks, int64_t N) {
  if (n_chunks <= 0 || N <= 0) return 0;
  return (size_t)n_chunks * (size_t)f16_ld_weight(N) * 8;
}

size_t dirotq_weight_panel_bytes(int32_t n_chunks, int64_t N) {
  if (n_chunks <= 0 || N <= 0) return 0;
  return panel_bytes(n_chunks, N);
}

int dirotq_expand_weight_panel_f16_layout(int32_t n_chunks, int64_t N, const void* w_codes, const void* w_mult, void* panel,
                                          int32_t half_chunks, void* stream) {
  if (n_chunks <= 0 || N <= 0 || !w_codes || !w_mult || !panel) return DIROTQ_E_ARG;
  if ((reinterpret_cast<uintptr_t>(w_codes) | reinterpret_cast<uintptr_t>(w_mult) | reinterpret_cast<uintptr_t>(panel)) & 15)
    return DIROTQ_E_ALIGN;
  return launch_expand_weight_panel(static_cast<const uint8_t*>(w_codes), n_chunks, N, w_mult, panel,
                                    static_cast<cudaStream_t>(stream), half_chunks ? 1 : 0);
}

int dirotq_expand_weight_panel_f16(int32_t n_chunks, int64_t N, const void* w_codes, const void* w_mult, void* panel,
                                   void* stream) {
  return dirotq_expand_weight_panel_f16_layout(n_chunks, N, w_codes, w_mult, panel, 0, stream);
}

size_t dirotq_gemm_w4a4_int_f16_workspace_bytes(int64_t M, int64_t N_panel, int32_t n_chunks, int32_t tail_pitch) {
  if (M < 0 || N_panel < 0 || n_chunks <= 0 || tail_pitch < 0) return 0;
  return carve_f16(M, n_chunks, tail_pitch, N_panel).total;
}

// Per-head groups of at most 32 channels (SANA: 28) fill less than half of their 64-slot chunk: the 16-bit-conversion GEMM
// then puts the first halves of two chunks into one operand stage (half the stages, and the stage count sets its time).
static bool half_chunk_geometry(const ActGeom& g) {
  return g.H > 0 && g.cpg == 1 && g.group <= 32 && !is_nvfp4(g.mode);
}

// Where the GEMM's epilogue also quantises its output for a following layer: that layer's activation buffers.
struct QuantOut {
  void* codes;
  void* scales;
  void* zeros;
  int64_t ldm;
  int64_t q_len;
  void* tail;
  int tail_pitch;
  int row_bytes;
  int mode;
  float clip;
  float T;            // NVFP4 consumer: its activation tensor scale
  int n_kb64_pad;     // NVFP4 consumer: 64-column blocks per row of its scale-factor tile array
};

// skip_fold != 0: the workspace already holds the activation records and the scaled tail of these codes
// (left there by an earlier call on the same activations).  qo != null: see QuantOut; y may then be null.
static int gemm_w4a4_int_f16_impl(int32_t a_mode, int64_t M, int64_t N, int32_t n_chunks, const void* x_codes,
                                  const void* x_scales, const void* x_zeros, const void* w_codes, const void* w_mult,
                                  const void* w_panel, const float* w_colscale, const void* x_tail,
                                  const void* w_tail_scaled, int32_t tail_total, int32_t tail_pitch, const void* bias,
                                  void* y, void* workspace, size_t workspace_bytes, int skip_fold, int act,
                                  int32_t* status, void* stream, const QuantOut* qo = nullptr, const ActGeom* geom = nullptr) {
  if (a_mode != DIROTQ_INT4_SYM && a_mode != DIROTQ_INT4_ASYM && a_mode != DIROTQ_INT8_ASYM) return DIROTQ_E_UNSUPPORTED;
  if (M < 0 || N <= 0 || n_chunks <= 0 || !x_codes || !x_scales || !w_colscale || (!y && !qo) || !workspace)
    return DIROTQ_E_ARG;
  if (!w_panel && (!w_codes || !w_mult)) return DIROTQ_E_ARG;
  if (N % 8 != 0) return DIROTQ_E_UNSUPPORTED;
  if (a_mode != DIROTQ_INT4_SYM && !x_zeros) return DIROTQ_E_ARG;
  if (tail_total < 0 || (tail_total > 0 && (!x_tail || !w_tail_scaled || tail_pitch < tail_total || tail_pitch % 8)))
    return DIROTQ_E_ARG;
  const uintptr_t al = reinterpret_cast<uintptr_t>(x_codes) | reinterpret_cast<uintptr_t>(w_codes) |
                       reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x_tail) |
                       reinterpret_cast<uintptr_t>(w_tail_scaled) | reinterpret_cast<uintptr_t>(w_mult) |
                       reinterpret_cast<uintptr_t>(w_panel);
  if (al & 15) return DIROTQ_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return DIROTQ_E_ALIGN;
  const int32_t tp = tail_total > 0 ? tail_pitch : 0;
  const F16Carve c = carve_f16(M, n_chunks, tp, w_panel ? 0 : N);
  if (workspace_bytes < c.total) return DIROTQ_E_ARG;
  if (M == 0) return DIROTQ_OK;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int hc = geom && half_chunk_geometry(*geom) ? 1 : 0;      // a resident panel of such a layer has the same layout
  __nv_bfloat16* tail_s = tail_total > 0 ? reinterpret_cast<__nv_bfloat16*>(ws + c.tail) : nullptr;
  const __nv_bfloat16* zeros_in = a_mode != DIROTQ_INT4_SYM ? static_cast<const __nv_bfloat16*>(x_zeros) : nullptr;
  const __nv_bfloat16* tail_in = tail_total > 0 ? static_cast<const __nv_bfloat16*>(x_tail) : nullptr;
  if (!skip_fold && !w_panel) {
    // both per-call preparations in one launch: activation scales folded into FMA operands, and the fp16 weight
    // panel rebuilt in scratch (the weights stay 4-bit in memory)
    int rc = launch_fold_act_and_expand(static_cast<const __nv_bfloat16*>(x_scales), zeros_in, n_chunks, M, ld_rows(M),
                                        ws + c.rec, reinterpret_cast<float*>(ws + c.rs), tail_in, tail_s, tp,
                                        static_cast<const uint8_t*>(w_codes), N, w_mult, ws + c.panel, st, hc);
    if (rc) return rc;
    w_panel = ws + c.panel;
  } else {
    if (!skip_fold) {
      int rc = launch_fold_act_scales(static_cast<const __nv_bfloat16*>(x_scales), zeros_in, n_chunks, M, ld_rows(M),
                                      ws + c.rec, reinterpret_cast<float*>(ws + c.rs), tail_in, tail_s, tp, st);
      if (rc) return rc;
    }
    if (!w_panel) {
      int rc = launch_expand_weight_panel(static_cast<const uint8_t*>(w_codes), n_chunks, N, w_mult, ws + c.panel, st, hc);
      if (rc) return rc;
      w_panel = ws + c.panel;
    }
  }
  GemmIntF16Args a;
  a.a_mode = a_mode;
  a.M = M;
  a.N = N;
  a.n_chunks = n_chunks;
  a.xq = static_cast<const uint8_t*>(x_codes);
  a.x_row_bytes = (int64_t)n_chunks * (a_mode == DIROTQ_INT8_ASYM ? 64 : 32);
  a.a_const = reinterpret_cast<const uint2*>(ws + c.rec);
  a.rs = reinterpret_cast<const float*>(ws + c.rs);
  a.ldm = f16_ld_act(M);
  a.w_panel = w_panel;
  a.cs = w_colscale;
  a.xt = tail_s;
  a.wt = static_cast<const __nv_bfloat16*>(w_tail_scaled);
  a.kt = tail_total;
  a.kt_pitch = tail_pitch;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.status = status;
  a.wait_limit_k = wait_limit_k();
  a.force_bn = 0;
  a.act = act;
  a.half_chunks = hc;
  if (qo) {
    a.q_codes = static_cast<uint8_t*>(qo->codes);
    a.q_scales = static_cast<__nv_bfloat16*>(qo->scales);
    a.q_zeros = static_cast<__nv_bfloat16*>(qo->zeros);
    a.q_ldm = qo->ldm;
    a.q_row_bytes = qo->row_bytes;
    a.q_len = qo->q_len;
    a.q_tail = static_cast<__nv_bfloat16*>(qo->tail);
    a.q_tail_pitch = qo->tail_pitch;
    a.q_mode = qo->mode;
    a.q_clip = qo->clip;
  }
  return launch_gemm_int_f16(a, st);
}

int dirotq_gemm_w4a4_int_f16(int32_t a_mode, int64_t M, int64_t N, int32_t n_chunks, const void* x_codes,
                             const void* x_scales, const void* x_zeros, const void* w_codes, const void* w_mult,
                             const void* w_panel, const float* w_colscale, const void* x_tail,
                             const void* w_tail_scaled, int32_t tail_total, int32_t tail_pitch, const void* bias, void* y,
                             void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  return gemm_w4a4_int_f16_impl(a_mode, M, N, n_chunks, x_codes, x_scales, x_zeros, w_codes, w_mult, w_panel, w_colscale,
                                x_tail, w_tail_scaled, tail_total, tail_pitch, bias, y, workspace, workspace_bytes, 0, 0,
                                status, stream);
}

static int gemm_w4a4_nvfp4_impl(int64_t M, int64_t N, int32_t n_chunks, const void* x_codes, const void* x_sf,
                                const void* w_codes, const void* w_sf, float out_scale, const float* w_colscale,
                                const void* x_tail,
                                const void* w_tail_scaled, int32_t tail_total, int32_t tail_pitch, const void* bias,
                                void* y, int act, int32_t* status, void* stream, const QuantOut* qo = nullptr) {
  if (M < 0 || N <= 0 || n_chunks <= 0 || !x_codes || !x_sf || !w_codes || !w_sf || (!y && !qo)) return DIROTQ_E_ARG;
  if (N % 8 != 0) return DIROTQ_E_UNSUPPORTED;
  if (tail_total < 0 || (tail_total > 0 && (!x_tail || !w_tail_scaled || tail_pitch < tail_total || tail_pitch % 8))) return DIROTQ_E_ARG;
  const uintptr_t al = reinterpret_cast<uintptr_t>(x_sf) | reinterpret_cast<uintptr_t>(w_sf) | reinterpret_cast<uintptr_t>(y) |
                       reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(x_codes) |
                       reinterpret_cast<uintptr_t>(w_codes) | reinterpret_cast<uintptr_t>(x_tail) |
                       reinterpret_cast<uintptr_t>(w_tail_scaled) | reinterpret_cast<uintptr_t>(w_colscale);
  if (al & 15) return DIROTQ_E_ALIGN;
  GemmFp4Args a;
  a.M = M;
  a.N = N;
  a.n_chunks = n_chunks;
  a.xq = static_cast<const uint8_t*>(x_codes);
  a.xsf = static_cast<const uint8_t*>(x_sf);
  a.wq = static_cast<const uint8_t*>(w_codes);
  a.wsf = static_cast<const uint8_t*>(w_sf);
  a.out_scale = out_scale;
  a.col_scale = w_colscale;
  a.xt = static_cast<const __nv_bfloat16*>(x_tail);
  a.wt = static_cast<const __nv_bfloat16*>(w_tail_scaled);
  a.kt = tail_total;
  a.kt_pitch = tail_pitch;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.status = status;
  a.wait_limit_k = wait_limit_k();
  a.act = act;
  if (qo) {
    a.q_codes = static_cast<uint8_t*>(qo->codes);
    a.q_sf = static_cast<uint8_t*>(qo->scales);
    a.q_len = qo->q_len;
    a.q_tail = static_cast<__nv_bfloat16*>(qo->tail);
    a.q_tail_pitch = qo->tail_pitch;
    a.q_row_bytes = qo->row_bytes;
    a.q_n_kb64_pad = qo->n_kb64_pad;
    a.q_clip = qo->clip;
    a.q_T = qo->T;
  }
  return launch_gemm_nvfp4(a, static_cast<cudaStream_t>(stream));
}

int dirotq_gemm_w4a4_nvfp4(int64_t M, int64_t N, int32_t n_chunks, const void* x_codes, const void* x_sf,
                           const void* w_codes, const void* w_sf, float out_scale, const float* w_colscale,
                           const void* x_tail, const void* w_tail_scaled, int32_t tail_total, int32_t tail_pitch,
                           const void* bias, void* y, int32_t* status, void* stream) {
  return gemm_w4a4_nvfp4_impl(M, N, n_chunks, x_codes, x_sf, w_codes, w_sf, out_scale, w_colscale, x_tail, w_tail_scaled,
                              tail_total, tail_pitch, bias, y, 0, status, stream);
}

struct WsCarve {
  size_t codes, scales, zeros, tail, xrot, fold, total;
};
// Layers whose quantiser cannot run in the rotation's epilogue rotate into a bf16 scratch tensor first and quantise
// from there: a channel selection after the rotation, one scale per row, integer groups of another size than the hidden
// epilogue's 64, or a per-head group whose 32-column reads would run past the head (head_dim - tail, rounded up to 32,
// above head_dim).
static bool rotates_then_quantises(const dirotq_linear* lin, const ActGeom& g) {
  if (!lin->rot_t) return false;
  if (lin->perm_idx || g.per_token) return true;
  if (is_nvfp4(g.mode)) return false;
  if (g.H == 0) return g.group != 64;
  return ((g.group + 31) / 32) * 32 > g.d;
}
static bool uses_f16_gemm(const dirotq_linear* lin, const ActGeom& g) {
  return lin->w_mult != nullptr &&
         (g.mode == DIROTQ_INT4_SYM || g.mode == DIROTQ_INT4_ASYM || g.mode == DIROTQ_INT8_ASYM);
}
static int carve(const dirotq_linear* lin, int64_t M, ActGeom* g, WsCarve* w) {
  int rc = make_geom(&lin->fmt, g);
  if (rc) return rc;
  dirotq_act_layout l;
  dirotq_act_layout_of(&lin->fmt, &l);
  w->codes = 0;
  w->scales = w->codes + dirotq_act_codes_bytes(&l, M);
  w->zeros = w->scales + dirotq_act_scales_bytes(&lin->fmt, &l, M);
  w->tail = w->zeros + dirotq_act_zeros_bytes(&lin->fmt, &l, M);
  w->xrot = w->tail + (g->tail_total > 0 ? dirotq_act_tail_bytes(&l, M) : 0);
  w->xrot = (w->xrot + 255) & ~size_t(255);
  w->fold = w->xrot + (rotates_then_quantises(lin, *g) ? pad256((size_t)M * (size_t)g->D * 2) : 0);
  w->fold = (w->fold + 255) & ~size_t(255);
  w->total = w->fold;
  if (uses_f16_gemm(lin, *g))
    w->total += dirotq_gemm_w4a4_int_f16_workspace_bytes(M, lin->w_panel_f16 ? 0 : lin->out_features, g->n_chunks,
                                                         g->tail_total > 0 ? g->tail_pitch : 0);
  return DIROTQ_OK;
}

size_t dirotq_linear_workspace_bytes(const dirotq_linear* lin, int64_t M) {
  ActGeom g;
  WsCarve w;
  if (!lin || M < 0 || carve(lin, M, &g, &w)) return 0;
  return w.total;
}

// Which producers can quantise in their epilogue, and for which consumer format: the 16-bit-conversion integer GEMM
// for 4-bit integer consumers, the block-scaled FP4 GEMM for NVFP4 consumers.
static bool produces_epilogue_codes(const dirotq_linear* lin, const ActGeom& g, int consumer_mode) {
  if (g.mode == DIROTQ_NVFP4_HW) return consumer_mode == DIROTQ_NVFP4_HW;
  if (!uses_f16_gemm(lin, g) || g.mode == DIROTQ_INT8_ASYM) return false;
  return consumer_mode == DIROTQ_INT4_SYM || consumer_mode == DIROTQ_INT4_ASYM;
}

// stages: 1 = rotate / quantise into the workspace, 2 = GEMM from the workspace, 3 = both; 4 (with 2) = the
// workspace holds codes, scales and zero points written by someone else (a producer's epilogue): the per-call
// folding of the scales, normally part of stage 1's bookkeeping, runs before the GEMM.
// qo != null: the GEMM's epilogue quantises its output into these buffers as well (16-bit-conversion INT path only).
static int linear_stages(const dirotq_linear* lin, const void* x, int64_t M, void* y, void* workspace,
                         size_t workspace_bytes, int stages, int32_t* status, void* stream,
                         const QuantOut* qo = nullptr) {
  if (!lin || !workspace || ((stages & 1) && !x) || ((stages & 2) && !y && !qo)) return DIROTQ_E_ARG;
  ActGeom g;
  WsCarve w;
  int rc = carve(lin, M, &g, &w);
  if (rc) return rc;
  if (workspace_bytes < w.total) return DIROTQ_E_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return DIROTQ_E_ALIGN;
  if (g.mode == DIROTQ_NVFP4_REF) return DIROTQ_E_UNSUPPORTED;   // bf16 scales cannot feed the FP4 tensor cores
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* codes = ws + w.codes;
  void* scales = ws + w.scales;
  void* zeros = is_asym(g.mode) ? ws + w.zeros : nullptr;
  void* tail = g.tail_total > 0 ? ws + w.tail : nullptr;
  if (stages & 1) {
    if (rotates_then_quantises(lin, g)) {
      void* x_rot = ws + w.xrot;
      rc = dirotq_rotate_quantize(&lin->fmt, x, lin->rot_t, M, x_rot, nullptr, nullptr, nullptr, nullptr, status, stream);
      if (!rc) rc = dirotq_quantize_act(&lin->fmt, x_rot, g.D, lin->perm_idx, M, codes, scales, zeros, tail, stream);
    } else if (lin->rot_t)
      rc = dirotq_rotate_quantize(&lin->fmt, x, lin->rot_t, M, nullptr, codes, scales, zeros, tail, status, stream);
    else
      rc = dirotq_quantize_act(&lin->fmt, x, g.D, lin->perm_idx, M, codes, scales, zeros, tail, stream);
    if (rc) return rc;
  }
  if (!(stages & 2)) return DIROTQ_OK;
  if (qo && !produces_epilogue_codes(lin, g, qo->mode)) return DIROTQ_E_UNSUPPORTED;
  if (g.mode == DIROTQ_NVFP4_HW)
    return gemm_w4a4_nvfp4_impl(M, lin->out_features, g.n_chunks, codes, scales, lin->w_codes, lin->w_scales,
                                lin->fmt.tensor_scale * lin->w_tensor_scale, lin->w_colscale, tail, lin->w_tail, g.tail_total,
                                g.tail_pitch, lin->bias, y, lin->epilogue_act, status, stream, qo);
  if (lin->epilogue_act < 0 || lin->epilogue_act > 1) return DIROTQ_E_ARG;
  if (uses_f16_gemm(lin, g)) {
    if (!lin->w_colscale || (g.tail_total > 0 && !lin->w_tail_f16)) return DIROTQ_E_ARG;
    // the activation-side folding belongs to the first stage: a GEMM-only call finds its results in place
    return gemm_w4a4_int_f16_impl(g.mode, M, lin->out_features, g.n_chunks, codes, scales, zeros, lin->w_codes,
                                  lin->w_mult, lin->w_panel_f16, lin->w_colscale, tail, lin->w_tail_f16, g.tail_total, g.tail_pitch,
                                  lin->bias, y, ws + w.fold, w.total - w.fold, (stages & 5) ? 0 : 1, lin->epilogue_act,
                                  status, stream, qo, &g);
  }
  if (lin->epilogue_act != 0) return DIROTQ_E_UNSUPPORTED;
  return dirotq_gemm_w4a4_int(g.mode, M, lin->out_features, g.n_chunks, codes, scales, zeros, lin->w_codes,
                              static_cast<const float*>(lin->w_scales), lin->w_sum, tail, lin->w_tail, g.tail_total,
                              g.tail_pitch, lin->bias, y, nullptr, status, stream);
}

int dirotq_linear_forward(const dirotq_linear* lin, const void* x, int64_t M, void* y, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream) {
  return linear_stages(lin, x, M, y, workspace, workspace_bytes, 3, status, stream);
}

int dirotq_linear_gemm(const dirotq_linear* lin, int64_t M, void* y, void* workspace, size_t workspace_bytes,
                       int32_t* status, void* stream) {
  return linear_stages(lin, nullptr, M, y, workspace, workspace_bytes, 2, status, stream);
}

// A following layer can take its activations from the producer's epilogue when its quantiser needs nothing but the
// producer's output row: 4-bit integer groups of 64 over the leading channels, the rest (a multiple of 64, possibly
// none) kept in 16 bits, no rotation, no channel selection, and the 16-bit-conversion GEMM (whose per-call folding
// step reads the scales back).
static int next_takes_epilogue_codes(const dirotq_linear* lin, const dirotq_linear* next, const ActGeom& gn) {
  if (next->rot_t || next->perm_idx) return 0;
  if (gn.H != 0 || gn.per_token || gn.q_len % 64 != 0 || gn.tail_total % 64 != 0) return 0;
  if (gn.D != lin->out_features) return 0;
  if (gn.mode == DIROTQ_NVFP4_HW) {
    uint32_t u;
    memcpy(&u, &gn.T, 4);
    return (u & 0x7FFFFFu) == 0u ? 1 : 0;            // the packed quantiser needs a power-of-two tensor scale
  }
  if (gn.mode != DIROTQ_INT4_SYM && gn.mode != DIROTQ_INT4_ASYM) return 0;
  if (gn.group != 64) return 0;
  return uses_f16_gemm(next, gn) ? 1 : 0;
}

int dirotq_linear_uses_half_chunks(const dirotq_linear* lin) {
  ActGeom g;
  if (!lin || make_geom(&lin->fmt, &g)) return 0;
  return (uses_f16_gemm(lin, g) && half_chunk_geometry(g)) ? 1 : 0;
}

int dirotq_linear_chain_supported(const dirotq_linear* lin, const dirotq_linear* next) {
  if (!lin || !next) return 0;
  ActGeom g, gn;
  if (make_geom(&lin->fmt, &g) || make_geom(&next->fmt, &gn)) return 0;
  if (!produces_epilogue_codes(lin, g, gn.mode)) return 0;
  return next_takes_epilogue_codes(lin, next, gn);
}

int dirotq_linear_forward_chain(const dirotq_linear* lin, const void* x, int64_t M, void* y, void* workspace,
                                size_t workspace_bytes, const dirotq_linear* next, void* next_workspace,
                                size_t next_workspace_bytes, int32_t* status, void* stream) {
  if (!lin || !next || !next_workspace) return DIROTQ_E_ARG;
  if (!dirotq_linear_chain_supported(lin, next)) return DIROTQ_E_UNSUPPORTED;
  ActGeom gn;
  WsCarve wn;
  int rc = carve(next, M, &gn, &wn);
  if (rc) return rc;
  if (next_workspace_bytes < wn.total) return DIROTQ_E_ARG;
  if (reinterpret_cast<uintptr_t>(next_workspace) & 255) return DIROTQ_E_ALIGN;
  uint8_t* nws = static_cast<uint8_t*>(next_workspace);
  QuantOut qo;
  qo.codes = nws + wn.codes;
  qo.scales = nws + wn.scales;
  qo.zeros = is_asym(gn.mode) ? nws + wn.zeros : nullptr;
  qo.ldm = ld_rows(M);
  qo.q_len = gn.q_len;
  qo.tail = gn.tail_total > 0 ? nws + wn.tail : nullptr;
  qo.tail_pitch = gn.tail_pitch;
  qo.row_bytes = gn.code_row_bytes;
  qo.mode = gn.mode;
  qo.clip = gn.clip;
  qo.T = gn.T;
  qo.n_kb64_pad = (gn.n_chunks + 3) & ~3;
  return linear_stages(lin, x, M, y, workspace, workspace_bytes, 3, status, stream, &qo);
}

int dirotq_linear_gemm_prequantised(const dirotq_linear* lin, int64_t M, void* y, void* workspace,
                                    size_t workspace_bytes, int32_t* status, void* stream) {
  return linear_stages(lin, nullptr, M, y, workspace, workspace_bytes, 2 | 4, status, stream);
}


// ---------------------------------------------------------------------------------------------
// Allocation-free variant of dirotq_linear_forward
// ---------------------------------------------------------------------------------------------
// Scratch for callers that cannot provide any: a fixed array in device global memory, part of the
// library image.  Every GPU that loads the library holds these bytes until the process exits.
#define DIROTQ_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[DIROTQ_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the real
// address is looked up once per device (with that device current) and published here.  Two host
// threads that make the first call on a device at the same time both look it up and store the same
// value.  The cache does not survive a device reset (cudaDeviceReset): a process that resets a
// device must not call this entry point on it afterwards.
static std::atomic<void*> g_static_scratch_addr[64];

static int static_scratch_ptr(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return DIROTQ_E_CUDA;
  if (dev >= 64) return DIROTQ_E_UNSUPPORTED;      // more device ordinals than this table holds
  void* p = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return DIROTQ_E_CUDA;
    g_static_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return DIROTQ_OK;
}

size_t dirotq_linear_forward_static_capacity(void) { return DIROTQ_STATIC_SCRATCH_BYTES; }

int dirotq_linear_forward_static(const dirotq_linear* lin, const void* x, int64_t M, void* y, int32_t* status,
                                 void* stream) {
  if (!lin || !x || !y || M < 0) return DIROTQ_E_ARG;
  ActGeom g;
  WsCarve w;
  int rc = carve(lin, M, &g, &w);
  if (rc) return rc;
  if (w.total > DIROTQ_STATIC_SCRATCH_BYTES) return DIROTQ_E_TOO_LARGE;
  void* ws = nullptr;
  rc = static_scratch_ptr(&ws);
  if (rc) return rc;
  // The array still holds whatever the previous call left.  Only the scale-factor tiles of the
  // NVFP4 format rely on zeros (their padding entries are never written), so that region is cleared
  // here, in stream order, before the kernels run.  Nothing else reads stale bytes: every tensor map
  // over the tail is built with tail_total columns and M rows (not tail_pitch / padded rows), so pad
  // columns and rows are zero-filled by the copy engine; pad code slots of a partial last group are
  // written as zero codes by the quantiser; scales of pad rows only feed output rows that are never
  // stored.
  if (g.mode == DIROTQ_NVFP4_HW) {
    if (cudaMemsetAsync(static_cast<uint8_t*>(ws) + w.scales, 0, w.zeros - w.scales,
                        static_cast<cudaStream_t>(stream)) != cudaSuccess)
      return DIROTQ_E_CUDA;
  }
  return dirotq_linear_forward(lin, x, M, y, ws, w.total, status, stream);
}

}  // extern "C"
