// C ABI glue: argument checks on the host, geometry, launches.  See include/dirotq_b200.h.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "layout.cuh"
#include "launchers.cuh"

using namespace dq;

extern "C" {

int dirotq_abi_version(void) { return DIROTQ_ABI_VERSION; }

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

}  // extern "C"
