// Host/device view of the activation / weight code layouts declared in include/dirotq_b200.h.
#pragma once
#include <cstdint>
#include "../../include/dirotq_b200.h"

namespace dq {

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t round_up64(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// Flattened, kernel-friendly description of one activation format.
struct ActGeom {
  int mode;
  int D;          // input width
  int H;          // 0 = hidden layout
  int d;          // head dim (H > 0)
  int hlen;       // tail per head (H > 0) or total (H == 0)
  int group;      // effective group size
  int q_len;
  int n_groups;
  int cpg;        // 64-chunks per group
  int n_chunks;
  int k_pad;
  int code_row_bytes;
  int tail_total;
  int tail_pitch;
  int n_scales;
  float clip;
  float T;        // NVFP4_HW tensor scale
  int per_token;  // integer modes, hidden layout: one scale (and zero point) per row, stored once per 64-chunk
};

inline bool is_nvfp4(int mode) { return mode == DIROTQ_NVFP4_REF || mode == DIROTQ_NVFP4_HW; }
inline bool is_asym(int mode) { return mode == DIROTQ_INT4_ASYM || mode == DIROTQ_INT8_ASYM; }

inline int make_geom(const dirotq_act_format* f, ActGeom* g) {
  if (!f || !g) return DIROTQ_E_ARG;
  if (f->mode < DIROTQ_INT4_SYM || f->mode > DIROTQ_NVFP4_HW) return DIROTQ_E_ARG;
  if (f->width <= 0 || f->width % 8 != 0 || f->tail_len < 0) return DIROTQ_E_ARG;
  g->mode = f->mode;
  g->D = f->width;
  g->per_token = 0;
  g->H = f->num_heads;
  g->d = f->head_dim;
  g->hlen = f->tail_len;
  g->clip = f->clip_ratio;
  g->T = f->tensor_scale;
  if (f->mode == DIROTQ_NVFP4_HW && !(f->tensor_scale > 0.f)) return DIROTQ_E_ARG;
  if (g->H > 0) {
    if (g->d <= 0 || g->H * g->d != g->D || g->d % 8 != 0) return DIROTQ_E_ARG;
    if (g->hlen <= 0 || g->hlen >= g->d) return DIROTQ_E_ARG;  // hlen == 0 is a hidden layout
    if (is_nvfp4(f->mode)) {
      // per head, the tensor-core form: the heads' low coefficients side by side in blocks of 16 (never straddling a
      // head), the heads' high coefficients behind them -- the reference's rearrangement
      // (dirotq_fused_unrotation_fast.py:94-99) with its one group per head cut into the hardware's scale blocks
      if (f->mode != DIROTQ_NVFP4_HW || (g->d - g->hlen) % 16 != 0 || g->d % 16 != 0) return DIROTQ_E_UNSUPPORTED;
      g->group = 16;
      g->q_len = g->H * (g->d - g->hlen);
      g->n_groups = g->q_len / 16;
    } else {
      g->group = g->d - g->hlen;
      g->q_len = g->H * g->group;
      g->n_groups = g->H;
    }
    g->tail_total = g->H * g->hlen;
  } else {
    if (g->hlen >= g->D) return DIROTQ_E_ARG;
    g->q_len = g->D - g->hlen;
    g->group = is_nvfp4(f->mode) ? 16 : f->group_size;
    if (is_nvfp4(f->mode) && f->group_size != 16) return DIROTQ_E_UNSUPPORTED;
    if (g->group <= 0) {
      // per-token scales (ActQuantizer with groupsize <= 0, utils/quant_utils.py:236-240, :242-271): the codes keep
      // the 64-slot chunk layout the GEMMs read and every chunk of a row carries the row's scale
      g->per_token = 1;
      g->group = 64;
    }
    g->n_groups = ceil_div(g->q_len, g->group);
    g->tail_total = g->hlen;
  }
  if (g->group > 128) return DIROTQ_E_UNSUPPORTED;
  if (is_nvfp4(f->mode)) {
    g->cpg = 1;
    g->n_chunks = ceil_div(g->q_len, 64);
    g->n_scales = g->n_groups;
  } else {
    g->cpg = ceil_div(g->group, 64);
    g->n_chunks = g->n_groups * g->cpg;
    g->n_scales = g->n_chunks;
  }
  g->k_pad = g->n_chunks * 64;
  g->code_row_bytes = (f->mode == DIROTQ_INT8_ASYM) ? g->k_pad : g->k_pad / 2;
  g->tail_pitch = (int)round_up64(g->tail_total, 8);
  return DIROTQ_OK;
}

inline int64_t ld_rows(int64_t M) { return round_up64(M, 8); }
inline size_t pad256(size_t b) { return (b + 255) / 256 * 256; }

// byte offset of a UE4M3 scale factor in the 128-row x 4-group tiling
__host__ __device__ inline int64_t sf_offset(int64_t row, int kblk16, int n_kb64_pad) {
  int64_t rb = row >> 7;
  int r = (int)(row & 127);
  return (rb * n_kb64_pad + (kblk16 >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kblk16 & 3);
}

}  // namespace dq
