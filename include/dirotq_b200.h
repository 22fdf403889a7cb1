/* dirotq_b200 -- C ABI of the B200 (sm_100a) quantized-linear path of DiRotQ.
 *
 * The reference project is pure Python and has no native ABI; each entry point below names the
 * reference code it replaces (paths inside the DiRotQ project).  All pointers are DEVICE pointers
 * unless the name ends in `_host`.  `stream` is a cudaStream_t passed as void*.  The library never
 * allocates, frees or caches device memory: every buffer, scratch included, is the caller's.
 *
 * Return value: 0 = launched, < 0 = argument rejected on the host before any launch (see
 * dirotq_error_string).  Device-side bounded waits that run out write a positive code into the
 * caller's `status` word (int32, device memory, must be zero before the call); the kernel then
 * unwinds and returns normally, so the context stays usable.
 */
#ifndef DIROTQ_B200_H
#define DIROTQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DIROTQ_ABI_VERSION 6

/* ---- activation quantiser modes (ActQuantizer.configure, utils/quant_utils.py:182-199) ---- */
enum {
  DIROTQ_INT4_SYM = 0,  /* bits=4 sym=True  : codes [-8,7], scale = amax/7            (:63-68, :204-209) */
  DIROTQ_INT4_ASYM = 1, /* bits=4 sym=False : codes [0,15] + zero point               (:75-81, :211-215) */
  DIROTQ_INT8_ASYM = 2, /* bits=8 sym=False : codes [0,255] + zero point (W4A8)                         */
  DIROTQ_NVFP4_REF = 3, /* quant_dtype="nvfp4": E2M1 codes + UNROUNDED bf16 group scale (:148-180);
                           bit-exact to the reference, not consumable by block-scaled tensor cores */
  DIROTQ_NVFP4_HW = 4   /* E2M1 codes + UE4M3 group scale relative to an fp32 tensor scale (the
                           two-level recipe of speedup/weight_only_nvfp4.py:42-72 applied to activations) */
};

/* Error codes (negative returns). */
enum {
  DIROTQ_OK = 0,
  DIROTQ_E_ARG = -1,        /* null pointer / bad size */
  DIROTQ_E_UNSUPPORTED = -2,/* combination not implemented */
  DIROTQ_E_ALIGN = -3,      /* pointer or pitch not aligned as required */
  DIROTQ_E_CUDA = -4,       /* a CUDA runtime / driver call failed */
  DIROTQ_E_TOO_LARGE = -5   /* exceeds a fixed capacity */
};

/* How one linear's input is split and grouped.  Mirrors what ActQuantWrapper + ActQuantizer carry
 * (utils/quant_utils.py:300-323, :101-106) after the per-head override of
 * dirotq_fused_unrotation_fast.py:89-93 (groupsize := head_dim - tail, tail := H * tail). */
typedef struct dirotq_act_format {
  int32_t mode;         /* DIROTQ_* above */
  int32_t width;        /* D, input features */
  int32_t num_heads;    /* 0: hidden layout [low | tail]; H > 0: per-head layout.  Per-head DIROTQ_NVFP4_HW (head_dim
                         * and head_dim - tail_len multiples of 16): every head's low coefficients in blocks of 16,
                         * side by side, the heads' high coefficients behind them; produced only by
                         * dirotq_rotate_quantize (dirotq_quantize_act returns DIROTQ_E_UNSUPPORTED). */
  int32_t head_dim;     /* d (per-head only; H * d == D) */
  int32_t tail_len;     /* high_bits_length: hidden = total, per-head = per head */
  int32_t group_size;   /* hidden: 1..128 (INT; a group takes one or two 64-slot chunks) or 16 (NVFP4); per-head:
                         * ignored, group = d - tail_len.  The fused rotate + quantise kernel quantises hidden INT
                         * groups of 64 and per-head groups with ceil32(d - tail_len) <= d; for the other integer
                         * formats dirotq_rotate_quantize returns DIROTQ_E_UNSUPPORTED with codes != NULL and
                         * dirotq_linear_forward rotates into scratch and quantises from there (M * D * 2 bytes of
                         * workspace more, counted by dirotq_linear_workspace_bytes).
                         * <= 0 (integer modes, hidden layout): ONE scale / zero point per row over the quantised
                         * channels, zero included in the extrema (ActQuantizer._find_params,
                         * utils/quant_utils.py:242-271); codes keep the 64-slot chunk layout and the row's scale
                         * is stored for every chunk, so the GEMMs read it like any other format.  The fused
                         * rotate + quantise kernel cannot produce it (a row spans several column tiles):
                         * dirotq_rotate_quantize returns DIROTQ_E_UNSUPPORTED with codes != NULL, and
                         * dirotq_linear_forward rotates into scratch and quantises from there. */
  float clip_ratio;     /* ActQuantizer.clip_ratio */
  float tensor_scale;   /* DIROTQ_NVFP4_HW only: fp32 per-tensor scale T (> 0) */
} dirotq_act_format;

/* Sizes derived from a format (all per row unless stated). */
typedef struct dirotq_act_layout {
  int32_t q_len;          /* quantised channels per row */
  int32_t group;          /* effective group size */
  int32_t n_groups;       /* reference groups per row (incl. a zero-padded last one) */
  int32_t chunks_per_group; /* 64-wide GEMM chunks per group (1, or 2 for groups of 65..128) */
  int32_t n_chunks;       /* INT: n_groups * chunks_per_group; NVFP4: ceil(q_len / 64) */
  int32_t k_pad;          /* code slots per row = n_chunks * 64 */
  int32_t code_row_bytes; /* k_pad / 2 (4-bit) or k_pad (8-bit) */
  int32_t tail_total;     /* passthrough channels per row */
  int32_t tail_pitch;     /* elements; tail_total rounded up to 8 */
  int32_t n_scales;       /* scale entries per row: INT n_chunks, NVFP4_REF q_len/16 (rounded up) */
} dirotq_act_layout;

/* Fills *out; returns DIROTQ_OK or an error for an unsupported format. */
int dirotq_act_layout_of(const dirotq_act_format* fmt, dirotq_act_layout* out);

/* Buffer sizes in bytes for M rows (each rounded up to 256 B).  Data layouts:
 *  codes : [M, code_row_bytes].  INT4: inside every block of 32 code slots, byte j holds slot j in
 *          its low nibble and slot 16+j in its high nibble.  NVFP4: slot 2j in the low nibble of
 *          byte j.  INT8: one byte per slot.  Slot of element e of group g: (g*chunks_per_group)*64+e.
 *  scales: INT / NVFP4_REF: bf16 [n_scales, ldm] (GROUP-major, ldm = M rounded up to 8).
 *          NVFP4_HW: UE4M3 bytes in 512-byte tiles of 128 rows x 4 groups:
 *            tile(rb, kb) at ((rb * ceil4(n_chunks)) + kb) * 512, inside it
 *            (row%32)*16 + (row%128/32)*4 + (group%4); buffers must be zeroed once by the caller
 *            (pad entries are never written).
 *  zeros : bf16 [n_scales, ldm] (asymmetric modes only).
 *  tail  : bf16 [M, tail_pitch].
 */
size_t dirotq_act_codes_bytes(const dirotq_act_layout* l, int64_t M);
size_t dirotq_act_scales_bytes(const dirotq_act_format* f, const dirotq_act_layout* l, int64_t M);
size_t dirotq_act_zeros_bytes(const dirotq_act_format* f, const dirotq_act_layout* l, int64_t M);
size_t dirotq_act_tail_bytes(const dirotq_act_layout* l, int64_t M);

/* ---------------------------------------------------------------------------------------------
 * Kernel 1a: quantise an already rotated (or permuted / unrotated) activation tensor.
 * Replaces ActQuantizer.find_params + ActQuantizer.forward (utils/quant_utils.py:112-180,
 * :201-240) and the perm_idx gather of dirotq_fused_unrotation_fast.py:130-134.
 *   x        : bf16 [M, width], row pitch x_pitch elements
 *   perm_idx : int64 [width] or NULL  (x[..., perm_idx] is quantised)
 * Per-head formats expect x in the interleaved [H, d] layout the wrapper receives.
 */
int dirotq_quantize_act(const dirotq_act_format* fmt, const void* x, int64_t x_pitch, const int64_t* perm_idx,
                        int64_t M, void* codes, void* scales, void* zeros, void* tail, void* stream);

/* Kernel 1: fused rotate + split + quantise.  Replaces `x_flat @ self.rotation` / the per-head
 * einsum followed by find_params + quantizer (dirotq_fused_unrotation_fast.py:69-104) and the
 * stand-alone rotation kernels speedup/kernels/{int8,fp8,bf16}_rotation.py.
 *   x     : bf16 [M, width] contiguous
 *   rot_t : bf16 [width, width] = TRANSPOSE of the rotation (row n = column n of U); for per-head
 *           formats the block-diagonal matrix of the H transposed d x d blocks
 *   x_rot : optional bf16 [M, width] output of the rotated tensor (may be NULL)
 *   codes/scales/zeros/tail: as above; all four NULL = rotation only (x_rot required)
 *   status: int32 device word (zero on entry)
 */
int dirotq_rotate_quantize(const dirotq_act_format* fmt, const void* x, const void* rot_t, int64_t M, void* x_rot,
                           void* codes, void* scales, void* zeros, void* tail, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Kernel 3: weight quantiser / packer.  Replaces speedup/nunchaku_pack.py:225-459
 * (convert_to_nunchaku_w4x4y16, convert_dirotq_low_weight_to_nunchaku[_fp4]) and the NVFP4 weight
 * quantiser speedup/weight_only_nvfp4.py:42-72; arithmetic of utils/quant_utils.py:714-767.
 *
 * INT4: w_low fp32 [N, n_low] in the rotated basis.  group = reference group size (any value in
 *   1..128).  scale_in fp32 [N, n_groups] or NULL (NULL: RTN scale = clamp(amax,1e-5)/7).
 *   w_is_codes != 0: w_low already holds integer codes in [-8,7] (scale_in required).
 *   Outputs: codes [N, k_pad/2] (same slot layout as activations), scales fp32 [n_chunks, ldn]
 *   (group-major, ldn = N rounded up to 8), wsum fp32 [n_chunks, ldn] = sum of the codes of a chunk.
 */
int dirotq_pack_weight_int4(const float* w_low, int64_t N, int64_t n_low, int32_t group, const float* scale_in,
                            int32_t w_is_codes, void* codes, float* scales, float* wsum, void* stream);

/* NVFP4: group 16, two-level scale.  tensor_scale T > 0 (fp32; the host picks a power of two).
 *   scale_in: UE4M3 bytes [N, n_low/16] or NULL (NULL: micro = e4m3(clamp(amax/6/T, 2^-9, 448))).
 *   w_is_codes != 0: w_low holds E2M1 nibble values 0..15 as floats (scale_in required).
 *   Outputs: codes [N, k_pad/2] sequential nibbles (k_pad = ceil64(n_low)), sf = tiled UE4M3 bytes
 *   (same tiling as activations, rows = N; zero the buffer once before the call).
 */
int dirotq_pack_weight_nvfp4(const float* w_low, int64_t N, int64_t n_low, float tensor_scale,
                             const uint8_t* scale_in, int32_t w_is_codes, void* codes, void* sf, void* stream);

/* NVFP4 with the reference's own two-level recipe, bit for bit (speedup/weight_only_nvfp4.py:42-72, _quantize_nvfp4):
 *   group_scale = max(amax_g / 6, 1e-12); gscale[n] = max(max_g(group_scale) / 448, 1e-12) per OUTPUT CHANNEL (fp32);
 *   micro = e4m3(group_scale / gscale[n]); codes = first argmin |w / (micro * gscale[n]) - codebook| (an exact
 *   midpoint goes to the value of smaller magnitude, no -0).
 *   Outputs: codes and sf as dirotq_pack_weight_nvfp4 (the reference packs its nibbles planar, column j with column
 *   j + K/2; here they are sequential, the order the tensor core reads); row_scale fp32 [N] = gscale rounded to bf16,
 *   the value the reference stores and dequantises with; row_scale_exact fp32 [N] = the unrounded gscale the codes
 *   were taken against (scratch the caller may discard).  The GEMMs take row_scale as their per-channel factor. */
int dirotq_pack_weight_nvfp4_rowscale(const float* w_low, int64_t N, int64_t n_low, void* codes, void* sf,
                                      float* row_scale, float* row_scale_exact, void* stream);

/* Hadamard front end of layers with use_hadamard (dirotq_fused_unrotation_fast.py:106-128;
 * utils/hadamard_utils.py:56-80): y[:, :low_dim] = FWHT(x[:, :low_dim] * sign_flips) / sqrt(low_dim) with
 * fp32 butterflies in the reference's stage order (bit-identical to it), y[:, low_dim:] = x[:, low_dim:].
 * x, y bf16 [M, width] (y != x); sign_flips bf16 [low_dim] of +-1 or NULL; low_dim a power of two in
 * [16, 8192].  The quantiser (dirotq_quantize_act / dirotq_linear_forward without rotation) runs on y. */
int dirotq_hadamard_low(const void* x, int64_t M, int32_t width, int32_t low_dim, const void* sign_flips, void* y,
                        void* stream);

/* ---------------------------------------------------------------------------------------------
 * Kernel 2: W4A4 GEMM + bf16 high-precision branch + dequant + bias.  Replaces the inner
 * `self.module(x)` of the fused forward (dirotq_fused_unrotation_fast.py:141) as a real 4-bit GEMM
 * (the reference's speed path calls the third-party nunchaku gemm_w4a4 for this).
 *
 * INT (exact int32 accumulation per 64-chunk, tcgen05 kind::i8):
 *   y[m,n] = sum_c xs[c,m] ws[c,n] (sum_k qx qw  -  xz[c,m] wsum[c,n]) + x_tail[m,:].w_tail[n,:] + bias[n]
 *   a_mode : DIROTQ_INT4_SYM / INT4_ASYM / INT8_ASYM (layout of x_codes / presence of x_zeros)
 *   w_tail : bf16 [N, tail_pitch]; x_tail bf16 [M, tail_pitch]; tail_total may be 0
 *   acc_dump: optional int32 [n_chunks, M, N] receiving the raw per-chunk accumulators (tests)
 */
int dirotq_gemm_w4a4_int(int32_t a_mode, int64_t M, int64_t N, int32_t n_chunks, const void* x_codes,
                         const void* x_scales, const void* x_zeros, const void* w_codes, const float* w_scales,
                         const float* w_sum, const void* x_tail, const void* w_tail, int32_t tail_total,
                         int32_t tail_pitch, const void* bias, void* y, int32_t* acc_dump, int32_t* status,
                         void* stream);

/* Integer activations at tensor rate (tcgen05 kind::f16): the same product as dirotq_gemm_w4a4_int for
 * 4-bit and 8-bit activation codes, computed the way the reference's own linear computes it -- a 16-bit GEMM with fp32
 * accumulation over the dequantised values s*(q-z) and s_w*q_w (dirotq_fused_unrotation_fast.py:141)
 * -- while both operands stay 4-bit in memory: activation codes are expanded to fp16 between shared
 * memory and the tensor core, weight codes once per call into an fp16 scratch panel that the GEMM's
 * tiles read through L2; one accumulator runs over the whole K, and nothing is drained per chunk.
 * Activation values are exact in fp16; weight values are rounded once to fp16 (the reference rounds
 * them to bf16).  Row / column powers of two keep every scale inside the fp16 range.
 *
 * dirotq_fold_weight_scales_f16 (once per layer): w_scales fp32 [n_chunks, ldn] ->
 *   w_mult: dirotq_fold_weight_records_bytes(n_chunks, N) bytes of 8-byte per-(chunk, channel)
 *   records (fp16 pairs: scale * 2^24 and -8 * scale, each divided by the channel's power of two), w_colscale fp32 [N]; w_tail bf16 [N, tail_pitch] -> w_tail_out = w_tail / colscale
 *   (may be NULL when tail_total == 0).
 * dirotq_expand_weight_panel_f16: w_codes + w_mult -> panel, fp16 [N, n_chunks * 64]
 *   (dirotq_weight_panel_bytes(n_chunks, N) bytes, 16-byte aligned): (q_w - 8) * s_w / colscale in the
 *   K order the activation converters produce.  A caller that prefers 2 bytes per weight of resident memory to a
 *   small per-call pre-pass builds it once and passes it as w_panel.
 * dirotq_gemm_w4a4_int_f16: a_mode DIROTQ_INT4_SYM, DIROTQ_INT4_ASYM or DIROTQ_INT8_ASYM; w_panel NULL: the panel
 *   is rebuilt from w_codes / w_mult in the workspace on every call (w_codes / w_mult may be NULL when w_panel
 *   is given); workspace of dirotq_gemm_w4a4_int_f16_workspace_bytes(M, N_panel, n_chunks, tail_pitch) bytes,
 *   256-byte aligned (per-call activation multipliers, the scaled copy of the tail and, for N_panel = N > 0,
 *   the panel; N_panel = 0 for callers that pass their own).
 */
size_t dirotq_fold_weight_records_bytes(int32_t n_chunks, int64_t N);
int dirotq_fold_weight_scales_f16(int32_t n_chunks, int64_t N, const float* w_scales, const void* w_tail,
                                  int32_t tail_total, int32_t tail_pitch, void* w_mult, float* w_colscale,
                                  void* w_tail_out, void* stream);
size_t dirotq_weight_panel_bytes(int32_t n_chunks, int64_t N);
int dirotq_expand_weight_panel_f16(int32_t n_chunks, int64_t N, const void* w_codes, const void* w_mult, void* panel,
                                   void* stream);
/* The same with the panel layout of layers whose per-head groups have at most 32 channels (half_chunks != 0; SANA's
 * 28): only the first 32 code slots of each chunk are expanded, two chunks per 64-wide stage, panel [N,
 * ceil(n_chunks / 2) * 64].  dirotq_linear_uses_half_chunks tells whether dirotq_linear_forward reads a resident
 * panel (dirotq_linear.w_panel_f16) of `lin` in that layout. */
int dirotq_expand_weight_panel_f16_layout(int32_t n_chunks, int64_t N, const void* w_codes, const void* w_mult, void* panel,
                                          int32_t half_chunks, void* stream);
size_t dirotq_gemm_w4a4_int_f16_workspace_bytes(int64_t M, int64_t N_panel, int32_t n_chunks, int32_t tail_pitch);
int dirotq_gemm_w4a4_int_f16(int32_t a_mode, int64_t M, int64_t N, int32_t n_chunks, const void* x_codes,
                             const void* x_scales, const void* x_zeros, const void* w_codes, const void* w_mult,
                             const void* w_panel, const float* w_colscale, const void* x_tail,
                             const void* w_tail_scaled, int32_t tail_total, int32_t tail_pitch, const void* bias, void* y,
                             void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* NVFP4 (tcgen05 kind::mxf4nvf4, UE4M3 scale factors in TMEM):
 *   y[m,n] = out_scale * c[n] * (sum_blocks sfx sfw (e2m1.e2m1) + x_tail . w_tail_scaled[n]) + bias[n]
 *   out_scale = Tx * Tw; w_colscale: optional fp32 [N] (16-byte aligned) per-channel weight scale c[n] (row_scale of
 *   dirotq_pack_weight_nvfp4_rowscale), NULL = 1; w_tail_scaled = w_tail / (out_scale * c[n]) (bf16, prepared once
 *   by the host).
 */
int dirotq_gemm_w4a4_nvfp4(int64_t M, int64_t N, int32_t n_chunks, const void* x_codes, const void* x_sf,
                           const void* w_codes, const void* w_sf, float out_scale, const float* w_colscale,
                           const void* x_tail, const void* w_tail_scaled, int32_t tail_total, int32_t tail_pitch,
                           const void* bias, void* y, int32_t* status, void* stream);

/* W4A16: bf16 activations x INT4 group-64 weights (PixArt ff.net.2 under --skip-quant-layers; the
 * reference's model of this layer is dequantise-then-GEMM, speedup/weight_only_nvfp4.py:128-178).
 * Weights in the dirotq_pack_weight_int4 format with group 64 (K = n_chunks * 64).  The weight is
 * dequantised to bf16 into `workspace` (N * K * 2 bytes, caller-owned scratch, 16-byte aligned) and
 * multiplied on the bf16 tensor cores; x bf16 [M, K], y bf16 [M, N]. */
size_t dirotq_gemm_w4a16_workspace_bytes(int64_t N, int64_t K);
int dirotq_gemm_w4a16(int64_t M, int64_t N, int64_t K, const void* x, const void* w_codes, const float* w_scales,
                      const void* bias, void* y, void* workspace, size_t workspace_bytes, int32_t* status,
                      void* stream);

/* The two halves of dirotq_gemm_w4a16 / dirotq_gemm_w4a16_nvfp4 on their own, for callers that keep the dequantised
 * weight (N * K * 2 bytes) resident instead of rebuilding it on every call -- worth it when the batch is small and the
 * dequantisation is a visible share of the layer (a 4096-row call of PixArt's 4608 -> 1152 ff.net.2: 13 of 58 us).
 *   dirotq_dequant_weight_int4: w_out bf16 [N, K] = code * scale, K = n_chunks * 64, one rounding per value (what
 *   WeightOnlyNVFP4Linear.dequant does for its format, speedup/weight_only_nvfp4.py:162-171).
 *   dirotq_gemm_bf16: y = x @ w^T + bias on the bf16 tensor cores; x [M, K], w [N, K] (K-major), y [M, N]. */
int dirotq_dequant_weight_int4(int64_t N, int64_t K, const void* w_codes, const float* w_scales, void* w_out, void* stream);
int dirotq_gemm_bf16(int64_t M, int64_t N, int64_t K, const void* x, const void* w, const void* bias, void* y,
                     int32_t* status, void* stream);
/* Same with an NVFP4 weight: the forward of the reference's WeightOnlyNVFP4Linear
 * (speedup/weight_only_nvfp4.py:128-178).  Codes / tiled UE4M3 scales from either NVFP4 packer; the second-level
 * scale is w_rowscale (fp32 [N], from dirotq_pack_weight_nvfp4_rowscale: the reference's per-channel gscale) when
 * given, else the scalar w_tensor_scale.  Dequantised value = bf16(e2m1 * (micro * scale)), one rounding, as the
 * reference's dequantiser computes it (:96-112). */
int dirotq_gemm_w4a16_nvfp4(int64_t M, int64_t N, int64_t K, const void* x, const void* w_codes, const void* w_sf,
                            float w_tensor_scale, const float* w_rowscale, const void* bias, void* y, void* workspace,
                            size_t workspace_bytes, int32_t* status, void* stream);

/* The dequantisation step of the call above alone: w_out bf16 [N, K] (K a multiple of 64).  Replaces
 * WeightOnlyNVFP4Linear.dequant (speedup/weight_only_nvfp4.py:75-125, 158-160). */
int dirotq_dequant_weight_nvfp4(int64_t N, int64_t K, const void* w_codes, const void* w_sf, float w_tensor_scale,
                                const float* w_rowscale, void* w_out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One wrapped linear end to end: what the patched ActQuantWrapper.forward runs
 * (dirotq_fused_unrotation_fast.py:56-141).  `workspace` holds codes / scales / zeros / tail. */
typedef struct dirotq_linear {
  dirotq_act_format fmt;
  int64_t out_features;
  const void* rot_t;        /* NULL: no rotation (quantise only) */
  const int64_t* perm_idx;  /* optional channel selection x[..., perm_idx].  With rot_t == NULL it is applied to the input
                             * (dirotq_fused_unrotation_fast.py:130-134); with rot_t != NULL to the ROTATED tensor
                             * (two launches: rotate into scratch, then gather + quantise) -- how a per-head
                             * rotation meets a format whose groups are not one per head. */
  const void* w_codes;
  const void* w_scales;     /* INT: fp32 [n_chunks, ldn]; NVFP4: tiled UE4M3 */
  const float* w_sum;       /* INT only */
  const void* w_tail;       /* bf16 [N, tail_pitch] (NVFP4: divided by out_scale) */
  const void* bias;         /* bf16 [N] or NULL */
  float w_tensor_scale;     /* NVFP4 only */
  /* Integer activations: all three from dirotq_fold_weight_scales_f16.  When w_mult is set the
   * forward runs dirotq_gemm_w4a4_int_f16; when NULL, the exact-integer dirotq_gemm_w4a4_int.
   * NVFP4: w_colscale alone may be set -- the per-channel scale of dirotq_pack_weight_nvfp4_rowscale (w_tail then
   * holds w_tail / (Tx * w_tensor_scale * w_colscale[n])). */
  const void* w_mult;
  const float* w_colscale;
  const void* w_tail_f16;
  /* Activation fused into the GEMM epilogue: 0 = none, 1 = GELU in its tanh form, applied to the bf16-rounded
   * output (what the activation module that follows the linear in the reference model computes:
   * diffusers' GELU(approximate="tanh") around ff.net.0.proj).  Supported by the tensor-rate integer GEMM
   * and the NVFP4 GEMM; DIROTQ_E_UNSUPPORTED on the exact-integer route. */
  int32_t epilogue_act;
  /* Optional resident fp16 weight panel from dirotq_expand_weight_panel_f16 (tensor-rate integer route only);
   * NULL: rebuilt in the workspace on every call. */
  const void* w_panel_f16;
} dirotq_linear;

size_t dirotq_linear_workspace_bytes(const dirotq_linear* lin, int64_t M);
int dirotq_linear_forward(const dirotq_linear* lin, const void* x, int64_t M, void* y, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream);

/* Second half of dirotq_linear_forward alone: the GEMM of `lin` on the quantised activations that an
 * earlier dirotq_linear_forward left in `workspace` (same M, a layer with the same activation format
 * and rotation -- e.g. to_k and to_v after to_q, which the reference rotates with the same matrix,
 * models/pixart-sigma/model_utils.py:84-92 -- and the same GEMM variant, i.e. w_mult set or not in
 * both).  The caller guarantees that the activations are unchanged since. */
int dirotq_linear_gemm(const dirotq_linear* lin, int64_t M, void* y, void* workspace, size_t workspace_bytes,
                       int32_t* status, void* stream);

/* Producer -> consumer hand-off inside a feed-forward pair (up-projection with its fused GELU, then
 * the down-projection; the reference runs them as two ActQuantWrapper forwards with the activation
 * between them, models/pixart-sigma/model_utils.py:120-127, utils/quant_utils.py:255-326): the
 * producer's GEMM epilogue quantises its own output rows for `next` -- codes, scales and zero points
 * land in next_workspace exactly as next's quantise stage would have left them, bit for bit -- so the
 * separate quantise launch and one round trip of the [M, out_features] tensor disappear.  `y` may be
 * NULL when nobody else reads the producer's output.  Afterwards dirotq_linear_gemm_prequantised
 * (next, M, ...) on next_workspace finishes the pair.
 *   Supported (dirotq_linear_chain_supported returns 1): `lin` a 4-bit integer layer on the
 * 16-bit-conversion GEMM (w_mult set); `next` a 4-bit integer layer, hidden layout, groups of 64, its
 * quantised part and its 16-bit tail both multiples of 64 channels (the tail may be empty), no
 * rotation, no channel selection, width == lin->out_features, w_mult set.  Anything else: DIROTQ_E_UNSUPPORTED, nothing launched. */
int dirotq_linear_uses_half_chunks(const dirotq_linear* lin);
int dirotq_linear_chain_supported(const dirotq_linear* lin, const dirotq_linear* next);
int dirotq_linear_forward_chain(const dirotq_linear* lin, const void* x, int64_t M, void* y, void* workspace,
                                size_t workspace_bytes, const dirotq_linear* next, void* next_workspace,
                                size_t next_workspace_bytes, int32_t* status, void* stream);
/* The GEMM of `lin` on codes / scales / zero points that a producer's epilogue wrote into `workspace`
 * (dirotq_linear_forward_chain): like dirotq_linear_gemm, plus the per-call folding of the scales
 * that dirotq_linear_forward does in its first half. */
int dirotq_linear_gemm_prequantised(const dirotq_linear* lin, int64_t M, void* y, void* workspace,
                                    size_t workspace_bytes, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Block glue: the row-wise passes between two wrapped linears of a DiT block.  Not part of the
 * ActQuantWrapper forward; the reference's model forwards run them as separate PyTorch / nunchaku
 * calls (speedup/report_flux_w4a4_no_rot_ffdown.py:199-228, :240-252, :261-276).  bf16 in and out,
 * fp32 inside, one rounding; every input is read once.
 *
 * dirotq_layernorm_modulate: y[r, :] = LayerNorm(x[r, :]) * (1 + scale[b, :]) + shift[b, :] with
 *   b = r / rows_per_sample; no affine parameters, biased variance.  scale / shift: bf16, sample b at
 *   scale + b * mod_pitch (elements; either may be NULL).  D % 8 == 0, D <= 4096.
 * dirotq_gated_residual: out = h + gate[b, :] * (y + y2); y2 and gate may be NULL (gate NULL: out =
 *   h + y + y2).  out may alias h.
 * dirotq_qkv_norm_rope: q, k, v bf16 [B * T, H * d] with a common row pitch (elements; columns of one
 *   fused projection output, or three tensors).  q and k: RMSNorm over each head's d values times
 *   w_q / w_k (bf16 [d], NULL: no normalisation), then the rotary embedding out[2i] = x[2i] cos[p, 2i]
 *   - x[2i+1] sin[p, 2i], out[2i+1] = x[2i+1] cos[p, 2i+1] + x[2i] sin[p, 2i+1] at position p = t0 + t
 *   (cos / sin bf16 [T_total, d], NULL: none); v is copied.  Outputs are token-major [B, T_total, H, d]
 *   and receive rows t0 .. t0 + T - 1 of every sample: two calls (text at t0 = 0, image at t0 = S)
 *   fill one buffer for a joint attention.  d = 64 or 128. */
int dirotq_layernorm_modulate(const void* x, int64_t M, int32_t D, int64_t rows_per_sample, const void* scale,
                              const void* shift, int64_t mod_pitch, float eps, void* y, void* stream);
int dirotq_gated_residual(const void* h, const void* y, const void* y2, const void* gate, int64_t mod_pitch, int64_t M,
                          int32_t D, int64_t rows_per_sample, void* out, void* stream);
int dirotq_qkv_norm_rope(const void* q, const void* k, const void* v, int64_t pitch, int64_t B, int64_t T, int32_t H,
                         int32_t d, const void* w_q, const void* w_k, const void* cos, const void* sin, int64_t T_total,
                         int64_t t0, float eps, void* out_q, void* out_k, void* out_v, void* stream);

/* Same computation as dirotq_linear_forward, for callers that can hand over nothing but the input
 * and the output.  (No counterpart in the reference: its eager forward allocates freely through
 * torch.)  Meant for hosts that give a plug-in no allocator at all -- an inference server whose
 * device memory is carved up once at start-up, or a latency-critical loop that cannot afford the
 * device-wide synchronisation a cudaMalloc / cudaFree may cause.  The codes / scales / zero points /
 * tail of the call live in a fixed array inside the library's device image
 * (dirotq_linear_forward_static_capacity() bytes, 32 MiB; each GPU that loads the library carries
 * it until the process exits).  The call allocates and frees nothing.
 *  - Sizes whose scratch need (dirotq_linear_workspace_bytes) exceeds the capacity are refused with
 *    DIROTQ_E_TOO_LARGE before anything is launched.
 *  - The first call on each device looks up the array's device address (a host-side runtime query);
 *    make that first call before starting any stream capture.  Host threads may race on that first
 *    call (each stores the same address).  The address is cached per device ordinal (0..63; higher
 *    ordinals are refused with DIROTQ_E_UNSUPPORTED) and does not survive a device reset.
 *  - All calls share the one array and it keeps the previous call's bytes; the entry point clears
 *    the part that must start at zero itself.  Two calls whose kernels may overlap on the GPU
 *    (different streams, no dependency) race on the array: serialise them. */
size_t dirotq_linear_forward_static_capacity(void);
int dirotq_linear_forward_static(const dirotq_linear* lin, const void* x, int64_t M, void* y, int32_t* status,
                                 void* stream);

/* ---- misc ---- */
int dirotq_abi_version(void);
/* Every device-side wait (on a shared-memory stage, an accumulator, scale factors) is bounded: after `cycles` SM clock
 * cycles (0 = the default of 3e9, about 1.5 s) the waiting role writes its code into the caller's status word, raises
 * the CTA's abort flag, the kernel awaits its copies in flight (bounded), frees its tensor memory and returns; the
 * context stays usable and the outputs of that launch are undefined.  The setting is process-wide and applies to
 * launches made after the call.  No counterpart in the reference (its eager kernels have no waits of their own). */
int dirotq_set_wait_limit_cycles(int64_t cycles);
const char* dirotq_error_string(int code);
/* Text for a positive device status code (which wait ran out). */
const char* dirotq_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* DIROTQ_B200_H */
