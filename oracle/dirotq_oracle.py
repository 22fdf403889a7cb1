"""CPU restatement of the DiRotQ quantized-linear forward (TEST INFRASTRUCTURE ONLY).

This file is the checker for the CUDA path.  Nothing in the shipped package
imports it: only the tests, the smoke entry and the CPU-baseline leg of the
benchmark do.  It restates, with plain torch CPU ops, the arithmetic of the
reference implementation and additionally exposes what the reference keeps
implicit: the integer / E2M1 *codes*, the group scales and zero points, and the
per-group int32 accumulators a real 4-bit GEMM produces.

Parity status: PINNED.  ``tests/golden/*.npz`` hold outputs of the unmodified
reference (imported from its checkout by ``tests/golden/make_golden.py``); the
CPU test-suite checks that ``scale * code`` from this file reproduces the
reference's fake-quant tensors, scales, zero points and layer outputs bit for
bit.

Reference citations (paths inside the DiRotQ project):
  utils/quant_utils.py:15-35     E2M1 codebook, bucketize rounding
  utils/quant_utils.py:63-85     STEQuantize / AsymSTEQuantize
  utils/quant_utils.py:112-180   ActQuantizer.forward (INT and NVFP4 grouped)
  utils/quant_utils.py:201-240   find_params (groupwise / per-token)
  utils/quant_utils.py:590-767   weight rotate / split / RTN
  dirotq_fused_unrotation.py:62-148       fp32 fused forward (CPU baseline)
  dirotq_fused_unrotation_fast.py:56-141  bf16 fused forward (bit contract)
  speedup/weight_only_nvfp4.py:42-72      two-level NVFP4 weight quantiser
  speedup/nunchaku_pack.py:63-70,324-459  packer-side quantisers
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F

# utils/quant_utils.py:15-16 -- 15-entry codebook, no negative zero.
E2M1_VALUES = [-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, 0.0,
               0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
E2M1_MAX = 6.0
# Hardware nibble for each codebook index: bit3 = sign, bits2..0 = magnitude
# index into [0, .5, 1, 1.5, 2, 3, 4, 6].
_MAG = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
E2M1_NIBBLE_OF_INDEX = [(8 | _MAG.index(-v)) if v < 0 else _MAG.index(v) for v in E2M1_VALUES]
E2M1_VALUE_OF_NIBBLE = _MAG + [-m for m in _MAG]


def e2m1_index(x_norm: torch.Tensor) -> torch.Tensor:
    """Codebook index of each element (quant_utils.py:30-35).

    ``bucketize`` with right=False sends an exact midpoint to the LOWER codebook
    value (toward -inf): 0.25 -> 0, -0.25 -> -0.5, 2.5 -> 2, -2.5 -> -3.
    """
    cb = torch.tensor(E2M1_VALUES, dtype=x_norm.dtype)
    mid = (cb[:-1] + cb[1:]) / 2
    return torch.bucketize(x_norm.contiguous(), mid)


def e2m1_nibbles(idx: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_NIBBLE_OF_INDEX, dtype=torch.uint8)
    return lut[idx]


def e2m1_values(nib: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUE_OF_NIBBLE, dtype=dtype)
    return lut[nib.long()]


# ---------------------------------------------------------------------------
# activation quantiser
# ---------------------------------------------------------------------------
@dataclass
class QuantCfg:
    """Mirror of the fields ActQuantizer.configure sets (quant_utils.py:182-199)."""
    bits: int = 4
    groupsize: int = 64
    sym: bool = True
    clip_ratio: float = 1.0
    high_bits_length: int = 0
    quant_dtype: str = "int"      # "int" | "nvfp4"

    def __post_init__(self):
        if self.quant_dtype == "nvfp4":
            self.sym = True

    @property
    def maxq(self) -> int:
        return 2 ** (self.bits - 1) - 1 if self.sym else 2 ** self.bits - 1


@dataclass
class ActQuantResult:
    codes: torch.Tensor            # [B,T,G,gs] int16 (INT: q or q-zero is NOT applied; raw q) / E2M1 nibble (NVFP4)
    scale: torch.Tensor            # [B,T,G,1]  x dtype
    zero: Optional[torch.Tensor]   # [B,T,G,1]  x dtype (asym INT) or None
    deq: torch.Tensor              # [B,T,q_len] x dtype, == reference fake-quant output on the low region
    tail: torch.Tensor             # [B,T,hlen] passthrough
    q_len: int
    full: torch.Tensor = field(default=None)  # cat(deq, tail) == ActQuantizer.forward output


def _group(x_l: torch.Tensor, gs: int) -> torch.Tensor:
    q_len = x_l.shape[-1]
    pad = (-q_len) % gs
    if pad:
        x_l = F.pad(x_l, (0, pad))          # quant_utils.py:129-131 / :167-169
    return x_l.reshape(x_l.shape[0], x_l.shape[1], -1, gs)


def act_quant_int(x: torch.Tensor, cfg: QuantCfg) -> ActQuantResult:
    """INT groupwise activation quantiser with explicit codes.

    find_params: quant_utils.py:201-216, :226-235.  Quantise: :63-85, :124-146.
    All arithmetic runs in ``x.dtype`` exactly as torch evaluates the reference
    expressions (bf16 ops round after every operation).
    """
    assert x.dim() == 3 and cfg.quant_dtype == "int"
    hlen = cfg.high_bits_length
    q_len = x.shape[-1] - hlen
    x_l, x_h = x[..., :q_len], x[..., q_len:]
    maxq = torch.tensor(cfg.maxq)           # 0-dim int64, does not promote
    if cfg.groupsize > 0:
        xg = _group(x_l, cfg.groupsize)
        xmax = torch.amax(xg, dim=-1, keepdim=True) * cfg.clip_ratio
        xmin = torch.amin(xg, dim=-1, keepdim=True) * cfg.clip_ratio
    else:
        # per-token scales (quant_utils.py:236-240 -> _find_params :242-271): one group = the whole quantised
        # region of a row; the extrema start from zero (:248-249)
        xg = x_l.reshape(x.shape[0], x.shape[1], 1, q_len)
        zero_ref = torch.zeros((), dtype=x.dtype)
        xmax = torch.maximum(torch.amax(xg, dim=-1, keepdim=True), zero_ref) * cfg.clip_ratio
        xmin = torch.minimum(torch.amin(xg, dim=-1, keepdim=True), zero_ref) * cfg.clip_ratio
    if cfg.sym:
        xmax = torch.maximum(torch.abs(xmin), xmax)
        tmp = xmax == 0
        scale = xmax / maxq
        scale[tmp] = 1
        scale = scale.to(x.dtype)
        q = torch.clamp(torch.round(xg / scale), -(maxq + 1), maxq)
        deq = scale * q
        zero = None
        codes = q
    else:
        tmp = (xmin == 0) & (xmax == 0)
        xmin[tmp] = -1
        xmax[tmp] = +1
        scale = (xmax - xmin).clamp(min=1e-5) / maxq
        zero = torch.round(-xmin / scale)
        scale, zero = scale.to(x.dtype), zero.to(x.dtype)
        q = torch.clamp(torch.round(xg / scale) + zero, 0, maxq)
        deq = scale * (q - zero)
        codes = q
    deq = deq.reshape(x.shape[0], x.shape[1], -1)[..., :q_len].to(x.dtype)
    full = deq if hlen == 0 else torch.cat([deq, x_h], dim=-1).to(x.dtype)
    return ActQuantResult(codes.to(torch.int16), scale, zero, deq, x_h, q_len, full)


def act_quant_nvfp4(x: torch.Tensor, cfg: QuantCfg) -> ActQuantResult:
    """Grouped E2M1 activation quantiser, unrounded scale (quant_utils.py:148-180)."""
    assert x.dim() == 3 and cfg.groupsize > 0
    hlen = cfg.high_bits_length
    q_len = x.shape[-1] - hlen
    x_l, x_h = x[..., :q_len], x[..., q_len:]
    xg = _group(x_l, cfg.groupsize)
    scale = torch.amax(xg.abs(), dim=-1, keepdim=True) * cfg.clip_ratio
    scale = (scale / E2M1_MAX).clamp(min=1e-5)
    idx = e2m1_index(xg / scale)
    cb = torch.tensor(E2M1_VALUES, dtype=x.dtype)
    deq = (cb[idx] * scale).reshape(x.shape[0], x.shape[1], -1)[..., :q_len]
    full = deq.to(x.dtype) if hlen == 0 else torch.cat([deq, x_h], dim=-1).to(x.dtype)
    return ActQuantResult(e2m1_nibbles(idx), scale, None, deq.to(x.dtype), x_h, q_len, full)


def e4m3_round(v: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to FP8 E4M3 (finite, saturating at 448), returned as fp32."""
    return v.float().clamp(max=448.0).to(torch.float8_e4m3fn).float()


def act_quant_nvfp4_hw(x: torch.Tensor, cfg: QuantCfg, tensor_scale: float = 1.0) -> ActQuantResult:
    """Two-level NVFP4 quantiser that block-scaled tensor cores can consume.

    The reference has this recipe only for weights (weight_only_nvfp4.py:42-72:
    micro = e4m3(group_scale / gscale), codes against the EFFECTIVE scale); the
    activation side of the reference keeps an unrounded scale.  Contract used by
    the CUDA path: s_g = amax_g * clip / 6 evaluated in fp32 from the bf16 inputs,
    micro_g = e4m3_rn(clamp(s_g / T, 2^-9, 448)) (0 for an all-zero group),
    codes = bucketize(x / (micro_g * T)) with the reference tie rule, in fp32.
    """
    assert x.dim() == 3 and cfg.groupsize == 16
    hlen = cfg.high_bits_length
    q_len = x.shape[-1] - hlen
    x_l, x_h = x[..., :q_len], x[..., q_len:]
    xg = _group(x_l, 16).float()
    amax = xg.abs().amax(dim=-1, keepdim=True) * float(cfg.clip_ratio)
    s = amax / E2M1_MAX
    T = torch.tensor(float(tensor_scale), dtype=torch.float32)
    micro = e4m3_round((s / T).clamp(min=2.0 ** -9))
    micro = torch.where(amax == 0, torch.zeros_like(micro), micro)
    eff = micro * T
    xn = torch.where(eff > 0, xg / torch.where(eff > 0, eff, torch.ones_like(eff)), torch.zeros_like(xg))
    idx = e2m1_index(xn)
    cb = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    deq = (cb[idx] * eff).reshape(x.shape[0], x.shape[1], -1)[..., :q_len]
    full = torch.cat([deq.to(x.dtype), x_h], dim=-1) if hlen else deq.to(x.dtype)
    return ActQuantResult(e2m1_nibbles(idx), micro, None, deq, x_h, q_len, full)


def act_quant(x: torch.Tensor, cfg: QuantCfg) -> ActQuantResult:
    if cfg.quant_dtype == "nvfp4":
        return act_quant_nvfp4(x, cfg)
    return act_quant_int(x, cfg)


# ---------------------------------------------------------------------------
# rotations
# ---------------------------------------------------------------------------
def rotate_hidden(x: torch.Tensor, U: torch.Tensor, fp32: bool) -> torch.Tensor:
    """x_rot = x @ U.  fp32=True: dirotq_fused_unrotation.py:78-79; else _fast.py:71-72."""
    shp = x.shape
    if fp32:
        return (x.float().reshape(-1, shp[-1]) @ U.float()).reshape(shp)
    return (x.reshape(-1, shp[-1]) @ U.to(x.dtype)).reshape(shp)


def rotate_per_head(x: torch.Tensor, U_ph: torch.Tensor, fp32: bool) -> torch.Tensor:
    """[..., H*d] -> [..., H, d] rotated per head (_fast.py:81-82; fp32: dirotq_fused_unrotation.py:90-91)."""
    H, d, _ = U_ph.shape
    xh = (x.float() if fp32 else x).reshape(*x.shape[:-1], H, d)
    return torch.einsum('...hd,hde->...he', xh, U_ph.float() if fp32 else U_ph.to(x.dtype))


def per_head_rearrange(x_rot_heads: torch.Tensor, hlen: int) -> torch.Tensor:
    """[*, H, d] -> [*, H*d_q | H*hlen]  (_fast.py:83-88)."""
    *bt, H, d = x_rot_heads.shape
    d_q = d - hlen
    return torch.cat([x_rot_heads[..., :d_q].reshape(*bt, H * d_q),
                      x_rot_heads[..., d_q:].reshape(*bt, H * hlen)], dim=-1)


def per_head_interleave(x_quant: torch.Tensor, H: int, d: int, hlen: int) -> torch.Tensor:
    """Inverse of per_head_rearrange (_fast.py:97-100)."""
    bt = x_quant.shape[:-1]
    d_q = d - hlen
    a = x_quant[..., :H * d_q].reshape(*bt, H, d_q)
    b = x_quant[..., H * d_q:].reshape(*bt, H, hlen)
    return torch.cat([a, b], dim=-1).reshape(*bt, H * d)


# ---------------------------------------------------------------------------
# fused forward (the drop-in boundary), functional form
# ---------------------------------------------------------------------------
@dataclass
class LayerSpec:
    """What ActQuantWrapper carries for one linear (quant_utils.py:300-323)."""
    weight: torch.Tensor                    # [N, D] fused weight in the rotated basis
    bias: Optional[torch.Tensor]
    cfg: QuantCfg
    rotation: Optional[torch.Tensor] = None          # [D, D]
    rotation_per_head: Optional[torch.Tensor] = None  # [H, d, d]
    perm_idx: Optional[torch.Tensor] = None
    hadamard_low_dim: Optional[int] = None            # use_hadamard layers (quant_utils.py:314-316)
    hadamard_sign_flips: Optional[torch.Tensor] = None


def fast_hadamard_transform(x: torch.Tensor) -> torch.Tensor:
    """Walsh-Hadamard transform along the last (power-of-two) dimension, divided by sqrt(D): butterflies
    (a + b, a - b) over blocks of size h = 1, 2, 4, ... in that order (utils/hadamard_utils.py:56-80)."""
    D = x.shape[-1]
    assert D & (D - 1) == 0
    lead = x.shape[:-1]
    h = 1
    while h < D:
        x = x.reshape(*lead, D // (2 * h), 2, h)
        a, b = x[..., 0, :], x[..., 1, :]
        x = torch.stack([a + b, a - b], dim=-2).reshape(*lead, D)
        h *= 2
    return x / (D ** 0.5)


def hadamard_low(x: torch.Tensor, low_dim: int, sign_flips: Optional[torch.Tensor], fp32: bool) -> torch.Tensor:
    """The use_hadamard branch of the forward up to the quantiser (dirotq_fused_unrotation_fast.py:106-125;
    fp32 variant dirotq_fused_unrotation.py:98-121)."""
    x_low, x_high = x[..., :low_dim], x[..., low_dim:]
    if fp32:
        x_low = x_low.float()
        if sign_flips is not None:
            x_low = x_low * sign_flips.float()
        y = fast_hadamard_transform(x_low)
        return torch.cat([y, x_high.float()], dim=-1) if x_high.shape[-1] else y
    if sign_flips is not None:
        x_low = x_low * sign_flips.to(x.dtype)
    y = fast_hadamard_transform(x_low.float()).to(x.dtype)
    return torch.cat([y, x_high], dim=-1) if x_high.shape[-1] else y


def quantized_input(x: torch.Tensor, spec: LayerSpec, fp32: bool):
    """Returns (x_fake_quant in the layout the fused weight expects, ActQuantResult, x_rot)."""
    cfg = spec.cfg
    if spec.rotation is not None:
        x_rot = rotate_hidden(x, spec.rotation, fp32)
        r = act_quant(x_rot, cfg)
        return r.full, r, x_rot
    if spec.rotation_per_head is not None:
        H, d, _ = spec.rotation_per_head.shape
        xr = rotate_per_head(x, spec.rotation_per_head, fp32)
        hlen = cfg.high_bits_length
        if fp32 or hlen == 0:
            # dirotq_fused_unrotation.py:86-96 does NOT rearrange: flat hlen / groupsize.
            flat = xr.reshape(*x.shape[:-1], H * d)
            r = act_quant(flat, cfg)
            return r.full, r, flat
        d_q = d - hlen
        xre = per_head_rearrange(xr, hlen)
        c2 = QuantCfg(cfg.bits, d_q if d_q > 0 else -1, cfg.sym, cfg.clip_ratio, H * hlen, cfg.quant_dtype)
        r = act_quant(xre, c2)
        return per_head_interleave(r.full, H, d, hlen), r, xre
    if spec.hadamard_low_dim is not None:
        x_rot = hadamard_low(x, spec.hadamard_low_dim, spec.hadamard_sign_flips, fp32)
        r = act_quant(x_rot, cfg)
        return r.full, r, x_rot
    if spec.perm_idx is not None:
        xp = x[..., spec.perm_idx]
        if fp32:
            xp = xp  # dirotq_fused_unrotation.py:129 keeps the input dtype here
        r = act_quant(xp, cfg)
        return r.full, r, xp
    r = act_quant(x, cfg)
    return r.full, r, x


def fused_forward(x: torch.Tensor, spec: LayerSpec, fp32: bool = False) -> torch.Tensor:
    """_fused_forward (fp32=True) / _fused_forward_fast (fp32=False) for a fused layer."""
    xq, _, _ = quantized_input(x, spec, fp32)
    xq = xq.to(x.dtype)
    return F.linear(xq, spec.weight, spec.bias).to(x.dtype)


# ---------------------------------------------------------------------------
# weight side
# ---------------------------------------------------------------------------
def weight_quant_int(W: torch.Tensor, bits: int, gs: int, sym: bool = True):
    """_quant_group_int (quant_utils.py:714-737), groupwise; returns (deq, codes, scale)."""
    out_f, in_f = W.shape
    W = W.float()
    pad = (-in_f) % gs
    if pad:
        W = F.pad(W, (0, pad))
    Wg = W.reshape(out_f, -1, gs)
    assert sym
    maxq = 2 ** (bits - 1) - 1
    scale = Wg.abs().amax(dim=-1, keepdim=True).clamp(min=1e-5) / maxq
    q = torch.clamp(torch.round(Wg / scale), -maxq - 1, maxq)
    deq = (q * scale).reshape(out_f, -1)[:, :in_f]
    return deq, q.to(torch.int8), scale.squeeze(-1)


def weight_quant_nvfp4(W: torch.Tensor, gs: int = 16):
    """_quant_group_nvfp4 (quant_utils.py:752-765); returns (deq, nibbles, scale)."""
    out_f, in_f = W.shape
    W = W.float()
    pad = (-in_f) % gs
    if pad:
        W = F.pad(W, (0, pad))
    Wg = W.reshape(out_f, -1, gs)
    scale = Wg.abs().amax(dim=-1, keepdim=True).clamp(min=1e-5) / E2M1_MAX
    idx = e2m1_index(Wg / scale)
    cb = torch.tensor(E2M1_VALUES)
    deq = (cb[idx] * scale).reshape(out_f, -1)[:, :in_f]
    return deq, e2m1_nibbles(idx), scale.squeeze(-1)


def pow2_tensor_scale(group_scale_max: float) -> float:
    """Per-tensor scale used by the CUDA packer: the smallest power of two T with
    max_g(s_g) / T <= 448, so dividing by T is exact in every float format."""
    if group_scale_max <= 0:
        return 1.0
    return float(2.0 ** math.ceil(math.log2(group_scale_max / 448.0)))


def weight_quant_nvfp4_hw(W: torch.Tensor, tensor_scale: Optional[float] = None):
    """Two-level NVFP4 weight quantiser (weight_only_nvfp4.py:42-72 recipe) with a
    per-TENSOR fp32 scale and the reference's bucketize tie rule.

    s_g = amax_g/6; micro_g = e4m3_rn(clamp(s_g/T, 2^-9)); eff = micro*T;
    codes = bucketize(W/eff).  Returns (deq, nibbles [N,K], micro [N,K/16] fp32, T).
    """
    N, K = W.shape
    assert K % 16 == 0
    Wg = W.float().reshape(N, K // 16, 16)
    amax = Wg.abs().amax(-1, keepdim=True)
    s = amax / E2M1_MAX
    T = pow2_tensor_scale(float(s.max())) if tensor_scale is None else float(tensor_scale)
    micro = e4m3_round((s / T).clamp(min=2.0 ** -9))
    micro = torch.where(amax == 0, torch.zeros_like(micro), micro)
    eff = micro * T
    xn = torch.where(eff > 0, Wg / torch.where(eff > 0, eff, torch.ones_like(eff)), torch.zeros_like(Wg))
    idx = e2m1_index(xn)
    cb = torch.tensor(E2M1_VALUES)
    deq = (cb[idx] * eff).reshape(N, K)
    return deq, e2m1_nibbles(idx).reshape(N, K), micro.squeeze(-1), T


# speedup/weight_only_nvfp4.py:35-36 -- codebook in hardware nibble order (index = nibble)
_E2M1_BY_NIBBLE = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def weight_quant_nvfp4_rowscale(W: torch.Tensor):
    """The reference's own two-level NVFP4 weight quantiser, _quantize_nvfp4 (speedup/weight_only_nvfp4.py:42-72),
    with the nibbles left unpacked:

        group_scale = max(amax_g / 6, 1e-12)      gscale[n] = max(max_g group_scale / 448, 1e-12)      (fp32)
        micro = e4m3(group_scale / gscale[n])     eff = float(micro) * gscale[n]
        nibble = first argmin_i |W / eff - codebook[i]|

    Returns (nibbles [N, K] uint8, micro [N, K/16] float8_e4m3fn, gscale [N] bf16, gscale_exact [N] fp32).
    The reference stores the nibbles planar (column j with column j + K/2 in one byte, :66-71): see
    ``pack_planar_halves``."""
    N, K = W.shape
    assert K % 16 == 0
    Wg = W.float().reshape(N, K // 16, 16)
    gs_full = (Wg.abs().amax(-1) / E2M1_MAX).clamp(min=1e-12)
    gscale = (gs_full.amax(-1) / 448.0).clamp(min=1e-12)
    micro = (gs_full / gscale[:, None]).to(torch.float8_e4m3fn)
    eff = micro.float() * gscale[:, None]
    # First argmin over [0 .5 1 1.5 2 3 4 6 -0 -.5 ... -6] restated as thresholds: the distances that compete are
    # exact in fp32, a tie keeps the earlier index = the smaller magnitude, +0 precedes -0 and every negative value
    # that rounds to zero, and a zero micro-scale (quotient inf / nan, all distances inf / nan) keeps index 0.
    v = Wg / eff.unsqueeze(-1)
    a = v.abs()
    m = torch.zeros_like(v, dtype=torch.uint8)
    for thr in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        m += (a > thr).to(torch.uint8)
    m = torch.where(torch.isfinite(v), m, torch.zeros_like(m))
    nib = torch.where((v < 0) & (m > 0), m + 8, m)
    return nib.reshape(N, K), micro, gscale.to(torch.bfloat16), gscale


def pack_planar_halves(nib: torch.Tensor) -> torch.Tensor:
    """[N, K] nibbles -> [N, K/2] bytes, byte j = column j | column j + K/2 << 4 (weight_only_nvfp4.py:66-71)."""
    K2 = nib.shape[1] // 2
    return (nib[:, :K2] | (nib[:, K2:] << 4)).contiguous()


def unpack_planar_halves(codes: torch.Tensor) -> torch.Tensor:
    return torch.cat([codes & 0xF, codes >> 4], dim=1)


def dequant_nvfp4_rowscale(nib: torch.Tensor, micro: torch.Tensor, gscale_bf16: torch.Tensor, eager: bool = False):
    """bf16 weight of WeightOnlyNVFP4Linear.  eager=False: the fused dequantiser the forward uses
    (weight_only_nvfp4.py:96-112: fp32 micro * gscale, times the codebook value, ONE rounding to bf16);
    eager=True: dequant_torch (:162-171: bf16 product of the scales, then a bf16 product with the value)."""
    N, K = nib.shape
    if eager:
        cb = torch.tensor(_E2M1_BY_NIBBLE, dtype=torch.bfloat16)
        scale = (micro.to(torch.bfloat16) * gscale_bf16[:, None]).repeat_interleave(16, dim=1)
        return cb[nib.long()] * scale
    cb = torch.tensor(_E2M1_BY_NIBBLE, dtype=torch.float32)
    scale = (micro.float() * gscale_bf16.float()[:, None]).repeat_interleave(16, dim=1)
    return (cb[nib.long()] * scale).to(torch.bfloat16)


def rotate_and_split_W(W: torch.Tensor, spec: LayerSpec):
    """_rotate_and_split_W (quant_utils.py:590-711), hidden / per-head / perm branches.
    Returns (W_low [N, n_low], W_tail [N, n_tail] or None, groupsize_override)."""
    Wf = W.float()
    out_f = Wf.shape[0]
    hlen = int(spec.cfg.high_bits_length)
    if spec.rotation is not None:
        Wr = Wf @ spec.rotation.float()
        if hlen > 0:
            n_low = Wr.shape[1] - hlen
            return Wr[:, :n_low].contiguous(), Wr[:, n_low:].contiguous(), None
        return Wr.contiguous(), None, None
    if spec.rotation_per_head is not None:
        H, d, _ = spec.rotation_per_head.shape
        Wr = torch.einsum('ohd,hde->ohe', Wf.reshape(out_f, H, d), spec.rotation_per_head.float())
        d_q = d - hlen
        if hlen > 0:
            return (Wr[:, :, :d_q].reshape(out_f, H * d_q).contiguous(),
                    Wr[:, :, d_q:].reshape(out_f, H * hlen).contiguous(), d_q)
        return Wr.reshape(out_f, H * d), None, d
    if spec.perm_idx is not None:
        Wp = Wf[:, spec.perm_idx]
        if hlen > 0:
            n_low = Wp.shape[1] - hlen
            return Wp[:, :n_low].contiguous(), Wp[:, n_low:].contiguous(), None
        return Wp.contiguous(), None, None
    return Wf.contiguous(), None, None


def stitch_fused_weight(W_low_q: torch.Tensor, W_tail: Optional[torch.Tensor], spec: LayerSpec):
    """stitch() closures of _rotate_and_split_W: hidden = cat; per-head = interleave per head."""
    if W_tail is None:
        return W_low_q
    if spec.rotation_per_head is not None:
        H, d, _ = spec.rotation_per_head.shape
        hlen = int(spec.cfg.high_bits_length)
        out_f = W_low_q.shape[0]
        return torch.cat([W_low_q.reshape(out_f, H, d - hlen), W_tail.reshape(out_f, H, hlen)],
                         dim=2).reshape(out_f, H * d)
    return torch.cat([W_low_q, W_tail], dim=1)


# ---------------------------------------------------------------------------
# what a real 4-bit GEMM computes
# ---------------------------------------------------------------------------
def int_group_accumulators(codes_x: torch.Tensor, codes_w: torch.Tensor) -> torch.Tensor:
    """acc[g, m, n] = sum_k codes_x[m, g, k] * codes_w[n, g, k]  (exact int32).

    codes_x [M, G, gs] (for asymmetric activations pass q - zero), codes_w [N, G, gs]."""
    return torch.einsum('mgk,ngk->gmn', codes_x.to(torch.int32), codes_w.to(torch.int32))


def w4a4_int_linear(codes_x, scale_x, codes_w, scale_w, x_tail, w_tail, bias, zero_x=None):
    """y = sum_g s_x[m,g] s_w[n,g] acc_g[m,n] + x_tail @ w_tail^T + bias, in fp32.

    codes_x [M,G,gs] int, scale_x [M,G], codes_w [N,G,gs], scale_w [N,G]."""
    cx = codes_x.to(torch.int32)
    if zero_x is not None:
        cx = cx - zero_x.to(torch.int32).reshape(cx.shape[0], cx.shape[1], 1)
    acc = int_group_accumulators(cx, codes_w).float()
    y = torch.einsum('gmn,mg,ng->mn', acc, scale_x.float(), scale_w.float())
    if x_tail is not None and x_tail.shape[-1] > 0:
        y = y + x_tail.float() @ w_tail.float().T
    if bias is not None:
        y = y + bias.float()
    return y


def w4a4_nvfp4_linear(nib_x, micro_x, Tx, nib_w, micro_w, Tw, x_tail, w_tail, bias):
    """y = Tx*Tw * sum_blocks micro_x micro_w (e2m1 . e2m1) + tail + bias, evaluated in fp64."""
    vx = e2m1_values(nib_x, torch.float64)          # [M, K]
    vw = e2m1_values(nib_w, torch.float64)          # [N, K]
    M, K = vx.shape
    sx = micro_x.double().reshape(M, K // 16, 1)
    sw = micro_w.double().reshape(vw.shape[0], K // 16, 1)
    dx = (vx.reshape(M, K // 16, 16) * sx).reshape(M, K)
    dw = (vw.reshape(-1, K // 16, 16) * sw).reshape(-1, K)
    y = (dx @ dw.T) * (float(Tx) * float(Tw))
    if x_tail is not None and x_tail.shape[-1] > 0:
        y = y + x_tail.double() @ w_tail.double().T
    if bias is not None:
        y = y + bias.double()
    return y.float()


def qsnr_db(ref: torch.Tensor, test: torch.Tensor) -> float:
    """10 log10(|ref|^2 / |ref - test|^2), the reference's layer-quality metric (diagnose_layer_qsnr.py:38-46)."""
    ref, test = ref.double(), test.double()
    noise = float(((ref - test) ** 2).sum())
    return float("inf") if noise == 0 else 10.0 * math.log10(float((ref ** 2).sum()) / noise)


def fused_forward_nvfp4_hw(x: torch.Tensor, spec: LayerSpec, tensor_scale: float = 1.0, x_rot: Optional[torch.Tensor] = None):
    """What the block-scaled tensor-core NVFP4 layer computes, in fp64: activations by the two-level recipe
    (act_quant_nvfp4_hw), the fused weight's low block put back on a 4-bit grid by the reference's own two-level
    weight recipe (weight_quant_nvfp4_rowscale), the 16-bit branch and bias added.  ``x_rot`` overrides the rotated
    tensor (pass the one the kernel produced to remove accumulation-order differences)."""
    cfg = spec.cfg
    if x_rot is None:
        x_rot = rotate_hidden(x, spec.rotation.to(x.dtype), fp32=False) if spec.rotation is not None else x
    lead = x_rot.shape[:-1]
    x3 = x_rot.reshape(1, -1, x_rot.shape[-1])
    r = act_quant_nvfp4_hw(x3, cfg, tensor_scale)
    M, q_len = x3.shape[1], r.q_len
    kq = (q_len + 15) // 16 * 16
    w_low = F.pad(spec.weight[:, :q_len].float(), (0, kq - q_len))
    nib_w, micro_w, g_bf16, _ = weight_quant_nvfp4_rowscale(w_low)
    N = w_low.shape[0]
    dw = (e2m1_values(nib_w, torch.float64).reshape(N, -1, 16) * (micro_w.double() * g_bf16.double()[:, None]).unsqueeze(-1))
    dx = F.pad(r.deq.double().reshape(M, q_len), (0, kq - q_len))
    y = dx @ dw.reshape(N, kq).T
    if cfg.high_bits_length > 0:
        y = y + r.tail.double().reshape(M, -1) @ spec.weight[:, q_len:].double().T
    if spec.bias is not None:
        y = y + spec.bias.double()
    return y.float().reshape(*lead, N)


# ---------------------------------------------------------------------------
# device data formats (restated here so tests can decode what the kernels emit)
# ---------------------------------------------------------------------------
def pack_planar32(codes: torch.Tensor) -> torch.Tensor:
    """INT codes [R, K] (K % 32 == 0, values taken mod 16) -> [R, K/2] uint8.
    Within each block of 32 codes, byte j holds code j in its low nibble and code
    16+j in its high nibble."""
    R, K = codes.shape
    c = (codes.to(torch.int16) & 0xF).to(torch.uint8).reshape(R, K // 32, 2, 16)
    return (c[:, :, 0, :] | (c[:, :, 1, :] << 4)).reshape(R, K // 2).contiguous()


def unpack_planar32(packed: torch.Tensor, signed: bool) -> torch.Tensor:
    R, Kh = packed.shape
    p = packed.reshape(R, Kh // 16, 16)
    lo, hi = (p & 0xF).to(torch.int16), (p >> 4).to(torch.int16)
    c = torch.stack([lo, hi], dim=2).reshape(R, Kh * 2)
    if signed:
        c = torch.where(c >= 8, c - 16, c)
    return c


def pack_seq_nibbles(nib: torch.Tensor) -> torch.Tensor:
    """E2M1 nibbles [R, K] -> [R, K/2] uint8; element 2j in the low nibble of byte j."""
    n = nib.to(torch.uint8)
    return (n[:, 0::2] | (n[:, 1::2] << 4)).contiguous()


def unpack_seq_nibbles(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(packed.shape[0], -1)


def sf_atom_offset(row: torch.Tensor, kblk: torch.Tensor, n_kblk64: int) -> torch.Tensor:
    """Byte offset of the scale factor of (row, 16-wide k-block) in the tiled layout the
    block-scaled tensor-core path reads: tiles of 128 rows x 4 scale factors (= 64 K
    elements), 512 bytes each, tile (rb, kb64) at (rb * n_kblk64 + kb64) * 512, and inside
    a tile  (row % 32) * 16 + (row % 128 // 32) * 4 + (kblk % 4)."""
    rb, r = row // 128, row % 128
    kb64, j = kblk // 4, kblk % 4
    return (rb * n_kblk64 + kb64) * 512 + (r % 32) * 16 + (r // 32) * 4 + j


def _sf_n_kb64_pad(nb16: int) -> int:
    """64-element k-blocks per row tile, padded to a multiple of 4 (one pipeline stage = 256 elements)."""
    return ((nb16 + 3) // 4 + 3) // 4 * 4


def sf_tile(sf: torch.Tensor) -> torch.Tensor:
    """[R, K/16] e4m3 bytes (uint8) -> flat tiled buffer (rows padded to 128, zeros in the padding)."""
    R, nb = sf.shape
    Rp, nkb = (R + 127) // 128 * 128, _sf_n_kb64_pad(nb)
    out = torch.zeros(Rp // 128 * nkb * 512, dtype=torch.uint8)
    rr = torch.arange(R).reshape(R, 1).expand(R, nb)
    kk = torch.arange(nb).reshape(1, nb).expand(R, nb)
    out[sf_atom_offset(rr, kk, nkb).reshape(-1)] = sf.reshape(-1)
    return out


def sf_untile(buf: torch.Tensor, R: int, nb: int) -> torch.Tensor:
    nkb = _sf_n_kb64_pad(nb)
    rr = torch.arange(R).reshape(R, 1).expand(R, nb)
    kk = torch.arange(nb).reshape(1, nb).expand(R, nb)
    return buf[sf_atom_offset(rr, kk, nkb).reshape(-1)].reshape(R, nb)


# ---------------------------------------------------------------------------
# synthetic inputs with the stated distributions (stand-ins for calibrated data)
# ---------------------------------------------------------------------------
def random_orthogonal(n: int, gen: torch.Generator) -> torch.Tensor:
    """QR of a seeded Gaussian with the sign fix of utils/hadamard_utils.py:25-28 (fp64)."""
    a = torch.randn(n, n, dtype=torch.float64, generator=gen)
    q, r = torch.linalg.qr(a)
    q = q * torch.sign(torch.diag(r)).unsqueeze(0)
    return q


def synth_activations(M: int, D: int, gen: torch.Generator, rank: int = 32, heavy: int = 8) -> torch.Tensor:
    """N(0,1) plus a planted rank-`rank` subspace with 20x variance and `heavy`
    Student-t(3) channels; bf16 [M, D]."""
    x = torch.randn(M, D, generator=gen)
    rank = min(rank, D)
    v = torch.linalg.qr(torch.randn(D, rank, generator=gen))[0]
    z = torch.randn(M, rank, generator=gen) * math.sqrt(19.0)
    x = x + z @ v.T
    ch = torch.randperm(D, generator=gen)[:heavy]
    num = torch.randn(M, heavy, generator=gen)
    chi = (torch.randn(M, heavy, 3, generator=gen) ** 2).sum(-1) / 3.0
    x[:, ch] = num / chi.sqrt()
    return x.to(torch.bfloat16)
