"""Host side of the weight packer: from a fused rotated weight (or explicit codes) to the device
buffers the GEMMs read.  Replaces speedup/nunchaku_pack.py (convert_dirotq_low_weight_to_nunchaku,
..._fp4) of the reference; the bit twiddling runs in the CUDA packer (csrc/pack.cu), the offline
grid recovery below stays in PyTorch like the rest of the calibration code.
"""
from __future__ import annotations

import math
import warnings
from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


@dataclass
class GridRecovery:
    scales: torch.Tensor        # fp32 [N, G]
    n_groups: int
    n_lossy: int                # groups whose values are not on a 4-bit grid within tolerance
    max_rel_residual: float


def recover_int4_grid(w_low: torch.Tensor, group: int, rel_tol: float = 2.0 ** -7) -> GridRecovery:
    """Recover per-group scales of an already quantised-and-dequantised weight.

    The reference keeps only ``q * s`` rounded to the model dtype (utils/gptq_utils.py:517,
    utils/quant_utils.py:799).  RTN uses s = amax/7; GPTQ fixes s from the pre-GPTQ weight and may
    use code -8, so amax/8 is tried as well; the scale is then refined by least squares on the
    recovered codes.  Groups that do not land on a grid are counted, never silently accepted.
    """
    w = w_low.float()
    N, K = w.shape
    pad = (-K) % group
    if pad:
        w = torch.nn.functional.pad(w, (0, pad))
    wg = w.reshape(N, -1, group)
    amax = wg.abs().amax(-1, keepdim=True).clamp(min=1e-5)
    best_s, best_r = None, None
    for denom in (7.0, 8.0):
        s0 = amax / denom
        q = torch.clamp(torch.round(wg / s0), -8, 7)
        den = (q * q).sum(-1, keepdim=True)
        s1 = torch.where(den > 0, (wg * q).sum(-1, keepdim=True) / den.clamp(min=1), s0)
        q1 = torch.clamp(torch.round(wg / s1), -8, 7)
        r = ((q1 * s1 - wg).abs().amax(-1, keepdim=True) / amax)
        if best_s is None:
            best_s, best_r = s1, r
        else:
            take = r < best_r
            best_s = torch.where(take, s1, best_s)
            best_r = torch.where(take, r, best_r)
    lossy = int((best_r > rel_tol).sum())
    return GridRecovery(best_s.squeeze(-1).contiguous(), wg.shape[1], lossy, float(best_r.max()))


def convert_dirotq_low_weight_to_b200(w_low: torch.Tensor, group_size: int = 64, scales: Optional[torch.Tensor] = None,
                                      codes: Optional[torch.Tensor] = None, strict: bool = False) -> ops.PackedWeightInt4:
    """INT4 weights of one layer -> packed device buffers.

    Either pass explicit ``codes`` [N, n_low] in [-8, 7] with ``scales`` [N, G], or a dequantised
    weight ``w_low`` whose grid is recovered (see recover_int4_grid)."""
    if codes is not None:
        assert scales is not None
        return ops.pack_weight_int4(codes.float().cuda(), group_size, scales=scales.float().cuda(), w_is_codes=True)
    if scales is None:
        rec = recover_int4_grid(w_low, group_size)
        if rec.n_lossy:
            msg = (f"{rec.n_lossy} of {rec.n_groups * w_low.shape[0]} weight groups are not on a 4-bit grid "
                   f"(max relative residual {rec.max_rel_residual:.3g}); they are re-quantised")
            if strict:
                raise ValueError(msg)
            warnings.warn(msg)
        scales = rec.scales
    return ops.pack_weight_int4(w_low.float().cuda(), group_size, scales=scales.float().cuda())


def pow2_tensor_scale(max_group_scale: float) -> float:
    """Smallest power of two T with max_group_scale / T <= 448 (division by T is exact)."""
    if max_group_scale <= 0:
        return 1.0
    return float(2.0 ** math.ceil(math.log2(max_group_scale / 448.0)))


def convert_dirotq_low_weight_to_b200_fp4(w_low: torch.Tensor, tensor_scale: Optional[float] = None,
                                          nibbles: Optional[torch.Tensor] = None,
                                          scales_e4m3: Optional[torch.Tensor] = None) -> ops.PackedWeightNvfp4:
    """NVFP4 (group 16, UE4M3 group scales, fp32 tensor scale) weights -> packed device buffers."""
    if nibbles is not None:
        assert scales_e4m3 is not None and tensor_scale is not None
        return ops.pack_weight_nvfp4(nibbles.float().cuda(), tensor_scale, scales_e4m3=scales_e4m3.cuda(),
                                     w_is_codes=True)
    if tensor_scale is None:
        K = w_low.shape[1]
        pad = (-K) % 16
        wf = torch.nn.functional.pad(w_low.float(), (0, pad)) if pad else w_low.float()
        smax = float(wf.reshape(w_low.shape[0], -1, 16).abs().amax(-1).max()) / 6.0
        tensor_scale = pow2_tensor_scale(smax)
    return ops.pack_weight_nvfp4(w_low.float().cuda(), tensor_scale)
