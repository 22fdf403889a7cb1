"""Weight-only NVFP4 linear (A16W4) on the B200 kernels.

Mirror of the reference's speedup/weight_only_nvfp4.py: the same class name, constructor helper and
methods (``from_linear``, ``forward``, ``dequant``, ``weight_bytes``), the same two-level quantiser
(:42-72 -- per-output-channel scale, E4M3 micro-scales per 16 weights, first-argmin codes), reproduced
bit for bit by the CUDA packer.  Storage differs on purpose: nibbles are sequential (the order the tensor
core and the dequantiser read), the micro-scales sit in 512-byte tiles, and the per-channel scale is kept
as the fp32 value of the reference's bf16 number.  ``to_reference_buffers`` converts back to the
reference's ``codes`` / ``micro`` / ``gscale`` tensors.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops

_GROUP = 16


class WeightOnlyNVFP4Linear(nn.Module):
    """bf16 activations x NVFP4 weights; forward = dequantise into scratch + bf16 tcgen05 GEMM."""

    def __init__(self, in_features: int, out_features: int, packed: ops.PackedWeightNvfp4, bias=None):
        super().__init__()
        if in_features % 64 or out_features % 8:
            raise ValueError("in_features must be a multiple of 64 and out_features of 8")
        self.in_features, self.out_features = in_features, out_features
        self.packed = packed
        self.bias = None if bias is None else bias.detach().to(device=packed.codes.device, dtype=torch.bfloat16).contiguous()
        self._scratch = None

    @classmethod
    def from_linear(cls, lin: nn.Linear, device="cuda") -> "WeightOnlyNVFP4Linear":
        W = lin.weight.data.to(device=device, dtype=torch.float32)
        return cls(lin.in_features, lin.out_features, ops.pack_weight_nvfp4_rowscale(W),
                   None if lin.bias is None else lin.bias.data)

    def dequant(self) -> torch.Tensor:
        """bf16 [out, in] weight: codebook value x (micro-scale x channel scale), rounded once."""
        return ops.dequant_weight_nvfp4(self.packed)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shp = x.shape
        x2d = x.reshape(-1, shp[-1]).to(torch.bfloat16).contiguous()
        if self._scratch is None:
            self._scratch = torch.empty(self.out_features * self.in_features * 2, dtype=torch.uint8, device=x2d.device)
        y = ops.gemm_w4a16_nvfp4(x2d, self.packed, self.bias, workspace=self._scratch)
        return y.reshape(*shp[:-1], self.out_features).to(x.dtype)

    def weight_bytes(self) -> int:
        # 4-bit codes + one E4M3 byte per 16 weights + a bf16 scale per channel, as the reference counts them
        return self.out_features * self.in_features // 2 + self.out_features * self.in_features // _GROUP + 2 * self.out_features

    def to_reference_buffers(self):
        """(codes [N, K/2] uint8 in the reference's planar order, micro [N, K/16] float8_e4m3fn, gscale [N] bf16)."""
        N, K = self.out_features, self.in_features
        p = self.packed.codes.cpu()[:, : K // 2]
        nib = torch.stack([p & 0xF, p >> 4], dim=-1).reshape(N, K)
        codes = (nib[:, : K // 2] | (nib[:, K // 2:] << 4)).contiguous()
        sf = self.packed.sf.cpu()
        nkb = (self.packed.n_chunks + 3) // 4 * 4
        rows = torch.arange(N).reshape(N, 1)
        kb = torch.arange(K // _GROUP).reshape(1, -1)
        off = ((rows // 128) * nkb + kb // 4) * 512 + (rows % 32) * 16 + (rows % 128 // 32) * 4 + kb % 4
        micro = sf[off.reshape(-1)].reshape(N, K // _GROUP).view(torch.float8_e4m3fn)
        return codes, micro, self.packed.row_scale.cpu()[:N].to(torch.bfloat16)
