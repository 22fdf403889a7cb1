"""Multi-GPU use of the quantized-linear path: one process per GPU (torchrun), NCCL over NVLink.

The path shards naturally: activations are quantised per token and per group, GEMM rows are
independent, so the image/latent batch is split across ranks with NO collective (data parallel).
Only FLUX-sized FFNs are additionally tensor-parallel: the up-projection is column-split, the
down-projection row-split, followed by ONE all-reduce of the [M, hidden] partial sums.  The reference
has no distributed code at all; its single-GPU forward (dirotq_fused_unrotation_fast.py:56-141) is
what every rank runs on its shard.

Row-splitting a quantised down-projection is exact with respect to the unsplit layer: group
boundaries (64 or 16 channels) never straddle a K-slice, so every rank produces the same codes and
scales the unsplit layer would, and the partial outputs sum to the unsplit output.  A dense online
rotation in front of the down-projection does not row-split (it mixes all K); in tensor-parallel mode
the down-projection therefore runs without rotation, as the reference's own speed path does
(speedup/report_flux_w4a4_no_rot_ffdown.py:10-12).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of `n` items owned by `rank`; remainders go to the lowest ranks."""
    base, rem = divmod(n, world)
    b = rank * base + min(rank, rem)
    return b, b + base + (1 if rank < rem else 0)


def shard_batch(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Data-parallel shard of a [B, T, D] batch along B (no communication)."""
    b, e = shard_range(x.shape[0], world, rank)
    return x[b:e]


def tp_slices(features: int, world: int, rank: int, granule: int = 64) -> Tuple[int, int]:
    """[begin, end) of a tensor-parallel split of `features` that keeps quantisation groups whole."""
    if features % (world * granule) != 0:
        raise ValueError(f"{features} features do not split into {world} slices of whole {granule}-wide groups")
    w = features // world
    return rank * w, (rank + 1) * w


@dataclass
class TPFeedForward:
    """Tensor-parallel FFN: y = down(act(up(x))), up column-split, down row-split, one all-reduce.

    up_fn   : x [M, D]          -> [M, F / world]   (this rank's columns of the up-projection)
    down_fn : h [M, F / world]  -> [M, D] partial   (this rank's K-slice; bias only on rank 0)
    """
    up_fn: Callable[[torch.Tensor], torch.Tensor]
    down_fn: Callable[[torch.Tensor], torch.Tensor]
    act_fn: Callable[[torch.Tensor], torch.Tensor]
    group: Optional[dist.ProcessGroup] = None
    reduce_dtype: Optional[torch.dtype] = None      # e.g. torch.float32 to sum partials in fp32

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        h = self.act_fn(self.up_fn(x))
        y = self.down_fn(h)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            out_dtype = y.dtype
            if self.reduce_dtype is not None and y.dtype != self.reduce_dtype:
                y = y.to(self.reduce_dtype)
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            y = y.to(out_dtype)
        return y


def build_flux_tp_ffn(world: int, rank: int, quant: str = "int4", device="cuda", seed: int = 3000, hidden: int = 3072,
                      inner: int = 12288, k: int = 384) -> TPFeedForward:
    """A FLUX-shaped FFN (3072 -> 12288 GELU-tanh -> 3072) split over `world` ranks, on the CUDA kernels.
    Every rank draws the FULL synthetic weight from the same seed and keeps its slice, so the split
    layer equals the unsplit one."""
    from . import backend, dit
    from .wrapper import ActQuantWrapper
    up_full = dit.make_wrapped_linear(dit.LayerDef("ff.net.0.proj", hidden, inner, tail=k), quant, seed, device)
    down_full = dit.make_wrapped_linear(dit.LayerDef("ff.net.2", inner, hidden, kind="norot", tail=0, source="ff"),
                                        quant, seed + 1, device)
    c0, c1 = tp_slices(inner, world, rank, 64)
    gran = 16 if quant == "nvfp4" else 64

    def slice_rows(ex, r0, r1):      # output-feature slice of an explicit weight
        out = {}
        for key, v in ex.items():
            if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == inner:
                out[key] = v[r0:r1].contiguous()
            else:
                out[key] = v
        return out

    def slice_cols(ex, k0, k1):      # input-feature (K) slice of an explicit weight, whole groups
        out = dict(ex)
        for key in ("codes", "nibbles"):
            if key in ex:
                out[key] = ex[key][:, k0:k1].contiguous()
        for key in ("scales", "scales_e4m3"):
            if key in ex:
                out[key] = ex[key][:, k0 // gran:k1 // gran].contiguous()
        if rank != 0:
            out["bias"] = None
        return out

    import torch.nn as nn
    up = ActQuantWrapper(nn.Linear(hidden, c1 - c0, bias=True, device="meta", dtype=torch.bfloat16))
    up.quantizer = up_full.quantizer
    up.rotation = up_full.rotation
    up._unrot_fused = True
    up._b200_explicit = slice_rows(up_full._b200_explicit, c0, c1)
    down = ActQuantWrapper(nn.Linear(c1 - c0, hidden, bias=True, device="meta", dtype=torch.bfloat16))
    down.quantizer = down_full.quantizer
    down._unrot_fused = True
    down._b200_explicit = slice_cols(down_full._b200_explicit, c0, c1)
    holder = nn.ModuleList([up, down])
    backend.preconvert_rotations_to_device(holder, device)
    gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh")
    return TPFeedForward(lambda x: up(x), lambda h: down(h), gelu)
