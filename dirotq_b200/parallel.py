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


class FluxLinearStep:
    """Every wrapped linear of one FLUX.1-dev denoising step (19 double-stream blocks on the image and
    the text stream, 38 single-stream blocks on their concatenation) at a FIXED global batch, split
    over `world` ranks (strong scaling).

    Token rows are independent through a quantised linear, so the attention-side linears (to_q/k/v,
    out-projection) run on this rank's M/world rows with no communication.  The FFN pairs
    (ff.net.0.proj -> GELU -> ff.net.2, and proj_mlp -> GELU -> proj_out.linears.1) run either the
    same way (ffn="dp") or tensor-parallel (ffn="tp"): all-gather the rows, column-split
    up-projection, row-split down-projection without rotation, reduce-scatter of the partial sums
    back to row shards - two NCCL collectives per FFN, none elsewhere.  Weights are synthetic and
    drawn per rank at the slice's shape; equality of a split FFN with the unsplit one is a property
    of the slicing (build_flux_tp_ffn), tested separately.
    """

    def __init__(self, world: int, rank: int, device, batch: int = 4, n_double: int = 19, n_single: int = 38,
                 ffn: str = "tp", quant: str = "int4", seed: int = 3000, k: int = 384):
        from . import dit
        import torch.nn as nn
        assert ffn in ("tp", "dp")
        self.world, self.rank, self.ffn = world, rank, ffn if world > 1 else "dp"
        self.rows = {"img": batch * 4096, "txt": batch * 512, "single": batch * 4608}
        for m in self.rows.values():
            if m % world:
                raise ValueError(f"{m} rows do not split over {world} ranks")
        self.hidden, self.inner = 3072, 12288
        tp = world if self.ffn == "tp" else 1
        tp_slices(self.inner, tp, 0, 64)
        ph = dict(kind="perhead", tail=16, heads=24, head_dim=128)
        attn = [dit.LayerDef(n, 3072, 3072, tail=k) for n in ("attn.to_q", "attn.to_k", "attn.to_v")] + \
               [dit.LayerDef("attn.to_out", 3072, 3072, **ph)]
        up = dit.LayerDef("ffn_up", 3072, self.inner // tp, tail=k)
        down = dit.LayerDef("ffn_down", self.inner // tp, 3072, kind="norot", tail=0, source="ff")
        self.census = []            # (stream, LayerDef at full size) for the operation count
        self.blocks = []            # (stream, [attn wrappers], up, down)
        layers = []
        tree = nn.ModuleList()
        s = seed + 104729 * rank
        for stream, n in (("img", n_double), ("txt", n_double), ("single", n_single)):
            for _ in range(n):
                ws = [dit.make_wrapped_linear(ld, dit.layer_quant(ld, quant), s + i, device) for i, ld in enumerate(attn)]
                for w_ in ws[1:3]:      # to_k, to_v: same input, same rotation as to_q (flux-schnell/model_utils.py:165-178)
                    w_.rotation = ws[0].rotation.clone()
                wu = dit.make_wrapped_linear(up, quant, s + 4, device)
                wd = dit.make_wrapped_linear(down, quant, s + 5, device)
                if self.ffn == "tp" and rank != 0:
                    wd._b200_explicit["bias"] = None        # the bias enters the reduced sum once
                s += 6
                self.blocks.append((stream, ws, wu, wd))
                blk = nn.Module()
                for ld, w_ in zip(attn + [up, down], ws + [wu, wd]):
                    dit._set_nested(blk, ld.name, w_)
                tree.append(blk)
                layers += ws + [wu, wd]
                self.census += [(stream, ld) for ld in attn]
                self.census += [(stream, dit.LayerDef("ffn_up", 3072, self.inner)),
                                (stream, dit.LayerDef("ffn_down", self.inner, 3072))]
        self.layers = tree               # module tree (blocks.i.attn.to_q ...); call order is in self.blocks
        self._flat = layers
        self._gather = {}
        self.fused_gelu = False
        # Tensor-parallel mode: CUDA-event pairs around every collective when `comm_pairs` is a list (bench.py sums
        # them into the NCCL time per step).  In single-stream blocks proj_mlp reads the SAME tokens as to_q / to_k /
        # to_v, so its all-gather does not depend on the attention linears and is issued on a side stream while they
        # run; in double-stream blocks the feed-forward reads what follows the attention, so nothing can be hoisted.
        self.comm_pairs = None
        self.overlap_gather = True
        self._comm_stream = None

    def fuse_gelu(self) -> int:
        """GELU of the FFN pairs into the up-projection's GEMM epilogue (call after the layers are prepared)."""
        n = 0
        for _, _, wu, _ in self.blocks:
            st = getattr(wu, "_b200_state", None)
            if st is None or (st.folded is None and st.fmt.mode != 4):
                return 0
        for _, _, wu, _ in self.blocks:
            wu._b200_state.epilogue_act, wu._b200_state._c = 1, None
            n += 1
        self.fused_gelu = n > 0
        return n

    def fuse_ffn_quantise(self) -> int:
        """The up-projections' epilogues quantise for their un-rotated down-projections (backend.fuse_ffn_quantise);
        the [M, inner] hidden tensor is never written, since only the down-projection reads it here.  Needs
        fuse_gelu first: the hand-off recognises the tensor the up-projection returned."""
        from . import backend
        if not self.fused_gelu:
            return 0
        return backend.fuse_ffn_quantise(pairs=[(wu, wd) for _, _, wu, wd in self.blocks], keep_hidden=False)

    def ops_per_step(self):
        """(linear, rotation) operations of the whole step at the global batch."""
        from . import dit
        lin = sum(dit.linear_ops(ld, self.rows[st]) for st, ld in self.census)
        rot = sum(2.0 * self.rows[st] * 3072 * (128 if ld.kind == "perhead" else 3072)
                  for st, ld in self.census if ld.in_f == 3072)
        return lin, rot

    def kernel_launches_per_step(self) -> int:
        from . import backend
        return sum(backend.kernel_launches(getattr(l, "_b200_state", None), getattr(l, "_b200_w4a16", None)) for l in self._flat)

    def rows_per_rank(self, stream: str) -> int:
        return self.rows[stream] // self.world

    def _buffers(self, x):
        m = x.shape[0]
        key = (m, x.dtype)
        if key not in self._gather:
            self._gather[key] = (torch.empty(self.world * m, self.hidden, dtype=x.dtype, device=x.device),
                                 torch.empty(m, self.hidden, dtype=x.dtype, device=x.device))
        return self._gather[key]

    def _timed(self, fn):
        if self.comm_pairs is None:
            return fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        self.comm_pairs.append((e0, e1))

    def _start_gather(self, x):
        """all-gather of this rank's rows on the side stream; returns the event the main stream waits for."""
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(x.device)
        full, _ = self._buffers(x)
        main = torch.cuda.current_stream(x.device)
        self._comm_stream.wait_stream(main)
        with torch.cuda.stream(self._comm_stream):
            self._timed(lambda: dist.all_gather_into_tensor(full, x.contiguous()))
            done = torch.cuda.Event()
            done.record(self._comm_stream)
        return done

    def _ffn(self, x, wu, wd, gathered=None):
        act = (lambda t: t) if self.fused_gelu else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
        if self.ffn == "dp":
            return wd(act(wu(x)))
        m = x.shape[0]
        full, out = self._buffers(x)
        if gathered is not None:
            torch.cuda.current_stream(x.device).wait_event(gathered)
        else:
            self._timed(lambda: dist.all_gather_into_tensor(full, x.contiguous()))
        part = wd(act(wu(full.unsqueeze(0)))).reshape(self.world * m, self.hidden)
        self._timed(lambda: dist.reduce_scatter_tensor(out, part, op=dist.ReduceOp.SUM))
        return out

    def __call__(self, x_rows: torch.Tensor) -> torch.Tensor:
        """x_rows: this rank's [rows_per_rank("single"), 3072] bf16 rows; image rows first, then text."""
        m_img = self.rows_per_rank("img")
        views = {"img": x_rows[:m_img], "txt": x_rows[m_img:], "single": x_rows}
        y = None
        for stream, ws, wu, wd in self.blocks:
            x = views[stream]
            x3 = x.unsqueeze(0)
            hoist = self.ffn == "tp" and self.overlap_gather and stream == "single"
            gathered = self._start_gather(x) if hoist else None
            for w in ws:
                y = w(x3)
            y = self._ffn(x, wu, wd, gathered) if self.ffn == "tp" else self._ffn(x3, wu, wd)
        return y
