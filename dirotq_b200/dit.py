"""Layer census of the DiT families the quantized-linear path runs in, and a builder of
random-initialised wrapped linears with those shapes.

Shapes follow the reference's model adapters (models/pixart-sigma/model_utils.py:164-290,
models/flux-schnell/model_utils.py, models/sana-1.6b/model_utils.py, models/*/config.yaml:6-11):
which linears are wrapped, which rotation they get (hidden [D,D] or per-head [H,d,d]) and how many
PCA coefficients stay 16-bit.  Weights are synthetic (random codes + scales): calibrated checkpoints
are not redistributable.  Every linear is an ActQuantWrapper, run through the patched forward.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from .wrapper import ActQuantWrapper


@dataclass(frozen=True)
class LayerDef:
    name: str
    in_f: int
    out_f: int
    kind: str = "hidden"        # "hidden" | "perhead" | "w4a16" | "norot"
    tail: int = 0               # hidden: total 16-bit channels; perhead: per head
    heads: int = 0
    head_dim: int = 0
    source: str = "x"           # which activation feeds it: "x" (block input) or "ff" (FFN hidden)


def pixart_block(k: int = 64, per_head_out: bool = False) -> List[LayerDef]:
    """One PixArt-Sigma block: hidden 1152, 16 heads x 72, FFN 4608 (config.yaml:6-11).  k = 16-bit
    PCA coefficients of the hidden-rotation layers; ff.net.2 runs W4A16 (activations not quantised)."""
    out_kw = dict(kind="perhead", tail=9, heads=16, head_dim=72) if per_head_out else dict(kind="hidden", tail=k)
    return [
        LayerDef("attn1.to_q", 1152, 1152, tail=k), LayerDef("attn1.to_k", 1152, 1152, tail=k),
        LayerDef("attn1.to_v", 1152, 1152, tail=k), LayerDef("attn1.to_out.0", 1152, 1152, **out_kw),
        LayerDef("attn2.to_q", 1152, 1152, tail=k), LayerDef("attn2.to_out.0", 1152, 1152, **out_kw),
        LayerDef("ff.net.0.proj", 1152, 4608, tail=k),
        LayerDef("ff.net.2", 4608, 1152, kind="w4a16", source="ff"),
    ]


def flux_double_block(k: int = 384, k_down: int = 1536, rotate_down: bool = False,
                      per_head_out: bool = True) -> List[LayerDef]:
    """One FLUX double-stream block, one stream (image and text streams have the same linears, at
    M_img and M_txt rows).  hidden 3072 = 24 heads x 128, MLP 12288.  The K = 12288 down-projection
    runs without a rotation on the speed path (speedup/report_flux_w4a4_no_rot_ffdown.py:10-12);
    the attention out-projection takes a per-head rotation (16 of 128 coefficients per head 16-bit)."""
    down = LayerDef("ff.net.2", 12288, 3072, kind="hidden" if rotate_down else "norot", tail=k_down, source="ff")
    out_kw = dict(kind="perhead", tail=16, heads=24, head_dim=128) if per_head_out else dict(kind="hidden", tail=k)
    return [LayerDef("attn.to_q", 3072, 3072, tail=k), LayerDef("attn.to_k", 3072, 3072, tail=k),
            LayerDef("attn.to_v", 3072, 3072, tail=k), LayerDef("attn.to_out.0", 3072, 3072, **out_kw),
            LayerDef("ff.net.0.proj", 3072, 12288, tail=k), down]


def flux_single_block(k: int = 384, k_down: int = 1536, per_head_out: bool = True) -> List[LayerDef]:
    """One FLUX single-stream block; proj_out is split into its attention part (linears.0) and its
    MLP part (linears.1), as speedup/split_proj_out.py:38-48 does."""
    out_kw = dict(kind="perhead", tail=16, heads=24, head_dim=128) if per_head_out else dict(kind="hidden", tail=k)
    return [LayerDef("attn.to_q", 3072, 3072, tail=k), LayerDef("attn.to_k", 3072, 3072, tail=k),
            LayerDef("attn.to_v", 3072, 3072, tail=k), LayerDef("proj_mlp", 3072, 12288, tail=k),
            LayerDef("proj_out.linears.0", 3072, 3072, **out_kw),
            LayerDef("proj_out.linears.1", 12288, 3072, kind="norot", tail=k_down, source="ff")]


def sana_block(k: int = 320) -> List[LayerDef]:
    """One SANA-1.6B block: hidden 2240, 70 heads x 32; the Mix-FFN convolutions are not quantised."""
    ph = dict(kind="perhead", tail=4, heads=70, head_dim=32)
    return [LayerDef("attn1.to_q", 2240, 2240, tail=k), LayerDef("attn1.to_k", 2240, 2240, tail=k),
            LayerDef("attn1.to_v", 2240, 2240, tail=k), LayerDef("attn1.to_out.0", 2240, 2240, **ph),
            LayerDef("attn2.to_q", 2240, 2240, tail=k), LayerDef("attn2.to_out.0", 2240, 2240, **ph)]


def per_head_nvfp4_ok(ld: LayerDef) -> bool:
    """Whether a per-head layer has a block-16 NVFP4 form (FLUX: 128 - 16 = 112; not PixArt's 63 or SANA's 28)."""
    return ld.kind == "perhead" and ld.head_dim % 16 == 0 and (ld.head_dim - ld.tail) % 16 == 0


def layer_quant(ld: LayerDef, quant: str) -> str:
    """The format a layer runs in under a model-wide choice: per-head layers without an NVFP4 form stay INT4."""
    return "int4" if (quant == "nvfp4" and ld.kind == "perhead" and not per_head_nvfp4_ok(ld)) else quant


def linear_ops(ld: LayerDef, M: int) -> float:
    """Algorithmic operations of the linear itself (4-bit part + 16-bit branch): 2 M N D."""
    return 2.0 * M * ld.in_f * ld.out_f


def rotation_ops(ld: LayerDef, M: int) -> float:
    if ld.kind == "hidden":
        return 2.0 * M * ld.in_f * ld.in_f
    if ld.kind == "perhead":
        return 2.0 * M * ld.heads * ld.head_dim * ld.head_dim
    return 0.0


def _random_orthogonal(n: int, gen: torch.Generator, device) -> torch.Tensor:
    """QR of a seeded Gaussian with the sign fix of the reference (utils/hadamard_utils.py:13-28)."""
    a = torch.randn(n, n, generator=gen, device=device, dtype=torch.float32)
    q, r = torch.linalg.qr(a)
    return q * torch.sign(torch.diagonal(r)).unsqueeze(0)


def make_wrapped_linear(ld: LayerDef, quant: str, seed: int, device="cuda", a_sym: bool = True) -> ActQuantWrapper:
    """quant: "int4" (group 64, W4A4), "int8" (W4A8 asymmetric) or "nvfp4" (group 16, E4M3 scales)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    lin = nn.Linear(ld.in_f, ld.out_f, bias=True, device="meta", dtype=torch.bfloat16)
    w = ActQuantWrapper(lin)
    N, D = ld.out_f, ld.in_f
    bias = (torch.randn(N, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
    if ld.kind == "w4a16":
        w.quantizer.configure(bits=16, groupsize=-1, sym=True)
        if quant == "nvfp4":          # weight-only NVFP4 (the reference's WeightOnlyNVFP4Linear)
            from .pack import pow2_tensor_scale
            nib = torch.randint(0, 16, (N, D), generator=gen, device=dev).to(torch.uint8)
            s_ = torch.exp(torch.randn(N, D // 16, generator=gen, device=dev) * 0.5 - 4.0)
            T = pow2_tensor_scale(float(s_.max()))
            micro = (s_ / T).clamp(min=2.0 ** -9, max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)
            w._b200_explicit = {"nibbles": nib, "scales_e4m3": micro, "tensor_scale": T, "bias": bias}
            return w
        codes = torch.randint(-8, 8, (N, D), generator=gen, device=dev)
        scales = (torch.rand(N, D // 64, generator=gen, device=dev) * 0.015 + 0.005).to(torch.float16).float()
        w._b200_explicit = {"codes": codes, "scales": scales, "bias": bias}
        return w
    if ld.kind == "perhead":
        H, d = ld.heads, ld.head_dim
        w.rotation_per_head = torch.stack([_random_orthogonal(d, gen, dev) for _ in range(H)])
        w.num_heads, w.head_dim = H, d
        n_low, group, tail_total = H * (d - ld.tail), d - ld.tail, H * ld.tail
    else:
        if ld.kind == "hidden":
            w.rotation = _random_orthogonal(D, gen, dev)
        tail_total = ld.tail
        n_low = D - ld.tail
        group = 16 if quant == "nvfp4" else 64
    w._unrot_fused = True
    w_tail = (torch.randn(N, tail_total, generator=gen, device=dev) * 0.02) if tail_total else None
    if quant == "nvfp4":
        assert ld.kind != "perhead" or per_head_nvfp4_ok(ld), "per-head NVFP4 needs head_dim and head_dim - tail in multiples of 16"
        w.quantizer.configure(bits=4, groupsize=16, high_bits_length=ld.tail, quant_dtype="nvfp4")
        nib = torch.randint(0, 16, (N, n_low), generator=gen, device=dev).to(torch.uint8)
        s = torch.exp(torch.randn(N, (n_low + 15) // 16, generator=gen, device=dev) * 0.5 - 4.0)
        from .pack import pow2_tensor_scale
        T = pow2_tensor_scale(float(s.max()))
        micro = (s / T).clamp(min=2.0 ** -9, max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        w._b200_explicit = {"nibbles": nib, "scales_e4m3": micro, "tensor_scale": T, "bias": bias}
    else:
        bits = 8 if quant == "int8" else 4
        w.quantizer.configure(bits=bits, groupsize=group, sym=(a_sym and bits == 4), high_bits_length=ld.tail,
                              quant_dtype="int")
        codes = torch.randint(-8, 8, (N, n_low), generator=gen, device=dev)
        scales = (torch.rand(N, (n_low + group - 1) // group, generator=gen, device=dev) * 0.015 + 0.005)
        w._b200_explicit = {"codes": codes, "scales": scales.to(torch.float16).float(), "bias": bias}
    if w_tail is not None:
        w._b200_explicit["w_tail"] = w_tail
    return w


class GeluProj(nn.Module):
    """Mirror of diffusers.models.activations.GELU as the reference's transformers use it for ff.net.0:
    a projection followed by GELU (here always the tanh form); `proj` is the wrapped linear."""

    def __init__(self, proj: nn.Module, approximate: str = "tanh"):
        super().__init__()
        self.proj = proj
        self.approximate = approximate

    def forward(self, hidden_states):
        return torch.nn.functional.gelu(self.proj(hidden_states), approximate=self.approximate)


def _set_nested(root: nn.Module, dotted: str, leaf: nn.Module):
    """root.a.b.c = leaf for dotted == "a.b.c", creating plain container modules on the way."""
    parts = dotted.split(".")
    m = root
    for p in parts[:-1]:
        if not hasattr(m, p):
            m.add_module(p, nn.Module())
        m = getattr(m, p)
    m.add_module(parts[-1], leaf)


class LinearPathStep(nn.Module):
    """All wrapped linears of one denoising step of a DiT, run in block order on the block input
    (and, for FFN down-projections, on the activated up-projection output).  Attention, norms and
    modulation are outside the quantized-linear path and are not part of this step."""

    def __init__(self, block: List[LayerDef], n_blocks: int, quant: str, device="cuda", seed: int = 1000,
                 a_sym: bool = True):
        super().__init__()
        self.block = block
        self.n_blocks = n_blocks
        self.blocks = nn.ModuleList()     # module tree with the reference's names (blocks.3.attn1.to_q ...)
        self.layers = []                  # the same wrappers in call order
        self.heads = {}                   # index in self.layers -> GeluProj module that owns that wrapper
        for b in range(n_blocks):
            blk = nn.Module()
            qkv_rotation = {}
            for i, ld in enumerate(block):
                w = make_wrapped_linear(ld, layer_quant(ld, quant), seed + b * len(block) + i, device, a_sym)
                # to_q / to_k / to_v of one attention see the same input and get the same rotation
                # (evec @ R1 of one basis: models/pixart-sigma/model_utils.py:84-92, flux-schnell:165-178)
                parent, _, leaf = ld.name.rpartition(".")
                if leaf in ("to_q", "to_k", "to_v") and ld.kind == "hidden":
                    if parent in qkv_rotation:
                        w.rotation = qkv_rotation[parent].clone()
                    else:
                        qkv_rotation[parent] = w.rotation
                if ld.out_f > ld.in_f:
                    head = GeluProj(w)                    # ff.net.0 = GELU(proj(x)), as in the reference models
                    _set_nested(blk, ld.name.rsplit(".", 1)[0] if ld.name.endswith(".proj") else ld.name + "_act", head)
                    self.heads[len(self.layers)] = head
                else:
                    _set_nested(blk, ld.name, w)
                self.layers.append(w)
            self.blocks.append(blk)

    def ops_per_step(self, M: int):
        lin = sum(linear_ops(ld, M) for ld in self.block) * self.n_blocks
        rot = sum(rotation_ops(ld, M) for ld in self.block) * self.n_blocks
        return lin, rot

    def kernel_launches_per_step(self) -> int:
        """Library kernels per step: rotate/quantise (or weight dequantise) + GEMM per linear, plus the
        scale-folding kernel of the tensor-rate INT4 GEMM where a layer uses it."""
        from . import backend
        return sum(backend.kernel_launches(getattr(lyr, "_b200_state", None), getattr(lyr, "_b200_w4a16", None)) for lyr in self.layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = x
        nb = len(self.block)
        for b in range(self.n_blocks):
            ff = None
            for i, ld in enumerate(self.block):
                lyr = self.layers[b * nb + i]
                if ld.source == "ff":
                    y = lyr(ff)
                elif b * nb + i in self.heads:
                    ff = y = self.heads[b * nb + i](x)        # projection + GELU (fused into the GEMM when enabled)
                else:
                    y = lyr(x)
        return y


class GraphedCall:
    """fn() captured once into a CUDA graph and replayed: for steps whose kernels are short enough that launching them
    from Python bounds the step (a batch shard of one sample per GPU: the model-shaped PixArt step is 30 % faster replayed
    than launched).  fn must be a pure function of device tensors that stay where they are (inputs, weights, the layers'
    workspaces, all allocated by an earlier call); it is called once on a side stream first, so that lazily built state
    (resident weight panels, workspaces) exists before the capture.  The status watch of the forward is off during the
    capture (an event query cannot be captured); call ops.check_status() after replays instead."""

    def __init__(self, fn):
        from . import backend
        self.fn, self.graph, self.out = fn, None, None
        saved = backend.WATCH_STATUS
        backend.WATCH_STATUS = False
        try:
            cur = torch.cuda.current_stream()
            side = torch.cuda.Stream()
            side.wait_stream(cur)
            with torch.cuda.stream(side), torch.no_grad():
                fn()
            cur.wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph), torch.no_grad():
                self.out = fn()
            self.graph = graph
        finally:
            backend.WATCH_STATUS = saved

    def __call__(self):
        self.graph.replay()
        return self.out


class HostStreamedStep:
    """Runs a step whose input and output live in pinned host memory: the host -> device copy of call i + 1 and the
    device -> host copy of call i run on side streams while the kernels of the neighbouring calls execute (two
    device input buffers; stream-ordered with events; every call copies its own input and its own result)."""

    def __init__(self, step, x_host: torch.Tensor, y_host: torch.Tensor, device):
        assert x_host.is_pinned() and y_host.is_pinned()
        self.step, self.x_host, self.y_host = step, x_host, y_host
        self.dev = torch.device(device)
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self.x_dev = [torch.empty(x_host.shape, dtype=x_host.dtype, device=self.dev) for _ in range(2)]
        self.in_ready = [torch.cuda.Event() for _ in range(2)]
        self.in_free = [torch.cuda.Event() for _ in range(2)]
        self.out_done = torch.cuda.Event()
        self.out_free = [torch.cuda.Event() for _ in range(2)]
        self.replay = None
        self.i = 0
        main = torch.cuda.current_stream(self.dev)
        for e in self.in_free + self.out_free:
            e.record(main)
        self.out_done.record(main)

    def enable_graphs(self):
        """Replay the step from a CUDA graph, one per input buffer (small batches: Python's launch cost shows).  The
        result of a replay lives in the graph's own memory; it is overwritten two calls later, after its copy to the
        host has completed."""
        self.replay = [GraphedCall(lambda b=b: self.step(self.x_dev[b])) for b in range(2)]

    def __call__(self):
        b = self.i & 1
        self.i += 1
        main = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.in_free[b])            # the kernels that last read this buffer are done
            self.x_dev[b].copy_(self.x_host, non_blocking=True)
            self.in_ready[b].record(self.s_in)
        main.wait_event(self.in_ready[b])
        if self.replay is not None:
            main.wait_event(self.out_free[b])                # the host copy of this graph's previous result is done
            y = self.replay[b]()
        else:
            y = self.step(self.x_dev[b])
        self.in_free[b].record(main)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            if self.replay is None:
                y.record_stream(self.s_out)
            self.y_host.copy_(y.reshape(self.y_host.shape), non_blocking=True)
            self.out_done.record(self.s_out)
            self.out_free[b].record(self.s_out)
        return y

    def finish(self):
        """Make the calling stream wait for the last result copy (call before reading y_host or stopping a timer)."""
        torch.cuda.current_stream(self.dev).wait_event(self.out_done)
