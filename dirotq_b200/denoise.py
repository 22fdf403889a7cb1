"""Model-shaped denoising steps: the wrapped linears in the dataflow they are called in.

The reference's hot loop is ``pipe.transformer(...)`` once per denoising step (apply_dirotq.py:79-125): every
wrapped linear is fed by its block's real dataflow -- norm / modulation -> q, k, v -> attention -> out-projection ->
feed-forward, with residuals and chaining from block to block.  The blocks below reproduce that dataflow for the
three DiT families of the reference with random-initialised weights of the models' shapes (checkpoints are not
redistributable): which linears are wrapped, which rotation they get and which layers stay 16-bit follow the
reference's adapters (models/pixart-sigma/model_utils.py:60-290, models/flux-schnell/model_utils.py:150-330 and
speedup/report_flux_w4a4_no_rot_ffdown.py:192-296, models/sana-1.6b/model_utils.py, models/*/config.yaml).

Everything that is not a wrapped linear -- layer / RMS norms, adaLN modulation, rotary embedding, softmax or linear
attention, depthwise convolution, residual adds -- is plain PyTorch in bf16: it lies outside the quantized-linear
path and is here so that the path can be timed, and checked, where it runs.  Module names mirror diffusers'
(attn1.to_q, ff.net.0.proj, attn.add_q_proj ...), so that backend.share_sibling_activations and
backend.fuse_gelu_modules find their patterns as they do in the reference's transformers.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .dit import GeluProj, LayerDef, layer_quant, linear_ops, make_wrapped_linear, rotation_ops
from .wrapper import ActQuantWrapper


# The row-wise passes between the wrapped linears (modulated LayerNorm, gated residuals, q / k RMSNorm + rotary embedding)
# run as single-pass kernels of the library (csrc/glue.cu) by default; False keeps them as chains of PyTorch elementwise
# kernels, the form the reference's model forwards have (speedup/report_flux_w4a4_no_rot_ffdown.py:199-252).
FUSED_GLUE = True


def _ln_mod(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    if FUSED_GLUE and x.is_cuda:
        from . import ops
        return ops.layernorm_modulate(x.contiguous(), scale, shift)
    return F.layer_norm(x, (x.shape[-1],), eps=1e-6) * (1 + scale) + shift


def _gated(h: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None):
    if FUSED_GLUE and h.is_cuda:
        from . import ops
        return ops.gated_residual(h.contiguous(), y, gate, y2)
    y = y if y2 is None else y + y2
    return h + (y if gate is None else gate * y)


def _heads(x: torch.Tensor, h: int) -> torch.Tensor:
    B, T, C = x.shape
    return x.view(B, T, h, C // h).transpose(1, 2)


def _merge(x: torch.Tensor) -> torch.Tensor:
    B, H, T, d = x.shape
    return x.transpose(1, 2).reshape(B, T, H * d)


def _bf16_linear(in_f: int, out_f: int, gen: torch.Generator, device, bias: bool = True) -> nn.Linear:
    """A layer the reference leaves 16-bit (cross-attention keys / values, modulation projections)."""
    lin = nn.Linear(in_f, out_f, bias=bias, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_((torch.randn(out_f, in_f, generator=gen, device=device) / math.sqrt(in_f)).to(torch.bfloat16))
        if bias:
            lin.bias.zero_()
    for p_ in lin.parameters():
        p_.requires_grad_(False)
    return lin


class _Census:
    """Bookkeeping shared by the blocks: the LayerDef of every wrapped linear and how many rows it sees."""

    def _init_census(self):
        self.census = []          # (LayerDef, rows-per-sample factor name)

    def _wrap(self, ld: LayerDef, quant: str, seed: int, device, rows: str = "img") -> ActQuantWrapper:
        w = make_wrapped_linear(ld, layer_quant(ld, quant), seed, device)     # PixArt / SANA per-head layers stay INT4
        self.census.append((ld, rows))
        return w


class _Attention(nn.Module):
    """Holder with diffusers' attribute names (to_q, to_k, to_v, to_out[0], optional add_* projections)."""


def _share_rotation(ws):
    """to_q / to_k / to_v of one attention are rotated by the same matrix (evec @ R1 of one basis:
    models/pixart-sigma/model_utils.py:84-92, models/flux-schnell/model_utils.py:165-190)."""
    for w in ws[1:]:
        w.rotation = ws[0].rotation.clone()


# ---------------------------------------------------------------------------------------------------------------------
# PixArt-Sigma
# ---------------------------------------------------------------------------------------------------------------------
class PixArtBlock(nn.Module, _Census):
    """diffusers BasicTransformerBlock in its ada_norm_single form (PixArt-Sigma): hidden 1152, 16 heads x 72,
    self-attention, cross-attention to the text tokens (keys / values 16-bit, not wrapped:
    models/pixart-sigma/config.yaml:32-33), GELU-tanh feed-forward 1152 -> 4608 -> 1152 whose down-projection
    runs W4A16 (--skip-quant-layers ff.net.2)."""

    def __init__(self, quant: str, seed: int, device, k: int = 64, per_head_out: bool = False, dim: int = 1152,
                 heads: int = 16, inner: int = 4608):
        super().__init__()
        self._init_census()
        self.dim, self.heads = dim, heads
        gen = torch.Generator(device=device).manual_seed(seed)
        out_kw = dict(kind="perhead", tail=9, heads=heads, head_dim=dim // heads) if per_head_out else dict(tail=k)
        self.attn1, self.attn2 = _Attention(), _Attention()
        qkv = [self._wrap(LayerDef(f"attn1.{n}", dim, dim, tail=k), quant, seed + i, device) for i, n in
               enumerate(("to_q", "to_k", "to_v"))]
        _share_rotation(qkv)
        self.attn1.to_q, self.attn1.to_k, self.attn1.to_v = qkv
        self.attn1.to_out = nn.ModuleList([self._wrap(LayerDef("attn1.to_out.0", dim, dim, **out_kw), quant, seed + 3, device)])
        self.attn2.to_q = self._wrap(LayerDef("attn2.to_q", dim, dim, tail=k), quant, seed + 4, device)
        self.attn2.to_k = _bf16_linear(dim, dim, gen, device)
        self.attn2.to_v = _bf16_linear(dim, dim, gen, device)
        self.attn2.to_out = nn.ModuleList([self._wrap(LayerDef("attn2.to_out.0", dim, dim, **out_kw), quant, seed + 5, device)])
        self.ff = nn.Module()
        up = self._wrap(LayerDef("ff.net.0.proj", dim, inner, tail=k), quant, seed + 6, device)
        down = self._wrap(LayerDef("ff.net.2", inner, dim, kind="w4a16", source="ff"), quant, seed + 7, device)
        self.ff.net = nn.ModuleList([GeluProj(up), nn.Identity(), down])
        self.scale_shift_table = nn.Parameter((torch.randn(6, dim, generator=gen, device=device) / math.sqrt(dim))
                                              .to(torch.bfloat16), requires_grad=False)

    def forward(self, h: torch.Tensor, enc: torch.Tensor, temb: torch.Tensor) -> torch.Tensor:
        """h [B, T, D] image tokens, enc [B, S, D] projected text tokens, temb [B, 6 D] adaLN-single embedding."""
        B, _, D = h.shape
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = (self.scale_shift_table[None] + temb.reshape(B, 6, D)).chunk(6, dim=1)
        n = _ln_mod(h, sc_a, sh_a)
        a = self.attn1
        o = F.scaled_dot_product_attention(_heads(a.to_q(n), self.heads), _heads(a.to_k(n), self.heads),
                                           _heads(a.to_v(n), self.heads))
        h = _gated(h, a.to_out[0](_merge(o)), g_a)
        c = self.attn2                                       # ada_norm_single: no norm in front of the cross-attention
        o = F.scaled_dot_product_attention(_heads(c.to_q(h), self.heads), _heads(c.to_k(enc), self.heads),
                                           _heads(c.to_v(enc), self.heads))
        h = _gated(h, c.to_out[0](_merge(o)))
        n = _ln_mod(h, sc_m, sh_m)
        return _gated(h, self.ff.net[2](self.ff.net[0](n)), g_m)


# ---------------------------------------------------------------------------------------------------------------------
# FLUX.1
# ---------------------------------------------------------------------------------------------------------------------
def rope_tables(T: int, d: int, device, theta: float = 10000.0):
    """cos / sin [T, d] of a 1-D rotary embedding (FLUX uses three axes; one is enough for the cost and the dataflow)."""
    pos = torch.arange(T, device=device, dtype=torch.float32)
    freq = theta ** (-torch.arange(0, d, 2, device=device, dtype=torch.float32) / d)
    ang = torch.outer(pos, freq).repeat_interleave(2, dim=1)
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    xr = torch.stack([-x[..., 1::2], x[..., 0::2]], dim=-1).flatten(-2)
    return x * cos + xr * sin


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class _FluxAttention(_Attention):
    pass


class FluxDoubleBlock(nn.Module, _Census):
    """diffusers FluxTransformerBlock: image and text streams with their own adaLN-Zero modulation, q / k / v
    projections (RMS-normalised per head, rotary), ONE joint attention over text + image tokens, out-projections,
    and GELU-tanh feed-forwards 3072 -> 12288 -> 3072.  Per-head rotation on the out-projections and no rotation in
    front of the K = 12288 down-projections, as the measured configuration has them."""

    def __init__(self, quant: str, seed: int, device, k: int = 384, dim: int = 3072, heads: int = 24, inner: int = 12288,
                 per_head_out: bool = True):
        super().__init__()
        self._init_census()
        self.dim, self.heads = dim, heads
        d = dim // heads
        gen = torch.Generator(device=device).manual_seed(seed)
        out_kw = dict(kind="perhead", tail=16, heads=heads, head_dim=d) if per_head_out else dict(tail=k)
        a = self.attn = _FluxAttention()
        img = [self._wrap(LayerDef(f"attn.{n}", dim, dim, tail=k), quant, seed + i, device) for i, n in
               enumerate(("to_q", "to_k", "to_v"))]
        txt = [self._wrap(LayerDef(f"attn.{n}", dim, dim, tail=k), quant, seed + 3 + i, device, rows="txt") for i, n in
               enumerate(("add_q_proj", "add_k_proj", "add_v_proj"))]
        _share_rotation(img)
        _share_rotation(txt)
        a.to_q, a.to_k, a.to_v = img
        a.add_q_proj, a.add_k_proj, a.add_v_proj = txt
        a.to_out = nn.ModuleList([self._wrap(LayerDef("attn.to_out.0", dim, dim, **out_kw), quant, seed + 6, device)])
        a.to_add_out = self._wrap(LayerDef("attn.to_add_out", dim, dim, **out_kw), quant, seed + 7, device, rows="txt")
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            setattr(a, n, nn.Parameter(torch.ones(d, device=device, dtype=torch.bfloat16), requires_grad=False))
        self.ff, self.ff_context = nn.Module(), nn.Module()
        for j, (ff, rows) in enumerate(((self.ff, "img"), (self.ff_context, "txt"))):
            up = self._wrap(LayerDef("ff.net.0.proj", dim, inner, tail=k), quant, seed + 8 + 2 * j, device, rows=rows)
            down = self._wrap(LayerDef("ff.net.2", inner, dim, kind="norot", tail=0, source="ff"), quant, seed + 9 + 2 * j,
                              device, rows=rows)
            ff.net = nn.ModuleList([GeluProj(up), nn.Identity(), down])
        self.norm1 = _bf16_linear(dim, 6 * dim, gen, device)           # AdaLayerNormZero's projection of the embedding
        self.norm1_context = _bf16_linear(dim, 6 * dim, gen, device)

    def forward(self, img: torch.Tensor, txt: torch.Tensor, temb: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        D, H, a = self.dim, self.heads, self.attn
        mi = self.norm1(F.silu(temb))[:, None].chunk(6, dim=-1)
        mt = self.norm1_context(F.silu(temb))[:, None].chunk(6, dim=-1)
        ni = _ln_mod(img, mi[1], mi[0])
        nt = _ln_mod(txt, mt[1], mt[0])
        S = txt.shape[1]
        if FUSED_GLUE and img.is_cuda:
            # text rows then image rows of q / k / v, normalised and rotated, straight into token-major buffers: no
            # concatenation, and the attention output comes back in the layout the out-projections read
            from . import ops
            B, T = img.shape[0], img.shape[1]
            bufs = tuple(torch.empty(B, S + T, H, D // H, dtype=img.dtype, device=img.device) for _ in range(3))
            ops.qkv_norm_rope(a.add_q_proj(nt), a.add_k_proj(nt), a.add_v_proj(nt), H, a.norm_added_q, a.norm_added_k,
                              cos, sin, out=bufs, t0=0)
            ops.qkv_norm_rope(a.to_q(ni), a.to_k(ni), a.to_v(ni), H, a.norm_q, a.norm_k, cos, sin, out=bufs, t0=S)
            o = _merge(F.scaled_dot_product_attention(*(t.transpose(1, 2) for t in bufs)))
        else:
            q = torch.cat([_rms(_heads(a.add_q_proj(nt), H), a.norm_added_q), _rms(_heads(a.to_q(ni), H), a.norm_q)], dim=2)
            kk = torch.cat([_rms(_heads(a.add_k_proj(nt), H), a.norm_added_k), _rms(_heads(a.to_k(ni), H), a.norm_k)], dim=2)
            v = torch.cat([_heads(a.add_v_proj(nt), H), _heads(a.to_v(ni), H)], dim=2)
            o = _merge(F.scaled_dot_product_attention(_rope(q, cos, sin), _rope(kk, cos, sin), v))
        txt = _gated(txt, a.to_add_out(o[:, :S]), mt[2])
        img = _gated(img, a.to_out[0](o[:, S:]), mi[2])
        ni = _ln_mod(img, mi[4], mi[3])
        nt = _ln_mod(txt, mt[4], mt[3])
        img = _gated(img, self.ff.net[2](self.ff.net[0](ni)), mi[5])
        txt = _gated(txt, self.ff_context.net[2](self.ff_context.net[0](nt)), mt[5])
        return img, txt


class FluxSingleBlock(nn.Module, _Census):
    """diffusers FluxSingleTransformerBlock with proj_out split into its attention half (linears.0) and its MLP half
    (linears.1), as the reference's split_proj_out does (models/flux-schnell/split_proj_out.py:22-71): q / k / v and
    proj_mlp read the same modulated tokens, attention and GELU(proj_mlp) feed the two halves, one gated residual."""

    def __init__(self, quant: str, seed: int, device, k: int = 384, dim: int = 3072, heads: int = 24, inner: int = 12288,
                 per_head_out: bool = True):
        super().__init__()
        self._init_census()
        self.dim, self.heads = dim, heads
        d = dim // heads
        gen = torch.Generator(device=device).manual_seed(seed)
        out_kw = dict(kind="perhead", tail=16, heads=heads, head_dim=d) if per_head_out else dict(tail=k)
        a = self.attn = _FluxAttention()
        qkv = [self._wrap(LayerDef(f"attn.{n}", dim, dim, tail=k), quant, seed + i, device) for i, n in
               enumerate(("to_q", "to_k", "to_v"))]
        _share_rotation(qkv)
        a.to_q, a.to_k, a.to_v = qkv
        a.norm_q = nn.Parameter(torch.ones(d, device=device, dtype=torch.bfloat16), requires_grad=False)
        a.norm_k = nn.Parameter(torch.ones(d, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.proj_mlp_act = GeluProj(self._wrap(LayerDef("proj_mlp", dim, inner, tail=k), quant, seed + 3, device))
        self.proj_out = nn.Module()
        self.proj_out.linears = nn.ModuleList([
            self._wrap(LayerDef("proj_out.linears.0", dim, dim, **out_kw), quant, seed + 4, device),
            self._wrap(LayerDef("proj_out.linears.1", inner, dim, kind="norot", tail=0, source="ff"), quant, seed + 5, device)])
        self.norm = _bf16_linear(dim, 3 * dim, gen, device)

    def forward(self, x: torch.Tensor, temb: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        D, H, a = self.dim, self.heads, self.attn
        shift, scale, gate = self.norm(F.silu(temb))[:, None].chunk(3, dim=-1)
        n = _ln_mod(x, scale, shift)
        if FUSED_GLUE and x.is_cuda:
            from . import ops
            q, kk, v = ops.qkv_norm_rope(a.to_q(n), a.to_k(n), a.to_v(n), H, a.norm_q, a.norm_k, cos, sin)
            o = _merge(F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), v.transpose(1, 2)))
        else:
            q, kk, v = _rms(_heads(a.to_q(n), H), a.norm_q), _rms(_heads(a.to_k(n), H), a.norm_k), _heads(a.to_v(n), H)
            o = _merge(F.scaled_dot_product_attention(_rope(q, cos, sin), _rope(kk, cos, sin), v))
        return _gated(x, self.proj_out.linears[0](o), gate, self.proj_out.linears[1](self.proj_mlp_act(n)))


# ---------------------------------------------------------------------------------------------------------------------
# SANA
# ---------------------------------------------------------------------------------------------------------------------
class SanaBlock(nn.Module, _Census):
    """SANA-1.6B block: ReLU linear self-attention (70 heads x 32), cross-attention to the text tokens, and the
    Mix-FFN (1x1 convolution 2240 -> 11200, 3x3 depthwise convolution, gated SiLU, 1x1 convolution 5600 -> 2240),
    which the reference does not quantise (models/sana-1.6b/config.yaml:10-11, 34)."""

    def __init__(self, quant: str, seed: int, device, k: int = 320, dim: int = 2240, heads: int = 70, ffn_ratio: float = 2.5):
        super().__init__()
        self._init_census()
        self.dim, self.heads = dim, heads
        d = dim // heads
        gen = torch.Generator(device=device).manual_seed(seed)
        ph = dict(kind="perhead", tail=4, heads=heads, head_dim=d)
        self.attn1, self.attn2 = _Attention(), _Attention()
        qkv = [self._wrap(LayerDef(f"attn1.{n}", dim, dim, tail=k), quant, seed + i, device) for i, n in
               enumerate(("to_q", "to_k", "to_v"))]
        _share_rotation(qkv)
        self.attn1.to_q, self.attn1.to_k, self.attn1.to_v = qkv
        self.attn1.to_out = nn.ModuleList([self._wrap(LayerDef("attn1.to_out.0", dim, dim, **ph), quant, seed + 3, device)])
        self.attn2.to_q = self._wrap(LayerDef("attn2.to_q", dim, dim, tail=k), quant, seed + 4, device)
        self.attn2.to_k = _bf16_linear(dim, dim, gen, device)
        self.attn2.to_v = _bf16_linear(dim, dim, gen, device)
        self.attn2.to_out = nn.ModuleList([self._wrap(LayerDef("attn2.to_out.0", dim, dim, **ph), quant, seed + 5, device)])
        inner = int(dim * ffn_ratio)
        self.ff = nn.Module()
        self.ff.conv_inverted = nn.Conv2d(dim, 2 * inner, 1, device=device, dtype=torch.bfloat16)
        self.ff.conv_depth = nn.Conv2d(2 * inner, 2 * inner, 3, padding=1, groups=2 * inner, device=device, dtype=torch.bfloat16)
        self.ff.conv_point = nn.Conv2d(inner, dim, 1, bias=False, device=device, dtype=torch.bfloat16)
        for p_ in self.ff.parameters():
            p_.requires_grad_(False)
        self.scale_shift_table = nn.Parameter((torch.randn(6, dim, generator=gen, device=device) / math.sqrt(dim))
                                              .to(torch.bfloat16), requires_grad=False)

    def _linear_attention(self, n: torch.Tensor) -> torch.Tensor:
        a, H = self.attn1, self.heads
        q, k, v = F.relu(_heads(a.to_q(n), H)).float(), F.relu(_heads(a.to_k(n), H)).float(), _heads(a.to_v(n), H).float()
        v1 = F.pad(v, (0, 1), value=1.0)                       # the extra column accumulates the normaliser
        o = q @ (k.transpose(-1, -2) @ v1)
        return _merge((o[..., :-1] / (o[..., -1:] + 1e-15)).to(n.dtype))

    def forward(self, h: torch.Tensor, enc: torch.Tensor, temb: torch.Tensor) -> torch.Tensor:
        B, T, D = h.shape
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = (self.scale_shift_table[None] + temb.reshape(B, 6, D)).chunk(6, dim=1)
        n = _ln_mod(h, sc_a, sh_a)
        h = _gated(h, self.attn1.to_out[0](self._linear_attention(n)), g_a)
        c, H = self.attn2, self.heads
        o = F.scaled_dot_product_attention(_heads(c.to_q(h), H), _heads(c.to_k(enc), H), _heads(c.to_v(enc), H))
        h = _gated(h, c.to_out[0](_merge(o)))
        n = _ln_mod(h, sc_m, sh_m)
        side = int(math.isqrt(T))
        f = self.ff.conv_depth(F.silu(self.ff.conv_inverted(n.transpose(1, 2).reshape(B, D, side, side))))
        f, gate = f.chunk(2, dim=1)
        f = self.ff.conv_point(f * F.silu(gate)).reshape(B, D, T).transpose(1, 2)
        return _gated(h, f, g_m)


# ---------------------------------------------------------------------------------------------------------------------
# whole steps
# ---------------------------------------------------------------------------------------------------------------------
class DenoiseStep(nn.Module):
    """One denoising step of a model-shaped transformer: `family` in {"pixart", "flux", "sana"}, blocks chained as the
    models chain them.  forward() takes this rank's batch shard; inputs are created by ``example_inputs``."""

    SHAPES = {"pixart": dict(dim=1152, tokens=4096, text=300), "sana": dict(dim=2240, tokens=1024, text=300),
              "flux": dict(dim=3072, tokens=4096, text=512)}

    def __init__(self, family: str, quant: str, device, n_blocks: Optional[int] = None, seed: int = 5000,
                 prepare: bool = False, **block_kw):
        """prepare=True packs every block for the device as soon as it is built and drops the synthetic dense data
        (explicit codes, fp32 rotations), so that a whole 57-block FLUX step never holds more than one block of it;
        the forward must be patched (backend.patch_forward) before the step is called either way."""
        super().__init__()
        self.family, self.quant = family, quant
        dev = torch.device(device)

        def build(cls, i):
            blk = cls(quant, seed + 16 * i, dev, **block_kw)
            if prepare:
                import contextlib, io
                from . import backend
                with contextlib.redirect_stdout(io.StringIO()):
                    backend.preconvert_rotations_to_device(blk, dev)
                for w in blk.modules():
                    if isinstance(w, ActQuantWrapper):
                        w._b200_explicit = None
                        w.rotation = w.rotation_per_head = None
            return blk

        if family == "pixart":
            n = 28 if n_blocks is None else n_blocks
            self.blocks = nn.ModuleList([build(PixArtBlock, i) for i in range(n)])
        elif family == "sana":
            n = 20 if n_blocks is None else n_blocks
            self.blocks = nn.ModuleList([build(SanaBlock, i) for i in range(n)])
        elif family == "flux":
            n = 19 if n_blocks is None else n_blocks           # double-stream blocks; twice as many single-stream ones
            self.blocks = nn.ModuleList([build(FluxDoubleBlock, i) for i in range(n)])
            self.single_blocks = nn.ModuleList([build(FluxSingleBlock, n + i) for i in range(2 * n)])
        else:
            raise ValueError(family)
        self.shape = self.SHAPES[family]

    def example_inputs(self, batch: int, device, seed: int = 0, tokens: Optional[int] = None, text: Optional[int] = None):
        from .synth import synth_activations
        s = self.shape
        T, S, D = tokens or s["tokens"], text or s["text"], s["dim"]
        g = torch.Generator().manual_seed(seed)
        h = synth_activations(batch * T, D, g).reshape(batch, T, D).to(device)
        enc = synth_activations(batch * S, D, g).reshape(batch, S, D).to(device)
        n_mod = D if self.family == "flux" else 6 * D
        temb = (torch.randn(batch, n_mod, generator=g) * 0.1).to(torch.bfloat16).to(device)
        return h, enc, temb

    def forward(self, h: torch.Tensor, enc: torch.Tensor, temb: torch.Tensor) -> torch.Tensor:
        if self.family != "flux":
            for blk in self.blocks:
                h = blk(h, enc, temb)
            return h
        S = enc.shape[1]
        cos, sin = rope_tables(S + h.shape[1], self.shape["dim"] // 24, h.device)
        img, txt = h, enc
        for blk in self.blocks:
            img, txt = blk(img, txt, temb, cos, sin)
        x = torch.cat([txt, img], dim=1)
        for blk in self.single_blocks:
            x = blk(x, temb, cos, sin)
        return x[:, S:]

    # ---- accounting ------------------------------------------------------------------------------------------------
    def all_blocks(self):
        return list(self.blocks) + list(getattr(self, "single_blocks", []))

    def wrapped(self) -> List[ActQuantWrapper]:
        return [m for m in self.modules() if isinstance(m, ActQuantWrapper)]

    def ops_per_step(self, batch: int, tokens: Optional[int] = None, text: Optional[int] = None):
        """(linear, rotation) operations of the wrapped linears of one step at this batch."""
        s = self.shape
        T, S = tokens or s["tokens"], text or s["text"]
        rows = {"img": batch * T, "txt": batch * S}
        lin = rot = 0.0
        for blk in self.all_blocks():
            single = isinstance(blk, FluxSingleBlock)
            for ld, r in blk.census:
                M = batch * (T + S) if single else rows[r]
                lin += linear_ops(ld, M)
                rot += rotation_ops(ld, M)
        return lin, rot

    def kernel_launches_per_step(self) -> int:
        from . import backend
        return sum(backend.kernel_launches(getattr(w, "_b200_state", None), getattr(w, "_b200_w4a16", None)) for w in self.wrapped())


def time_wrapped_linears(step: nn.Module, inputs, classes=(ActQuantWrapper,)) -> float:
    """Device milliseconds one forward of `step` spends inside its wrapped linears (CUDA events around every call,
    recorded on the current stream): the quantized-linear path's share of a model-shaped step."""
    pairs, handles = [], []

    def pre(_m, _a):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        pairs.append([e, None])

    def post(_m, _a, _o):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        pairs[-1][1] = e

    for m in step.modules():
        if isinstance(m, classes):
            handles.append(m.register_forward_pre_hook(pre))
            handles.append(m.register_forward_hook(post))
    try:
        step(*inputs)
        torch.cuda.synchronize()
    finally:
        for h in handles:
            h.remove()
    return sum(a.elapsed_time(b) for a, b in pairs)
