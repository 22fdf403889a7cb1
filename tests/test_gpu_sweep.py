"""Seeded random sweeps over layer geometries through the patched ActQuantWrapper.forward (the C ABI underneath), each case
checked against the oracle.  The fixed-shape tests pin the model configurations; these walk the API surface around them:
ragged row counts, output widths that are not tile multiples, every integer group size the layout takes, tails of any
length, per-head shapes whose groups do or do not fit the fused epilogue, Hadamard and permutation front ends.

Bounds.  Hidden layers: rel-L2 <= 1e-2 and cosine >= 0.999 against the reference quantiser + linear applied to the rotated
bf16 tensor the kernel produced (NVFP4: the two-level hardware recipe, 2e-2).  Per-head / Hadamard / permutation layers are
compared with the oracle's end-to-end forward, whose rotated tensor comes from other arithmetic, so the bound is 1.5 x the
distance between the reference's own fp32 and bf16 forwards on that layer (never below 1e-2); NVFP4 there: 0.12 / 0.99,
the bounds of the fixed-shape NVFP4 tests."""
import random

import pytest
import torch
import torch.nn as nn

from conftest import rel_l2, cosine
from oracle import dirotq_oracle as O

pytestmark = pytest.mark.gpu

QUANTS = ("int4s", "int4a", "int8", "nvfp4")


@pytest.fixture(autouse=True)
def _patched():
    from dirotq_b200 import backend
    from dirotq_b200.wrapper import ActQuantWrapper
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    yield
    ActQuantWrapper.forward = saved


def _grid_weight(W_low, gs, nvfp4, g):
    """Low block of a fused weight that lies on a 4-bit grid with groups of gs along its last dimension."""
    if nvfp4:
        q_len = W_low.shape[-1]
        pad = (q_len + 15) // 16 * 16 - q_len
        return O.weight_quant_nvfp4(torch.nn.functional.pad(W_low, (0, pad)))[0][:, :q_len]
    q_len = W_low.shape[-1]
    ng = (q_len + gs - 1) // gs
    Wp = torch.nn.functional.pad(W_low, (0, ng * gs - q_len)).reshape(*W_low.shape[:-1], ng, gs)
    s = (Wp.abs().amax(-1, keepdim=True) / 7).clamp(min=1e-5).to(torch.float16).float()
    return ((Wp / s).round().clamp(-8, 7) * s).reshape(*W_low.shape[:-1], ng * gs)[..., :q_len]


def _wrap(W, bias, quant, gs, k, g):
    from dirotq_b200.wrapper import ActQuantWrapper
    N, D = W.shape
    lin = nn.Linear(D, N, bias=bias).to(torch.bfloat16)
    lin.weight.data.copy_(W.to(torch.bfloat16))
    if bias:
        lin.bias.data.copy_((torch.randn(N, generator=g) * 0.1).to(torch.bfloat16))
    w = ActQuantWrapper(lin)
    bits, sym = (8 if quant == "int8" else 4), quant in ("int4s", "nvfp4")
    w.quantizer.configure(bits=bits, groupsize=gs, sym=sym, high_bits_length=k,
                          quant_dtype="nvfp4" if quant == "nvfp4" else "int")
    w._unrot_fused = True
    cfg = O.QuantCfg(bits, gs, sym, 1.0, k, "nvfp4" if quant == "nvfp4" else "int")
    return w, lin, cfg


def test_hidden_layers_of_random_geometry():
    from dirotq_b200 import ops
    rnd = random.Random(20)
    bad = []
    for case in range(48):
        D = rnd.choice([128, 256, 320, 576, 1000, 1152, 1536, 2240])
        k = rnd.choice([v for v in (0, 8, 16, 64, 72, 144, 320) if v < D // 2])
        N, M = rnd.choice([8, 16, 64, 200, 1152, 1160, 3000]), rnd.choice([1, 7, 128, 129, 500, 2048, 4100])
        quant, rot, bias = rnd.choice(QUANTS), rnd.random() < 0.67, rnd.random() < 0.8
        gs = 16 if quant == "nvfp4" else rnd.choice([64, 64, 64, 32, 128])
        g = torch.Generator().manual_seed(1000 + case)
        x = O.synth_activations(M, D, g).reshape(1, M, D)
        U = O.random_orthogonal(D, g).float() if rot else None
        deq = _grid_weight(torch.randn(N, D - k, generator=g) * 0.05, gs, quant == "nvfp4", g)
        W = torch.cat([deq, torch.randn(N, k, generator=g) * 0.02], dim=1)
        w, lin, cfg = _wrap(W, bias, quant, gs, k, g)
        if rot:
            w.rotation = U
        y = w(x.cuda()).float().cpu()
        ops.check_status()
        st = w._b200_state
        x_rot = ops.rotate(x.reshape(M, D).cuda(), st.rot_t).cpu().reshape(x.shape) if rot else x
        Wb, bb = lin.weight.data.cpu(), (lin.bias.data.cpu() if bias else None)
        if quant == "nvfp4":
            y_ref = O.fused_forward_nvfp4_hw(x, O.LayerSpec(Wb, bb, cfg, rotation=U), st.fmt.tensor_scale, x_rot=x_rot).float()
            tol = 2e-2
        else:
            r = O.act_quant(x_rot, cfg)
            y_ref = torch.nn.functional.linear(r.full.float(), Wb.float(), None if bb is None else bb.float())
            tol = 1e-2
        rl, cs = rel_l2(y, y_ref), cosine(y, y_ref)
        if not (rl <= tol and cs >= 0.999 and bool(torch.isfinite(y).all()) and st.n_lossy_groups == 0):
            bad.append((case, D, k, N, M, quant, gs, rot, bias, rl, cs, st.n_lossy_groups))
    assert not bad, bad


def test_per_head_layers_of_random_geometry():
    """Weight columns per head [low | high] (the reference re-interleaves before its linear,
    dirotq_fused_unrotation_fast.py:99-102).  Per-head NVFP4 needs head_dim and head_dim - tail in multiples of 16: the
    other shapes must be refused with NotImplementedError, not run."""
    from dirotq_b200 import ops
    rnd = random.Random(21)
    bad, ran, refused = [], 0, 0
    for case in range(40):
        H, d = rnd.choice([(16, 72), (24, 128), (70, 32), (8, 64), (4, 96), (12, 40), (3, 128), (5, 48)])
        t = rnd.choice([0, 1, 4, 8, 9, 16])
        t = 4 if t >= d // 2 else t
        N, M, quant = rnd.choice([8, 64, 200, 1152, 1160]), rnd.choice([1, 7, 128, 129, 500, 2048]), rnd.choice(QUANTS)
        D, gl = H * d, d - t
        g = torch.Generator().manual_seed(5000 + case)
        x = O.synth_activations(M, D, g).reshape(1, M, D)
        Uph = torch.stack([O.random_orthogonal(d, g).float() for _ in range(H)])
        fp4_ok = gl % 16 == 0 and d % 16 == 0
        W_low = torch.randn(N, H, gl, generator=g) * 0.05
        deq = _grid_weight(W_low, gl, False, g) if quant != "nvfp4" else (
            _grid_weight(W_low.reshape(N, H * gl), 16, True, g).reshape(N, H, gl) if fp4_ok else W_low)
        W = torch.cat([deq, torch.randn(N, H, t, generator=g) * 0.02], dim=2).reshape(N, D)
        w, lin, cfg = _wrap(W, True, quant, 16 if quant == "nvfp4" else gl, t, g)
        w.rotation_per_head, w.num_heads, w.head_dim = Uph, H, d
        if quant == "nvfp4" and not fp4_ok:
            with pytest.raises(NotImplementedError):
                w(x.cuda())
            refused += 1
            continue
        y = w(x.cuda()).float().cpu()
        ops.check_status()
        ran += 1
        spec = O.LayerSpec(lin.weight.data.cpu(), lin.bias.data.cpu(), cfg, rotation_per_head=Uph)
        y_fast, y_slow = O.fused_forward(x, spec, fp32=False).float(), O.fused_forward(x, spec, fp32=True).float()
        gap = rel_l2(y_fast, y_slow)
        rl, cs = rel_l2(y, y_fast), cosine(y, y_fast)
        bound, cmin = (max(0.12, 1.5 * gap), 0.99) if quant == "nvfp4" else (max(1e-2, 1.5 * gap), 0.995)
        if not (rl <= bound and cs >= cmin and bool(torch.isfinite(y).all()) and w._b200_state.n_lossy_groups == 0):
            bad.append((case, H, d, t, N, M, quant, rl, cs, gap))
    assert not bad, bad
    assert ran >= 25 and refused >= 1


def test_hadamard_and_permutation_layers_of_random_geometry():
    from dirotq_b200 import ops
    rnd = random.Random(22)
    bad = []
    for case in range(36):
        kind, quant = rnd.choice(["hadamard", "perm"]), rnd.choice(QUANTS)
        M, N = rnd.choice([1, 7, 128, 129, 500, 2048]), rnd.choice([8, 64, 200, 1152, 1160])
        gs = 16 if quant == "nvfp4" else 64
        if kind == "hadamard":
            low, extra = rnd.choice([64, 256, 512, 1024, 2048]), rnd.choice([0, 64, 72, 512, 8])
            D, k = low + extra, (extra if rnd.random() < 0.7 else rnd.choice([0, 8, 64]))
        else:
            D, k = rnd.choice([256, 576, 1152, 1000]), rnd.choice([0, 8, 64, 72])
        g = torch.Generator().manual_seed(9000 + case)
        x = O.synth_activations(M, D, g).reshape(1, M, D)
        deq = _grid_weight(torch.randn(N, D - k, generator=g) * 0.05, gs, quant == "nvfp4", g)
        W = torch.cat([deq, torch.randn(N, k, generator=g) * 0.02], dim=1)
        w, lin, cfg = _wrap(W, True, quant, gs, k, g)
        spec = O.LayerSpec(lin.weight.data.cpu(), lin.bias.data.cpu(), cfg)
        if kind == "hadamard":
            flips = (torch.randint(0, 2, (low,), generator=g).float() * 2 - 1) if rnd.random() < 0.7 else None
            w.use_hadamard, w.hadamard_low_dim, w.hadamard_sign_flips = True, low, flips
            spec.hadamard_low_dim, spec.hadamard_sign_flips = low, flips
        else:
            w.perm_idx = spec.perm_idx = torch.randperm(D, generator=g)
        y = w(x.cuda()).float().cpu()
        ops.check_status()
        y_fast, y_slow = O.fused_forward(x, spec, fp32=False).float(), O.fused_forward(x, spec, fp32=True).float()
        gap = rel_l2(y_fast, y_slow)
        rl, cs = rel_l2(y, y_fast), cosine(y, y_fast)
        bound, cmin = (max(0.12, 1.5 * gap), 0.99) if quant == "nvfp4" else (max(1e-2, 1.5 * gap), 0.995)
        if not (rl <= bound and cs >= cmin and bool(torch.isfinite(y).all())):
            bad.append((case, kind, D, k, N, M, quant, rl, cs, gap))
    assert not bad, bad


def test_widths_the_kernels_do_not_take_are_refused_before_any_launch():
    """Channel counts that are not multiples of 8 (16-byte rows are the kernels' unit of access): a clean error from the
    library's own validation, the status word untouched."""
    import warnings
    from dirotq_b200 import ops
    g = torch.Generator().manual_seed(3)
    for D, k, N in [(100, 0, 8), (1001, 3, 8), (1156, 0, 64), (256, 64, 7), (256, 64, 1001)]:
        W = torch.randn(N, D, generator=g) * 0.05
        w, _, _ = _wrap(W, True, "int4s", 64, k, g)
        w.rotation = torch.eye(D)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")                     # these random weights are not on a 4-bit grid
            with pytest.raises((RuntimeError, ValueError, NotImplementedError)):
                w(torch.zeros(1, 4, D, dtype=torch.bfloat16, device="cuda"))
    ops.check_status()
