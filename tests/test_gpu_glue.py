"""GPU parity of the block-glue kernels (csrc/glue.cu): floating-point kernels, so the reference is plain PyTorch in
fp64 on the same bf16 inputs.  Tolerance: the result is the correctly rounded bf16 of the fp64 value up to one bf16 ulp
(relative 2^-7 on values that are not tiny), and never further from it than the chain of PyTorch bf16 kernels the
reference's model forwards run (speedup/report_flux_w4a4_no_rot_ffdown.py:199-252)."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _close_to_fp64(got, want64, eager):
    got, eager = got.double().cpu(), eager.double().cpu()
    want = want64.cpu()
    err, err_eager = (got - want).abs(), (eager - want).abs()
    tol = want.abs() * 2.0 ** -7 + 1e-3                       # one bf16 ulp, and an absolute floor for cancellations
    assert bool((err <= tol).all()), float((err - tol).max())
    assert float(err.pow(2).sum()) <= 1.05 * float(err_eager.pow(2).sum()) + 1e-12


@pytest.mark.parametrize("B,T,D", [(2, 300, 1152), (3, 129, 3072), (1, 77, 2240), (2, 64, 4096), (1, 5, 64)])
def test_layernorm_modulate(B, T, D):
    from dirotq_b200 import ops
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(B, T, D, generator=g) * 2 + torch.randn(B, T, 1, generator=g)).to(torch.bfloat16).cuda()
    mod = (torch.randn(B, 6 * D, generator=g) * 0.3).to(torch.bfloat16).cuda()
    shift, scale = mod[:, None].chunk(6, dim=-1)[:2]          # strided views, as the blocks pass them
    y = ops.layernorm_modulate(x, scale, shift)
    x64 = x.double()
    want = F.layer_norm(x64, (D,), eps=1e-6) * (1 + scale.double()) + shift.double()
    eager = F.layer_norm(x, (D,), eps=1e-6) * (1 + scale) + shift
    _close_to_fp64(y, want, eager)
    # plain LayerNorm, and a scale shared by all samples
    y0 = ops.layernorm_modulate(x)
    _close_to_fp64(y0, F.layer_norm(x64, (D,), eps=1e-6), F.layer_norm(x, (D,), eps=1e-6))
    s1 = scale[:1].contiguous()
    y1 = ops.layernorm_modulate(x, s1, None)
    _close_to_fp64(y1, F.layer_norm(x64, (D,), eps=1e-6) * (1 + s1.double()), F.layer_norm(x, (D,), eps=1e-6) * (1 + s1))


@pytest.mark.parametrize("B,T,D", [(2, 300, 1152), (3, 129, 3072), (1, 5, 64)])
def test_gated_residual(B, T, D):
    from dirotq_b200 import ops
    g = torch.Generator().manual_seed(4)
    h, y, y2 = [(torch.randn(B, T, D, generator=g)).to(torch.bfloat16).cuda() for _ in range(3)]
    gate = (torch.randn(B, 3 * D, generator=g) * 0.5).to(torch.bfloat16).cuda()[:, None].chunk(3, dim=-1)[2]
    out = ops.gated_residual(h, y, gate)
    _close_to_fp64(out, h.double() + gate.double() * y.double(), h + gate * y)
    out = ops.gated_residual(h, y, gate, y2)
    _close_to_fp64(out, h.double() + gate.double() * (y.double() + y2.double()), h + gate * (y + y2))
    out = ops.gated_residual(h, y)
    assert torch.equal(out, h + y)                            # one add: the same single rounding
    yt = y.transpose(1, 2).contiguous().transpose(1, 2)       # a non-contiguous branch output (SANA's Mix-FFN)
    assert torch.equal(ops.gated_residual(h, yt, gate), ops.gated_residual(h, y, gate))


@pytest.mark.parametrize("B,S,T,H,d", [(2, 40, 200, 24, 128), (1, 0, 77, 6, 64), (3, 16, 33, 5, 128)])
def test_qkv_norm_rope_fills_a_joint_buffer(B, S, T, H, d):
    from dirotq_b200 import denoise, ops
    g = torch.Generator().manual_seed(5)
    C = H * d
    cos, sin = denoise.rope_tables(S + T, d, "cuda")
    wq, wk = [(1 + 0.2 * torch.randn(d, generator=g)).to(torch.bfloat16).cuda() for _ in range(2)]
    fused_img = torch.randn(B * T, 3 * C, generator=g).to(torch.bfloat16).cuda()       # one fused q | k | v projection output
    qi, ki, vi = [fused_img[:, j * C:(j + 1) * C].reshape(B, T, C) for j in range(3)]
    bufs = tuple(torch.full((B, S + T, H, d), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(3))
    if S:
        qt, kt, vt = [torch.randn(B, S, C, generator=g).to(torch.bfloat16).cuda() for _ in range(3)]   # separate tensors
        ops.qkv_norm_rope(qt, kt, vt, H, wq, wk, cos, sin, out=bufs, t0=0)
    ops.qkv_norm_rope(qi, ki, vi, H, wq, wk, cos, sin, out=bufs, t0=S)

    def ref(x, w, dt):
        xh = x.to(dt).view(x.shape[0], x.shape[1], H, d)
        xn = xh * torch.rsqrt(xh.pow(2).mean(-1, keepdim=True) + 1e-6) * w.to(dt)
        return xn

    def rope(x, dt, pos0):
        c, s_ = cos[pos0:pos0 + x.shape[1]].to(dt)[None, :, None], sin[pos0:pos0 + x.shape[1]].to(dt)[None, :, None]
        xr = torch.stack([-x[..., 1::2], x[..., 0::2]], dim=-1).flatten(-2)
        return x * c + xr * s_

    def eager(x, w, pos0):                                     # the blocks' PyTorch chain, bf16 between the steps
        xh = x.view(x.shape[0], x.shape[1], H, d)
        xn = (xh.float() * torch.rsqrt(xh.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype) * w
        return rope(xn, torch.bfloat16, pos0)

    for j, (src_t, src_i, w) in enumerate(((qt if S else None, qi, wq), (kt if S else None, ki, wk))):
        _close_to_fp64(bufs[j][:, S:], rope(ref(src_i, w, torch.float64), torch.float64, S), eager(src_i, w, S))
        if S:
            _close_to_fp64(bufs[j][:, :S], rope(ref(src_t, w, torch.float64), torch.float64, 0), eager(src_t, w, 0))
    assert torch.equal(bufs[2][:, S:], vi.view(B, T, H, d))
    if S:
        assert torch.equal(bufs[2][:, :S], vt.view(B, S, H, d))
    assert not any(torch.isnan(b.float()).any() for b in bufs)   # every row of the joint buffers was written


@pytest.mark.parametrize("family", ["pixart", "flux", "sana"])
def test_blocks_with_fused_glue_follow_the_pytorch_chain(family, monkeypatch):
    """A model-shaped step with the glue kernels.  (1) Every glue call inside the blocks is compared, on the inputs it
    actually received (strided modulation views, fused q | k | v columns, token offsets), with the PyTorch chain it
    replaces: bf16-rounding distance.  (2) End to end against the step on PyTorch's chains: the roundings between the steps
    of a chain move a few 4-bit codes in the linears that follow, so the bound is the block-drift bound the library's
    linears keep against the reference arithmetic (cosine >= 0.99, relative L2 <= 0.15)."""
    from dirotq_b200 import backend, denoise, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    calls = {"ln": 0, "gate": 0, "qkv": 0}
    ln, gr, qk = ops.layernorm_modulate, ops.gated_residual, ops.qkv_norm_rope

    def close(a, b, what):
        r = rel_l2(a.float().cpu(), b.float().cpu())
        assert r < 6e-3, (what, r)

    def ln_checked(x, scale=None, shift=None, eps=1e-6):
        y = ln(x, scale, shift, eps)
        close(y, F.layer_norm(x, (x.shape[-1],), eps=eps) * (1 + scale) + shift, "layernorm_modulate")
        calls["ln"] += 1
        return y

    def gr_checked(h, y, gate=None, y2=None):
        out = gr(h, y, gate, y2)
        yy = y if y2 is None else y + y2
        close(out, h + (yy if gate is None else gate * yy), "gated_residual")
        calls["gate"] += 1
        return out

    def qk_checked(q, k, v, heads, w_q, w_k, cos, sin, out=None, t0=0, eps=1e-6):
        res = qk(q, k, v, heads, w_q, w_k, cos, sin, out=out, t0=t0, eps=eps)
        T = q.shape[1]
        for j, (x, w) in enumerate(((q, w_q), (k, w_k))):
            e = denoise._rope(denoise._rms(denoise._heads(x, heads), w), cos[t0:t0 + T], sin[t0:t0 + T])    # [B, H, T, d]
            close(res[j][:, t0:t0 + T].transpose(1, 2), e, "qkv_norm_rope")
        assert torch.equal(res[2][:, t0:t0 + T], v.reshape(v.shape[0], T, heads, -1))
        calls["qkv"] += 1
        return res

    try:
        step = denoise.DenoiseStep(family, "int4", "cuda", n_blocks=1, seed=7300, prepare=True)
        inputs = step.example_inputs(1, "cuda", seed=2, tokens=256 if family == "sana" else 320, text=64)
        with torch.no_grad():
            denoise.FUSED_GLUE = False
            y_eager = step(*inputs)
            denoise.FUSED_GLUE = True
            monkeypatch.setattr(ops, "layernorm_modulate", ln_checked)
            monkeypatch.setattr(ops, "gated_residual", gr_checked)
            monkeypatch.setattr(ops, "qkv_norm_rope", qk_checked)
            y_fused = step(*inputs)
        ops.check_status()
    finally:
        denoise.FUSED_GLUE = True
        ActQuantWrapper.forward = saved
    assert calls["ln"] >= 2 and calls["gate"] >= 2 and (calls["qkv"] >= 3 if family == "flux" else calls["qkv"] == 0)
    a, b = y_fused.float().cpu(), y_eager.float().cpu()
    cos = float((a * b).sum() / (a.norm() * b.norm()))
    assert cos >= 0.99 and rel_l2(a, b) <= 0.15, (cos, rel_l2(a, b))
