"""GPU parity of the drop-in boundary: the patched ActQuantWrapper.forward against outputs of the
reference's own forwards (golden fixtures) and against the oracle at BASELINE config 0.
Tolerance from the task statement, rel-L2 <= 1e-2 and cosine >= 0.999 on layer outputs, is asserted against the
reference quantiser + bf16 linear applied to the SAME rotated bf16 tensor (the one the kernel produced).  Against
the reference's stored outputs, whose rotated tensor comes from another GEMM (last-bit differences flip 4-bit
codes), the bound is 1.5 x the distance between the reference's own fp32 and bf16 forwards on that layer; NVFP4
layers, whose scale format the reference's activation quantiser does not have, are bounded by QSNR instead."""
import pytest
import torch
import torch.nn as nn

from conftest import load_golden, rel_l2, cosine
from oracle import dirotq_oracle as O

pytestmark = pytest.mark.gpu

REL, COS = 1e-2, 0.999


def _wrapper_from_golden(g):
    from dirotq_b200.wrapper import ActQuantWrapper
    bits, gs, sym, hlen, is_fp4 = [int(v) for v in g["cfg"]]
    N, D = g["weight"].shape
    lin = nn.Linear(D, N, bias=True).to(torch.bfloat16)
    lin.weight.data.copy_(g["weight"])
    lin.bias.data.copy_(g["bias"])
    w = ActQuantWrapper(lin)
    w.quantizer.configure(bits=bits, groupsize=gs, sym=bool(sym), high_bits_length=hlen,
                          quant_dtype="nvfp4" if is_fp4 else "int")
    if "rotation" in g:
        w.rotation = g["rotation"]
    if "rotation_per_head" in g:
        w.rotation_per_head = g["rotation_per_head"]
        w.num_heads, w.head_dim = g["rotation_per_head"].shape[0], g["rotation_per_head"].shape[1]
    w._unrot_fused = True
    return w


@pytest.fixture(autouse=True)
def _patched():
    from dirotq_b200 import backend
    from dirotq_b200.wrapper import ActQuantWrapper
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    yield
    ActQuantWrapper.forward = saved


@pytest.mark.parametrize("name", ["hidden_int4_sym", "hidden_int4_asym", "hidden_int4_pad_notail",
                                  "hidden_int8_asym", "perhead_int4_sym", "perhead_int4_asym",
                                  "perhead_d32_int4_sym"])
def test_forward_matches_reference_int(name):
    from dirotq_b200 import backend, ops
    g = load_golden(name)
    w = _wrapper_from_golden(g)
    holder = nn.ModuleDict({"l": w})
    n = backend.preconvert_rotations_to_device(holder, "cuda")
    assert n == 1 and w._b200_state.n_lossy_groups == 0
    y = w(g["x"].cuda())
    ops.check_status()
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == tuple(g["y_fast"].shape)
    yc = y.float().cpu()
    # (1) exact-path check: the reference quantiser + bf16 linear applied to the x_rot OUR kernel produced
    st = w._b200_state
    x2d = g["x"].reshape(-1, g["x"].shape[-1]).cuda()
    _, x_rot = ops.rotate_quantize(x2d, st.rot_t, st.fmt, want_x_rot=True)
    from gpu_helpers import to_reference_layout, oracle_cfg
    xin = to_reference_layout(x_rot, st.fmt)
    r = O.act_quant(xin, oracle_cfg(st.fmt, st.layout))
    xq = r.full
    if st.fmt.num_heads:
        xq = O.per_head_interleave(xq, st.fmt.num_heads, st.fmt.head_dim, st.fmt.tail_len)
    y_same = torch.nn.functional.linear(xq.to(torch.bfloat16), g["weight"], g["bias"]).float().reshape(yc.shape)
    assert rel_l2(yc, y_same) <= REL and cosine(yc, y_same) >= COS, name
    # (2) against the reference's outputs.  x_rot from tensor cores and from the CPU GEMM differ in
    # the last bf16 bit for some elements, which flips 4-bit codes; on these tiny layers the
    # reference's own fp32 and bf16 forwards differ by 2.5-7e-2 for the same reason, so the bound is
    # that distance (the 1e-2 bound is asserted at BASELINE config 0 below).
    gap = rel_l2(g["y_fast"].float(), g["y_slow"].float())
    assert rel_l2(yc, g["y_fast"].float()) <= max(REL, 1.5 * gap), name
    assert cosine(yc, g["y_fast"].float()) >= 0.995, name
    if not name.startswith("perhead"):   # the reference's fp32 forward does not rearrange per-head layers
        assert rel_l2(yc, g["y_slow"].float()) <= max(REL, 1.5 * gap), name


@pytest.mark.parametrize("name", ["hidden_int4_sym_pertoken", "hidden_int4_asym_pertoken", "hidden_int4_asym_pertoken_pad"])
def test_per_token_activation_scales(name):
    """groupsize <= 0: one scale (and zero point) per token (ActQuantizer._find_params, utils/quant_utils.py:242-271).
    The layer rotates into scratch and quantises from there; codes, scale and zero point are bit-exact against the
    reference quantiser applied to the rotated tensor the kernel produced, the output within the layer tolerance."""
    from dirotq_b200 import backend, ops
    from gpu_helpers import decode_act, oracle_cfg
    g = load_golden(name)
    w = _wrapper_from_golden(g)
    holder = nn.ModuleDict({"l": w})
    assert backend.preconvert_rotations_to_device(holder, "cuda") == 1
    st = w._b200_state
    assert st.fmt.group_size <= 0 and st.n_lossy_groups == 0
    y = w(g["x"].cuda())
    ops.check_status()
    yc = y.float().cpu()
    x2d = g["x"].reshape(-1, g["x"].shape[-1]).cuda()
    M = x2d.shape[0]
    x_rot = ops.rotate(x2d, st.rot_t)
    with pytest.raises(RuntimeError):                       # the fused kernel cannot see a whole row
        ops.rotate_quantize(x2d, st.rot_t, st.fmt)
    buf = ops.quantize_act(x_rot, st.fmt)
    d = decode_act(buf)
    cfg = oracle_cfg(st.fmt, st.layout)
    assert cfg.groupsize == -1
    r = O.act_quant(x_rot.cpu().unsqueeze(0), cfg)
    q_len = st.layout.q_len
    assert torch.equal(d["codes_padded"].reshape(M, -1)[:, :q_len], r.codes.reshape(M, q_len))
    assert not d["codes_padded"].reshape(M, -1)[:, q_len:].any() or not cfg.sym   # symmetric padding slots hold code 0
    want_s = r.scale.reshape(M, 1).expand(M, st.layout.n_chunks).contiguous()
    assert torch.equal(d["scale_chunks"].view(torch.int16), want_s.view(torch.int16))
    if not cfg.sym:
        want_z = r.zero.reshape(M, 1).expand(M, st.layout.n_chunks).contiguous()
        assert torch.equal(d["zero"].view(torch.int16), want_z.view(torch.int16))
    if st.layout.tail_total:
        assert torch.equal(d["tail"].view(torch.int16), r.tail.reshape(M, -1).contiguous().view(torch.int16))
    y_same = torch.nn.functional.linear(r.full.to(torch.bfloat16), g["weight"], g["bias"]).float().reshape(yc.shape)
    assert rel_l2(yc, y_same) <= REL and cosine(yc, y_same) >= COS
    gap = rel_l2(g["y_fast"].float(), g["y_slow"].float())
    assert rel_l2(yc, g["y_fast"].float()) <= max(REL, 1.5 * gap) and cosine(yc, g["y_fast"].float()) >= 0.995
    # the allocation-free entry point sizes the extra scratch from the same layout
    assert torch.equal(backend.linear_forward_static(st, x2d), y.reshape(M, -1))


@pytest.mark.parametrize("gs,sym,bits,D,k,N,M", [(128, True, 4, 1152, 8, 1160, 128), (32, False, 4, 576, 16, 64, 2048),
                                                (32, True, 4, 2240, 320, 1160, 7), (128, False, 8, 576, 72, 200, 129),
                                                (32, False, 8, 1000, 72, 1152, 128)])
def test_hidden_rotation_with_other_integer_group_sizes(gs, sym, bits, D, k, N, M):
    """The reference's quantiser takes any groupsize (ActQuantizer.configure, utils/quant_utils.py:182-199); the rotation
    kernel's epilogue quantises groups of 64 only.  Other sizes rotate into scratch and quantise from there: codes and
    scales bit-exact against the reference quantiser on the rotated tensor the kernel produced, output within the
    layer tolerance."""
    from dirotq_b200 import backend, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    from gpu_helpers import assert_act_matches_oracle
    g = torch.Generator().manual_seed(gs * 7 + D)
    x = O.synth_activations(M, D, g).reshape(1, M, D)
    U = O.random_orthogonal(D, g).float()
    q_len = D - k
    ng = (q_len + gs - 1) // gs
    Wp = torch.nn.functional.pad(torch.randn(N, q_len, generator=g) * 0.05, (0, ng * gs - q_len)).reshape(N, ng, gs)
    s = (Wp.abs().amax(-1, keepdim=True) / 7).clamp(min=1e-5).to(torch.float16).float()
    deq = ((Wp / s).round().clamp(-8, 7) * s).reshape(N, -1)[:, :q_len]
    lin = nn.Linear(D, N, bias=True).to(torch.bfloat16)
    lin.weight.data.copy_(torch.cat([deq, torch.randn(N, k, generator=g) * 0.02], dim=1).to(torch.bfloat16))
    lin.bias.data.copy_((torch.randn(N, generator=g) * 0.1).to(torch.bfloat16))
    w = ActQuantWrapper(lin)
    w.quantizer.configure(bits=bits, groupsize=gs, sym=sym, high_bits_length=k, quant_dtype="int")
    w.rotation = U
    w._unrot_fused = True
    y = w(x.cuda())
    ops.check_status()
    st = w._b200_state
    assert st.fmt.group_size == gs and backend.kernel_launches(st) >= 4      # rotate, quantise, tail copy, (fold +) GEMM
    x2d = x.reshape(M, D).cuda()
    x_rot = ops.rotate(x2d, st.rot_t)
    with pytest.raises(RuntimeError):                       # the fused epilogue has groups of 64 only
        ops.rotate_quantize(x2d, st.rot_t, st.fmt)
    assert_act_matches_oracle(ops.quantize_act(x_rot, st.fmt), x_rot)
    r = O.act_quant(x_rot.cpu().unsqueeze(0), O.QuantCfg(bits, gs, sym, 1.0, k, "int"))
    y_same = torch.nn.functional.linear(r.full.to(torch.bfloat16), lin.weight.data.cpu(), lin.bias.data.cpu()).float()
    assert rel_l2(y.float().cpu(), y_same) <= REL and cosine(y.float().cpu(), y_same) >= COS
    assert torch.equal(backend.linear_forward_static(st, x2d), y.reshape(M, -1))


@pytest.mark.parametrize("H,d,t,bits,sym,N,M", [(5, 48, 8, 4, True, 1160, 128), (16, 72, 1, 8, False, 200, 500),
                                                (12, 40, 1, 4, False, 64, 1), (5, 48, 9, 4, True, 1152, 500)])
def test_per_head_groups_that_do_not_fit_the_fused_epilogue(H, d, t, bits, sym, N, M):
    """The per-head epilogue of the rotation kernel reads a head's group 32 columns at a time; a group whose rounded-up
    width exceeds the head (head_dim 48 with 8 high channels, 72 with 1, ...) rotates into scratch and quantises from
    there instead.  Weight columns are per head [low | high] (the reference re-interleaves before its linear,
    dirotq_fused_unrotation_fast.py:99-102)."""
    from dirotq_b200 import backend, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    from gpu_helpers import assert_act_matches_oracle
    g = torch.Generator().manual_seed(H * 100 + d + t)
    D, gl = H * d, d - t
    x = O.synth_activations(M, D, g).reshape(1, M, D)
    Uph = torch.stack([O.random_orthogonal(d, g).float() for _ in range(H)])
    W_low = torch.randn(N, H, gl, generator=g) * 0.05
    s = (W_low.abs().amax(-1, keepdim=True) / 7).clamp(min=1e-5).to(torch.float16).float()
    deq = (W_low / s).round().clamp(-8, 7) * s
    W = torch.cat([deq, torch.randn(N, H, t, generator=g) * 0.02], dim=2).reshape(N, D).to(torch.bfloat16)
    lin = nn.Linear(D, N, bias=True).to(torch.bfloat16)
    lin.weight.data.copy_(W)
    lin.bias.data.copy_((torch.randn(N, generator=g) * 0.1).to(torch.bfloat16))
    w = ActQuantWrapper(lin)
    w.quantizer.configure(bits=bits, groupsize=64, sym=sym, high_bits_length=t, quant_dtype="int")
    w.rotation_per_head = Uph
    w.num_heads, w.head_dim = H, d
    w._unrot_fused = True
    y = w(x.cuda())
    ops.check_status()
    st = w._b200_state
    assert st.n_lossy_groups == 0 and backend._rotates_then_quantises(st)
    x2d = x.reshape(M, D).cuda()
    with pytest.raises(RuntimeError):
        ops.rotate_quantize(x2d, st.rot_t, st.fmt)
    x_rot = ops.rotate(x2d, st.rot_t, H, d)
    # rotation-only launches under a per-head rotation: whole-head tile widths (144 for 72-wide heads) are not multiples
    # of the epilogue's 32-column store patches
    want_rot = O.rotate_per_head(x, Uph, fp32=True).reshape(M, D)
    assert rel_l2(x_rot.float().cpu(), want_rot) <= 5e-3
    assert_act_matches_oracle(ops.quantize_act(x_rot, st.fmt), x_rot)
    spec = O.LayerSpec(lin.weight.data.cpu(), lin.bias.data.cpu(), O.QuantCfg(bits, 64, sym, 1.0, t, "int"), rotation_per_head=Uph)
    y_fast, y_slow = O.fused_forward(x, spec, fp32=False).float(), O.fused_forward(x, spec, fp32=True).float()
    gap = rel_l2(y_fast, y_slow)
    yc = y.float().cpu()
    assert rel_l2(yc, y_fast) <= max(REL, 1.5 * gap) and cosine(yc, y_fast) >= 0.995
    assert torch.equal(backend.linear_forward_static(st, x2d), y.reshape(M, -1))


@pytest.mark.parametrize("fused", [True, False])
def test_per_head_rotation_with_nvfp4_activations(fused, monkeypatch):
    """Per-head rotation + NVFP4 (head_dim - tail a multiple of 16): the heads' low coefficients side by side in blocks
    of 16, by the rotation kernel's per-head epilogue (fused) or by a block-diagonal rotation into scratch followed by
    gather + quantise (two launches).  Bit contract: the hardware-recipe oracle on the gathered tensor; against the
    reference (one unrounded scale per head group) the layer is pinned by QSNR."""
    from dirotq_b200 import backend, ops
    monkeypatch.setattr(backend, "PER_HEAD_NVFP4_FUSED", fused)
    g = load_golden("perhead_nvfp4")
    w = _wrapper_from_golden(g)
    y = w(g["x"].cuda()).float().cpu()
    ops.check_status()
    st = w._b200_state
    H, d, hl = 4, 64, 16
    assert st.layout.tail_total == H * hl and st.layout.q_len == H * (d - hl)
    assert (st.fmt.num_heads == H and st.perm_idx is None) if fused else (st.fmt.num_heads == 0 and st.perm_idx is not None)
    if not fused:
        cols = torch.arange(H * d).reshape(H, d)
        assert torch.equal(st.perm_idx.cpu(), torch.cat([cols[:, : d - hl].reshape(-1), cols[:, d - hl:].reshape(-1)]))
    x2d = g["x"].reshape(-1, H * d).cuda()
    x_rot = ops.rotate(x2d, st.rot_t).cpu()
    xre = O.per_head_rearrange(x_rot.reshape(-1, H, d), hl).reshape(g["x"].shape)     # [H * (d - hl) | H * hl]
    W3 = g["weight"].float().reshape(-1, H, d)
    W_re = torch.cat([W3[:, :, : d - hl].reshape(-1, H * (d - hl)), W3[:, :, d - hl:].reshape(-1, H * hl)], 1).to(torch.bfloat16)
    spec = O.LayerSpec(W_re, g["bias"], O.QuantCfg(4, 16, True, 1.0, H * hl, "nvfp4"))
    y_hw = O.fused_forward_nvfp4_hw(xre, spec, st.fmt.tensor_scale, x_rot=xre)
    assert rel_l2(y, y_hw) <= 5e-3 and cosine(y, y_hw) >= 0.9999
    y_fp = torch.nn.functional.linear(xre.float(), W_re.float(), g["bias"].float())
    q_ref, q_ours = O.qsnr_db(y_fp, g["y_fast"].float()), O.qsnr_db(y_fp, y)
    print(f"perhead_nvfp4: QSNR reference fake-quant {q_ref:.2f} dB, B200 NVFP4 {q_ours:.2f} dB")
    assert q_ours >= q_ref - 0.5


def test_forward_nvfp4_against_hw_oracle_and_reference():
    """The tensor-core format needs UE4M3 group scales, which the reference's activation quantiser does not have.
    Bit contract: the hw oracle (two-level recipe on the activations, the reference's own two-level weight recipe
    on the weights).  Against the reference's unrounded-scale forward the layer is pinned by QUALITY: its QSNR
    (diagnose_layer_qsnr.py:38-46) against the unquantised-activation fp32 linear must be within 0.5 dB of the
    QSNR the reference's own fake-quant forward reaches on the same layer."""
    from dirotq_b200 import backend, ops
    g = load_golden("hidden_nvfp4")
    w = _wrapper_from_golden(g)
    y = w(g["x"].cuda()).float().cpu()
    ops.check_status()
    st = w._b200_state
    assert st.w_rowscale is not None and st.w_tensor_scale == 1.0
    cfg = O.QuantCfg(4, 16, True, 1.0, 48, "nvfp4")
    spec = O.LayerSpec(g["weight"], g["bias"], cfg, rotation=g["rotation"])
    x2d = g["x"].reshape(-1, g["x"].shape[-1]).cuda()
    x_rot = ops.rotate(x2d, st.rot_t).cpu().reshape(g["x"].shape)
    y_hw = O.fused_forward_nvfp4_hw(g["x"], spec, st.fmt.tensor_scale, x_rot=x_rot)
    assert rel_l2(y, y_hw) <= 5e-3 and cosine(y, y_hw) >= 0.9999      # same rotated tensor: accumulation order + bf16 output
    y_fp = torch.nn.functional.linear(x_rot.float(), g["weight"].float(), g["bias"].float())
    q_ref, q_ours = O.qsnr_db(y_fp, g["y_fast"].float()), O.qsnr_db(y_fp, y)
    print(f"hidden_nvfp4: QSNR reference fake-quant {q_ref:.2f} dB, B200 NVFP4 {q_ours:.2f} dB")
    assert q_ours >= q_ref - 0.5


@pytest.mark.parametrize("D,N,k,M", [(1152, 1152, 64, 2048), (1152, 1152, 144, 2048), (3072, 3072, 384, 1024)])
def test_nvfp4_layer_quality_not_worse_than_reference_fake_quant(D, N, k, M):
    """BASELINE config 0 / 2 inputs (planted subspace, heavy-tailed channels), random dense weight: QSNR against the
    UNQUANTISED fp32 linear of (i) the reference's forward -- _quant_group_nvfp4 weights (utils/quant_utils.py:752-767)
    and _forward_nvfp4_grouped activations (:148-180), both with unrounded scales -- and (ii) this library's layer
    on the same fused weight.  (ii) re-rounds both operands' group scales to E4M3; it must stay within 0.5 dB."""
    from dirotq_b200 import backend, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    g = torch.Generator().manual_seed(7)
    x = O.synth_activations(M, D, g).reshape(2, M // 2, D)
    U = O.random_orthogonal(D, g).float()
    W_rot = (torch.randn(N, D, generator=g) * 0.05) @ U
    deq, _, _ = O.weight_quant_nvfp4(W_rot[:, : D - k])
    Wf = torch.cat([deq, W_rot[:, D - k:]], dim=1).to(torch.bfloat16)
    lin = nn.Linear(D, N, bias=False).to(torch.bfloat16)
    lin.weight.data.copy_(Wf)
    w = ActQuantWrapper(lin)
    w.quantizer.configure(bits=4, groupsize=16, sym=True, high_bits_length=k, quant_dtype="nvfp4")
    w.rotation = U
    w._unrot_fused = True
    y = w(x.cuda()).float().cpu()
    ops.check_status()
    spec = O.LayerSpec(Wf, None, O.QuantCfg(4, 16, True, 1.0, k, "nvfp4"), rotation=U)
    y_ref = O.fused_forward(x, spec, fp32=False).float()
    y_fp = ((x.float().reshape(-1, D) @ U) @ W_rot.T).reshape(y.shape)
    q_ref, q_ours = O.qsnr_db(y_fp, y_ref), O.qsnr_db(y_fp, y)
    print(f"D={D} k={k}: QSNR reference fake-quant {q_ref:.2f} dB, B200 NVFP4 {q_ours:.2f} dB")
    assert q_ours >= q_ref - 0.5
    # and the bit contract on the tensor the kernel itself rotated
    st = w._b200_state
    x_rot = ops.rotate(x.reshape(-1, D).cuda(), st.rot_t).cpu().reshape(x.shape)
    y_hw = O.fused_forward_nvfp4_hw(x, spec, st.fmt.tensor_scale, x_rot=x_rot)
    assert rel_l2(y, y_hw) <= 5e-3 and cosine(y, y_hw) >= 0.9999


def _config0(seed=0, M=8192, D=1152, N=1152, k=64):
    g = torch.Generator().manual_seed(seed)
    x = O.synth_activations(M, D, g).reshape(2, M // 2, D)
    U = O.random_orthogonal(D, g).float()
    qw = torch.randint(-8, 8, (N, D - k), generator=g)
    sw = (torch.rand(N, (D - k) // 64, generator=g) * 0.015 + 0.005).to(torch.float16).float()
    w_tail = (torch.randn(N, k, generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    w_low = (qw.reshape(N, -1, 64).float() * sw.unsqueeze(-1)).reshape(N, -1)
    W = torch.cat([w_low, w_tail.float()], dim=1).to(torch.bfloat16)
    return x, U, qw, sw, w_tail, bias, W


@pytest.mark.parametrize("sym", [True, False])
def test_config0_layer_against_fp32_reference_path(sym):
    """BASELINE config 0: one PixArt attention linear, [2,4096,1152], k=64, INT4 g64, explicit codes."""
    from dirotq_b200 import backend, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    x, U, qw, sw, w_tail, bias, W = _config0()
    lin = nn.Linear(1152, 1152, bias=True).to(torch.bfloat16)
    lin.weight.data.copy_(W)
    lin.bias.data.copy_(bias)
    w = ActQuantWrapper(lin)
    w.quantizer.configure(bits=4, groupsize=64, sym=sym, high_bits_length=64, quant_dtype="int")
    w.rotation = U
    w._unrot_fused = True
    w._b200_explicit = {"codes": qw, "scales": sw}
    y = w(x.cuda()).float().cpu()
    ops.check_status()
    spec = O.LayerSpec(W, bias, O.QuantCfg(4, 64, sym, 1.0, 64, "int"), rotation=U)
    # (1) the stated tolerance, on the same rotated bf16 tensor: reference quantiser + bf16 linear applied
    #     to the x_rot our kernel produced
    st = w._b200_state
    _, x_rot = ops.rotate_quantize(x.reshape(-1, 1152).cuda(), st.rot_t, st.fmt, want_x_rot=True)
    r = O.act_quant(x_rot.cpu().reshape(x.shape), spec.cfg)
    y_same = torch.nn.functional.linear(r.full, W, bias).float()
    assert rel_l2(y, y_same) <= REL and cosine(y, y_same) >= COS
    # (2) against the reference forwards run end to end on the CPU.  Their own fp32 and bf16 variants
    #     differ by ~3.3e-2 on this input (codes flip where x_rot rounds differently), so that gap,
    #     not 1e-2, bounds any comparison across rotation arithmetic.
    y_slow = O.fused_forward(x, spec, fp32=True).float()
    y_fast = O.fused_forward(x, spec, fp32=False).float()
    gap = rel_l2(y_fast, y_slow)
    assert rel_l2(y, y_slow) <= 1.5 * gap and cosine(y, y_slow) >= COS
    assert rel_l2(y, y_fast) <= 1.5 * gap and cosine(y, y_fast) >= COS


def test_bits16_and_unfused_layers():
    from dirotq_b200 import ops
    from dirotq_b200.wrapper import ActQuantWrapper
    g = torch.Generator().manual_seed(3)
    lin = nn.Linear(256, 128).to(torch.bfloat16).cuda()
    w = ActQuantWrapper(lin)
    x = torch.randn(2, 50, 256, generator=g).to(torch.bfloat16).cuda()
    assert torch.equal(w(x), lin(x))                       # bits == 16: plain module
    # not fused (no rotation), quantised: the reference fake-quantises x and calls the module
    w.quantizer.configure(bits=4, groupsize=64, sym=True, high_bits_length=64, quant_dtype="int")
    Wq, _, _ = O.weight_quant_int(lin.weight.data.float().cpu()[:, :192], 4, 64)
    lin.weight.data[:, :192] = Wq.to(torch.bfloat16).cuda()
    y = w(x).float().cpu()
    ops.check_status()
    spec = O.LayerSpec(lin.weight.data.cpu(), lin.bias.data.cpu(), O.QuantCfg(4, 64, True, 1.0, 64, "int"))
    y_ref = O.fused_forward(x.cpu(), spec, fp32=False).float()
    assert rel_l2(y, y_ref) <= REL


def test_fp16_pipeline_dtype_roundtrip():
    from dirotq_b200 import ops
    g = load_golden("hidden_int4_sym")
    w = _wrapper_from_golden(g)
    y = w(g["x"].to(torch.float16).cuda())
    assert y.dtype == torch.float16
    assert rel_l2(y.float().cpu(), g["y_fast"].float()) <= REL


def test_rotation_api_signature():
    from dirotq_b200.rotation import prepare_U_bf16, bf16_rotation_forward
    g = torch.Generator().manual_seed(4)
    U = O.random_orthogonal(384, g).float().cuda()
    x = torch.randn(500, 384, generator=g).to(torch.bfloat16).cuda()
    Up, sc = prepare_U_bf16(U)
    assert sc is None
    y = bf16_rotation_forward(x, Up, sc, scale_x=None)
    assert rel_l2(y.float().cpu(), (x.float() @ U).cpu()) < 4e-3


@pytest.mark.parametrize("quant", ["int4", "nvfp4"])
def test_sibling_layers_share_one_rotate_quantise_pass(quant):
    """to_q / to_k / to_v carry the same rotation (models/pixart-sigma/model_utils.py:84-92) and are called on
    one tensor: the first call rotates and quantises, the other two run their GEMM on the same codes.  Outputs
    are bit-identical to layers prepared without sharing; a changed or different input is never served from
    the shared codes."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations

    def build():
        attn = nn.Module()
        ws = []
        for i, leaf in enumerate(("to_q", "to_k", "to_v")):
            w = dit.make_wrapped_linear(dit.LayerDef("attn1." + leaf, 384, 256 + 64 * i, tail=64), quant, 77 + i, "cuda")
            if ws:
                w.rotation = ws[0].rotation.clone()
            attn.add_module(leaf, w)
            ws.append(w)
        root = nn.Module()
        root.add_module("attn1", attn)
        return root, ws

    root, ws = build()
    backend.preconvert_rotations_to_device(root, "cuda")
    grp = ws[0]._b200_state.shared
    assert grp is not None and all(w._b200_state.shared is grp for w in ws)
    root2, ws2 = build()
    backend.SHARE_SIBLING_ACTIVATIONS = False
    try:
        backend.preconvert_rotations_to_device(root2, "cuda")
    finally:
        backend.SHARE_SIBLING_ACTIVATIONS = True
    assert all(w._b200_state.shared is None for w in ws2)

    x = synth_activations(300, 384, torch.Generator().manual_seed(9)).reshape(1, 300, 384).cuda()
    ys = [w(x) for w in ws]
    ops.check_status()
    assert (grp.misses, grp.hits) == (1, 2) and grp.x_ref is None
    for y, w2 in zip(ys, ws2):
        assert torch.equal(y, w2(x))
    # the same tensor again: a new pass (every member has used the old codes), then two hits
    ys_again = [w(x) for w in ws]
    assert (grp.misses, grp.hits) == (2, 4)
    assert all(torch.equal(a, b) for a, b in zip(ys, ys_again))
    # in-place change between siblings: the version counter moves, the codes are not reused
    y_q = ws[0](x)
    x.mul_(0.5)
    y_k = ws[1](x)
    assert grp.misses == 4
    assert torch.equal(y_k, ws2[1](x)) and torch.equal(y_q, ys[0])
    # a different tensor
    x2 = synth_activations(300, 384, torch.Generator().manual_seed(10)).reshape(1, 300, 384).cuda()
    assert torch.equal(ws[2](x2), ws2[2](x2))
    # calling one member twice on the same tensor recomputes rather than reusing its own stale slot
    a = ws[0](x2)
    b = ws[0](x2)
    assert torch.equal(a, b)
    ops.check_status()


@pytest.mark.parametrize("name", ["hadamard_int4_sym", "hadamard_int4_sym_n128"])
def test_hadamard_layers(name):
    """use_hadamard layers: the FWHT front end is bit-identical to the reference's fp32 butterflies, so the
    quantised activations and the layer output follow the reference's bf16 forward exactly up to the GEMM's
    accumulation order."""
    from dirotq_b200 import ops
    g = load_golden(name)
    w = _wrapper_from_golden(g)
    low_dim = int(g["low_dim"][0])
    w.use_hadamard, w.hadamard_low_dim, w.hadamard_sign_flips = True, low_dim, g["sign_flips"]
    x = g["x"].cuda()
    x_rot = ops.hadamard_low(x.reshape(-1, x.shape[-1]), low_dim, g["sign_flips"].to(torch.bfloat16).cuda())
    assert torch.equal(x_rot.cpu().view(torch.int16), g["x_rot_fast"].reshape(x_rot.shape).view(torch.int16))
    y = w(x)
    ops.check_status()
    assert w._b200_state.n_lossy_groups == 0
    yc = y.float().cpu()
    assert rel_l2(yc, g["y_fast"].float()) <= REL and cosine(yc, g["y_fast"].float()) >= COS


@pytest.mark.parametrize("D,low_dim", [(4608, 4096), (12288, 8192), (2048, 2048), (576, 512)])
def test_hadamard_front_end_model_sizes(D, low_dim):
    """PixArt ff.net.2 (4608 -> FWHT over 4096) and FLUX-sized widths: bit-identical to the oracle."""
    from dirotq_b200 import ops
    from dirotq_b200.synth import synth_activations
    g = torch.Generator().manual_seed(D)
    x = synth_activations(300, D, g)
    flips = (torch.randint(0, 2, (low_dim,), generator=g).float() * 2 - 1).to(torch.bfloat16)
    y = ops.hadamard_low(x.cuda(), low_dim, flips.cuda()).cpu()
    ref = O.hadamard_low(x, low_dim, flips, fp32=False)
    assert torch.equal(y.view(torch.int16), ref.view(torch.int16))
    y2 = ops.hadamard_low(x.cuda(), low_dim, None).cpu()
    assert torch.equal(y2.view(torch.int16), O.hadamard_low(x, low_dim, None, fp32=False).view(torch.int16))


@pytest.mark.parametrize("quant", ["int4", "int8", "nvfp4"])
def test_gelu_fused_into_the_gemm_epilogue(quant):
    """ff.net.0 = GELU(proj(x)): with the activation fused into the up-projection's epilogue the module returns
    what PyTorch's gelu(approximate="tanh") makes of the unfused bf16 output, up to the hardware tanh."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    ld = dit.LayerDef("ff.net.0.proj", 384, 1536, tail=64)
    w = dit.make_wrapped_linear(ld, quant, 31, "cuda")
    head = dit.GeluProj(w)
    root = nn.Module()
    root.add_module("ff0", head)
    backend.preconvert_rotations_to_device(root, "cuda")
    x = synth_activations(520, 384, torch.Generator().manual_seed(3)).reshape(1, 520, 384).cuda()
    y_plain = head(x)                                           # gelu as a separate PyTorch kernel
    assert backend.fuse_gelu_modules(root) == 1
    assert backend.fuse_gelu_modules(root) == 0                 # idempotent
    y_fused = head(x)
    ops.check_status()
    assert y_fused.dtype == torch.bfloat16 and y_fused.shape == y_plain.shape
    a, b = y_fused.float().cpu(), y_plain.float().cpu()
    assert rel_l2(a, b) < 2e-3 and cosine(a, b) > 0.9999
    # at most one bf16 ulp apart wherever the value is not tiny
    big = b.abs() > 1e-2
    assert float(((a - b).abs()[big] / b.abs()[big]).max()) < 2 ** -6


def test_empty_batch_through_the_wrapper():
    from dirotq_b200 import dit
    w = dit.make_wrapped_linear(dit.LayerDef("attn1.to_q", 256, 128, tail=64), "int4", 5, "cuda")
    y = w(torch.zeros(2, 0, 256, dtype=torch.bfloat16, device="cuda"))
    assert tuple(y.shape) == (2, 0, 128) and y.dtype == torch.bfloat16


def test_resident_weight_panel_through_the_wrapper():
    """backend.CACHE_WEIGHT_PANEL: the layer keeps its fp16 weight panel instead of rebuilding it per call; same bits."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    ld = dit.LayerDef("attn1.to_q", 384, 256, tail=64)
    x = synth_activations(300, 384, torch.Generator().manual_seed(4)).reshape(1, 300, 384).cuda()
    ys = []
    for cache in (False, True):
        old = backend.CACHE_WEIGHT_PANEL
        backend.CACHE_WEIGHT_PANEL = cache
        try:
            w = dit.make_wrapped_linear(ld, "int4", 33, "cuda")
            root = nn.Module()
            root.add_module("to_q", w)
            backend.preconvert_rotations_to_device(root, "cuda")
            ys.append(w(x))
            assert (w._b200_state.folded.panel is not None) == cache
        finally:
            backend.CACHE_WEIGHT_PANEL = old
    ops.check_status()
    assert torch.equal(ys[0].view(torch.int16), ys[1].view(torch.int16))


def test_packed_weight_cache_round_trip(tmp_path, monkeypatch):
    """save_packed_weights / load_packed_weights: a fresh model that loads the file produces the same bits
    without running the grid recovery or the packing kernels again."""
    from dirotq_b200 import backend, dit, ops, pack
    from dirotq_b200.synth import synth_activations

    def build():
        root = nn.Module()
        root.add_module("to_q", dit.make_wrapped_linear(dit.LayerDef("attn1.to_q", 384, 256, tail=64), "int4", 51, "cuda"))
        root.add_module("to_out", dit.make_wrapped_linear(dit.LayerDef("attn1.to_out.0", 384, 384, tail=4, kind="perhead",
                                                                         heads=12, head_dim=32), "int4", 52, "cuda"))
        root.add_module("fp4", dit.make_wrapped_linear(dit.LayerDef("attn2.to_q", 384, 256, tail=64), "nvfp4", 53, "cuda"))
        root.add_module("ff2", dit.make_wrapped_linear(dit.LayerDef("ff.net.2", 512, 384, kind="w4a16"), "int4", 54, "cuda"))
        return root

    x = synth_activations(260, 384, torch.Generator().manual_seed(6)).reshape(1, 260, 384).cuda()
    x2 = synth_activations(260, 512, torch.Generator().manual_seed(7)).reshape(1, 260, 512).cuda()
    a = build()
    backend.preconvert_rotations_to_device(a, "cuda")
    ya = [a.to_q(x), a.to_out(x), a.fp4(x), a.ff2(x2)]
    path = tmp_path / "packed.pt"
    assert backend.save_packed_weights(a, path) == 4

    b = build()
    assert backend.load_packed_weights(b, path) == 4

    def boom(*args, **kw):
        raise AssertionError("the packers must not run when a packed cache entry exists")
    for mod, name in ((ops, "pack_weight_int4"), (ops, "pack_weight_nvfp4"), (pack, "recover_int4_grid"),
                      (pack, "convert_dirotq_low_weight_to_b200"), (pack, "convert_dirotq_low_weight_to_b200_fp4")):
        monkeypatch.setattr(mod, name, boom)
    backend.preconvert_rotations_to_device(b, "cuda")
    yb = [b.to_q(x), b.to_out(x), b.fp4(x), b.ff2(x2)]
    ops.check_status()
    for u, v in zip(ya, yb):
        assert torch.equal(u.view(torch.int16), v.view(torch.int16))

    # a layer configured differently from the cached entry is refused
    c = build()
    backend.load_packed_weights(c, path)
    c.to_q.quantizer.high_bits_length = 128
    with pytest.raises(RuntimeError, match="does not match"):
        backend.preconvert_rotations_to_device(c, "cuda")


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """Failure detection without a fault: with the wait limit set to a few thousand cycles, the epilogue warps of a
    GEMM give up waiting for their first accumulator (a main loop of this size takes far longer), write their code to
    the status word, the kernel drains its copies, frees its tensor memory and RETURNS.  The status is positive and
    has a text; the forward's own watch raises at the next call; after the limit is restored the same call gives
    bit-identical results to a run before the incident."""
    from dirotq_b200 import _lib, backend, dit, ops
    from dirotq_b200.synth import synth_activations
    torch.cuda.synchronize()
    ops.check_status()
    # K = 12288: a tile's main loop runs for tens of microseconds, longer than one suspended poll of a waiting warp
    # (20 us), so the epilogue's wait for its first accumulator is certain to see the limit exceeded
    w = dit.make_wrapped_linear(dit.LayerDef("probe", 12288, 3072, kind="norot", tail=0, source="ff"), "int4", 77, "cuda")
    st = backend.prepare_layer(w, "cuda", w._b200_explicit)
    x = synth_activations(2048, 12288, torch.Generator().manual_seed(2)).cuda()
    y_good = backend.linear_forward(st, x).clone()
    torch.cuda.synchronize()
    ops.check_status()
    try:
        ops.set_wait_limit_cycles(4096)
        backend.linear_forward(st, x)                  # launches; some wait inside runs out and the kernels return
        torch.cuda.synchronize()                       # returns: nothing hangs
    finally:
        ops.set_wait_limit_cycles(0)
    code = int(ops.status_word("cuda")[0].item())
    assert 1 <= code <= 6 and b"timeout" in _lib.lib().dirotq_status_string(code)
    with pytest.raises(RuntimeError, match="timeout"):
        backend.linear_forward(st, x)                  # the product path's own watch reports it, one call later
    torch.cuda.synchronize()
    assert int(ops.status_word("cuda")[0].item()) == 0  # the watch cleared the word when it raised
    y_again = backend.linear_forward(st, x)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(y_again, y_good)
