"""Pins the CPU oracle against outputs of the unmodified reference (tests/golden)."""
import pytest
import torch

from conftest import bits_equal, load_golden, rel_l2
from oracle import dirotq_oracle as O

HIDDEN = ["hidden_int4_sym", "hidden_int4_asym", "hidden_int4_pad_notail", "hidden_int8_asym", "hidden_nvfp4",
          "hidden_int4_sym_pertoken", "hidden_int4_asym_pertoken", "hidden_int4_asym_pertoken_pad"]
PERHEAD = ["perhead_int4_sym", "perhead_int4_asym", "perhead_d32_int4_sym", "perhead_nvfp4"]
HADAMARD = ["hadamard_int4_sym", "hadamard_int4_sym_n128"]


def spec_of(g):
    bits, gs, sym, hlen, is_fp4 = [int(v) for v in g["cfg"]]
    cfg = O.QuantCfg(bits, gs, bool(sym), 1.0, hlen, "nvfp4" if is_fp4 else "int")
    spec = O.LayerSpec(g["weight"], g["bias"], cfg, g.get("rotation"), g.get("rotation_per_head"))
    if "low_dim" in g:
        spec.hadamard_low_dim = int(g["low_dim"][0])
        spec.hadamard_sign_flips = g["sign_flips"]
    return spec


@pytest.mark.parametrize("name", HIDDEN + PERHEAD + HADAMARD)
def test_fast_path_bit_exact(name):
    g = load_golden(name)
    spec = spec_of(g)
    xq, r, x_rot = O.quantized_input(g["x"], spec, fp32=False)
    assert bits_equal(x_rot, g["x_rot_fast"])
    assert bits_equal(r.full, g["xq_fast"])
    if "scale_fast" in g:
        assert bits_equal(r.scale.reshape(g["scale_fast"].shape), g["scale_fast"])
        if not spec.cfg.sym:
            assert bits_equal(r.zero.reshape(g["zero_fast"].shape), g["zero_fast"])
    assert bits_equal(O.fused_forward(g["x"], spec, fp32=False), g["y_fast"])


@pytest.mark.parametrize("name", HIDDEN + PERHEAD + HADAMARD)
def test_slow_fp32_path_bit_exact(name):
    g = load_golden(name)
    assert bits_equal(O.fused_forward(g["x"], spec_of(g), fp32=True), g["y_slow"])


@pytest.mark.parametrize("name", HIDDEN)
def test_codes_reconstruct_fake_quant(name):
    """scale * code (and scale * (code - zero)) must BE the reference's fake-quant tensor."""
    g = load_golden(name)
    spec = spec_of(g)
    _, r, _ = O.quantized_input(g["x"], spec, fp32=False)
    B, T, _ = g["x"].shape
    if spec.cfg.quant_dtype == "nvfp4":
        vals = O.e2m1_values(r.codes, torch.bfloat16)
        deq = (vals * r.scale).reshape(B, T, -1)[..., :r.q_len]
    elif spec.cfg.sym:
        deq = (r.scale * r.codes.to(torch.bfloat16)).reshape(B, T, -1)[..., :r.q_len]
        assert int(r.codes.min()) >= -8 and int(r.codes.max()) <= 7
    else:
        deq = (r.scale * (r.codes.to(torch.bfloat16) - r.zero)).reshape(B, T, -1)[..., :r.q_len]
        assert int(r.codes.min()) >= 0 and int(r.codes.max()) <= spec.cfg.maxq
    # value equality: an integer code cannot carry the sign of a -0.0 the fake-quant tensor may hold
    assert torch.equal(deq.to(torch.bfloat16), g["xq_fast"][..., :r.q_len])


def test_quantizer_edge_cases():
    g = load_golden("quantizer_edge")
    xr = g["x_rot"]
    for tag, cfg in [("int4_sym", O.QuantCfg(4, 64, True, 1.0, 64)),
                     ("int4_asym", O.QuantCfg(4, 64, False, 1.0, 64)),
                     ("int8_asym", O.QuantCfg(8, 64, False, 1.0, 64))]:
        r = O.act_quant_int(xr, cfg)
        assert bits_equal(r.full, g["xq_" + tag]), tag
        assert bits_equal(r.scale, g["scale_" + tag]), tag
        if not cfg.sym:
            assert bits_equal(r.zero, g["zero_" + tag]), tag
    r = O.act_quant_int(xr.float(), O.QuantCfg(4, 64, True, 1.0, 64))
    assert bits_equal(r.full, g["xq_int4_sym_f32"])
    # all-zero group -> scale 1, tiny group keeps a tiny scale
    r = O.act_quant_int(xr, O.QuantCfg(4, 64, True, 1.0, 64))
    assert float(r.scale[0, 3, 1, 0]) == 1.0
    # ties land on .5 after the bf16 quotient: round-half-even
    assert bool(((r.codes[0, :, 0, 1:64].float() * 2) % 2 == 0).all())
    rn = O.act_quant_nvfp4(g["x_rot_nvfp4"], O.QuantCfg(4, 16, True, 1.0, 16, "nvfp4"))
    assert bits_equal(rn.full, g["xq_nvfp4"])
    # exact midpoints go to the lower codebook value
    v = O.e2m1_values(rn.codes[0, 0, 0, 1:15])
    assert v.tolist() == [-6, -4, -3, -2, -1.5, -1, -0.5, 0, 0.5, 1, 1.5, 2, 3, 4]


def test_weight_side():
    g = load_golden("weights")
    W = g["W"]
    deq, q, s = O.weight_quant_int(W, 4, 64)
    assert bits_equal(deq, g["wq_int4_g64"])
    assert torch.equal((q.float() * s.unsqueeze(-1)).reshape(48, -1), g["wq_int4_g64"])
    deq, _, _ = O.weight_quant_int(W[:, :189], 4, 63)
    assert bits_equal(deq, g["wq_int4_g63"])
    deq, nib, s = O.weight_quant_nvfp4(W, 16)
    assert bits_equal(deq, g["wq_nvfp4_g16"])
    assert torch.equal((O.e2m1_values(nib) * s.unsqueeze(-1)).reshape(48, -1), g["wq_nvfp4_g16"])


def test_packer_side_tie_rule_differs():
    """speedup/nunchaku_pack.py:63-70 rounds ties toward zero; the accuracy path rounds toward -inf."""
    g = load_golden("weights")
    if "fp_quantize_in" not in g:
        pytest.skip("vectors not generated")
    x = g["fp_quantize_in"]
    ref_idx = g["fp_quantize_idx"]
    cb = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
    ours = O.e2m1_values(O.e2m1_nibbles(O.e2m1_index(x)))
    theirs = cb[ref_idx]
    assert ours.tolist()[:7] == [0.0, -0.5, 0.5, 2.0, -3.0, 4.0, -6.0]
    assert theirs.tolist()[:7] == [0.0, 0.0, 0.5, 2.0, -2.0, 4.0, -4.0]


def test_two_level_nvfp4_weight_quantizer_close_to_reference_recipe():
    """weight_only_nvfp4.py:42-72 uses a per-ROW global scale; ours a per-tensor power of two.
    Both must reconstruct W to E2M1 accuracy and ours must be self-consistent."""
    g = load_golden("weights")
    W = g["W"]
    deq, nib, micro, T = O.weight_quant_nvfp4_hw(W)
    assert T == 2.0 ** round(torch.log2(torch.tensor(T)).item())
    assert float(micro.max()) <= 448.0
    assert rel_l2(deq, W) < 0.12
    again = (O.e2m1_values(nib).reshape(48, -1, 16) * (micro * T).unsqueeze(-1)).reshape(48, -1)
    assert bits_equal(again, deq)


@pytest.mark.parametrize("name", ["weights", "weights_nvfp4_rowscale"])
def test_reference_two_level_nvfp4_weight_recipe_bit_exact(name):
    """speedup/weight_only_nvfp4.py:42-72 (_quantize_nvfp4): codes (planar nibble order), E4M3 micro-scales and the
    per-channel bf16 scale of the unmodified reference, bit for bit -- incl. micro-scales that round to zero, an
    all-zero row and every codebook midpoint of both signs (second fixture)."""
    g = load_golden(name)
    nib, micro, gscale, _ = O.weight_quant_nvfp4_rowscale(g["W"])
    assert torch.equal(O.pack_planar_halves(nib), g["wo_codes"])
    assert torch.equal(micro.view(torch.uint8), g["wo_micro_u8"])
    assert bits_equal(gscale, g["wo_gscale"])
    assert torch.equal(O.unpack_planar_halves(g["wo_codes"]), nib)
    if "wo_dequant_torch" in g:
        # eager dequantiser of the reference (:162-171), bit for bit; the fused one (:96-112) rounds once instead of twice
        assert bits_equal(O.dequant_nvfp4_rowscale(nib, micro, gscale, eager=True), g["wo_dequant_torch"])
        one = O.dequant_nvfp4_rowscale(nib, micro, gscale).float()
        two = g["wo_dequant_torch"].float()
        assert float((one - two).abs().max() / two.abs().max()) < 2.0 ** -7
        if name == "weights_nvfp4_rowscale":
            assert int((micro.float() == 0).sum()) > 0              # the zero-micro-scale rule is exercised
            assert nib[6, :16].tolist() == [7, 0, 0, 1, 9, 2, 10, 3, 11, 4, 12, 5, 13, 6, 14, 0]


def test_formats_roundtrip():
    g = torch.Generator().manual_seed(0)
    c = torch.randint(-8, 8, (5, 128), generator=g)
    assert (O.unpack_planar32(O.pack_planar32(c), True) == c).all()
    n = torch.randint(0, 16, (5, 64), generator=g).to(torch.uint8)
    assert (O.unpack_seq_nibbles(O.pack_seq_nibbles(n)) == n).all()
    sf = torch.randint(1, 255, (130, 17), generator=g).to(torch.uint8)
    buf = O.sf_tile(sf)
    assert buf.numel() == 2 * 8 * 512
    assert (O.sf_untile(buf, 130, 17) == sf).all()


def test_int_linear_matches_fake_quant_linear():
    """The integer GEMM formulation equals the reference's bf16 fake-quant GEMM within tolerance."""
    g = load_golden("hidden_int4_sym")
    spec = spec_of(g)
    _, r, _ = O.quantized_input(g["x"], spec, fp32=False)
    M = g["x"].shape[0] * g["x"].shape[1]
    q_len = r.q_len
    Wl = g["weight"][:, :q_len].float()
    _, qw, sw = O.weight_quant_int(Wl, 4, 64)     # fused weight is already on the grid
    assert rel_l2(qw.float().reshape(96, -1) * sw.repeat_interleave(64, 1), Wl) < 5e-3
    y = O.w4a4_int_linear(r.codes.reshape(M, -1, 64), r.scale.reshape(M, -1), qw, sw,
                          r.tail.reshape(M, -1), g["weight"][:, q_len:], g["bias"])
    assert rel_l2(y, g["y_fast"].reshape(M, -1)) < 1e-2
