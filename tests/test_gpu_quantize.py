"""GPU parity: kernel 1a (quantise), kernel 1 (fused rotate+quantise), kernel 3 (packers) vs the oracle.
Bit-exact for codes, scales, zero points and the passthrough tail."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import dirotq_oracle as O

pytestmark = pytest.mark.gpu


def _ops():
    from dirotq_b200 import ops
    return ops


def _fmts(ops, D=1152):
    return {
        "int4_sym": ops.ActFormat(ops.INT4_SYM, D, tail_len=64),
        "int4_asym": ops.ActFormat(ops.INT4_ASYM, D, tail_len=64),
        "int8_asym": ops.ActFormat(ops.INT8_ASYM, D, tail_len=64),
        "nvfp4_ref": ops.ActFormat(ops.NVFP4_REF, D, tail_len=144, group_size=16),
        "nvfp4_hw": ops.ActFormat(ops.NVFP4_HW, D, tail_len=144, group_size=16, tensor_scale=0.5),
        "int4_sym_pad": ops.ActFormat(ops.INT4_SYM, D, tail_len=0 if D % 64 else 40),
        "perhead72": ops.ActFormat(ops.INT4_SYM, D, tail_len=9, num_heads=D // 72, head_dim=72),
        "perhead72_asym": ops.ActFormat(ops.INT4_ASYM, D, tail_len=9, num_heads=D // 72, head_dim=72),
    }


@pytest.mark.parametrize("name", ["int4_sym", "int4_asym", "int8_asym", "nvfp4_ref", "nvfp4_hw", "int4_sym_pad",
                                  "perhead72", "perhead72_asym"])
def test_quantize_only_bit_exact(name):
    ops = _ops()
    from gpu_helpers import assert_act_matches_oracle
    g = torch.Generator().manual_seed(5)
    M, D = 777, 1152
    x = O.synth_activations(M, D, g)
    x[5, :64] = 0            # all-zero group
    x[6, 64:128] = 1e-7      # tiny group
    fmt = _fmts(ops, D)[name]
    buf = ops.quantize_act(x.cuda(), fmt)
    torch.cuda.synchronize()
    assert_act_matches_oracle(buf, x)


def test_quantize_edge_vectors():
    """Reference-generated adversarial vectors: exact .5 ties, all-zero / tiny / negative-only groups."""
    ops = _ops()
    from gpu_helpers import assert_act_matches_oracle, decode_act
    g = load_golden("quantizer_edge")
    xr = g["x_rot"][0]                                 # [64, 256]
    for mode, tag in [(ops.INT4_SYM, "int4_sym"), (ops.INT4_ASYM, "int4_asym"), (ops.INT8_ASYM, "int8_asym")]:
        fmt = ops.ActFormat(mode, 256, tail_len=64)
        buf = ops.quantize_act(xr.cuda(), fmt)
        dec, r = assert_act_matches_oracle(buf, xr)
        # and directly against the reference's fake-quant output
        s = dec["scale"].unsqueeze(-1)
        c = dec["codes"].to(torch.bfloat16)
        deq = s * c if mode == ops.INT4_SYM else s * (c - dec["zero"].unsqueeze(-1))
        assert torch.equal(deq.reshape(64, -1).to(torch.bfloat16), g["xq_" + tag][0, :, :192])
    xn = g["x_rot_nvfp4"][0]
    buf = ops.quantize_act(xn.cuda(), ops.ActFormat(ops.NVFP4_REF, 64, tail_len=16, group_size=16))
    dec, _ = assert_act_matches_oracle(buf, xn)
    deq = O.e2m1_values(dec["codes"], torch.bfloat16) * dec["scale"].unsqueeze(-1)
    assert torch.equal(deq.reshape(32, -1), g["xq_nvfp4"][0, :, :48])


def test_quantize_with_permutation():
    ops = _ops()
    from gpu_helpers import assert_act_matches_oracle
    g = torch.Generator().manual_seed(6)
    x = O.synth_activations(300, 256, g)
    perm = torch.randperm(256, generator=g)
    fmt = ops.ActFormat(ops.INT4_SYM, 256, tail_len=64)
    buf = ops.quantize_act(x.cuda(), fmt, perm_idx=perm.cuda())
    assert_act_matches_oracle(buf, x[:, perm])


@pytest.mark.parametrize("M,D", [(128, 128), (300, 256), (1000, 1152), (4096, 3072)])
def test_rotation_only(M, D):
    ops = _ops()
    g = torch.Generator().manual_seed(7)
    x = O.synth_activations(M, D, g).cuda()
    U = O.random_orthogonal(D, g).to(torch.bfloat16).cuda()
    y = ops.rotate(x, U.T.contiguous())
    ops.check_status()
    ref = (x.float() @ U.float())
    assert rel_l2(y.float().cpu(), ref.cpu()) < 4e-3     # bf16 output rounding
    ref_bf = (x @ U)
    assert rel_l2(y.float().cpu(), ref_bf.float().cpu()) < 4e-3


@pytest.mark.parametrize("name,M,D", [("int4_sym", 1000, 1152), ("int4_asym", 520, 1152), ("int8_asym", 520, 1152),
                                      ("nvfp4_ref", 520, 1152), ("nvfp4_hw", 1000, 1152), ("int4_sym", 300, 2240),
                                      ("int4_sym_pad", 260, 1152), ("int4_sym", 2048, 3072)])
def test_fused_rotate_quantize_hidden(name, M, D):
    """x_rot = bf16(x @ U) computed on tensor cores; the quantiser applied to THAT tensor must be bit-exact."""
    ops = _ops()
    from gpu_helpers import assert_act_matches_oracle
    g = torch.Generator().manual_seed(8)
    x = O.synth_activations(M, D, g).cuda()
    U = O.random_orthogonal(D, g).to(torch.bfloat16).cuda()
    fmt = _fmts(ops, D)[name]
    buf, x_rot = ops.rotate_quantize(x, U.T.contiguous(), fmt, want_x_rot=True)
    ops.check_status()
    assert rel_l2(x_rot.float().cpu(), (x.float() @ U.float()).cpu()) < 4e-3
    assert_act_matches_oracle(buf, x_rot.cpu())


@pytest.mark.parametrize("H,d,hlen,mode", [(16, 72, 9, "sym"), (16, 72, 9, "asym"), (70, 32, 4, "sym"),
                                           (24, 128, 16, "sym"), (24, 128, 16, "nvfp4"), (5, 64, 16, "nvfp4"),
                                           (9, 64, 32, "nvfp4")])     # 5 x 48 and 9 x 32 slots: a partly filled last chunk
def test_fused_rotate_quantize_per_head(H, d, hlen, mode):
    ops = _ops()
    from gpu_helpers import assert_act_matches_oracle
    g = torch.Generator().manual_seed(9)
    M, D = 390, H * d
    x = O.synth_activations(M, D, g).cuda()
    U_ph = torch.stack([O.random_orthogonal(d, g) for _ in range(H)]).to(torch.bfloat16)
    rot_t = torch.block_diag(*[U_ph[h].T for h in range(H)]).contiguous().cuda()
    if mode == "nvfp4":
        fmt = ops.ActFormat(ops.NVFP4_HW, D, tail_len=hlen, num_heads=H, head_dim=d, group_size=16, tensor_scale=0.5)
        with pytest.raises(RuntimeError):                     # this layout exists only fused with its rotation
            ops.quantize_act(x, fmt)
    else:
        fmt = ops.ActFormat(ops.INT4_SYM if mode == "sym" else ops.INT4_ASYM, D, tail_len=hlen, num_heads=H, head_dim=d)
    buf, x_rot = ops.rotate_quantize(x, rot_t, fmt, want_x_rot=True)
    ops.check_status()
    ref = O.rotate_per_head(x.cpu().unsqueeze(0), U_ph, fp32=True).reshape(M, D)
    assert rel_l2(x_rot.float().cpu(), ref) < 4e-3
    assert_act_matches_oracle(buf, x_rot.cpu())


def test_pack_weight_int4_matches_reference_rtn():
    ops = _ops()
    g = load_golden("weights")
    W = g["W"]                                           # [48, 192] fp32
    for group, ncols in [(64, 192), (63, 189)]:
        pk = ops.pack_weight_int4(W[:, :ncols].cuda(), group)
        deq_ref, q_ref, s_ref = O.weight_quant_int(W[:, :ncols], 4, group)
        codes = O.unpack_planar32(pk.codes.cpu(), True).reshape(48, -1, 64)[:, :, :group]
        assert torch.equal(codes.to(torch.int8), q_ref)
        assert torch.equal(pk.scales.cpu()[:, :48].T, s_ref)
        assert torch.equal(pk.wsum.cpu()[:, :48].T, q_ref.float().sum(-1))
        deq = (codes.float() * pk.scales.cpu()[:, :48].T.unsqueeze(-1)).reshape(48, -1)[:, :ncols]
        assert torch.equal(deq, g["wq_int4_g64" if group == 64 else "wq_int4_g63"])
    # explicit codes + scales round-trip
    q = torch.randint(-8, 8, (40, 128))
    s = torch.rand(40, 2) * 0.015 + 0.005
    pk = ops.pack_weight_int4(q.float().cuda(), 64, scales=s.cuda(), w_is_codes=True)
    assert torch.equal(O.unpack_planar32(pk.codes.cpu(), True), q.to(torch.int16))
    assert torch.equal(pk.scales.cpu()[:, :40].T, s)


def test_pack_weight_nvfp4_matches_oracle():
    ops = _ops()
    g = load_golden("weights")
    W = g["W"]
    deq, nib, micro, T = O.weight_quant_nvfp4_hw(W)
    pk = ops.pack_weight_nvfp4(W.cuda(), T)
    got = O.unpack_seq_nibbles(pk.codes.cpu())[:, :192]
    assert torch.equal(got, nib)
    sf = O.sf_untile(pk.sf.cpu(), 48, 12)
    assert torch.equal(sf.view(torch.float8_e4m3fn).float(), micro)
