"""GPU parity of the W4A16 layer (dequantise + bf16 tcgen05 GEMM) and of the DiT step builder."""
import pytest
import torch

from conftest import bits_equal, load_golden, rel_l2
from oracle import dirotq_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(300, 256, 128), (1000, 1152, 4608), (130, 136, 192)])
def test_w4a16(M, N, K):
    from dirotq_b200 import ops
    g = torch.Generator().manual_seed(21)
    x = O.synth_activations(M, K, g)
    q = torch.randint(-8, 8, (N, K), generator=g)
    s = (torch.rand(N, K // 64, generator=g) * 0.015 + 0.005).to(torch.float16).float()
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    pk = ops.pack_weight_int4(q.float().cuda(), 64, scales=s.cuda(), w_is_codes=True)
    y = ops.gemm_w4a16(x.cuda(), pk, bias.cuda())
    ops.check_status()
    W = (q.reshape(N, -1, 64).float() * s.unsqueeze(-1)).reshape(N, K).to(torch.bfloat16)   # the reference's module.weight
    y_ref = torch.nn.functional.linear(x.float(), W.float(), bias.float())
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3


def test_pixart_step_builder_runs_and_matches_layerwise():
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    try:
        for quant in ("int4", "nvfp4"):
            step = dit.LinearPathStep(dit.pixart_block(), 1, quant, device="cuda", seed=5)
            n = backend.preconvert_rotations_to_device(step, "cuda")
            assert n == 7
            g = torch.Generator().manual_seed(1)
            x = O.synth_activations(512, 1152, g).reshape(2, 256, 1152).cuda()
            y = step(x)
            ops.check_status()
            assert tuple(y.shape) == (2, 256, 1152) and bool(torch.isfinite(y.float()).all())
            lin, rot = step.ops_per_step(512)
            assert lin == 2 * 512 * (6 * 1152 * 1152 + 2 * 1152 * 4608) and rot == 2 * 512 * 7 * 1152 * 1152
    finally:
        ActQuantWrapper.forward = saved


@pytest.mark.parametrize("M,N,K", [(300, 256, 128), (1000, 1152, 4608), (130, 136, 192)])
def test_w4a16_nvfp4_weight(M, N, K):
    """Weight-only NVFP4 (speedup/weight_only_nvfp4.py:128-178): E2M1 codes x UE4M3 group scales x tensor scale,
    dequantised once to bf16, then the bf16 GEMM."""
    from dirotq_b200 import ops
    g = torch.Generator().manual_seed(22)
    x = O.synth_activations(M, K, g)
    nib = torch.randint(0, 16, (N, K), generator=g).to(torch.uint8)
    s = torch.exp(torch.randn(N, K // 16, generator=g) * 0.5 - 4.0)
    T = O.pow2_tensor_scale(float(s.max()))
    micro = O.e4m3_round(s / T)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    pk = ops.pack_weight_nvfp4(nib.float().cuda(), T, scales_e4m3=micro.to(torch.float8_e4m3fn).view(torch.uint8).cuda(),
                               w_is_codes=True)
    y = ops.gemm_w4a16_nvfp4(x.cuda(), pk, bias.cuda())
    ops.check_status()
    W = (O.e2m1_values(nib, torch.float32).reshape(N, -1, 16) * (micro.float() * T).unsqueeze(-1)).reshape(N, K)
    y_ref = torch.nn.functional.linear(x.float(), W.to(torch.bfloat16).float(), bias.float())
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3


def _unpack_rowscale(pk, N, K):
    nib = O.unpack_seq_nibbles(pk.codes.cpu())[:, :K]
    micro = O.sf_untile(pk.sf.cpu(), N, pk.n_chunks * 4)[:, : K // 16]
    return nib, micro, pk.row_scale.cpu()[:N]


@pytest.mark.parametrize("name", ["weights", "weights_nvfp4_rowscale"])
def test_rowscale_packer_bit_exact_vs_reference_vectors(name):
    """dirotq_pack_weight_nvfp4_rowscale against the unmodified reference's _quantize_nvfp4 outputs
    (speedup/weight_only_nvfp4.py:42-72): codes (after undoing its planar nibble order), E4M3 micro-scales and the
    bf16 per-channel scale, bit for bit."""
    from dirotq_b200 import ops
    g = load_golden(name)
    W = g["W"]
    N, K = W.shape
    pk = ops.pack_weight_nvfp4_rowscale(W.cuda())
    nib, micro, rs = _unpack_rowscale(pk, N, K)
    assert torch.equal(nib, O.unpack_planar_halves(g["wo_codes"]))
    assert torch.equal(micro, g["wo_micro_u8"])
    assert bits_equal(rs.to(torch.bfloat16), g["wo_gscale"]) and torch.equal(rs, g["wo_gscale"].float())


@pytest.mark.parametrize("M,N,K", [(300, 256, 128), (1000, 1152, 4608), (130, 136, 192)])
def test_w4a16_nvfp4_rowscale_matches_reference_linear(M, N, K):
    """WeightOnlyNVFP4Linear (speedup/weight_only_nvfp4.py:128-178) end to end: quantise with the reference recipe,
    dequantise + bf16 GEMM.  Codes / scales bit-exact against the oracle restatement (itself pinned to the
    reference's vectors); the dequantised weight bit-exact against the fused dequantiser's arithmetic; the output
    within rel-L2 3e-3 of that dequantiser followed by a linear."""
    from dirotq_b200 import ops
    g = torch.Generator().manual_seed(23)
    x = O.synth_activations(M, K, g)
    W = torch.randn(N, K, generator=g) * 0.05 * torch.exp(torch.randn(N, K // 16, 1, generator=g)).expand(N, K // 16, 16).reshape(N, K)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    pk = ops.pack_weight_nvfp4_rowscale(W.cuda())
    nib, micro_u8, rs = _unpack_rowscale(pk, N, K)
    r_nib, r_micro, r_g, _ = O.weight_quant_nvfp4_rowscale(W)
    assert torch.equal(nib, r_nib) and torch.equal(micro_u8, r_micro.view(torch.uint8)) and torch.equal(rs, r_g.float())
    y = ops.gemm_w4a16_nvfp4(x.cuda(), pk, bias.cuda())
    ops.check_status()
    # identity input rows read the dequantised weight back through the GEMM: bf16 values survive exactly
    if K <= 192:
        eye = torch.eye(K, dtype=torch.bfloat16)
        w_back = ops.gemm_w4a16_nvfp4(eye.cuda(), pk, None).cpu().T.contiguous()
        assert bits_equal(w_back, O.dequant_nvfp4_rowscale(r_nib, r_micro, r_g))
    # the reference's forward dequantises with its fused kernel (one rounding per weight): that is the target
    Wd = O.dequant_nvfp4_rowscale(r_nib, r_micro, r_g)
    y_ref = torch.nn.functional.linear(x.float(), Wd.float(), bias.float())
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3
    # its eager cross-check dequantiser (dequant_torch) rounds the scale product to bf16 first, which moves about a
    # third of the weights by one bf16 ulp: the two reference dequantisers are themselves 2.5e-3 apart
    We = O.dequant_nvfp4_rowscale(r_nib, r_micro, r_g, eager=True)
    y_eager = torch.nn.functional.linear(x.float(), We.float(), bias.float())
    assert rel_l2(y.float().cpu(), y_eager) < 3e-3 + rel_l2(y_ref, y_eager)


def test_weight_only_nvfp4_linear_class_mirrors_reference():
    """Same surface as the reference's WeightOnlyNVFP4Linear (from_linear / forward / dequant / weight_bytes); its
    buffers converted back to the reference's layout equal the reference's own vectors bit for bit."""
    from dirotq_b200.weight_only_nvfp4 import WeightOnlyNVFP4Linear
    g = load_golden("weights_nvfp4_rowscale")
    W = g["W"]
    lin = torch.nn.Linear(W.shape[1], W.shape[0], bias=True)
    lin.weight.data.copy_(W)
    m = WeightOnlyNVFP4Linear.from_linear(lin)
    codes, micro, gscale = m.to_reference_buffers()
    assert torch.equal(codes, g["wo_codes"]) and torch.equal(micro.view(torch.uint8), g["wo_micro_u8"])
    assert bits_equal(gscale, g["wo_gscale"])
    nib, mic, gs, _ = O.weight_quant_nvfp4_rowscale(W)
    assert bits_equal(m.dequant().cpu(), O.dequant_nvfp4_rowscale(nib, mic, gs))
    x = O.synth_activations(200, W.shape[1], torch.Generator().manual_seed(3)).reshape(2, 100, -1)
    y = m(x.cuda()).float().cpu()
    y_ref = torch.nn.functional.linear(x.float(), g["wo_dequant_torch"].float(), lin.bias.data.to(torch.bfloat16).float())
    assert tuple(y.shape) == (2, 100, W.shape[0]) and rel_l2(y, y_ref) < 6e-3     # eager dequantiser: see above
    assert m.weight_bytes() == W.numel() // 2 + W.numel() // 16 + 2 * W.shape[0]
