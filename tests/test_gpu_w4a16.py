"""GPU parity of the W4A16 layer (dequantise + bf16 tcgen05 GEMM) and of the DiT step builder."""
import pytest
import torch

from conftest import rel_l2
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
