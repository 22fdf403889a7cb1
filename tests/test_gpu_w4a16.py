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
