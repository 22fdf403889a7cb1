"""Multi-GPU (NCCL) checks, skipped on a single-GPU box: tensor-parallel FFN (column/row split + one
all-reduce) equals the unsplit layer; batch shards need no communication."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_ffn_and_dp_on_two_gpus():
    port = 29600 + os.getpid() % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    for quant, r in res.items():
        assert r["dp_equal"], quant
        assert r["tp_rel_l2"] < 1e-2, (quant, r)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_two_devices():
    """Per-device set-up inside the library (shared-memory attribute of every kernel, SM count, status word): the
    same small layers on cuda:0 and then on cuda:1 from ONE process, both against the oracle.  No peer access."""
    import torch.nn as nn
    from dirotq_b200 import backend, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    from oracle import dirotq_oracle as O
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    try:
        g = torch.Generator().manual_seed(11)
        M, D, N, k = 300, 256, 128, 64
        x = O.synth_activations(M, D, g).reshape(1, M, D)
        U = O.random_orthogonal(D, g).float()
        for quant, gs in (("int", 64), ("nvfp4", 16)):
            W_rot = (torch.randn(N, D, generator=g) * 0.05) @ U
            deq = O.weight_quant_int(W_rot[:, : D - k], 4, gs)[0] if quant == "int" else O.weight_quant_nvfp4(W_rot[:, : D - k])[0]
            W = torch.cat([deq, W_rot[:, D - k:]], dim=1).to(torch.bfloat16)
            bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
            outs = []
            for dev in ("cuda:0", "cuda:1"):
                with torch.cuda.device(dev):
                    lin = nn.Linear(D, N).to(torch.bfloat16)
                    lin.weight.data.copy_(W)
                    lin.bias.data.copy_(bias)
                    w = ActQuantWrapper(lin)
                    w.quantizer.configure(bits=4, groupsize=gs, sym=True, high_bits_length=k, quant_dtype=quant)
                    w.rotation, w._unrot_fused = U, True
                    y = w(x.to(dev))
                    ops.check_status(dev)
                    outs.append(y.float().cpu())
            assert torch.equal(outs[0], outs[1]), quant
            if quant == "int":
                spec = O.LayerSpec(W, bias, O.QuantCfg(4, gs, True, 1.0, k, quant), rotation=U)
                y_ref = O.fused_forward(x, spec, fp32=False).float()
                assert float((outs[1] - y_ref).norm() / y_ref.norm()) < 0.05
    finally:
        ActQuantWrapper.forward = saved
