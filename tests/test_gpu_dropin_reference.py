"""The drop-in claim on the reference's REAL classes: a module wrapped by the reference's add_actquant, weights
quantised by its rtn_quantize_weights / nvfp4_rtn_quantize_weights, forward swapped by this package's patch_forward +
preconvert_rotations_to_device (the two names apply_dirotq.py:188-194 imports, called at :406 and :415) -- against the
reference's own _fused_forward_fast on the CPU.  Needs the unmodified reference under oracle/_ref (placed there by
oracle/make_ref.py, which the build entry runs wherever a checkout of the reference exists)."""
import pytest
import torch
import torch.nn as nn

from conftest import rel_l2, cosine
from oracle import dirotq_oracle as O
from oracle import make_ref

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not make_ref.available(), reason="oracle/_ref not populated")]


class _Attn(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
        self.to_out = nn.ModuleList([nn.Linear(dim, dim), nn.Identity()])


class _Block(nn.Module):
    def __init__(self, dim, inner):
        super().__init__()
        self.attn1 = _Attn(dim)
        self.proj = nn.Linear(dim, inner)


@pytest.mark.parametrize("quant", ["int_sym", "int_asym", "nvfp4"])
def test_reference_wrapper_runs_on_the_b200_backend(quant):
    from dirotq_b200 import backend, ops
    qu, slow, fast = make_ref.load()
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(5)
    dim, inner, heads, M = 256, 512, 4, 300
    model = nn.ModuleDict({"transformer_blocks": nn.ModuleList([_Block(dim, inner)])}).to(torch.bfloat16)
    qu.add_actquant(model)                                                   # the reference's own wrapping pass
    layers = qu.find_qlayers(model, layers=[qu.ActQuantWrapper])
    assert len(layers) == 5 and all(type(w) is qu.ActQuantWrapper for w in layers.values())
    U = O.random_orthogonal(dim, g).float()
    Uh = torch.stack([O.random_orthogonal(dim // heads, g).float() for _ in range(heads)])
    fp4 = quant == "nvfp4"
    for name, w in layers.items():
        if name.endswith("to_out.0") and not fp4:
            w.rotation_per_head, w.num_heads, w.head_dim = Uh, heads, dim // heads
            w.quantizer.configure(bits=4, groupsize=64, sym=(quant == "int_sym"), high_bits_length=8, quant_dtype="int")
        else:
            w.rotation = U
            w.quantizer.configure(bits=4, groupsize=16 if fp4 else 64, sym=(quant != "int_asym"), high_bits_length=64,
                                  quant_dtype="nvfp4" if fp4 else "int")
    if fp4:
        qu.nvfp4_rtn_quantize_weights(model, groupsize=16)
    else:
        qu.rtn_quantize_weights(model, bits=4, groupsize=64, sym=True)       # sets _unrot_fused, weights in the rotated basis
    assert all(w._unrot_fused for w in layers.values())
    x = O.synth_activations(M, dim, g).reshape(2, M // 2, dim)
    saved = qu.ActQuantWrapper.forward
    try:
        # the reference's forward, on the CPU
        qu.ActQuantWrapper.forward = fast._fused_forward_fast
        fast.preconvert_rotations_to_device(model, "cpu", torch.bfloat16)
        with torch.no_grad():
            y_fast = {n: w(x).float() for n, w in layers.items()}
        qu.ActQuantWrapper.forward = slow._fused_forward
        for w in layers.values():                                            # the slow forward wants fp32 rotations
            if w.rotation is not None:
                w.rotation = w.rotation.float()
            if w.rotation_per_head is not None:
                w.rotation_per_head = w.rotation_per_head.float()
        with torch.no_grad():
            y_slow = {n: w(x).float() for n, w in layers.items()}
        # this package's backend on the same objects, exactly as apply_dirotq.py would call it
        backend.patch_forward()
        assert qu.ActQuantWrapper.forward is backend._fused_forward_b200
        n = backend.preconvert_rotations_to_device(model, "cuda")
        assert n == 5
        for name, w in layers.items():
            st = w._b200_state
            assert st.n_lossy_groups == 0, name                              # the RTN grid is recovered without loss
            y = w(x.cuda())
            ops.check_status()
            assert y.dtype == torch.bfloat16 and tuple(y.shape) == tuple(y_fast[name].shape)
            yc = y.float().cpu()
            if fp4:
                # E4M3 group scales are not what the reference's activation quantiser uses: quality bound (QSNR against
                # the unquantised-activation linear no more than 0.5 dB below the reference's own)
                W = w.module.weight.data.float()
                y_fp = torch.nn.functional.linear((x.float().reshape(-1, dim) @ U), W, w.module.bias.data.float()).reshape(yc.shape)
                assert O.qsnr_db(y_fp, yc) >= O.qsnr_db(y_fp, y_fast[name]) - 0.5, name
                assert cosine(yc, y_fast[name]) >= 0.99
            else:
                # the reference's own two forwards differ by `gap` on these small layers (4-bit codes flip where the
                # rotated tensor rounds differently); the backend must be no further from either
                gap = rel_l2(y_fast[name], y_slow[name]) if not name.endswith("to_out.0") else 0.0
                bound = max(1e-2, 1.5 * gap) if gap else 8e-2
                assert rel_l2(yc, y_fast[name]) <= bound and cosine(yc, y_fast[name]) >= 0.995, (name, rel_l2(yc, y_fast[name]), gap)
        groups = {id(w._b200_state.shared) for w in layers.values() if w._b200_state.shared is not None}
        assert len(groups) == 1                                              # to_q / to_k / to_v share one rotate + quantise
    finally:
        qu.ActQuantWrapper.forward = saved
