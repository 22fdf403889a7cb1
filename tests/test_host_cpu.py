"""CPU-only checks of the host side: the C-ABI library loads and exports what include/*.h declares,
layout arithmetic, wrapper API, weight-grid recovery.  No compute calls (no GPU here)."""
import ctypes as C
import os
import re

import pytest
import torch
import torch.nn as nn

from conftest import ROOT, load_golden


def test_library_exports_every_declared_symbol():
    from dirotq_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "dirotq_b200.h")).read()
    declared = set(re.findall(r"\b(dirotq_[a-z0-9_]+)\s*\(", hdr))
    declared -= {"dirotq_linear"}
    assert declared, "no declarations parsed"
    l = C.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(l, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.lib().dirotq_abi_version() == _lib.ABI_VERSION == int(re.search(r"DIROTQ_ABI_VERSION (\d+)", hdr).group(1))
    assert b"aligned" in _lib.lib().dirotq_error_string(-3)


def test_layouts():
    from dirotq_b200 import ops
    l = ops.act_layout(ops.ActFormat(ops.INT4_SYM, 1152, 64))
    assert (l.q_len, l.n_groups, l.n_chunks, l.code_row_bytes, l.tail_pitch) == (1088, 17, 17, 544, 64)
    l = ops.act_layout(ops.ActFormat(ops.INT4_ASYM, 1152, 9, num_heads=16, head_dim=72))
    assert (l.q_len, l.group, l.n_groups, l.k_pad, l.tail_total) == (1008, 63, 16, 1024, 144)
    l = ops.act_layout(ops.ActFormat(ops.INT4_SYM, 3072, 16, num_heads=24, head_dim=128))
    assert (l.group, l.chunks_per_group, l.n_chunks) == (112, 2, 48)
    l = ops.act_layout(ops.ActFormat(ops.INT8_ASYM, 2240, 320))
    assert (l.q_len, l.code_row_bytes) == (1920, 1920)
    l = ops.act_layout(ops.ActFormat(ops.NVFP4_HW, 1152, 144, group_size=16))
    assert (l.q_len, l.n_groups, l.n_chunks) == (1008, 63, 16)
    with pytest.raises(RuntimeError):
        ops.act_layout(ops.ActFormat(ops.NVFP4_HW, 1152, 9, num_heads=16, head_dim=72))   # per-head NVFP4
    with pytest.raises(RuntimeError):
        ops.act_layout(ops.ActFormat(ops.INT4_SYM, 1150, 64))                              # width % 8


def test_wrapper_api_matches_reference_contract():
    from dirotq_b200.wrapper import ActQuantWrapper, add_actquant, find_qlayers

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.to_q = nn.Linear(16, 16)
            self.to_out = nn.ModuleList([nn.Linear(16, 16), nn.Dropout(0.0)])
            self.skip_me = nn.Linear(16, 16)

    m = nn.ModuleDict({"b0": Blk(), "b1": Blk()})
    add_actquant(m, skip_names=["skip_me"])
    q = find_qlayers(m, layers=[ActQuantWrapper])
    assert sorted(q) == ["b0.to_out.0", "b0.to_q", "b1.to_out.0", "b1.to_q"]
    w = q["b0.to_q"]
    for attr in ["rotation", "rotation_per_head", "num_heads", "head_dim", "use_hadamard", "hadamard_sign_flips",
                 "hadamard_low_dim", "perm_idx", "module", "quantizer", "weight", "bias"]:
        assert hasattr(w, attr)
    w.quantizer.configure(bits=4, groupsize=64, sym=False, high_bits_length=64, quant_dtype="int")
    assert int(w.quantizer.maxq) == 15 and w.quantizer.high_bits_length == 64
    w.quantizer.configure(bits=4, groupsize=16, quant_dtype="nvfp4")
    assert w.quantizer.sym and int(w.quantizer.maxq) == 7
    x = torch.randn(2, 3, 16)
    with pytest.raises(RuntimeError):
        w(x)                                            # quantised + unpatched: no eager fallback
    w.quantizer.configure(bits=16)
    assert torch.equal(w(x), w.module(x))


def test_patch_forward_patches_both_classes(monkeypatch):
    import sys
    import types
    from dirotq_b200 import backend
    from dirotq_b200.wrapper import ActQuantWrapper
    fake = types.ModuleType("utils.quant_utils")

    class RefWrapper(nn.Module):
        pass
    fake.ActQuantWrapper = RefWrapper
    monkeypatch.setitem(sys.modules, "utils.quant_utils", fake)
    saved = ActQuantWrapper.forward
    try:
        backend.patch_forward()
        assert ActQuantWrapper.forward is backend._fused_forward_b200
        assert RefWrapper.forward is backend._fused_forward_b200
    finally:
        ActQuantWrapper.forward = saved


def test_grid_recovery_on_reference_quantised_weights():
    from dirotq_b200.pack import recover_int4_grid
    from oracle import dirotq_oracle as O
    g = load_golden("weights")
    wq = g["wq_int4_g64"]                                  # reference RTN output (fp32, exactly q*s)
    rec = recover_int4_grid(wq.to(torch.bfloat16), 64)     # as stored in a bf16 module.weight
    assert rec.n_lossy == 0
    _, q_ref, s_ref = O.weight_quant_int(g["W"], 4, 64)
    q = torch.clamp(torch.round(wq.reshape(48, -1, 64) / rec.scales.unsqueeze(-1)), -8, 7)
    assert torch.equal(q.to(torch.int8), q_ref)
    assert float(((rec.scales - s_ref).abs() / s_ref).max()) < 2.0 ** -8
    # a weight that is NOT on a grid is reported
    rec2 = recover_int4_grid(g["W"], 64)
    assert rec2.n_lossy > 0
    # golden layer weights from the reference pipeline (hidden + per-head layouts)
    gl = load_golden("hidden_int4_sym")
    assert recover_int4_grid(gl["weight"][:, :128], 64).n_lossy == 0
    gp = load_golden("perhead_int4_sym")
    wl = gp["weight"].reshape(96, 4, 72)[:, :, :63].reshape(96, -1)
    assert recover_int4_grid(wl, 63).n_lossy == 0


def test_shared_activation_bookkeeping():
    """The record that lets to_k / to_v reuse to_q's quantised activations: same storage + shape + in-place
    version and a member that has not used it yet; anything else is a miss."""
    import torch
    from dirotq_b200.backend import SharedActivation
    g = SharedActivation(3)
    x = torch.zeros(4, 8)
    assert not g.lookup(x, 0)
    g.store(x, 0)
    assert g.x_ref is x
    assert g.lookup(x.view(4, 8), 1)              # another view of the same storage and shape
    assert not g.lookup(x, 1)                     # member 1 has used it already
    assert not g.lookup(x[:2], 2)                 # different shape
    x.add_(1)                                     # in-place change: version moves
    assert not g.lookup(x, 2)
    g.store(x, 2)
    assert g.lookup(x, 0) and g.lookup(x, 1)
    assert g.x_ref is None                        # every member served: the reference is dropped
    y = torch.zeros(4, 8)
    assert not g.lookup(y, 0)
    assert (g.hits, g.misses) == (3, 2)


def test_shared_activation_survives_reused_output_buffers():
    """A buffer the library itself fills through a raw pointer (out=) must not be mistaken for the tensor quantised
    before: to_q and to_k run on `buf`, a library call then overwrites `buf`, to_v must miss.  And a group whose
    members do not all see the same tensor lets go of it on release()."""
    import torch
    from dirotq_b200 import ops
    from dirotq_b200.backend import SharedActivation
    g = SharedActivation(3)
    buf = torch.zeros(4, 8)
    g.store(buf, 0)
    assert g.lookup(buf, 1)
    ops.mark_written(buf)                          # what every out= path of the library does after its launch
    assert not g.lookup(buf, 2)
    g.store(buf, 2)
    assert g.lookup(buf, 0)
    assert g.x_ref is buf                          # member 1 never came: still held ...
    g.release()
    assert g.x_ref is None and not g.lookup(buf, 1)  # ... until released


def test_sibling_grouping_needs_equal_rotations_and_formats():
    import torch
    import torch.nn as nn
    from dirotq_b200 import backend, ops

    class FakeState:
        def __init__(self, rot, fmt, folded=None):
            self.rot_t, self.fmt, self.folded = rot, fmt, folded
            self.shared, self.member_id, self._c, self._ws = None, 0, None, {}

    class Wrapped(nn.Module):
        pass

    def attn(rots, fmts):
        m = nn.Module()
        for leaf, r, f in zip(("to_q", "to_k", "to_v"), rots, fmts):
            w = Wrapped()
            object.__setattr__(w, "_b200_state", FakeState(r, f))
            m.add_module(leaf, w)
        return m

    f4 = ops.ActFormat(ops.INT4_SYM, 64, tail_len=16)
    f8 = ops.ActFormat(ops.INT8_ASYM, 64, tail_len=16)
    r = torch.eye(64)
    root = nn.Module()
    root.add_module("a", attn([r, r.clone(), r.clone()], [f4, f4, f4]))          # all three equal
    root.add_module("b", attn([r, r.clone(), r * 2], [f4, f4, f4]))              # to_v rotates differently
    root.add_module("c", attn([r, r.clone(), r.clone()], [f4, f8, f4]))          # to_k has another format
    assert backend.share_sibling_activations(root, classes=(Wrapped,)) == 3
    sa = [m._b200_state for m in root.a.children()]
    assert sa[0].shared is sa[1].shared is sa[2].shared and [s.member_id for s in sa] == [0, 1, 2]
    sb = [m._b200_state for m in root.b.children()]
    assert sb[0].shared is sb[1].shared and sb[2].shared is None and sb[0].shared.n_members == 2
    sc = [m._b200_state for m in root.c.children()]
    assert sc[0].shared is sc[2].shared and sc[1].shared is None
