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


def _linear_c(fmt, out_features, rot=False, perm=False, w_mult=True):
    """A dirotq_linear with dummy (never dereferenced) pointers: enough for the host-side checks of the C ABI."""
    from dirotq_b200._lib import LinearC
    p = lambda on: C.c_void_p(0x1000 if on else 0)
    return LinearC(fmt.c(), out_features, p(rot), p(perm), p(True), p(True), p(True), p(True), p(False), 1.0,
                   p(w_mult), p(True), p(True), 0, p(False))


def test_per_token_layout_and_two_step_workspace():
    """groupsize <= 0: chunks of 64 code slots, one scale slot per chunk; a rotated per-token layer (and a rotated layer
    with a channel selection) asks for M * D * 2 more workspace bytes: the rotation's scratch."""
    from dirotq_b200 import _lib, ops
    tok = ops.ActFormat(ops.INT4_ASYM, 1152, 64, group_size=-1)
    g64 = ops.ActFormat(ops.INT4_ASYM, 1152, 64, group_size=64)
    lt, lg = ops.act_layout(tok), ops.act_layout(g64)
    assert (lt.q_len, lt.group, lt.n_chunks, lt.n_scales, lt.code_row_bytes) == (lg.q_len, 64, lg.n_chunks, lg.n_scales, lg.code_row_bytes)
    l = ops.act_layout(ops.ActFormat(ops.INT4_SYM, 160, 0, group_size=0))
    assert (l.q_len, l.n_chunks, l.k_pad) == (160, 3, 192)
    with pytest.raises(RuntimeError):
        ops.act_layout(ops.ActFormat(ops.NVFP4_HW, 1152, 64, group_size=-1))      # no block-scaled per-token form
    L = _lib.lib()
    M = 1000
    ws = lambda lin: int(L.dirotq_linear_workspace_bytes(C.byref(lin), M))
    base = ws(_linear_c(g64, 1152, rot=True))
    assert ws(_linear_c(tok, 1152, rot=True)) >= base + M * 1152 * 2
    assert ws(_linear_c(g64, 1152, rot=True, perm=True)) >= base + M * 1152 * 2
    assert ws(_linear_c(tok, 1152, rot=False)) == ws(_linear_c(g64, 1152, rot=False))
    # other formats the rotation's epilogue does not quantise: integer groups of 32 / 128 under a hidden rotation, and
    # per-head groups whose 32-column reads would leave the head (72-wide heads with 1 high channel; not with 9)
    for gs in (32, 128):
        f = ops.ActFormat(ops.INT4_SYM, 1152, 64, group_size=gs)
        assert ws(_linear_c(f, 1152, rot=True)) >= ws(_linear_c(f, 1152, rot=False)) + M * 1152 * 2
    ph = lambda t: ops.ActFormat(ops.INT4_SYM, 1152, t, num_heads=16, head_dim=72)
    assert ws(_linear_c(ph(1), 1152, rot=True)) >= ws(_linear_c(ph(1), 1152, rot=False)) + M * 1152 * 2
    assert ws(_linear_c(ph(9), 1152, rot=True)) == ws(_linear_c(ph(9), 1152, rot=False))
    f16 = ops.ActFormat(ops.NVFP4_HW, 1152, 64, group_size=16)
    assert ws(_linear_c(f16, 1152, rot=True, w_mult=False)) == ws(_linear_c(f16, 1152, rot=False, w_mult=False))


def test_chain_support_matrix():
    """Which producer / consumer pairs the epilogue hand-off accepts (dirotq_linear_chain_supported); refusals of
    dirotq_linear_forward_chain come back before anything is launched."""
    from dirotq_b200 import _lib, ops
    L = _lib.lib()
    ok = lambda a, b: bool(L.dirotq_linear_chain_supported(C.byref(a), C.byref(b)))
    up = _linear_c(ops.ActFormat(ops.INT4_SYM, 3072, 384), 12288, rot=True)
    down = lambda **kw: _linear_c(ops.ActFormat(kw.pop("mode", ops.INT4_SYM), 12288, kw.pop("tail", 0), group_size=kw.pop("gs", 64)),
                                  3072, **kw)
    assert ok(up, down()) and ok(up, down(tail=1536)) and ok(up, down(mode=ops.INT4_ASYM))
    assert not ok(up, down(rot=True))                       # a rotation mixes the whole row
    assert not ok(up, down(perm=True))
    assert not ok(up, down(tail=1000))                      # tail not a multiple of 64
    assert not ok(up, down(gs=-1))                          # per-token scale needs the whole row
    assert not ok(up, down(mode=ops.INT8_ASYM))
    assert not ok(up, down(w_mult=False))                   # consumer on the exact-integer GEMM: no folding step
    assert not ok(_linear_c(ops.ActFormat(ops.INT4_SYM, 3072, 384), 12288, rot=True, w_mult=False), down())
    assert not ok(up, _linear_c(ops.ActFormat(ops.INT4_SYM, 6144, 0), 3072))          # width != producer's out_features
    fp4 = lambda D, N, tail, **kw: _linear_c(ops.ActFormat(ops.NVFP4_HW, D, tail, group_size=16, tensor_scale=kw.pop("T", 1.0)),
                                            N, w_mult=False, **kw)
    assert ok(fp4(3072, 12288, 384, rot=True), fp4(12288, 3072, 0))
    assert ok(fp4(3072, 12288, 384, rot=True), fp4(12288, 3072, 1536, T=0.5))
    assert not ok(fp4(3072, 12288, 384, rot=True), fp4(12288, 3072, 0, T=0.75))       # packed quantiser: power-of-two scale
    assert not ok(fp4(3072, 12288, 384, rot=True), down())                            # formats do not mix
    assert not ok(up, fp4(12288, 3072, 0))
    bad = _linear_c(ops.ActFormat(ops.INT4_SYM, 12288, 0), 3072, rot=True)
    rc = L.dirotq_linear_forward_chain(C.byref(up), C.c_void_p(0x1000), 128, None, C.c_void_p(0x1000), 1 << 30, C.byref(bad),
                                       C.c_void_p(0x1000), 1 << 30, None, None)
    assert rc == -2 and b"not supported" in L.dirotq_error_string(rc)


def test_modulation_vectors_are_taken_through_their_views():
    """ops._mod_vec: the per-sample pitch of a modulation vector given as a chunk of a larger tensor (no copy)."""
    from dirotq_b200 import ops
    B, D = 3, 64
    mod = torch.zeros(B, 6 * D, dtype=torch.bfloat16)
    shift, scale = mod[:, None].chunk(6, dim=-1)[:2]                       # [B, 1, D] views, sample stride 6 D
    v, pitch = ops._mod_vec(scale, B, D)
    assert pitch == 6 * D and v.data_ptr() == scale.data_ptr() and v.shape == (B, D)
    table = torch.zeros(B, 6, D, dtype=torch.bfloat16).chunk(6, dim=1)[3]  # adaLN-single: [B, 1, D] of a [B, 6, D] tensor
    v, pitch = ops._mod_vec(table, B, D)
    assert pitch == 6 * D and v.data_ptr() == table.data_ptr()
    v, pitch = ops._mod_vec(torch.zeros(1, D, dtype=torch.bfloat16), B, D)   # one vector shared by all samples
    assert pitch == 0
    assert ops._mod_vec(None, B, D) == (None, 0)
