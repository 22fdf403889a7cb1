"""GPU parity of the producer-side fusions.  (1) The feed-forward hand-off: the up-projection's GEMM epilogue quantises GELU(up(x)) for the
down-projection (dirotq_linear_forward_chain + dirotq_linear_gemm_prequantised).  Integer work: the codes, group
scales, zero points and 16-bit channels it leaves must equal, bit for bit, what the reference quantiser
(utils/quant_utils.py:255-326, restated in the oracle) makes of the unfused hidden tensor, and the pair's output
must equal the two-step forward's exactly.  (2) q / k / v as one GEMM on weights concatenated along the output
dimension: every member's columns must equal its own GEMM's output exactly."""
import ctypes as C

import pytest
import torch
import torch.nn as nn

from oracle import dirotq_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _patched():
    from dirotq_b200 import backend
    from dirotq_b200.wrapper import ActQuantWrapper
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    yield
    ActQuantWrapper.forward = saved


def _pair(inner, tail_down, a_sym, seed, dim=384, k=64, quant="int4"):
    from dirotq_b200 import backend, dit
    up = dit.make_wrapped_linear(dit.LayerDef("ff.net.0.proj", dim, inner, tail=k), quant, seed, "cuda", a_sym=a_sym)
    down = dit.make_wrapped_linear(dit.LayerDef("ff.net.2", inner, dim, kind="norot", tail=tail_down, source="ff"),
                                   quant, seed + 1, "cuda", a_sym=a_sym)
    ff = nn.Module()
    ff.net = nn.ModuleList([dit.GeluProj(up), nn.Identity(), down])
    root = nn.Module()
    root.add_module("ff", ff)
    backend.preconvert_rotations_to_device(root, "cuda")
    assert backend.fuse_gelu_modules(root) == 1
    return root, ff, up, down


def _regions(st, M):
    """(name, offset, bytes) of the activation buffers at the head of a layer's workspace."""
    from dirotq_b200 import _lib
    L = _lib.lib()
    fmt = st.fmt.c()
    l = _lib.ActLayoutC()
    assert L.dirotq_act_layout_of(C.byref(fmt), C.byref(l)) == 0
    sizes = [("codes", L.dirotq_act_codes_bytes(C.byref(l), M)), ("scales", L.dirotq_act_scales_bytes(C.byref(fmt), C.byref(l), M)),
             ("zeros", L.dirotq_act_zeros_bytes(C.byref(fmt), C.byref(l), M)),
             ("tail", L.dirotq_act_tail_bytes(C.byref(l), M) if l.tail_total > 0 else 0)]
    out, off = [], 0
    for name, n in sizes:
        out.append((name, off, int(n)))
        off += int(n)
    return out, l


@pytest.mark.parametrize("quant,a_sym", [("int4", True), ("int4", False), ("nvfp4", True)])
@pytest.mark.parametrize("M,inner,tail_down", [(520, 1536, 0), (300, 1536, 128), (129, 1472, 64),
                                                (4700, 1536, 128)])     # the last one takes 192-wide column tiles
def test_epilogue_quantises_for_the_down_projection(quant, a_sym, M, inner, tail_down):
    from dirotq_b200 import backend, ops
    from dirotq_b200.synth import synth_activations
    root, ff, up, down = _pair(inner, tail_down, a_sym, 71, quant=quant)
    x = synth_activations(M, 384, torch.Generator().manual_seed(9)).reshape(1, M, 384).cuda()
    hidden = ff.net[0](x)
    y_two_step = ff.net[2](hidden)
    ops.check_status()
    sd = down._b200_state
    ws_two_step = sd.workspace(M, x.device).clone()

    assert backend.fuse_ffn_quantise(root) == 1
    assert backend.fuse_ffn_quantise(root) == 0                 # idempotent
    sd.workspace(M, x.device).zero_()
    hidden2 = ff.net[0](x)
    regions, lay = _regions(sd, M)
    ws_chain = sd.workspace(M, x.device).clone()
    y_chain = ff.net[2](hidden2)
    ops.check_status()
    assert sd.chain_hits == 1
    assert torch.equal(hidden2, hidden)                         # keep_hidden: the bf16 tensor is written as before
    assert torch.equal(y_chain, y_two_step)

    # what the producer's epilogue left, against the quantise-only kernel's buffers ...
    for name, off, n in regions:
        if n == 0:
            continue
        a, b = ws_chain[off:off + n].cpu(), ws_two_step[off:off + n].cpu()
        if name == "scales" and quant == "nvfp4":               # UE4M3 tiles: padding entries are zero in both
            pass
        elif name in ("scales", "zeros"):                       # [n_chunks, ldm] bf16, rows beyond M are padding
            ldm = (M + 7) // 8 * 8
            a = a[:lay.n_scales * ldm * 2].view(torch.int16).reshape(lay.n_scales, ldm)[:, :M]
            b = b[:lay.n_scales * ldm * 2].view(torch.int16).reshape(lay.n_scales, ldm)[:, :M]
        elif name == "codes":
            a, b = a[:M * lay.code_row_bytes], b[:M * lay.code_row_bytes]
        else:
            a, b = a[:M * lay.tail_pitch * 2], b[:M * lay.tail_pitch * 2]
        assert torch.equal(a, b), name

    # ... and against the reference quantiser (the two-level hardware recipe for NVFP4) applied to the hidden tensor
    from gpu_helpers import assert_act_matches_oracle
    view = lambda k: ws_chain[regions[k][1]:regions[k][1] + regions[k][2]] if regions[k][2] else None
    buf = ops.ActBuffers(sd.fmt, sd.layout, M, view(0), view(1), view(2), view(3))
    assert_act_matches_oracle(buf, hidden.reshape(M, -1))


def test_hidden_tensor_not_written_when_nobody_else_reads_it():
    from dirotq_b200 import backend, ops
    from dirotq_b200.synth import synth_activations
    M = 700
    root, ff, up, down = _pair(1536, 128, True, 83)
    x = synth_activations(M, 384, torch.Generator().manual_seed(2)).reshape(1, M, 384).cuda()
    y_two_step = ff.net[2](ff.net[0](x))
    assert backend.fuse_ffn_quantise(root, keep_hidden=False) == 1
    y_chain = ff.net[2](ff.net[0](x))
    ops.check_status()
    assert torch.equal(y_chain, y_two_step)
    # a pair fused before its first forward (the down-projection's workspace and resident panel do not exist yet)
    root_b, ff_b, _, down_b = _pair(1536, 128, True, 83)
    assert backend.fuse_ffn_quantise(root_b, keep_hidden=False) == 1
    y_first = ff_b.net[2](ff_b.net[0](x))
    ops.check_status()
    assert down_b._b200_state.chain_hits == 1 and torch.equal(y_first, y_two_step)
    # a tensor that is not the producer's output takes the ordinary path, and the stale hand-off is dropped
    ff.net[0](x)
    other = torch.randn(1, M, 1536, device="cuda").to(torch.bfloat16)
    hits = down._b200_state.chain_hits
    y_other = ff.net[2](other)
    assert down._b200_state.chain_hits == hits and down._b200_state.handed is None
    y_plain = backend.linear_forward(down._b200_state, other.reshape(M, 1536))
    assert torch.equal(y_other.reshape(M, -1), y_plain)


def test_unsupported_pairs_are_left_alone():
    from dirotq_b200 import backend, dit
    # a rotated down-projection needs the whole row before it can quantise: no hand-off
    up = dit.make_wrapped_linear(dit.LayerDef("ff.net.0.proj", 384, 1536, tail=64), "int4", 5, "cuda")
    down = dit.make_wrapped_linear(dit.LayerDef("ff.net.2", 1536, 384, tail=64, source="ff"), "int4", 6, "cuda")
    ff = nn.Module()
    ff.net = nn.ModuleList([dit.GeluProj(up), nn.Identity(), down])
    root = nn.Module()
    root.add_module("ff", ff)
    backend.preconvert_rotations_to_device(root, "cuda")
    backend.fuse_gelu_modules(root)
    assert backend.fuse_ffn_quantise(root) == 0
    assert not backend.chain_supported(up._b200_state, down._b200_state)


@pytest.mark.parametrize("quant", ["int4", "nvfp4"])
def test_flux_blocks_give_the_same_step_with_the_hand_off(quant):
    """One double-stream and two single-stream FLUX blocks: every feed-forward pair (image, text, single) hands its
    activations over in the epilogue and the step's output does not change by a bit."""
    from dirotq_b200 import backend, denoise, ops
    step = denoise.DenoiseStep("flux", quant, "cuda", n_blocks=1, seed=6100, prepare=True)
    assert backend.fuse_gelu_modules(step) == 4
    inputs = step.example_inputs(1, "cuda", seed=4, tokens=640, text=128)
    with torch.no_grad():
        y_two_step = step(*inputs)
        before = step.kernel_launches_per_step()
        assert backend.fuse_ffn_quantise(step, keep_hidden=False) == 4
        y_chain = step(*inputs)
    ops.check_status()
    assert torch.equal(y_chain, y_two_step)
    assert step.kernel_launches_per_step() == before - 4


@pytest.mark.parametrize("quant,widths", [("int4", (256, 320, 192)), ("nvfp4", (256, 384, 128)), ("int8", (128, 128, 128))])
def test_sibling_layers_run_as_one_gemm(quant, widths):
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations

    def build(seed0):
        attn = nn.Module()
        ws = []
        for i, leaf in enumerate(("to_q", "to_k", "to_v")):
            w = dit.make_wrapped_linear(dit.LayerDef("attn1." + leaf, 384, widths[i], tail=64), quant, seed0 + i, "cuda")
            if ws:
                w.rotation = ws[0].rotation.clone()
            attn.add_module(leaf, w)
            ws.append(w)
        root = nn.Module()
        root.add_module("attn1", attn)
        backend.preconvert_rotations_to_device(root, "cuda")
        return root, ws

    root, ws = build(177)
    root2, ws2 = build(177)                                     # same weights, separate GEMMs
    before = sum(backend.kernel_launches(w._b200_state) for w in ws)
    assert backend.fuse_sibling_gemms(root) == 1
    assert backend.fuse_sibling_gemms(root) == 0                # idempotent
    grp = ws[0]._b200_state.shared
    assert grp.fused is not None and grp.fused.out_features == sum(widths)
    after = sum(backend.kernel_launches(w._b200_state) for w in ws)
    assert after <= before - 2                                  # two GEMM launches fewer (at least)
    M = 700
    x = synth_activations(M, 384, torch.Generator().manual_seed(19)).reshape(1, M, 384).cuda()
    ys = [w(x) for w in ws]
    ops.check_status()
    assert (grp.misses, grp.hits) == (1, 2) and grp.x_ref is None and grp.y_all is None
    for y, w2, n in zip(ys, ws2, widths):
        assert y.shape == (1, M, n)
        assert torch.equal(y, w2(x))
    # head split as the attention does it: a view of the strided columns
    q = ys[0].view(1, -1, widths[0] // 64, 64).transpose(1, 2)
    assert q.shape == (1, widths[0] // 64, M, 64)
    # a group whose members see different tensors gives correct results and stops fusing
    xs = [synth_activations(M, 384, torch.Generator().manual_seed(30 + i)).reshape(1, M, 384).cuda() for i in range(8)]
    for i, xi in enumerate(xs):
        w, w2 = ws[i % 3], ws2[i % 3]
        assert torch.equal(w(xi), w2(xi))
    assert grp.fused is None
    ops.check_status()


def test_step_replayed_from_a_cuda_graph():
    """dit.GraphedCall: a linear-path step with all fusions on, captured once and replayed, returns what the launched
    step returns, follows in-place changes of its input buffer, and leaves the status word clean."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    step = dit.LinearPathStep(dit.flux_double_block(k_down=0), 1, "int4", device="cuda", seed=4100)
    backend.preconvert_rotations_to_device(step, "cuda")
    assert backend.fuse_gelu_modules(step) == 1 and backend.fuse_ffn_quantise(step, keep_hidden=False) == 1
    assert backend.fuse_sibling_gemms(step) == 1
    x = synth_activations(640, 3072, torch.Generator().manual_seed(1)).reshape(1, 640, 3072).cuda()
    with torch.no_grad():
        y_launched = step(x).clone()
        replay = dit.GraphedCall(lambda: step(x))
        assert torch.equal(replay(), y_launched)
        x2 = synth_activations(640, 3072, torch.Generator().manual_seed(2)).reshape(1, 640, 3072).cuda()
        x.copy_(x2)                                             # same buffer, new contents
        y_replayed = replay().clone()
        y2 = step(x2)
    ops.check_status()
    assert torch.equal(y_replayed, y2) and not torch.equal(y_replayed, y_launched)
    assert backend.WATCH_STATUS is True


def test_fusions_at_the_edges():
    """Empty and one-row batches through fused q/k/v groups and feed-forward hand-offs; an explicit output buffer for a
    member of a fused group; dropping held tensors between steps."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    step = dit.LinearPathStep(dit.flux_double_block(k_down=0), 1, "int4", device="cuda", seed=4300)
    backend.preconvert_rotations_to_device(step, "cuda")
    backend.fuse_gelu_modules(step)
    assert backend.fuse_ffn_quantise(step, keep_hidden=False) == 1 and backend.fuse_sibling_gemms(step) == 1
    ref = dit.LinearPathStep(dit.flux_double_block(k_down=0), 1, "int4", device="cuda", seed=4300)   # same weights, no fusion
    backend.preconvert_rotations_to_device(ref, "cuda")
    backend.fuse_gelu_modules(ref)
    for M in (0, 1, 77):
        x = synth_activations(max(M, 1), 3072, torch.Generator().manual_seed(M))[:M].reshape(1, M, 3072).cuda()
        with torch.no_grad():
            y, y_ref = step(x), ref(x)
        assert y.shape == (1, M, 3072) and torch.equal(y, y_ref)
    ops.check_status()
    # a member of a fused group asked to write into the caller's buffer
    q = step.layers[0]._b200_state
    x2d = synth_activations(64, 3072, torch.Generator().manual_seed(5)).cuda()
    out = torch.empty(64, q.out_features, dtype=torch.bfloat16, device="cuda")
    got = backend.linear_forward(q, x2d, out=out)
    assert got is out and torch.equal(out, backend.linear_forward(ref.layers[0]._b200_state, x2d))
    assert backend.release_shared_activations(step) >= 1 and q.shared.x_ref is None and q.shared.y_all is None
    ops.check_status()


def test_sibling_gemm_on_dense_nvfp4_weights_with_per_channel_scales():
    """Dense NVFP4 layers (the reference's quantised cache holds dequantised weights) are packed by the two-level recipe
    with one scale per output channel: a fused q / k / v layer carries the members' scales side by side and the 16-bit
    branch divided by them; every member's columns equal its own GEMM's output."""
    from dirotq_b200 import backend, ops
    from dirotq_b200.wrapper import ActQuantWrapper
    g = torch.Generator().manual_seed(21)
    D, k = 384, 64
    U = O.random_orthogonal(D, g).float()

    def build():
        attn = nn.Module()
        gw = torch.Generator().manual_seed(22)
        for i, (leaf, N) in enumerate((("to_q", 256), ("to_k", 128), ("to_v", 384))):
            W_rot = (torch.randn(N, D, generator=gw) * 0.05 * (1 + i)) @ U
            deq, _, _ = O.weight_quant_nvfp4(W_rot[:, : D - k])
            lin = nn.Linear(D, N, bias=(i != 1)).to(torch.bfloat16)
            lin.weight.data.copy_(torch.cat([deq, W_rot[:, D - k:]], dim=1).to(torch.bfloat16))
            if lin.bias is not None:  # nn.Linear draws its bias from the global generator: both copies take this one
                lin.bias.data.copy_(torch.randn(N, generator=gw).to(torch.bfloat16))
            w = ActQuantWrapper(lin)
            w.quantizer.configure(bits=4, groupsize=16, sym=True, high_bits_length=k, quant_dtype="nvfp4")
            w.rotation = U.clone()
            w._unrot_fused = True
            attn.add_module(leaf, w)
        root = nn.Module()
        root.add_module("attn1", attn)
        backend.preconvert_rotations_to_device(root, "cuda")
        return root, [attn.to_q, attn.to_k, attn.to_v]

    root, ws = build()
    root2, ws2 = build()
    assert all(w._b200_state.w_rowscale is not None for w in ws)
    assert backend.fuse_sibling_gemms(root) == 1
    x = O.synth_activations(500, D, g).reshape(1, 500, D).to(torch.bfloat16).cuda()
    for w, w2 in zip(ws, ws2):
        assert torch.equal(w(x), w2(x))
    assert ws[0]._b200_state.shared.hits == 2
    ops.check_status()


def test_fused_layers_over_changing_row_counts():
    """Workspaces, resident weight panels, shared activations and hand-offs are reused from call to call: a fused q / k / v
    group and a fused feed-forward pair called with a sequence of different row counts return, every time, exactly what
    freshly built, unfused layers return for that input."""
    import contextlib
    import io
    import random
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    rnd = random.Random(5)

    def quiet(fn, *a, **k):
        with contextlib.redirect_stdout(io.StringIO()):
            return fn(*a, **k)

    for case in range(6):
        quant, a_sym = rnd.choice(["int4", "nvfp4", "int8"]), rnd.random() < 0.5
        dim, inner, k = rnd.choice([(384, 1536, 64), (1152, 4608, 64), (256, 512, 0)])

        def build():
            attn = nn.Module()
            ws = [dit.make_wrapped_linear(dit.LayerDef(n, dim, dim, tail=k), quant, 40 + case * 9 + i, "cuda", a_sym=a_sym)
                  for i, n in enumerate(("to_q", "to_k", "to_v"))]
            for n, w in zip(("to_q", "to_k", "to_v"), ws):
                w.rotation = ws[0].rotation
                attn.add_module(n, w)
            up = dit.make_wrapped_linear(dit.LayerDef("ff.net.0.proj", dim, inner, tail=k), quant, 44 + case * 9, "cuda", a_sym=a_sym)
            down = dit.make_wrapped_linear(dit.LayerDef("ff.net.2", inner, dim, kind="norot", tail=0, source="ff"), quant,
                                           45 + case * 9, "cuda", a_sym=a_sym)
            ff = nn.Module()
            ff.net = nn.ModuleList([dit.GeluProj(up), nn.Identity(), down])
            root = nn.Module()
            root.add_module("attn1", attn)
            root.add_module("ff", ff)
            quiet(backend.preconvert_rotations_to_device, root, "cuda")
            quiet(backend.fuse_gelu_modules, root)
            return root, ws, ff

        def run(ws_, ff_, x):
            return [w(x).clone() for w in ws_] + [ff_.net[2](ff_.net[0](x)).clone()]

        root, ws, ff = build()
        assert quiet(backend.fuse_sibling_gemms, root) == 1
        quiet(backend.fuse_ffn_quantise, root, keep_hidden=False)
        for j in range(5):
            M = rnd.choice([1, 7, 129, 500, 2048, 4100, 9000])
            x = synth_activations(M, dim, torch.Generator().manual_seed(case * 100 + j)).reshape(1, M, dim).cuda()
            got = run(ws, ff, x)
            _, ws_f, ff_f = build()
            want = run(ws_f, ff_f, x)
            ops.check_status()
            assert all(torch.equal(a, b) for a, b in zip(got, want)), (case, quant, a_sym, dim, M)
