"""Model-shaped blocks through the patched forward: every wrapped linear of one FLUX.1-dev double- and
single-stream block (hidden 3072, 24 x 128 heads, MLP 12288, per-head out-projection), one SANA-1.6B
block (hidden 2240, 70 x 32 heads; W4A4 and W4A8) and one PixArt-Sigma block with per-head
out-projections.  Each layer is checked against the reference quantiser (oracle) + a dense fp32 linear
on the rotated tensor the kernel produced: rel-L2 <= 1e-2, cosine >= 0.999; the quantised activations
themselves are compared bit for bit."""
import pytest
import torch

from conftest import rel_l2, cosine
from oracle import dirotq_oracle as O
from gpu_helpers import assert_act_matches_oracle, dense_reference_weight, oracle_cfg, to_reference_layout

pytestmark = pytest.mark.gpu

REL, COS = 1e-2, 0.999


@pytest.fixture(autouse=True)
def _patched():
    from dirotq_b200 import backend
    from dirotq_b200.wrapper import ActQuantWrapper
    saved = ActQuantWrapper.forward
    backend.patch_forward()
    yield
    ActQuantWrapper.forward = saved


def _check_layer(w, ld, x):
    """x [B, T, D] on the GPU -> y on the GPU, after comparing with the oracle."""
    from dirotq_b200 import ops
    y = w(x)
    ops.check_status()
    assert y.dtype == x.dtype and tuple(y.shape) == (*x.shape[:-1], ld.out_f)
    x2d = x.reshape(-1, ld.in_f)
    W = dense_reference_weight(w, ld)
    bias = w._b200_explicit["bias"].float().cpu()
    if ld.kind == "w4a16":
        y_ref = x2d.float().cpu() @ W.T + bias
    else:
        st = w._b200_state
        if st.rot_t is not None:
            buf, x_rot = ops.rotate_quantize(x2d, st.rot_t, st.fmt, want_x_rot=True)
        else:
            buf, x_rot = ops.quantize_act(x2d, st.fmt), x2d
        assert_act_matches_oracle(buf, x_rot)
        r = O.act_quant(to_reference_layout(x_rot, st.fmt), oracle_cfg(st.fmt, st.layout))
        xq = r.full
        if st.fmt.num_heads:
            xq = O.per_head_interleave(xq, st.fmt.num_heads, st.fmt.head_dim, st.fmt.tail_len)
        y_ref = xq.float().reshape(-1, ld.in_f) @ W.T + bias
    yc = y.float().cpu().reshape(-1, ld.out_f)
    e, c = rel_l2(yc, y_ref), cosine(yc, y_ref)
    assert e <= REL and c >= COS, (ld.name, e, c)
    return y


def _run_block(block, quant, M, seed):
    from dirotq_b200 import dit
    from dirotq_b200.synth import synth_activations
    step = dit.LinearPathStep(block, 1, quant, device="cuda", seed=seed)
    D = block[0].in_f
    x = synth_activations(M, D, torch.Generator().manual_seed(seed)).reshape(1, M, D).cuda()
    ff = None
    for ld, w in zip(block, step.layers):
        if ld.source == "ff":
            _check_layer(w, ld, ff)
        else:
            y = _check_layer(w, ld, x)
            if ld.out_f > ld.in_f:
                ff = torch.nn.functional.gelu(y, approximate="tanh") * 0.25


def test_flux_double_stream_block():
    from dirotq_b200 import dit
    _run_block(dit.flux_double_block(), "int4", 392, 3000)


def test_flux_single_stream_block():
    from dirotq_b200 import dit
    _run_block(dit.flux_single_block(), "int4", 264, 3100)


def test_flux_rotated_down_projection():
    """The dense [12288, 12288] rotation before ff.net.2 (k = 1536), as the accuracy path runs it."""
    from dirotq_b200 import dit
    blk = [ld for ld in dit.flux_double_block(rotate_down=True) if ld.name.startswith("ff.")]
    _run_block(blk, "int4", 200, 3200)


@pytest.mark.parametrize("quant", ["int4", "int8"])
def test_sana_block(quant):
    from dirotq_b200 import dit
    _run_block(dit.sana_block(), quant, 520, 4000)


def test_pixart_block_with_per_head_out_projections():
    from dirotq_b200 import dit
    _run_block(dit.pixart_block(per_head_out=True), "int4", 300, 1000)


def test_pixart_block_nvfp4_layers_run():
    """NVFP4 block (hidden-rotation layers; the per-head ones stay INT4): finite outputs, status clean.
    Bit parity of the NVFP4 formats is covered by the quantiser and GEMM tests."""
    from dirotq_b200 import dit, ops
    from dirotq_b200.synth import synth_activations
    step = dit.LinearPathStep(dit.pixart_block(), 1, "nvfp4", device="cuda", seed=2000)
    x = synth_activations(512, 1152, torch.Generator().manual_seed(2)).reshape(2, 256, 1152).cuda()
    y = step(x)
    ops.check_status()
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("quant", ["int4", "nvfp4"])
def test_full_size_rows_are_independent(quant):
    """BASELINE config 1 size (M = 8 x 4096 rows): a quantised linear treats every token on its own, so
    (1) the forward of the whole batch equals, bit for bit, the forwards of its shards put together (the
    property data-parallel sharding relies on), and (2) permuting the rows permutes the output."""
    from dirotq_b200 import dit, ops
    from dirotq_b200.synth import synth_activations
    M, D = 32768, 1152
    w = dit.make_wrapped_linear(dit.LayerDef("attn1.to_q", D, D, tail=64), quant, 4242, "cuda")
    x = synth_activations(M, D, torch.Generator().manual_seed(42)).cuda()
    y = w(x.reshape(8, 4096, D)).reshape(M, D)
    ops.check_status()
    assert torch.isfinite(y.float()).all()
    parts = [w(x[i * 4096:(i + 1) * 4096].reshape(1, 4096, D)).reshape(4096, D) for i in range(8)]
    assert torch.equal(torch.cat(parts), y)
    odd = torch.cat([w(x[:12345].reshape(1, 12345, D)).reshape(12345, D),
                     w(x[12345:].reshape(1, M - 12345, D)).reshape(M - 12345, D)])      # ragged split
    assert torch.equal(odd, y)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(1)).cuda()
    assert torch.equal(w(x[perm].reshape(1, M, D)).reshape(M, D), y[perm])
    ops.check_status()


def test_host_streamed_step_returns_the_same_result():
    """dit.HostStreamedStep: input copied from pinned memory and result copied back on side streams, call after call."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    step = dit.LinearPathStep(dit.pixart_block(64), 1, "int4", "cuda", seed=1000)
    backend.preconvert_rotations_to_device(step, "cuda")
    x_host = synth_activations(512, 1152, torch.Generator().manual_seed(9)).reshape(1, 512, 1152).pin_memory()
    y_ref = step(x_host.cuda())
    y_host = torch.empty(tuple(y_ref.shape), dtype=torch.bfloat16).pin_memory()
    run = dit.HostStreamedStep(step, x_host, y_host, "cuda")
    for _ in range(3):
        run()
    run.finish()
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(y_host.view(torch.int16), y_ref.cpu().view(torch.int16))
    # the same replayed from CUDA graphs (one per input buffer), with a new input on every call
    run.enable_graphs()
    for seed in (10, 11, 12, 13, 14):
        x_new = synth_activations(512, 1152, torch.Generator().manual_seed(seed)).reshape(1, 512, 1152)
        torch.cuda.synchronize()                            # the previous call's copy of x_host has been made
        x_host.copy_(x_new)
        run()
        run.finish()
        torch.cuda.synchronize()
        assert torch.equal(y_host.view(torch.int16), step(x_new.cuda()).cpu().view(torch.int16)), seed
    ops.check_status()


@pytest.mark.parametrize("quant,a_sym", [("int4", True), ("int4", False), ("int8", False)])
@pytest.mark.parametrize("H,M", [(70, 300), (5, 300), (7, 9000)])
def test_short_per_head_groups_share_operand_stages(quant, a_sym, H, M, monkeypatch):
    """Per-head groups of 28 channels (SANA: d = 32, 4 of them 16-bit) occupy 64-slot chunks that are half padding; the
    16-bit-conversion GEMM packs the first halves of two chunks into one operand stage.  Odd and even head counts,
    a small batch (resident weight panel) and a large one (panel rebuilt per call), all three activation formats."""
    from dirotq_b200 import _lib, backend, dit
    from dirotq_b200.synth import synth_activations
    import ctypes as C
    monkeypatch.setattr(backend, "PANEL_CACHE_BUDGET_FRACTION", 0.0)      # large batches rebuild the panel per call
    ld = dit.LayerDef("attn1.to_out.0", H * 32, 256, kind="perhead", tail=4, heads=H, head_dim=32)
    w = dit.make_wrapped_linear(ld, quant, 900 + H, "cuda", a_sym=a_sym)
    holder = torch.nn.ModuleDict({"l": w})
    backend.preconvert_rotations_to_device(holder, "cuda")
    st = w._b200_state
    assert _lib.lib().dirotq_linear_uses_half_chunks(C.byref(st.c_struct())) == 1
    x = synth_activations(M, H * 32, torch.Generator().manual_seed(H)).reshape(1, M, H * 32).cuda()
    y = _check_layer(w, ld, x)
    assert (st.folded.panel is not None) == (M <= backend.PANEL_CACHE_MAX_ROWS)
    if st.folded.panel is not None:
        assert st.folded.panel.shape == (256, (H + 1) // 2 * 64)
    assert torch.equal(w(x), y)                                 # second call: same result with the panel in place
    if M > backend.PANEL_CACHE_MAX_ROWS:
        # with room in the device's budget for 16-bit weight copies a large batch keeps its panel too: same bits
        monkeypatch.setattr(backend, "PANEL_CACHE_BUDGET_FRACTION", 1.0 / 16)
        st.panel_declined = False
        assert torch.equal(w(x), y) and st.folded.panel is not None and st.folded.panel.shape == (256, (H + 1) // 2 * 64)
        assert torch.equal(w(x), y)
