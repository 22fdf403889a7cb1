"""GPU parity of kernel 2: int32 per-chunk accumulators bit-exact, layer outputs within bf16 rounding
of the exact-arithmetic oracle (rel-L2 <= 3e-3 here; the end-to-end bound vs the reference is 1e-2)."""
import pytest
import torch

from conftest import rel_l2, cosine
from oracle import dirotq_oracle as O

pytestmark = pytest.mark.gpu


def _setup_int(ops, M, N, fmt, seed):
    from gpu_helpers import decode_act
    g = torch.Generator().manual_seed(seed)
    x = O.synth_activations(M, fmt.width, g)
    act = ops.quantize_act(x.cuda(), fmt)
    lay = act.layout
    dec = decode_act(act)
    n_low = lay.n_groups * lay.group if fmt.num_heads else lay.q_len
    qw = torch.randint(-8, 8, (N, n_low), generator=g)
    n_groups_w = (n_low + lay.group - 1) // lay.group
    sw = (torch.rand(N, n_groups_w, generator=g) * 0.015 + 0.005).to(torch.float16).float()
    pk = ops.pack_weight_int4(qw.float().cuda(), lay.group, scales=sw.cuda(), w_is_codes=True)
    w_tail = (torch.randn(N, lay.tail_total, generator=g) * 0.02).to(torch.bfloat16) if lay.tail_total else None
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    return x, act, dec, qw, sw, pk, w_tail, bias


def _oracle_int(dec, lay, qw, sw, w_tail, bias, asym):
    M = dec["codes"].shape[0]
    N = qw.shape[0]
    pad = lay.n_groups * lay.group - qw.shape[1]
    qwp = torch.nn.functional.pad(qw, (0, pad)).reshape(N, lay.n_groups, lay.group)
    cx = dec["codes"].clone()
    # slots beyond q_len in a partial last group hold no data
    if pad:
        cx[:, -1, lay.group - pad:] = 0
    zero = dec["zero"].float() if asym else None
    y = O.w4a4_int_linear(cx, dec["scale"].float(), qwp, sw, dec.get("tail"), w_tail, bias, zero_x=zero)
    cxi = cx.to(torch.int32)
    if asym:
        cxi = cxi - zero.to(torch.int32).unsqueeze(-1)
        if pad:
            cxi[:, -1, lay.group - pad:] = 0
    acc = O.int_group_accumulators(cxi, qwp)
    return y, acc


@pytest.mark.parametrize("mode,M,N,D,tail", [("sym", 300, 256, 320, 64), ("sym", 1000, 1152, 1152, 64),
                                             ("asym", 520, 384, 1152, 64), ("int8", 520, 384, 1152, 64),
                                             ("sym", 260, 128, 256, 0), ("sym", 200, 136, 160, 0),
                                             ("sym", 2048, 3072, 3072, 384)])
def test_int_gemm_hidden(mode, M, N, D, tail):
    from dirotq_b200 import ops
    m = {"sym": ops.INT4_SYM, "asym": ops.INT4_ASYM, "int8": ops.INT8_ASYM}[mode]
    fmt = ops.ActFormat(m, D, tail_len=tail)
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, M, N, fmt, 11)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    y, dump = ops.gemm_w4a4_int(act, pk, wt, bias.cuda(), dump_acc=True)
    ops.check_status()
    y_ref, acc_ref = _oracle_int(dec, lay, qw, sw, w_tail, bias, mode != "sym")
    assert torch.equal(dump.cpu(), acc_ref.to(torch.int32)), "int32 accumulators differ"
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3
    assert cosine(y.float().cpu(), y_ref) > 0.9999


@pytest.mark.parametrize("H,d,hlen", [(16, 72, 9), (6, 32, 4), (4, 128, 16)])
def test_int_gemm_per_head(H, d, hlen):
    from dirotq_b200 import ops
    fmt = ops.ActFormat(ops.INT4_SYM, H * d, tail_len=hlen, num_heads=H, head_dim=d)
    M, N = 390, 256
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, M, N, fmt, 12)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    y, dump = ops.gemm_w4a4_int(act, pk, wt, bias.cuda(), dump_acc=True)
    ops.check_status()
    y_ref, acc_ref = _oracle_int(dec, lay, qw, sw, w_tail, bias, False)
    cpg = lay.chunks_per_group
    got = dump.cpu().reshape(lay.n_groups, cpg, M, N).sum(1)
    assert torch.equal(got, acc_ref.to(torch.int32))
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3


@pytest.mark.parametrize("M,N,D,tail", [(128, 128, 320, 64), (300, 256, 320, 64), (1000, 1152, 1152, 144),
                                        (520, 384, 1152, 64), (260, 128, 256, 0), (2048, 3072, 3072, 384)])
def test_nvfp4_gemm(M, N, D, tail):
    from dirotq_b200 import ops
    from gpu_helpers import decode_act
    g = torch.Generator().manual_seed(13)
    Tx = 0.5
    fmt = ops.ActFormat(ops.NVFP4_HW, D, tail_len=tail, group_size=16, tensor_scale=Tx)
    x = O.synth_activations(M, D, g)
    act = ops.quantize_act(x.cuda(), fmt)
    lay = act.layout
    dec = decode_act(act)
    nib_w = torch.randint(0, 16, (N, lay.q_len), generator=g).to(torch.uint8)
    # log-normal group scales rounded to E4M3, fp32 (power-of-two) tensor scale
    s = torch.exp(torch.randn(N, lay.n_groups, generator=g) * 0.5 - 4.0)
    Tw = O.pow2_tensor_scale(float(s.max()))
    micro_w = O.e4m3_round(s / Tw)
    pk = ops.pack_weight_nvfp4(nib_w.float().cuda(), Tw,
                               scales_e4m3=micro_w.to(torch.float8_e4m3fn).view(torch.uint8).cuda(), w_is_codes=True)
    w_tail = (torch.randn(N, lay.tail_total, generator=g) * 0.02).to(torch.bfloat16) if tail else None
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    wts = None
    if tail:
        wts = ops.pad_tail_weight((w_tail.float() / (Tx * Tw)).to(torch.bfloat16), lay.tail_pitch, N, "cuda")
        assert torch.equal(wts[:, :tail].float().cpu() * (Tx * Tw), w_tail.float())   # power of two: exact
    y = ops.gemm_w4a4_nvfp4(act, pk, wts, bias.cuda())
    ops.check_status()
    nib_x = dec["codes"].reshape(M, -1)[:, : lay.q_len]
    pad = (-lay.q_len) % 16
    if pad:
        nib_x = torch.nn.functional.pad(nib_x, (0, pad)); nib_w = torch.nn.functional.pad(nib_w, (0, pad))
    y_ref = O.w4a4_nvfp4_linear(nib_x, dec["scale"], Tx, nib_w, micro_w, Tw, dec.get("tail"), w_tail, bias)
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3
    assert cosine(y.float().cpu(), y_ref) > 0.9999


@pytest.mark.parametrize("M,N,D,tail", [(300, 256, 320, 64), (1000, 1152, 1152, 144), (260, 136, 256, 0)])
def test_nvfp4_gemm_per_channel_weight_scale(M, N, D, tail):
    """Weights by the reference's two-level recipe (per-output-channel scale, speedup/weight_only_nvfp4.py:42-72):
    the GEMM applies the channel scale in its epilogue, the 16-bit branch is pre-divided by it."""
    from dirotq_b200 import ops
    from gpu_helpers import decode_act
    g = torch.Generator().manual_seed(14)
    Tx = 1.0
    fmt = ops.ActFormat(ops.NVFP4_HW, D, tail_len=tail, group_size=16, tensor_scale=Tx)
    x = O.synth_activations(M, D, g)
    act = ops.quantize_act(x.cuda(), fmt)
    lay = act.layout
    dec = decode_act(act)
    W = torch.randn(N, lay.q_len, generator=g) * 0.05 * torch.exp(torch.randn(N, 1, generator=g))   # channel scales vary
    pk = ops.pack_weight_nvfp4_rowscale(W.cuda())
    nib_w, micro_w, g_bf16, _ = O.weight_quant_nvfp4_rowscale(W)
    assert torch.equal(O.unpack_seq_nibbles(pk.codes.cpu())[:, : lay.q_len], nib_w)
    assert torch.equal(pk.row_scale.cpu()[:N], g_bf16.float())
    w_tail = (torch.randn(N, lay.tail_total, generator=g) * 0.02).to(torch.bfloat16) if tail else None
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    wts = None
    if tail:
        wts = ops.pad_tail_weight((w_tail.float() / (Tx * g_bf16.float()[:, None])).to(torch.bfloat16), lay.tail_pitch, N, "cuda")
    y = ops.gemm_w4a4_nvfp4(act, pk, wts, bias.cuda())
    ops.check_status()
    nib_x = dec["codes"].reshape(M, -1)[:, : lay.q_len]
    eff_w = micro_w.float().double() * g_bf16.double()[:, None]           # per-group effective weight scale
    y_ref = O.w4a4_nvfp4_linear(nib_x, dec["scale"], Tx, nib_w, eff_w, 1.0, dec.get("tail"), w_tail, bias)
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3
    assert cosine(y.float().cpu(), y_ref) > 0.9999


# ---- INT4 at tensor rate: codes expanded to fp16 next to the tensor core, one fp32 accumulator ----------
@pytest.mark.parametrize("mode,M,N,D,tail", [("sym", 300, 256, 320, 64), ("sym", 1000, 1152, 1152, 64),
                                             ("asym", 520, 384, 1152, 64), ("sym", 260, 128, 256, 0),
                                             ("sym", 200, 136, 160, 0), ("asym", 130, 512, 256, 8),
                                             ("sym", 2048, 3072, 3072, 384), ("sym", 700, 4608, 1152, 64),
                                             ("int8", 520, 384, 1152, 64), ("int8", 300, 256, 320, 0),
                                             ("int8", 1000, 2240, 2240, 320), ("int8", 200, 136, 160, 0)])
def test_int4_f16_gemm_hidden(mode, M, N, D, tail):
    from dirotq_b200 import ops
    m = {"sym": ops.INT4_SYM, "asym": ops.INT4_ASYM, "int8": ops.INT8_ASYM}[mode]
    fmt = ops.ActFormat(m, D, tail_len=tail)
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, M, N, fmt, 21)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, lay.tail_total)
    y = ops.gemm_w4a4_int_f16(act, pk, folded, bias.cuda())
    ops.check_status()
    y_ref, _ = _oracle_int(dec, lay, qw, sw, w_tail, bias, mode != "sym")
    y_int = ops.gemm_w4a4_int(act, pk, wt, bias.cuda())
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3
    assert cosine(y.float().cpu(), y_ref) > 0.9999
    # against the exact-integer kernel: both round the same fp32 value to bf16 up to the weights' fp16 rounding
    assert rel_l2(y.float().cpu(), y_int.float().cpu()) < 3e-3


@pytest.mark.parametrize("H,d,hlen,mode", [(16, 72, 9, "sym"), (6, 32, 4, "sym"), (4, 128, 16, "sym"), (6, 32, 4, "int8")])
def test_int4_f16_gemm_per_head(H, d, hlen, mode):
    from dirotq_b200 import ops
    fmt = ops.ActFormat(ops.INT8_ASYM if mode == "int8" else ops.INT4_SYM, H * d, tail_len=hlen, num_heads=H, head_dim=d)
    M, N = 390, 256
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, M, N, fmt, 22)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, lay.tail_total)
    y = ops.gemm_w4a4_int_f16(act, pk, folded, bias.cuda())
    ops.check_status()
    y_ref, _ = _oracle_int(dec, lay, qw, sw, w_tail, bias, mode == "int8")
    assert rel_l2(y.float().cpu(), y_ref) < 3e-3


def test_int4_f16_gemm_wide_dynamic_range():
    """Rows and columns whose scales differ by many orders of magnitude: the per-row / per-column powers
    of two keep every fp16 operand in range; the result still matches exact arithmetic."""
    from dirotq_b200 import ops
    from gpu_helpers import decode_act
    M, N, D, tail = 256, 256, 576, 64
    g = torch.Generator().manual_seed(23)
    x = O.synth_activations(M, D, g).float()
    x *= torch.logspace(-6, 5, M).unsqueeze(1)               # rows from 1e-6 to 1e5
    x[:, 64:128] *= 300.0                                    # one loud group, one nearly silent
    x[:, 128:192] *= 1e-3
    x = x.to(torch.bfloat16)
    fmt = ops.ActFormat(ops.INT4_SYM, D, tail_len=tail)
    act = ops.quantize_act(x.cuda(), fmt)
    lay = act.layout
    dec = decode_act(act)
    qw = torch.randint(-8, 8, (N, lay.q_len), generator=g)
    sw = (torch.rand(N, lay.n_groups, generator=g) * 0.015 + 0.005) * torch.logspace(-5, 3, N).unsqueeze(1)
    pk = ops.pack_weight_int4(qw.float().cuda(), 64, scales=sw.cuda(), w_is_codes=True)
    w_tail = (torch.randn(N, tail, generator=g) * 0.02 * torch.logspace(-5, 3, N).unsqueeze(1)).to(torch.bfloat16)
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, tail)
    y = ops.gemm_w4a4_int_f16(act, pk, folded, None).float().cpu()
    ops.check_status()
    y_ref, _ = _oracle_int(dec, lay, qw, sw, w_tail, None, False)
    assert torch.isfinite(y).all()
    # row-wise: every row, however small, is resolved (a global norm would hide the small rows)
    err = (y - y_ref).norm(dim=1) / y_ref.norm(dim=1).clamp_min(1e-30)
    assert float(err.max()) < 6e-3, float(err.max())


@pytest.mark.parametrize("mode,M,N,D,tail", [("sym", 1, 8, 64, 0), ("sym", 127, 8, 128, 64), ("asym", 129, 200, 192, 8),
                                             ("int8", 1, 16, 64, 0), ("int8", 130, 24, 128, 64), ("sym", 5, 1152, 1152, 64),
                                             ("sym", 300, 200, 64, 0), ("int8", 64, 192, 384, 320)])
def test_int_f16_gemm_edge_shapes(mode, M, N, D, tail):
    """Single rows, output widths below one tile, one- and two-chunk K, tails wider than the quantised part."""
    from dirotq_b200 import ops
    m = {"sym": ops.INT4_SYM, "asym": ops.INT4_ASYM, "int8": ops.INT8_ASYM}[mode]
    fmt = ops.ActFormat(m, D, tail_len=tail)
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, M, N, fmt, 31)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, lay.tail_total)
    y = ops.gemm_w4a4_int_f16(act, pk, folded, bias.cuda())
    ops.check_status()
    y_ref, _ = _oracle_int(dec, lay, qw, sw, w_tail, bias, mode != "sym")
    assert rel_l2(y.float().cpu(), y_ref) < 4e-3


def test_int_f16_gemm_empty_batch():
    from dirotq_b200 import ops
    fmt = ops.ActFormat(ops.INT4_SYM, 128, tail_len=64)
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, 8, 16, fmt, 32)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, 16, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, lay.tail_total)
    empty = ops.quantize_act(x[:0].cuda(), fmt)
    y = ops.gemm_w4a4_int_f16(empty, pk, folded, bias.cuda())
    assert tuple(y.shape) == (0, 16)
    ops.check_status()


# K order of a 64-slot chunk in the expanded operands: per planar-32 block (byte j = code j | code 16+j << 4),
# per 32-bit word wi of the block: low nibbles of bytes 0 and 2, high nibbles of bytes 0 and 2, then bytes 1 and 3
def _panel_k_order():
    order = []
    for b in range(2):
        for wi in range(4):
            for j in (4 * wi, 4 * wi + 2, 16 + 4 * wi, 16 + 4 * wi + 2, 4 * wi + 1, 4 * wi + 3, 16 + 4 * wi + 1, 16 + 4 * wi + 3):
                order.append(32 * b + j)
    return torch.tensor(order)


@pytest.mark.parametrize("N,D,tail", [(256, 320, 64), (1152, 1152, 64), (136, 160, 0)])
def test_weight_panel_f16_is_the_single_rounding_of_the_folded_product(N, D, tail):
    """dirotq_expand_weight_panel_f16: element = fp16((q + 8) * 2^-24 * mult - 8 s') with ONE rounding, mult and the
    addend being the fp16 record of its (chunk, channel); checked bit for bit against float64 arithmetic."""
    from dirotq_b200 import ops
    fmt = ops.ActFormat(ops.INT4_SYM, D, tail_len=tail)
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, 8, N, fmt, 41)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, N, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, lay.tail_total)
    panel = ops.expand_weight_panel_f16(pk, folded).cpu()
    assert panel.dtype == torch.float16 and tuple(panel.shape) == (N, lay.n_chunks * 64)
    ldn = folded.mult.numel() // (8 * lay.n_chunks)
    rec = folded.mult.cpu().view(torch.float16).reshape(lay.n_chunks, ldn, 4)[:, :N]       # {mult, mult, add, add}
    mult, add = rec[..., 0].double().t(), rec[..., 2].double().t()                          # [N, n_chunks]
    assert torch.equal(rec[..., 0], rec[..., 1]) and torch.equal(rec[..., 2], rec[..., 3])
    q = torch.zeros(N, lay.n_chunks * 64, dtype=torch.float64)
    q[:, : qw.shape[1]] = qw.double()
    q = q.reshape(N, lay.n_chunks, 64)[:, :, _panel_k_order()]
    # codes are stored offset-binary (q + 8) as subnormal fp16 (q + 8) * 2^-24
    want = ((q + 8.0) * 2.0 ** -24 * mult.unsqueeze(-1) + add.unsqueeze(-1)).to(torch.float16).reshape(N, -1)
    assert torch.equal(panel.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("mode", ["sym", "asym", "int8"])
def test_resident_weight_panel_gives_the_same_bits_as_the_per_call_one(mode):
    from dirotq_b200 import ops
    m = {"sym": ops.INT4_SYM, "asym": ops.INT4_ASYM, "int8": ops.INT8_ASYM}[mode]
    fmt = ops.ActFormat(m, 1152, tail_len=64)
    x, act, dec, qw, sw, pk, w_tail, bias = _setup_int(ops, 700, 384, fmt, 42)
    lay = act.layout
    wt = ops.pad_tail_weight(w_tail, lay.tail_pitch, 384, "cuda")
    folded = ops.fold_weight_scales_f16(pk, wt, lay.tail_total)
    y0 = ops.gemm_w4a4_int_f16(act, pk, folded, bias.cuda())
    folded.panel = ops.expand_weight_panel_f16(pk, folded)
    y1 = ops.gemm_w4a4_int_f16(act, pk, folded, bias.cuda())
    ops.check_status()
    assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
