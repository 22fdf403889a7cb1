"""Torch-tensor front end of the C ABI: allocates outputs as torch tensors, passes raw device
pointers and the current CUDA stream, raises on any non-zero return code.

Buffer layouts are documented in include/dirotq_b200.h.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import ActFormatC, ActLayoutC, check

INT4_SYM, INT4_ASYM, INT8_ASYM, NVFP4_REF, NVFP4_HW = 0, 1, 2, 3, 4
_ASYM = (INT4_ASYM, INT8_ASYM)


@dataclass(frozen=True)
class ActFormat:
    mode: int
    width: int
    tail_len: int = 0
    group_size: int = 64
    num_heads: int = 0
    head_dim: int = 0
    clip_ratio: float = 1.0
    tensor_scale: float = 1.0

    def c(self) -> ActFormatC:
        return ActFormatC(self.mode, self.width, self.num_heads, self.head_dim, self.tail_len, self.group_size,
                          self.clip_ratio, self.tensor_scale)


@dataclass(frozen=True)
class ActLayout:
    q_len: int
    group: int
    n_groups: int
    chunks_per_group: int
    n_chunks: int
    k_pad: int
    code_row_bytes: int
    tail_total: int
    tail_pitch: int
    n_scales: int


def act_layout(fmt: ActFormat) -> ActLayout:
    out = ActLayoutC()
    check(_lib.lib().dirotq_act_layout_of(C.byref(fmt.c()), C.byref(out)), "dirotq_act_layout_of")
    return ActLayout(*[getattr(out, f) for f, _ in ActLayoutC._fields_])


def mark_written(t: torch.Tensor):
    """Advance a tensor's in-place version counter after the library wrote it through a raw pointer: torch has not
    seen that write, and callers (backend.SharedActivation) use the counter to tell whether a tensor changed."""
    torch.autograd.graph.increment_version(t)


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


_status = {}


def status_word(device) -> torch.Tensor:
    """int32 device word the kernels write a timeout code into (zero = healthy)."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(8, dtype=torch.int32, device=f"cuda:{key}")
    return _status[key]


class StatusWatch:
    """Consumer of the status word on the product path, without a synchronisation: after a forward the word is copied
    to pinned host memory on the forward's stream; before the next forward the copy, if it has landed, is looked at.
    A bounded device-side wait that ran out therefore surfaces as an exception one call later at the latest
    (or at the next check_status), instead of feeding a pipeline with undefined outputs in silence."""

    def __init__(self, device):
        self.dev = torch.device(device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False

    def poll(self):
        """Raises if the last landed copy shows a non-zero status.  Never blocks."""
        if self.pending and self.event.query():
            self.pending = False
            s = int(self.host[0])
            if s != 0:
                status_word(self.dev).zero_()
                self.host.zero_()
                raise RuntimeError("dirotq_b200 kernel reported: " + _lib.lib().dirotq_status_string(s).decode())

    def post(self):
        """Queue the copy of the status word behind the kernels just launched on the current stream."""
        if self.pending and not self.event.query():
            return                      # an earlier copy is still in flight: it will be looked at first
        self.host.copy_(status_word(self.dev)[:1], non_blocking=True)
        self.event.record()
        self.pending = True


_watch = {}


def status_watch(device) -> StatusWatch:
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _watch:
        _watch[key] = StatusWatch(torch.device("cuda", key))
    return _watch[key]


def set_wait_limit_cycles(cycles: int):
    """Process-wide bound of the device-side waits in SM clock cycles (0 = default, about 1.5 s)."""
    check(_lib.lib().dirotq_set_wait_limit_cycles(int(cycles)), "dirotq_set_wait_limit_cycles")


def check_status(device=None):
    """Synchronising read of the status word; raises if a bounded device-side wait ran out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    s = int(status_word(dev)[0].item())
    if s != 0:
        status_word(dev).zero_()
        raise RuntimeError("dirotq_b200 kernel reported: " + _lib.lib().dirotq_status_string(s).decode())


@dataclass
class ActBuffers:
    fmt: ActFormat
    layout: ActLayout
    M: int
    codes: torch.Tensor
    scales: torch.Tensor
    zeros: Optional[torch.Tensor]
    tail: Optional[torch.Tensor]

    @property
    def ldm(self):
        return (self.M + 7) // 8 * 8


def alloc_act(fmt: ActFormat, M: int, device) -> ActBuffers:
    """Zero-initialised code / scale / zero / tail buffers for M rows (pad entries must stay zero)."""
    lay = act_layout(fmt)
    l = _lib.lib()
    fc, lc = fmt.c(), ActLayoutC(*[getattr(lay, f) for f, _ in ActLayoutC._fields_])
    nb = lambda fn, *a: int(fn(*a))
    codes = torch.zeros(nb(l.dirotq_act_codes_bytes, C.byref(lc), M), dtype=torch.uint8, device=device)
    scales = torch.zeros(nb(l.dirotq_act_scales_bytes, C.byref(fc), C.byref(lc), M), dtype=torch.uint8, device=device)
    zb = nb(l.dirotq_act_zeros_bytes, C.byref(fc), C.byref(lc), M)
    zeros = torch.zeros(zb, dtype=torch.uint8, device=device) if zb else None
    tb = nb(l.dirotq_act_tail_bytes, C.byref(lc), M)
    tail = torch.zeros(tb, dtype=torch.uint8, device=device) if lay.tail_total > 0 else None
    return ActBuffers(fmt, lay, M, codes, scales, zeros, tail)


def quantize_act(x2d: torch.Tensor, fmt: ActFormat, perm_idx: Optional[torch.Tensor] = None,
                 out: Optional[ActBuffers] = None) -> ActBuffers:
    """Kernel 1a: quantise an already rotated / permuted [M, D] bf16 tensor."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.dim() == 2 and x2d.stride(1) == 1
    M = x2d.shape[0]
    buf = out if out is not None else alloc_act(fmt, M, x2d.device)
    if M == 0:
        return buf
    check(_lib.lib().dirotq_quantize_act(C.byref(fmt.c()), _ptr(x2d), x2d.stride(0), _ptr(perm_idx), M,
                                         _ptr(buf.codes), _ptr(buf.scales), _ptr(buf.zeros), _ptr(buf.tail),
                                         _stream()), "dirotq_quantize_act")
    return buf


def rotate_quantize(x2d: torch.Tensor, rot_t: torch.Tensor, fmt: ActFormat, want_x_rot: bool = False,
                    out: Optional[ActBuffers] = None):
    """Kernel 1: fused rotate + split + quantise.  rot_t = rotation transposed ([D_out, D_in] bf16)."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous()
    assert rot_t.dtype == torch.bfloat16 and rot_t.is_contiguous()
    M = x2d.shape[0]
    buf = out if out is not None else alloc_act(fmt, M, x2d.device)
    x_rot = torch.empty_like(x2d) if want_x_rot else None
    if M == 0:
        return (buf, x_rot) if want_x_rot else buf
    check(_lib.lib().dirotq_rotate_quantize(C.byref(fmt.c()), _ptr(x2d), _ptr(rot_t), M, _ptr(x_rot),
                                            _ptr(buf.codes), _ptr(buf.scales), _ptr(buf.zeros), _ptr(buf.tail),
                                            _ptr(status_word(x2d.device)), _stream()), "dirotq_rotate_quantize")
    return (buf, x_rot) if want_x_rot else buf


def hadamard_low(x2d: torch.Tensor, low_dim: int, sign_flips: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Hadamard front end: FWHT over the first low_dim channels (after +-1 sign flips), rest copied."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous() and x2d.dim() == 2
    if sign_flips is not None:
        assert sign_flips.dtype == torch.bfloat16 and sign_flips.numel() == low_dim and sign_flips.is_contiguous()
    y = out if out is not None else torch.empty_like(x2d)
    check(_lib.lib().dirotq_hadamard_low(_ptr(x2d), x2d.shape[0], x2d.shape[1], low_dim, _ptr(sign_flips), _ptr(y),
                                         _stream()), "dirotq_hadamard_low")
    if out is not None:
        mark_written(out)
    return y


def rotate(x2d: torch.Tensor, rot_t: torch.Tensor, num_heads: int = 0, head_dim: int = 0) -> torch.Tensor:
    """Rotation only (bf16 tcgen05 GEMM): y = x @ rot_t.T."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous()
    D = x2d.shape[1]
    fmt = ActFormat(INT4_SYM, D, tail_len=1 if num_heads else 0, num_heads=num_heads, head_dim=head_dim)
    y = torch.empty_like(x2d)
    check(_lib.lib().dirotq_rotate_quantize(C.byref(fmt.c()), _ptr(x2d), _ptr(rot_t), x2d.shape[0], _ptr(y),
                                            None, None, None, None, _ptr(status_word(x2d.device)), _stream()),
          "dirotq_rotate_quantize(rotation only)")
    return y


@dataclass
class PackedWeightInt4:
    N: int
    n_low: int
    group: int
    n_chunks: int
    codes: torch.Tensor     # uint8 [N, n_chunks*32]
    scales: torch.Tensor    # fp32 [n_chunks, ldn]
    wsum: torch.Tensor      # fp32 [n_chunks, ldn]


def pack_weight_int4(w_low: torch.Tensor, group: int, scales: Optional[torch.Tensor] = None,
                     w_is_codes: bool = False) -> PackedWeightInt4:
    """Kernel 3 (INT4).  w_low fp32 [N, n_low] rotated weight (or integer codes if w_is_codes)."""
    w = w_low.to(torch.float32).contiguous()
    N, n_low = w.shape
    n_groups = (n_low + group - 1) // group
    n_chunks = n_groups * ((group + 63) // 64)
    ldn = (N + 7) // 8 * 8
    codes = torch.zeros(N, n_chunks * 32, dtype=torch.uint8, device=w.device)
    sc = torch.zeros(n_chunks, ldn, dtype=torch.float32, device=w.device)
    ws = torch.zeros(n_chunks, ldn, dtype=torch.float32, device=w.device)
    s_in = None if scales is None else scales.to(torch.float32).contiguous()
    if s_in is not None:
        assert s_in.shape == (N, n_groups)
    check(_lib.lib().dirotq_pack_weight_int4(_ptr(w), N, n_low, group, _ptr(s_in), int(w_is_codes), _ptr(codes),
                                             _ptr(sc), _ptr(ws), _stream()), "dirotq_pack_weight_int4")
    return PackedWeightInt4(N, n_low, group, n_chunks, codes, sc, ws)


@dataclass
class PackedWeightNvfp4:
    N: int
    n_low: int
    n_chunks: int
    tensor_scale: float
    codes: torch.Tensor     # uint8 [N, n_chunks*32]
    sf: torch.Tensor        # uint8 tiled UE4M3
    row_scale: Optional[torch.Tensor] = None   # fp32 [ldn]: per-channel second-level scale (reference recipe)


def pack_weight_nvfp4_rowscale(w_low: torch.Tensor) -> PackedWeightNvfp4:
    """Kernel 3 (NVFP4) with the reference's own two-level weight recipe (speedup/weight_only_nvfp4.py:42-72):
    per-output-channel scale gscale[n] (kept as its bf16 value in fp32), E4M3 micro-scales relative to it, codes by
    first-argmin against micro * gscale."""
    w = w_low.to(torch.float32).contiguous()
    N, n_low = w.shape
    n_chunks = (n_low + 63) // 64
    ldn = (N + 7) // 8 * 8
    codes = torch.zeros(N, n_chunks * 32, dtype=torch.uint8, device=w.device)
    sf = torch.zeros(((N + 127) // 128) * ((n_chunks + 3) // 4 * 4) * 512, dtype=torch.uint8, device=w.device)
    rs = torch.ones(ldn, dtype=torch.float32, device=w.device)
    rs_exact = torch.ones(ldn, dtype=torch.float32, device=w.device)
    check(_lib.lib().dirotq_pack_weight_nvfp4_rowscale(_ptr(w), N, n_low, _ptr(codes), _ptr(sf), _ptr(rs), _ptr(rs_exact),
                                                       _stream()), "dirotq_pack_weight_nvfp4_rowscale")
    return PackedWeightNvfp4(N, n_low, n_chunks, 1.0, codes, sf, rs)


def pack_weight_nvfp4(w_low: torch.Tensor, tensor_scale: float, scales_e4m3: Optional[torch.Tensor] = None,
                      w_is_codes: bool = False) -> PackedWeightNvfp4:
    """Kernel 3 (NVFP4, group 16, two-level scale)."""
    w = w_low.to(torch.float32).contiguous()
    N, n_low = w.shape
    n_chunks = (n_low + 63) // 64
    codes = torch.zeros(N, n_chunks * 32, dtype=torch.uint8, device=w.device)
    sf = torch.zeros(((N + 127) // 128) * ((n_chunks + 3) // 4 * 4) * 512, dtype=torch.uint8, device=w.device)
    s_in = None
    if scales_e4m3 is not None:
        s_in = scales_e4m3.contiguous()
        assert s_in.dtype == torch.uint8 and s_in.shape == (N, (n_low + 15) // 16)
    check(_lib.lib().dirotq_pack_weight_nvfp4(_ptr(w), N, n_low, float(tensor_scale), _ptr(s_in), int(w_is_codes),
                                              _ptr(codes), _ptr(sf), _stream()), "dirotq_pack_weight_nvfp4")
    return PackedWeightNvfp4(N, n_low, n_chunks, float(tensor_scale), codes, sf)


def pad_tail_weight(w_tail: Optional[torch.Tensor], tail_pitch: int, N: int, device) -> Optional[torch.Tensor]:
    """bf16 [N, tail_total] -> bf16 [N, tail_pitch] (zero padded), the layout the GEMMs read."""
    if w_tail is None or tail_pitch == 0:
        return None
    out = torch.zeros(N, tail_pitch, dtype=torch.bfloat16, device=device)
    out[:, : w_tail.shape[1]] = w_tail.to(device=device, dtype=torch.bfloat16)
    return out


def gemm_w4a4_int(act: ActBuffers, w: PackedWeightInt4, w_tail: Optional[torch.Tensor],
                  bias: Optional[torch.Tensor], dump_acc: bool = False):
    """Kernel 2 (INT).  Returns y bf16 [M, N] (and the int32 per-chunk accumulators if dump_acc)."""
    lay, M, N = act.layout, act.M, w.N
    assert lay.n_chunks == w.n_chunks, (lay.n_chunks, w.n_chunks)
    dev = act.codes.device
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    dump = torch.zeros(lay.n_chunks, M, N, dtype=torch.int32, device=dev) if dump_acc else None
    if lay.tail_total > 0:
        assert w_tail is not None and tuple(w_tail.shape) == (N, lay.tail_pitch) and w_tail.dtype == torch.bfloat16
    check(_lib.lib().dirotq_gemm_w4a4_int(act.fmt.mode, M, N, lay.n_chunks, _ptr(act.codes), _ptr(act.scales),
                                          _ptr(act.zeros), _ptr(w.codes), _ptr(w.scales), _ptr(w.wsum),
                                          _ptr(act.tail), _ptr(w_tail), lay.tail_total, lay.tail_pitch, _ptr(bias),
                                          _ptr(y), _ptr(dump), _ptr(status_word(dev)), _stream()),
          "dirotq_gemm_w4a4_int")
    return (y, dump) if dump_acc else y


@dataclass
class FoldedWeightF16:
    """Weight-side constants of the tensor-rate INT4 GEMM (dirotq_fold_weight_scales_f16)."""
    mult: torch.Tensor                    # uint8: 8-byte records per (chunk, channel)
    colscale: torch.Tensor                # fp32 [ldn]
    tail: Optional[torch.Tensor]          # bf16 [N, tail_pitch] = w_tail / colscale
    panel: Optional[torch.Tensor] = None  # fp16 [N, n_chunks * 64]: resident expanded weights (optional)


def fold_weight_scales_f16(w: PackedWeightInt4, w_tail: Optional[torch.Tensor], tail_total: int) -> FoldedWeightF16:
    """Per-layer preparation for gemm_w4a4_int_f16: fp16 multipliers, column powers of two, scaled tail."""
    dev = w.scales.device
    ldn = w.scales.shape[1]
    mult = torch.zeros(int(_lib.lib().dirotq_fold_weight_records_bytes(w.n_chunks, w.N)), dtype=torch.uint8, device=dev)
    cs = torch.ones(ldn, dtype=torch.float32, device=dev)
    tail_out, pitch = None, 0
    if tail_total > 0:
        assert w_tail is not None and w_tail.dtype == torch.bfloat16 and w_tail.is_contiguous()
        pitch = w_tail.shape[1]
        tail_out = torch.zeros_like(w_tail)
    check(_lib.lib().dirotq_fold_weight_scales_f16(w.n_chunks, w.N, _ptr(w.scales), _ptr(w_tail), tail_total, pitch,
                                                   _ptr(mult), _ptr(cs), _ptr(tail_out), _stream()),
          "dirotq_fold_weight_scales_f16")
    return FoldedWeightF16(mult, cs, tail_out)


def expand_weight_panel_f16(w: PackedWeightInt4, folded: FoldedWeightF16, half_chunks: bool = False) -> torch.Tensor:
    """fp16 [N, n_chunks * 64] panel of (q_w - 8) * s_w / colscale, in the K order of the GEMM's activation
    converters: what dirotq_gemm_w4a4_int_f16 otherwise rebuilds in its workspace on every call.  half_chunks: the
    layout of layers with per-head groups of at most 32 channels, [N, ceil(n_chunks / 2) * 64]."""
    n = int(_lib.lib().dirotq_weight_panel_bytes(w.n_chunks, w.N))
    panel = torch.empty(n // 2, dtype=torch.float16, device=w.codes.device)
    check(_lib.lib().dirotq_expand_weight_panel_f16_layout(w.n_chunks, w.N, _ptr(w.codes), _ptr(folded.mult), _ptr(panel),
                                                           1 if half_chunks else 0, _stream()),
          "dirotq_expand_weight_panel_f16_layout")
    cols = ((w.n_chunks + 1) // 2 if half_chunks else w.n_chunks) * 64
    return panel[: w.N * cols].view(w.N, cols)


def f16_workspace_bytes(act: ActBuffers, N_panel: int = 0) -> int:
    """N_panel = the layer's out_features when the call has to rebuild the weight panel; 0 with a resident one."""
    lay = act.layout
    tp = lay.tail_pitch if lay.tail_total > 0 else 0
    return max(256, int(_lib.lib().dirotq_gemm_w4a4_int_f16_workspace_bytes(act.M, N_panel, lay.n_chunks, tp)))


def gemm_w4a4_int_f16(act: ActBuffers, w: PackedWeightInt4, folded: FoldedWeightF16, bias: Optional[torch.Tensor],
                      workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Kernel 2 (INT4, tensor-rate variant): codes expanded to fp16 in shared memory, one fp32 accumulator."""
    lay, M, N = act.layout, act.M, w.N
    assert act.fmt.mode in (INT4_SYM, INT4_ASYM, INT8_ASYM) and lay.n_chunks == w.n_chunks
    dev = act.codes.device
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    tp = lay.tail_pitch if lay.tail_total > 0 else 0
    need = int(_lib.lib().dirotq_gemm_w4a4_int_f16_workspace_bytes(M, 0 if folded.panel is not None else N,
                                                                   lay.n_chunks, tp))
    ws = workspace if workspace is not None else torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
    if M == 0:
        return y
    check(_lib.lib().dirotq_gemm_w4a4_int_f16(act.fmt.mode, M, N, lay.n_chunks, _ptr(act.codes), _ptr(act.scales),
                                              _ptr(act.zeros), _ptr(w.codes), _ptr(folded.mult), _ptr(folded.panel),
                                              _ptr(folded.colscale),
                                              _ptr(act.tail), _ptr(folded.tail), lay.tail_total, lay.tail_pitch,
                                              _ptr(bias), _ptr(y), _ptr(ws), ws.numel(), _ptr(status_word(dev)),
                                              _stream()), "dirotq_gemm_w4a4_int_f16")
    return y


def gemm_w4a4_nvfp4(act: ActBuffers, w: PackedWeightNvfp4, w_tail_scaled: Optional[torch.Tensor],
                    bias: Optional[torch.Tensor]) -> torch.Tensor:
    """Kernel 2 (NVFP4).  w_tail_scaled = w_tail / (Tx * Tw [* w.row_scale[n]]), bf16 [N, tail_pitch]."""
    lay, M, N = act.layout, act.M, w.N
    assert act.fmt.mode == NVFP4_HW and lay.n_chunks == w.n_chunks
    dev = act.codes.device
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    out_scale = float(act.fmt.tensor_scale) * float(w.tensor_scale)
    check(_lib.lib().dirotq_gemm_w4a4_nvfp4(M, N, lay.n_chunks, _ptr(act.codes), _ptr(act.scales), _ptr(w.codes),
                                            _ptr(w.sf), out_scale, _ptr(w.row_scale), _ptr(act.tail), _ptr(w_tail_scaled),
                                            lay.tail_total, lay.tail_pitch, _ptr(bias), _ptr(y),
                                            _ptr(status_word(dev)), _stream()), "dirotq_gemm_w4a4_nvfp4")
    return y


def gemm_w4a16_nvfp4(x2d: torch.Tensor, w: "PackedWeightNvfp4", bias: Optional[torch.Tensor],
                     workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """W4A16 linear with an NVFP4 weight: bf16 x [M, K] (K = n_chunks * 64) times E2M1 codes x UE4M3 group scales
    x tensor scale (dequantised into scratch, then the tcgen05 bf16 GEMM)."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous()
    M, K = x2d.shape
    assert K == w.n_chunks * 64
    need = int(_lib.lib().dirotq_gemm_w4a16_workspace_bytes(w.N, K))
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x2d.device)
    y = torch.empty(M, w.N, dtype=torch.bfloat16, device=x2d.device)
    if M == 0:
        return y
    check(_lib.lib().dirotq_gemm_w4a16_nvfp4(M, w.N, K, _ptr(x2d), _ptr(w.codes), _ptr(w.sf), float(w.tensor_scale),
                                             _ptr(w.row_scale), _ptr(bias), _ptr(y), _ptr(ws), ws.numel(), _ptr(status_word(x2d.device)),
                                             _stream()), "dirotq_gemm_w4a16_nvfp4")
    return y


def dequant_weight_nvfp4(w: "PackedWeightNvfp4") -> torch.Tensor:
    """bf16 [N, K] weight of a packed NVFP4 layer (K = n_chunks * 64), one rounding per value."""
    K = w.n_chunks * 64
    out = torch.empty(w.N, K, dtype=torch.bfloat16, device=w.codes.device)
    check(_lib.lib().dirotq_dequant_weight_nvfp4(w.N, K, _ptr(w.codes), _ptr(w.sf), float(w.tensor_scale),
                                                 _ptr(w.row_scale), _ptr(out), _stream()), "dirotq_dequant_weight_nvfp4")
    return out


def dequant_weight_int4(w: PackedWeightInt4) -> torch.Tensor:
    """bf16 [N, K] weight of a packed INT4 group-64 layer (K = n_chunks * 64), one rounding per value."""
    assert w.group == 64
    K = w.n_chunks * 64
    out = torch.empty(w.N, K, dtype=torch.bfloat16, device=w.codes.device)
    check(_lib.lib().dirotq_dequant_weight_int4(w.N, K, _ptr(w.codes), _ptr(w.scales), _ptr(out), _stream()),
          "dirotq_dequant_weight_int4")
    return out


def gemm_bf16(x2d: torch.Tensor, w_dense: torch.Tensor, bias: Optional[torch.Tensor],
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w^T + bias on the bf16 tensor cores (the GEMM half of the W4A16 layers, on a resident dequantised weight)."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous()
    assert w_dense.dtype == torch.bfloat16 and w_dense.is_contiguous() and w_dense.shape[1] == x2d.shape[1]
    M, K = x2d.shape
    N = w_dense.shape[0]
    y = out if out is not None else torch.empty(M, N, dtype=torch.bfloat16, device=x2d.device)
    check(_lib.lib().dirotq_gemm_bf16(M, N, K, _ptr(x2d), _ptr(w_dense), _ptr(bias), _ptr(y), _ptr(status_word(x2d.device)),
                                      _stream()), "dirotq_gemm_bf16")
    if out is not None:
        mark_written(out)
    return y


def gemm_w4a16(x2d: torch.Tensor, w: PackedWeightInt4, bias: Optional[torch.Tensor],
               workspace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """W4A16 linear: bf16 x [M, K] times INT4 group-64 weights (dequantised into scratch, then tcgen05 bf16 GEMM)."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous() and w.group == 64
    M, K = x2d.shape
    assert K == w.n_chunks * 64
    need = int(_lib.lib().dirotq_gemm_w4a16_workspace_bytes(w.N, K))
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x2d.device)
    y = out if out is not None else torch.empty(M, w.N, dtype=torch.bfloat16, device=x2d.device)
    check(_lib.lib().dirotq_gemm_w4a16(M, w.N, K, _ptr(x2d), _ptr(w.codes), _ptr(w.scales), _ptr(bias), _ptr(y),
                                       _ptr(ws), ws.numel(), _ptr(status_word(x2d.device)), _stream()),
          "dirotq_gemm_w4a16")
    if out is not None:
        mark_written(out)
    return y




# ---------------------------------------------------------------------------------------------------------------------
# block glue (row-wise passes between two wrapped linears)
# ---------------------------------------------------------------------------------------------------------------------
def _mod_vec(v: Optional[torch.Tensor], B: int, D: int):
    """(pointer tensor, per-sample pitch) of a modulation vector given as [B, D], [B, 1, D] or [1, D] / [D] (shared)."""
    if v is None:
        return None, 0
    v2 = v.reshape(-1, D) if v.dim() != 2 else v
    assert v2.dtype == torch.bfloat16 and v2.stride(1) == 1 and v2.shape[0] in (1, B)
    return v2, (0 if v2.shape[0] == 1 else v2.stride(0))


def layernorm_modulate(x: torch.Tensor, scale: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
                       eps: float = 1e-6) -> torch.Tensor:
    """y = LayerNorm(x) * (1 + scale) + shift over the last dimension, no affine parameters; x bf16 [B, T, D], scale /
    shift per sample ([B, D] or [B, 1, D], views into a larger tensor allowed).  One pass, fp32 inside."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 3
    B, T, D = x.shape
    sc, p1 = _mod_vec(scale, B, D)
    sh, p2 = _mod_vec(shift, B, D)
    if sc is not None and sh is not None and p1 != p2:
        sh = sh.expand(B, D).contiguous() if p2 == 0 else sh.contiguous()
        sc = sc.expand(B, D).contiguous() if p1 == 0 else sc.contiguous()
        p1 = p2 = D
    y = torch.empty_like(x)
    check(_lib.lib().dirotq_layernorm_modulate(_ptr(x), B * T, D, T, _ptr(sc), _ptr(sh), p1 if sc is not None else p2,
                                               float(eps), _ptr(y), _stream()), "dirotq_layernorm_modulate")
    return y


def gated_residual(h: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor] = None,
                   y2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h + gate * (y + y2): h, y, y2 bf16 [B, T, D]; gate per sample ([B, D] / [B, 1, D]) or None."""
    assert h.is_cuda and h.dtype == torch.bfloat16 and h.is_contiguous() and h.dim() == 3
    B, T, D = h.shape
    y = y.reshape(B, T, D)
    y = y if y.is_contiguous() else y.contiguous()
    if y2 is not None:
        y2 = y2.reshape(B, T, D)
        y2 = y2 if y2.is_contiguous() else y2.contiguous()
    g, pitch = _mod_vec(gate, B, D)
    out = torch.empty_like(h)
    check(_lib.lib().dirotq_gated_residual(_ptr(h), _ptr(y), _ptr(y2), _ptr(g), pitch, B * T, D, T, _ptr(out), _stream()),
          "dirotq_gated_residual")
    return out


def qkv_norm_rope(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, w_q: Optional[torch.Tensor],
                  w_k: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                  out: Optional[tuple] = None, t0: int = 0, eps: float = 1e-6):
    """q, k, v bf16 [B, T, H * d] (columns of one fused projection output or separate tensors, common row pitch): RMSNorm
    per head times w_q / w_k and the rotary embedding on q and k, v copied, all written token-major into
    out = (q, k, v) buffers [B, T_total, H, d] at token offset t0 (allocated with T_total = T when out is None)."""
    B, T, C = q.shape
    d = C // heads
    pitch = q.stride(1)
    for t in (q, k, v):
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.shape == q.shape and t.stride(2) == 1
        assert t.stride(1) == pitch and (B == 1 or t.stride(0) == T * pitch), "q, k, v: rows of all samples at one pitch"
    if out is None:
        out = tuple(torch.empty(B, T, heads, d, dtype=torch.bfloat16, device=q.device) for _ in range(3))
    T_total = out[0].shape[1]
    for o in out:
        assert o.is_contiguous() and o.shape == (B, T_total, heads, d)
    if cos is not None:
        assert cos.shape == (T_total, d) and sin.shape == (T_total, d) and cos.is_contiguous() and sin.is_contiguous()
        assert cos.dtype == torch.bfloat16 and sin.dtype == torch.bfloat16, "rotary tables: bf16 [T_total, d]"
    for w_ in (w_q, w_k):
        assert w_ is None or (w_.dtype == torch.bfloat16 and w_.shape == (d,) and w_.is_contiguous()), "norm weights: bf16 [d]"
    check(_lib.lib().dirotq_qkv_norm_rope(_ptr(q), _ptr(k), _ptr(v), pitch, B, T, heads, d, _ptr(w_q), _ptr(w_k), _ptr(cos),
                                          _ptr(sin), T_total, t0, float(eps), _ptr(out[0]), _ptr(out[1]), _ptr(out[2]),
                                          _stream()), "dirotq_qkv_norm_rope")
    return out
