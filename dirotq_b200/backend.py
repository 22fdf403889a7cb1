"""Drop-in backend for the reference's fused-unrotation forward.

Exports the two names apply_dirotq.py imports from its backend module
(dirotq_fused_unrotation_fast.py:25, :144; selected at apply_dirotq.py:188-194):

    patch_forward()                                   -> ActQuantWrapper.forward = B200 path
    preconvert_rotations_to_device(transformer, ...)  -> int

The forward keeps the reference's contract (dirotq_fused_unrotation_fast.py:56-141): rotate into the
layer's PCA basis, keep the top-k coefficients in bf16, quantise the rest to 4 bit, multiply by the
fused weight, add bias, return x.dtype.  Here those steps are two CUDA kernels behind one C-ABI
call (dirotq_linear_forward); the quantised weight is packed once, when the layer is prepared.
"""
from __future__ import annotations

import ctypes as C
import sys
import warnings
import weakref
import dataclasses
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from . import _lib, ops, pack
from ._lib import LinearC, check
from .wrapper import ActQuantWrapper

_HW_NVFP4_ACT_SCALE = 1.0   # static fp32 tensor scale of NVFP4 activations (UE4M3 then covers amax up to 2688)


class SharedActivation:
    """Quantised activations shared by sibling layers that see the same input through the same rotation
    and format (attn.to_q / to_k / to_v: the reference gives all three `evec @ R1` of one basis,
    models/pixart-sigma/model_utils.py:84-92, and diffusers calls them on one hidden_states tensor).
    The first member called on a tensor rotates and quantises it into the group's workspace; members
    called next on the SAME tensor run only their GEMM.  "Same" = same storage address, shape and
    in-place version counter, with a reference held so that the storage cannot be recycled in between;
    the reference is dropped once every member has used it (or by release()).  Buffers that this library
    itself fills through raw pointers (`out=` arguments) have their version counter advanced explicitly
    (ops.mark_written), so a reused output buffer is never mistaken for the tensor quantised before."""

    def __init__(self, n_members: int):
        self.n_members = n_members
        self.members: list = []          # the LayerStates: the workspace is sized for the largest of them
        self.ws: Dict[int, torch.Tensor] = {}
        self.x_ref: Optional[torch.Tensor] = None
        self.key = None
        self.seen = set()
        self.hits = 0
        self.misses = 0
        self.fused: Optional["LayerState"] = None     # one layer over the members' weights, concatenated along N
        self.offsets: list = []                        # first output column of each member in the fused layer
        self.y_all: Optional[torch.Tensor] = None      # [M, sum N]: output of the fused GEMM for the held tensor
        self.incomplete = 0                            # fused passes whose result some member never picked up

    @staticmethod
    def _key(x: torch.Tensor):
        stream = torch.cuda.current_stream(x.device).cuda_stream if x.is_cuda else 0
        return (x.data_ptr(), x._version, tuple(x.shape), tuple(x.stride()), x.dtype, x.device.index, stream)

    def lookup(self, x: torch.Tensor, member_id: int) -> bool:
        """True if the workspace already holds this tensor's codes and `member_id` has not used them yet."""
        hit = self.x_ref is not None and self.key == self._key(x) and member_id not in self.seen
        if hit:
            self.hits += 1
            self.seen.add(member_id)
            if len(self.seen) == self.n_members:
                self.x_ref, self.key = None, None
        return hit

    def store(self, x: torch.Tensor, member_id: int):
        self.misses += 1
        if self.x_ref is not None and len(self.seen) < self.n_members:
            self.incomplete += 1
        self.x_ref, self.key, self.seen = x, self._key(x), {member_id}

    def release(self):
        """Forget the held activation tensor (it stays referenced until every member has used it, which never
        happens when the members of a group do not all see the same input, e.g. a cross-attention)."""
        self.x_ref, self.key, self.seen, self.y_all = None, None, set(), None


@dataclass
class LayerState:
    """Device-resident packed form of one wrapped linear."""
    fmt: ops.ActFormat
    layout: ops.ActLayout
    out_features: int
    rot_t: Optional[torch.Tensor]
    perm_idx: Optional[torch.Tensor]
    w_codes: torch.Tensor
    w_scales: torch.Tensor
    w_sum: Optional[torch.Tensor]
    w_tail: Optional[torch.Tensor]
    bias: Optional[torch.Tensor]
    w_tensor_scale: float = 1.0
    n_lossy_groups: int = 0
    folded: Optional[ops.FoldedWeightF16] = None     # INT4 activations: constants of the tensor-rate GEMM
    shared: Optional[SharedActivation] = None
    member_id: int = 0
    epilogue_act: int = 0                            # 1: GELU (tanh form) fused into the GEMM epilogue
    hadamard_low_dim: int = 0                        # use_hadamard layers: FWHT over the first channels
    hadamard_flips: Optional[torch.Tensor] = None
    w_rowscale: Optional[torch.Tensor] = None        # NVFP4: fp32 per-channel weight scale (reference recipe)
    chain_next: Optional["LayerState"] = None        # this layer's GEMM epilogue quantises its output for that layer
    chain_keep_output: bool = True                   # False: the bf16 output itself is never written (nobody else reads it)
    handed: Optional[torch.Tensor] = None            # consumer side: the producer's output whose codes the workspace holds
    handed_key: Optional[tuple] = None
    chain_hits: int = 0
    chain_fed: bool = False                          # a producer's epilogue quantises for this layer
    panel_declined: bool = False                     # a large-batch call found the resident-panel budget spent
    _c: Optional[LinearC] = None
    _ws: Dict[int, torch.Tensor] = field(default_factory=dict)

    def c_struct(self) -> LinearC:
        if self._c is None:
            p = lambda t: C.c_void_p(0 if t is None else t.data_ptr())
            f = self.folded
            self._c = LinearC(self.fmt.c(), self.out_features, p(self.rot_t), p(self.perm_idx), p(self.w_codes),
                              p(self.w_scales), p(self.w_sum), p(self.w_tail), p(self.bias), self.w_tensor_scale,
                              p(f.mult if f else None), p(f.colscale if f else self.w_rowscale), p(f.tail if f else None),
                              int(self.epilogue_act), p(f.panel if f else None))
        return self._c

    def workspace(self, M: int, device) -> torch.Tensor:
        if self.shared is not None:
            ws = self.shared.ws.get(M)
            if ws is None:
                n = max(int(_lib.lib().dirotq_linear_workspace_bytes(C.byref(m.c_struct()), M))
                        for m in (self.shared.members or [self]))
                ws = torch.zeros(max(n, 256), dtype=torch.uint8, device=device)
                self.shared.ws = {M: ws}
                self.shared.x_ref, self.shared.key = None, None
            return ws
        ws = self._ws.get(M)
        if ws is None:
            n = int(_lib.lib().dirotq_linear_workspace_bytes(C.byref(self.c_struct()), M))
            # zero once: padding entries of the scale-factor tiles are never written afterwards
            ws = torch.zeros(max(n, 256), dtype=torch.uint8, device=device)
            self._ws = {M: ws}          # keep one size; diffusion steps reuse the same M
        return ws


def kernel_launches(st: Optional[LayerState], w4a16=None) -> int:
    """Library kernels one forward of a wrapped linear launches.  A W4A16 layer (no LayerState): weight
    dequantisation + GEMM.  W4A4: rotate/quantise + GEMM; the tensor-rate integer GEMM adds one preparation launch
    (scale folding and, unless the layer keeps a resident panel, the weight-panel pre-pass); a sibling that reuses the
    activations of the layer before it runs only its own GEMM (and pre-pass)."""
    if st is None:
        return 1 if (w4a16 is not None and w4a16.dense is not None) else 2    # resident dequantised weight: GEMM only
    if st.shared is not None and st.shared.fused is not None:
        return kernel_launches(st.shared.fused) if st.member_id == 0 else 0     # one pass and one GEMM for the group
    n = 1 if (st.shared is not None and st.member_id > 0) else 2
    if st.chain_fed:
        n -= 1                              # its activations arrive quantised from the producer's epilogue
    if st.folded is not None:
        # scale folding (first user of the activations only) and the weight-panel pre-pass (unless resident): one launch
        # when both are due, else one each
        fold = not (st.shared is not None and st.member_id > 0)
        n += 1 if (fold or st.folded.panel is None) else 0
    follower = (st.shared is not None and st.member_id > 0) or st.chain_fed
    two_step = _rotates_then_quantises(st)
    if two_step and not follower:
        n += 1                              # rotation into scratch, then the quantise kernel
    if (st.rot_t is None or two_step) and st.layout.tail_total > 0 and not follower:
        n += 1                              # the quantise kernel copies the passthrough channels in a launch of its own
    if st.hadamard_low_dim:
        n += 1
    return n


def _rotates_then_quantises(st: LayerState) -> bool:
    """Mirror of the library's routing: formats the rotation kernel's epilogue cannot quantise (a channel selection after
    the rotation, per-token scales, integer groups other than 64 under a hidden rotation, per-head groups whose 32-column
    reads would leave the head) rotate into scratch and quantise in a second launch."""
    f = st.fmt
    if st.rot_t is None:
        return False
    if st.perm_idx is not None or f.group_size <= 0:
        return True
    if f.mode in (ops.NVFP4_HW, ops.NVFP4_REF):
        return False
    if f.num_heads == 0:
        return f.group_size != 64
    return (f.head_dim - f.tail_len + 31) // 32 * 32 > f.head_dim


def linear_forward(st: LayerState, x2d: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One wrapped linear through the C ABI: x2d bf16 [M, D] -> bf16 [M, N]."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous()
    M = x2d.shape[0]
    if M == 0:
        return out if out is not None else torch.empty(0, st.out_features, dtype=torch.bfloat16, device=x2d.device)
    grp = st.shared
    if grp is not None and grp.fused is not None:
        # siblings fused into one layer: the first member called on a tensor runs it, the others take their columns
        if grp.incomplete > 2:
            grp.fused, grp.y_all = None, None            # the members do not see the same tensor after all: separate GEMMs
        else:
            if not grp.lookup(x2d, st.member_id):
                grp.store(x2d, st.member_id)
                grp.y_all = linear_forward(grp.fused, x2d)
            off = grp.offsets[st.member_id]
            part = grp.y_all[:, off:off + st.out_features]
            if grp.x_ref is None:
                grp.y_all = None                         # every member has its view
            if out is not None:
                out.copy_(part)
                return out
            return part
    y = out if out is not None else torch.empty(M, st.out_features, dtype=torch.bfloat16, device=x2d.device)
    if st.hadamard_low_dim:
        x2d = ops.hadamard_low(x2d, st.hadamard_low_dim, st.hadamard_flips)
    if (CACHE_WEIGHT_PANEL == "auto" and st.folded is not None and st.folded.panel is None and not st.panel_declined and
            _panel_budget_take(st, x2d.device, 2 * st.out_features * st.layout.n_chunks * 64, M <= PANEL_CACHE_MAX_ROWS)):
        pk = ops.PackedWeightInt4(st.out_features, st.layout.q_len, st.layout.group, st.layout.n_chunks, st.w_codes,
                                  st.w_scales, st.w_sum)
        half = bool(_lib.lib().dirotq_linear_uses_half_chunks(C.byref(st.c_struct())))
        st.folded.panel = ops.expand_weight_panel_f16(pk, st.folded, half)
        st._c = None
        if st.shared is None and st.handed is None:
            st._ws = {}                 # the workspace no longer needs room for a per-call panel
    elif CACHE_WEIGHT_PANEL == "auto" and st.folded is not None and st.folded.panel is None and M > PANEL_CACHE_MAX_ROWS:
        st.panel_declined = True        # over the budget: asked once, not on every call
    ws = st.workspace(M, x2d.device)
    watch = ops.status_watch(x2d.device) if WATCH_STATUS else None
    if watch is not None:
        watch.poll()                    # a wait that ran out in an earlier call surfaces here (no synchronisation)
    status = C.c_void_p(ops.status_word(x2d.device).data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if st.handed is not None:
        hit = st.handed_key == SharedActivation._key(x2d)
        st.handed, st.handed_key = None, None
        if hit:
            # the producer's epilogue left this tensor's codes, scales and 16-bit channels in the workspace
            st.chain_hits += 1
            check(_lib.lib().dirotq_linear_gemm_prequantised(C.byref(st.c_struct()), M, C.c_void_p(y.data_ptr()),
                                                             C.c_void_p(ws.data_ptr()), ws.numel(), status, stream),
                  "dirotq_linear_gemm_prequantised")
            if out is not None:
                ops.mark_written(out)
            if watch is not None:
                watch.post()
            return y
    nxt = st.chain_next
    if nxt is not None and st.shared is None and not nxt.hadamard_low_dim:
        nws = nxt.workspace(M, x2d.device)
        yp = C.c_void_p(y.data_ptr() if st.chain_keep_output else 0)
        check(_lib.lib().dirotq_linear_forward_chain(C.byref(st.c_struct()), C.c_void_p(x2d.data_ptr()), M, yp,
                                                     C.c_void_p(ws.data_ptr()), ws.numel(), C.byref(nxt.c_struct()),
                                                     C.c_void_p(nws.data_ptr()), nws.numel(), status, stream),
              "dirotq_linear_forward_chain")
        if out is not None:
            ops.mark_written(out)
        nxt.handed, nxt.handed_key = y, SharedActivation._key(y)
        if watch is not None:
            watch.post()
        return y
    if st.shared is not None:
        if st.shared.lookup(x2d, st.member_id):
            check(_lib.lib().dirotq_linear_gemm(C.byref(st.c_struct()), M, C.c_void_p(y.data_ptr()),
                                                C.c_void_p(ws.data_ptr()), ws.numel(),
                                                C.c_void_p(ops.status_word(x2d.device).data_ptr()),
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                  "dirotq_linear_gemm")
            if out is not None:
                ops.mark_written(out)
            if watch is not None:
                watch.post()
            return y
        st.shared.store(x2d, st.member_id)
    check(_lib.lib().dirotq_linear_forward(C.byref(st.c_struct()), C.c_void_p(x2d.data_ptr()), M,
                                           C.c_void_p(y.data_ptr()), C.c_void_p(ws.data_ptr()), ws.numel(),
                                           C.c_void_p(ops.status_word(x2d.device).data_ptr()),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream)),
          "dirotq_linear_forward")
    if out is not None:
        ops.mark_written(out)
    if watch is not None:
        watch.post()
    return y


def linear_forward_static(st: LayerState, x2d: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """linear_forward without any scratch from the caller: the library's built-in device array is used
    (see dirotq_linear_forward_static in include/dirotq_b200.h for the capacity and the sharing rules)."""
    assert x2d.is_cuda and x2d.dtype == torch.bfloat16 and x2d.is_contiguous()
    M = x2d.shape[0]
    y = out if out is not None else torch.empty(M, st.out_features, dtype=torch.bfloat16, device=x2d.device)
    check(_lib.lib().dirotq_linear_forward_static(C.byref(st.c_struct()), C.c_void_p(x2d.data_ptr()), M,
                                                  C.c_void_p(y.data_ptr()),
                                                  C.c_void_p(ops.status_word(x2d.device).data_ptr()),
                                                  C.c_void_p(torch.cuda.current_stream().cuda_stream)),
          "dirotq_linear_forward_static")
    return y


def _act_format(w) -> ops.ActFormat:
    q = w.quantizer
    D = w.module.in_features
    hlen = int(q.high_bits_length)
    nvfp4 = q.quant_dtype == "nvfp4"
    if nvfp4:
        mode = ops.NVFP4_HW
    elif q.bits == 8 and not q.sym:
        mode = ops.INT8_ASYM
    elif q.bits == 4:
        mode = ops.INT4_SYM if q.sym else ops.INT4_ASYM
    else:
        raise NotImplementedError(f"activation format bits={q.bits} sym={q.sym} has no sm_100a kernel")
    per_head = w.rotation_per_head is not None and getattr(w, "_unrot_fused", False) and hlen > 0
    if per_head:
        if nvfp4:
            # The reference quantises each head's d - tail coefficients as one E2M1 group
            # (dirotq_fused_unrotation_fast.py:89-93).  The tensor cores scale blocks of 16: the heads' low
            # coefficients are gathered in front (as the reference's rearrangement does, :94-99) and quantised in
            # blocks of 16, which never straddle a head when d - tail is a multiple of 16.
            H, d = int(w.num_heads), int(w.head_dim)
            if (d - hlen) % 16:
                raise NotImplementedError(f"per-head NVFP4 with head_dim - tail = {d - hlen}: not a multiple of the "
                                          "16-element scale block of the FP4 tensor cores; use INT4 for this layer")
            if PER_HEAD_NVFP4_FUSED and d % 16 == 0:
                # the rotation kernel's own per-head epilogue writes this layout (one launch)
                return ops.ActFormat(mode, D, tail_len=hlen, num_heads=H, head_dim=d, group_size=16,
                                     clip_ratio=float(q.clip_ratio), tensor_scale=_HW_NVFP4_ACT_SCALE)
            # rotation into scratch, then gather + quantise (two launches): hidden layout + channel selection
            return ops.ActFormat(mode, D, tail_len=H * hlen, group_size=16, clip_ratio=float(q.clip_ratio),
                                 tensor_scale=_HW_NVFP4_ACT_SCALE)
        return ops.ActFormat(mode, D, tail_len=hlen, num_heads=int(w.num_heads), head_dim=int(w.head_dim),
                             clip_ratio=float(q.clip_ratio))
    gs = int(q.groupsize)
    if gs <= 0:
        if nvfp4:
            raise NotImplementedError("per-token NVFP4 (one bf16 scale per row, no block scales) has no block-scaled "
                                      "tensor-core form; use groupsize=16")
        gs = -1                         # per-token scales: ActQuantizer._find_params (utils/quant_utils.py:242-271)
    return ops.ActFormat(mode, D, tail_len=hlen, group_size=gs, clip_ratio=float(q.clip_ratio),
                         tensor_scale=_HW_NVFP4_ACT_SCALE)


# Per-head rotation + NVFP4: True = the rotation kernel's per-head NVFP4 epilogue (head_dim a multiple of 16); False = the
# general two-launch form (rotate into scratch, gather + quantise), which also serves head dims the epilogue does not take.
PER_HEAD_NVFP4_FUSED = True


def _per_head_selection(w):
    """(H, d, tail) for a per-head layer whose format is expressed as rotation + channel selection (NVFP4), else None."""
    q = w.quantizer
    if (q.quant_dtype == "nvfp4" and w.rotation_per_head is not None and getattr(w, "_unrot_fused", False)
            and int(q.high_bits_length) > 0 and not (PER_HEAD_NVFP4_FUSED and int(w.head_dim) % 16 == 0)):
        return int(w.num_heads), int(w.head_dim), int(q.high_bits_length)
    return None


# The forward watches the device status word without synchronising (ops.StatusWatch): a bounded device-side wait that
# ran out raises at the next forward on that device.  False leaves the check to explicit ops.check_status() calls.
WATCH_STATUS = True

# How a dense NVFP4 weight (the reference's cache holds only dequantised weights) is put back on a 4-bit grid:
# "rowscale" = the reference's own two-level recipe, per-output-channel scale + E4M3 micro-scales
# (speedup/weight_only_nvfp4.py:42-72); "tensor" = one power-of-two scale per tensor with the accuracy path's tie rule.
NVFP4_WEIGHT_RECIPE = "rowscale"

# Integer-activation layers (W4A4 and W4A8) run the tensor-rate GEMM (codes expanded to fp16 next to the
# tensor core).  Set to False to route them through the exact-integer kind::i8 kernel instead.
INT4_TENSOR_RATE_GEMM = True
# The tensor-rate GEMM reads the weight as an fp16 panel.  False: the panel is rebuilt from the 4-bit codes in
# scratch on every call (weights stay 4-bit in memory; a pre-pass of N x K work per M x N x K GEMM).  True: built once
# per layer and kept (2 bytes per weight of device memory, no pre-pass).  "auto" (default): kept by layers that are
# called with few rows (at most PANEL_CACHE_MAX_ROWS: a batch shard on one of several GPUs, a small batch), where the
# pre-pass, whose cost does not shrink with the batch, is a fifth of the call; and by layers called with more rows for
# as long as all 16-bit weight copies on the device (these panels and the dense weights of W4A16 layers) stay within
# PANEL_CACHE_BUDGET_FRACTION of its memory (a sixteenth: 11 GB of a B200's 180 -- every PixArt / SANA layer, where the
# pre-pass is 2-3 % of a batch-8 step; two thirds of a 12-billion-parameter FLUX, whose long GEMMs hardly notice it);
# layers beyond the budget keep 0.5 byte per weight and rebuild per call.
CACHE_WEIGHT_PANEL = "auto"
PANEL_CACHE_MAX_ROWS = 8192
PANEL_CACHE_BUDGET_FRACTION = 1.0 / 16
_PANEL_RESIDENT_BYTES: Dict[int, int] = {}


def resident_weight_copy_bytes(device=None) -> int:
    """Bytes of 16-bit weight copies (fp16 panels, dense W4A16 weights) currently kept on the device."""
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    return _PANEL_RESIDENT_BYTES.get(idx, 0)


def _panel_budget_release(idx: int, nbytes: int):
    _PANEL_RESIDENT_BYTES[idx] = max(0, _PANEL_RESIDENT_BYTES.get(idx, 0) - nbytes)


def _panel_budget_take(owner, device, nbytes: int, always: bool) -> bool:
    """Account nbytes of 16-bit weight copy to `owner` (released when it is collected); False when a large-batch layer
    would exceed the device's budget."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    used = _PANEL_RESIDENT_BYTES.get(idx, 0)
    if not always and used + nbytes > PANEL_CACHE_BUDGET_FRACTION * torch.cuda.get_device_properties(idx).total_memory:
        return False
    _PANEL_RESIDENT_BYTES[idx] = used + nbytes
    weakref.finalize(owner, _panel_budget_release, idx, nbytes)
    return True


def _half_chunks(fmt: ops.ActFormat, lay: ops.ActLayout) -> bool:
    """dirotq_linear_uses_half_chunks for a layer on the 16-bit-conversion GEMM, before its LayerState exists."""
    return fmt.num_heads > 0 and lay.chunks_per_group == 1 and lay.group <= 32 and fmt.mode != ops.NVFP4_HW


def prepare_layer(w, device="cuda", explicit: Optional[dict] = None) -> LayerState:
    """Build the packed device state of one ActQuantWrapper.

    explicit: optional dict with the true quantised weight instead of the dequantised
    ``module.weight``: INT {"codes" [N,n_low] int, "scales" [N,G]}, NVFP4 {"nibbles" [N,n_low],
    "scales_e4m3" uint8 [N,n_low/16], "tensor_scale" float}; optional "w_tail" [N, tail_total]."""
    fmt = _act_format(w)
    lay = ops.act_layout(fmt)
    ph_sel = _per_head_selection(w)
    fused = getattr(w, "_unrot_fused", False)
    N, D = w.module.out_features, w.module.in_features
    dev = torch.device(device)
    rot_t = perm = None
    had_dim, had_flips = 0, None
    if fused and getattr(w, "use_hadamard", False):
        # same branch order as the reference forward (rotation, per-head, Hadamard, permutation)
        if w.rotation is None and w.rotation_per_head is None:
            had_dim = int(w.hadamard_low_dim)
            if getattr(w, "hadamard_sign_flips", None) is not None:
                had_flips = w.hadamard_sign_flips.to(device=dev, dtype=torch.bfloat16).contiguous()
    if fused and w.rotation is not None:
        rot_t = w.rotation.to(device=dev, dtype=torch.float32).t().contiguous().to(torch.bfloat16)
    elif fused and w.rotation_per_head is not None:
        U = w.rotation_per_head.to(device=dev, dtype=torch.float32)
        rot_t = torch.block_diag(*[U[h].t() for h in range(U.shape[0])]).contiguous().to(torch.bfloat16)
        if ph_sel is not None:
            H, d, hl = ph_sel
            cols = torch.arange(H * d, device=dev).reshape(H, d)
            perm = torch.cat([cols[:, : d - hl].reshape(-1), cols[:, d - hl:].reshape(-1)]).to(torch.int64).contiguous()
    elif fused and not had_dim and getattr(w, "perm_idx", None) is not None:
        perm = w.perm_idx.to(device=dev, dtype=torch.int64).contiguous()
    packed = getattr(w, "_b200_packed", None)
    if packed is not None:
        if packed.get("kind") != "w4a4" or packed["fmt"] != dataclasses.asdict(fmt) or packed["out_features"] != N:
            raise RuntimeError("packed-weight cache entry does not match this layer's quantiser configuration "
                               f"(cached {packed.get('fmt')}, layer {dataclasses.asdict(fmt)}): rebuild the cache")
        t = lambda v: None if v is None else v.to(dev).contiguous()
        w_codes, w_scales, w_sum = t(packed["w_codes"]), t(packed["w_scales"]), t(packed["w_sum"])
        w_tail_p, bias = t(packed["w_tail"]), t(packed["bias"])
        folded = None
        if INT4_TENSOR_RATE_GEMM and fmt.mode in (ops.INT4_SYM, ops.INT4_ASYM, ops.INT8_ASYM):
            pk = ops.PackedWeightInt4(N, lay.q_len, lay.group, lay.n_chunks, w_codes, w_scales, w_sum)
            folded = ops.fold_weight_scales_f16(pk, w_tail_p, lay.tail_total)
            if CACHE_WEIGHT_PANEL is True:
                folded.panel = ops.expand_weight_panel_f16(pk, folded, _half_chunks(fmt, lay))
        return LayerState(fmt, lay, N, rot_t, perm, w_codes, w_scales, w_sum, w_tail_p, bias,
                          float(packed["w_tensor_scale"]), int(packed["n_lossy_groups"]), folded,
                          hadamard_low_dim=had_dim, hadamard_flips=had_flips, w_rowscale=t(packed.get("w_rowscale")))
    have_codes = bool(explicit) and ("codes" in explicit or "nibbles" in explicit)
    have_tail = lay.tail_total == 0 or (bool(explicit) and "w_tail" in explicit)
    w_low = w_tail = None
    if not (have_codes and have_tail):
        # split the fused weight into the quantised block and the 16-bit tail (quant_utils.py:574-587, :659-685)
        Wf = w.module.weight.data.to(device=dev, dtype=torch.float32)
        if fmt.num_heads > 0 or ph_sel is not None:
            H, d, hl = ph_sel if ph_sel is not None else (fmt.num_heads, fmt.head_dim, fmt.tail_len)
            W3 = Wf.reshape(N, H, d)
            w_low = W3[:, :, : d - hl].reshape(N, H * (d - hl)).contiguous()
            w_tail = W3[:, :, d - hl:].reshape(N, H * hl).contiguous()
        else:
            w_low = Wf[:, : lay.q_len].contiguous()
            w_tail = Wf[:, lay.q_len:].contiguous() if lay.tail_total else None
    if explicit and "w_tail" in explicit:
        w_tail = explicit["w_tail"].to(device=dev, dtype=torch.float32)
    n_lossy, Tw, w_sum, w_rowscale = 0, 1.0, None, None
    if fmt.mode == ops.NVFP4_HW:
        if explicit and "nibbles" in explicit:
            pk = pack.convert_dirotq_low_weight_to_b200_fp4(None, explicit["tensor_scale"], explicit["nibbles"],
                                                            explicit["scales_e4m3"])
        elif NVFP4_WEIGHT_RECIPE == "rowscale":
            pk = ops.pack_weight_nvfp4_rowscale(w_low.to(dev))
        else:
            pk = pack.convert_dirotq_low_weight_to_b200_fp4(w_low)
        Tw = pk.tensor_scale
        w_codes, w_scales, w_rowscale = pk.codes, pk.sf, pk.row_scale
        out_scale = fmt.tensor_scale * Tw
        if w_tail is None:
            wt = None
        elif w_rowscale is not None:
            # the GEMM multiplies the whole accumulator by out_scale * scale[n]: the 16-bit branch is divided by it here
            wt = (w_tail.to(dev) / (out_scale * w_rowscale[:N, None])).to(torch.bfloat16)
        else:
            wt = (w_tail / out_scale).to(torch.bfloat16)
    else:
        if explicit and "codes" in explicit:
            pk = pack.convert_dirotq_low_weight_to_b200(None, lay.group, scales=explicit["scales"], codes=explicit["codes"])
        else:
            rec = pack.recover_int4_grid(w_low, lay.group)
            n_lossy = rec.n_lossy
            if n_lossy:
                warnings.warn(f"{n_lossy} weight groups of a [{N},{D}] layer are not on a 4-bit grid; re-quantised")
            pk = ops.pack_weight_int4(w_low, lay.group, scales=rec.scales.to(dev))
        w_codes, w_scales, w_sum = pk.codes, pk.scales, pk.wsum
        wt = None if w_tail is None else w_tail.to(torch.bfloat16)
    w_tail_p = ops.pad_tail_weight(wt, lay.tail_pitch, N, dev)
    if explicit and "bias" in explicit:
        bias = None if explicit["bias"] is None else explicit["bias"].to(device=dev, dtype=torch.bfloat16).contiguous()
    else:
        bias = None if w.module.bias is None else w.module.bias.data.to(device=dev, dtype=torch.bfloat16).contiguous()
    folded = None
    if INT4_TENSOR_RATE_GEMM and fmt.mode in (ops.INT4_SYM, ops.INT4_ASYM, ops.INT8_ASYM):
        folded = ops.fold_weight_scales_f16(pk, w_tail_p, lay.tail_total)
        if CACHE_WEIGHT_PANEL is True:
            folded.panel = ops.expand_weight_panel_f16(pk, folded, _half_chunks(fmt, lay))
    return LayerState(fmt, lay, N, rot_t, perm, w_codes, w_scales, w_sum, w_tail_p, bias, Tw, n_lossy, folded,
                      hadamard_low_dim=had_dim, hadamard_flips=had_flips, w_rowscale=w_rowscale)


@dataclass
class W4A16State:
    """A layer whose activations stay 16-bit while its weight is 4-bit (bits == 16 under
    --skip-quant-layers, e.g. PixArt ff.net.2): INT4 group-64 weight, or NVFP4 weight as in the reference's
    WeightOnlyNVFP4Linear (speedup/weight_only_nvfp4.py:128-178)."""
    w: object                       # ops.PackedWeightInt4 or ops.PackedWeightNvfp4
    bias: Optional[torch.Tensor]
    dense: Optional[torch.Tensor] = None      # resident dequantised weight (bf16 [N, K]), see w4a16_forward
    declined: bool = False                    # a large-batch call found the budget for resident 16-bit copies spent


# Dequantised weights of W4A16 layers follow the policy of CACHE_WEIGHT_PANEL: resident (2 bytes per weight) for layers
# called with at most PANEL_CACHE_MAX_ROWS rows, where the dequantisation is a visible share of the call, and for the
# others while the device's budget lasts; otherwise rebuilt on every call in ONE scratch buffer per device and stream,
# shared by all layers (stream order keeps it safe).
_W4A16_SCRATCH: Dict[tuple, torch.Tensor] = {}


def _w4a16_scratch(nbytes: int, device) -> torch.Tensor:
    key = (torch.device(device).index, torch.cuda.current_stream(device).cuda_stream)
    buf = _W4A16_SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _W4A16_SCRATCH[key] = buf
    return buf


def w4a16_forward(s16: W4A16State, x2d: torch.Tensor) -> torch.Tensor:
    """bf16 activations x 4-bit weight: x2d bf16 [M, K] -> bf16 [M, N]."""
    M = x2d.shape[0]
    nvfp4 = isinstance(s16.w, ops.PackedWeightNvfp4)
    resident = s16.dense is not None or CACHE_WEIGHT_PANEL is True
    if not resident and CACHE_WEIGHT_PANEL == "auto" and not s16.declined:
        resident = _panel_budget_take(s16, x2d.device, 2 * s16.w.N * s16.w.n_chunks * 64, M <= PANEL_CACHE_MAX_ROWS)
        s16.declined = not resident and M > PANEL_CACHE_MAX_ROWS
    if resident:
        if s16.dense is None:
            s16.dense = ops.dequant_weight_nvfp4(s16.w) if nvfp4 else ops.dequant_weight_int4(s16.w)
        return ops.gemm_bf16(x2d, s16.dense, s16.bias)
    K = s16.w.n_chunks * 64
    scratch = _w4a16_scratch(int(_lib.lib().dirotq_gemm_w4a16_workspace_bytes(s16.w.N, K)), x2d.device)
    if nvfp4:
        return ops.gemm_w4a16_nvfp4(x2d, s16.w, s16.bias, workspace=scratch)
    return ops.gemm_w4a16(x2d, s16.w, s16.bias, workspace=scratch)


def prepare_w4a16(w, device="cuda", explicit: Optional[dict] = None, group: int = 64) -> Optional[W4A16State]:
    """Pack the 4-bit weight of an activation-unquantised layer, if its weight IS on a 4-bit grid."""
    N, K = w.module.out_features, w.module.in_features
    if K % 64 or N % 8 or group != 64:
        return None
    dev = torch.device(device)
    packed = getattr(w, "_b200_packed", None)
    if packed is not None:
        if packed.get("kind") != "w4a16" or packed["N"] != N or packed["K"] != K:
            raise RuntimeError("packed-weight cache entry does not match this 16-bit-activation layer: rebuild the cache")
        t = lambda v: None if v is None else v.to(dev).contiguous()
        if packed["weight"] == "nvfp4":
            pk = ops.PackedWeightNvfp4(N, K, K // 64, float(packed["tensor_scale"]), t(packed["codes"]), t(packed["sf"]),
                                       t(packed.get("row_scale")))
        else:
            pk = ops.PackedWeightInt4(N, K, 64, K // 64, t(packed["codes"]), t(packed["scales"]), t(packed["wsum"]))
        return W4A16State(pk, t(packed["bias"]))
    if explicit and "nibbles" in explicit:
        pk = pack.convert_dirotq_low_weight_to_b200_fp4(None, explicit["tensor_scale"], explicit["nibbles"],
                                                        explicit["scales_e4m3"])
        bias = explicit.get("bias")
    elif explicit and "codes" in explicit:
        pk = pack.convert_dirotq_low_weight_to_b200(None, 64, scales=explicit["scales"], codes=explicit["codes"])
        bias = explicit.get("bias")
    else:
        W = w.module.weight.data.to(device=dev, dtype=torch.float32)
        rec = pack.recover_int4_grid(W, 64)
        if rec.n_lossy:
            return None            # a genuine 16-bit layer: stays an nn.Linear
        pk = ops.pack_weight_int4(W, 64, scales=rec.scales.to(dev))
        bias = w.module.bias.data if w.module.bias is not None else None
    bias = None if bias is None else bias.to(device=dev, dtype=torch.bfloat16).contiguous()
    return W4A16State(pk, bias)


def _fused_forward_b200(self, x):
    """ActQuantWrapper.forward on the B200 kernels (contract: dirotq_fused_unrotation_fast.py:56-141)."""
    if self.quantizer.bits >= 16:
        s16 = getattr(self, "_b200_w4a16", None)
        if s16 is None and getattr(self, "_b200_explicit", None) is not None:
            s16 = prepare_w4a16(self, x.device, self._b200_explicit)     # synthetic layer: no dense weight
            object.__setattr__(self, "_b200_w4a16", s16)
        if s16 is None:
            return self.module(x).to(x.dtype)
        shp = x.shape
        x2d = x.reshape(-1, shp[-1]).to(torch.bfloat16).contiguous()
        y = w4a16_forward(s16, x2d)
        return y.reshape(*shp[:-1], s16.w.N).to(x.dtype)
    st = getattr(self, "_b200_state", None)
    if st is None:
        st = prepare_layer(self, x.device, getattr(self, "_b200_explicit", None))
        object.__setattr__(self, "_b200_state", st)
    x_dtype = x.dtype
    shp = x.shape
    x2d = x.reshape(-1, shp[-1])
    if x2d.dtype != torch.bfloat16:
        x2d = x2d.to(torch.bfloat16)     # the kernels compute in bf16 (fp16 pipelines are converted here)
    y = linear_forward(st, x2d.contiguous())
    return y.reshape(*shp[:-1], st.out_features).to(x_dtype)


# Sibling layers with equal rotation and format (to_q / to_k / to_v) rotate and quantise their common
# input once.  Set to False to give every layer its own pass.
SHARE_SIBLING_ACTIVATIONS = True
# groups of leaf names whose members read one tensor through one rotation: the image-stream and (FLUX double blocks,
# models/flux-schnell/model_utils.py:180-186) the text-stream projections of an attention
_SIBLING_GROUPS = (("to_q", "to_k", "to_v"), ("add_q_proj", "add_k_proj", "add_v_proj"))


def share_sibling_activations(transformer, classes=None) -> int:
    """Group prepared sibling wrappers (same parent module, names to_q / to_k / to_v or add_q_proj / add_k_proj /
    add_v_proj) whose rotations are equal element for element and whose activation formats are identical.  Returns
    the number of groups."""
    classes = tuple(classes or _wrapper_classes())
    buckets: Dict[str, list] = {}
    for name, mod in transformer.named_modules():
        if not isinstance(mod, classes):
            continue
        st = getattr(mod, "_b200_state", None)
        parent, _, leaf = name.rpartition(".")
        gid = next((i for i, grp in enumerate(_SIBLING_GROUPS) if leaf in grp), None)
        if st is None or st.rot_t is None or gid is None:
            continue
        buckets.setdefault((parent, gid), []).append(st)
    n_groups = 0
    for members in buckets.values():
        first = members[0]
        same = [first] + [m for m in members[1:]
                          if m.fmt == first.fmt and (m.folded is None) == (first.folded is None)
                          and m.rot_t.shape == first.rot_t.shape and torch.equal(m.rot_t, first.rot_t)]
        if len(same) < 2:
            continue
        grp = SharedActivation(len(same))
        grp.members = list(same)
        for i, m in enumerate(same):
            m.shared, m.member_id = grp, i
            m.rot_t = first.rot_t            # one copy of the rotation on the device
            m._c = None
            m._ws = {}
        n_groups += 1
    return n_groups


def _concat_states(members) -> Optional[LayerState]:
    """One LayerState whose weight is the members' weights stacked along the output dimension (same activation format,
    rotation and GEMM variant).  None where the packed layouts do not concatenate (NVFP4 scale tiles span 128 output
    channels; the members' weight tensor scales and epilogues must agree)."""
    first = members[0]
    fmt, lay, dev = first.fmt, first.layout, first.w_codes.device
    if any(m.hadamard_low_dim or m.perm_idx is not None or m.epilogue_act != first.epilogue_act or m.chain_next is not None
           or m.w_tensor_scale != first.w_tensor_scale or (m.w_rowscale is None) != (first.w_rowscale is None)
           or (m.folded is None) != (first.folded is None) or m.out_features % 8 for m in members):
        return None
    nvfp4 = fmt.mode == ops.NVFP4_HW
    if nvfp4 and any(m.out_features % 128 for m in members):
        return None
    N = sum(m.out_features for m in members)
    w_codes = torch.cat([m.w_codes[: m.out_features] for m in members], 0).contiguous()
    has_bias = any(m.bias is not None for m in members)
    bias = None
    if has_bias:
        bias = torch.cat([m.bias if m.bias is not None else torch.zeros(m.out_features, dtype=torch.bfloat16, device=dev)
                          for m in members]).contiguous()
    w_tail = None
    if lay.tail_total > 0:
        w_tail = torch.cat([m.w_tail[: m.out_features] for m in members], 0).contiguous()
    if nvfp4:
        w_scales = torch.cat([m.w_scales for m in members]).contiguous()              # whole 128-channel tiles
        rs = None
        if first.w_rowscale is not None:
            rs = torch.cat([m.w_rowscale[: m.out_features] for m in members]).contiguous()
        return LayerState(fmt, lay, N, first.rot_t, None, w_codes, w_scales, None, w_tail, bias, first.w_tensor_scale,
                          0, None, epilogue_act=first.epilogue_act, w_rowscale=rs)
    w_scales = torch.cat([m.w_scales[:, : m.out_features] for m in members], 1).contiguous()
    w_sum = torch.cat([m.w_sum[:, : m.out_features] for m in members], 1).contiguous()
    folded = None
    if first.folded is not None:
        pk = ops.PackedWeightInt4(N, lay.q_len, lay.group, lay.n_chunks, w_codes, w_scales, w_sum)
        folded = ops.fold_weight_scales_f16(pk, w_tail, lay.tail_total)                # per-channel: same constants
    return LayerState(fmt, lay, N, first.rot_t, None, w_codes, w_scales, w_sum, w_tail, bias, first.w_tensor_scale, 0,
                      folded, epilogue_act=first.epilogue_act)


def fuse_sibling_gemms(transformer, classes=None) -> int:
    """Sibling layers that already share one rotate + quantise pass (share_sibling_activations: to_q / to_k / to_v,
    add_q_proj / add_k_proj / add_v_proj) also run as ONE GEMM on their weights concatenated along the output
    dimension -- the shape the reference's speed path gives its fused qkv projection
    (speedup/report_flux_w4a4_no_rot_ffdown.py:336-345).  The first member called on a tensor launches the pass and
    the GEMM; every member returns its own columns of the [M, sum N] result (a strided view; values are bit-identical
    to the separate GEMMs, whose per-element arithmetic does not depend on the tiling).  A group whose members turn out
    to see different tensors (a cross-attention) falls back to separate GEMMs after three unconsumed passes; for that
    the members keep their own packed weights, so a fused group holds its 4-bit weights twice.
    Returns the number of fused groups."""
    classes = tuple(classes or _wrapper_classes())
    groups = {}
    for _, mod in transformer.named_modules():
        st = getattr(mod, "_b200_state", None) if isinstance(mod, classes) else None
        if st is not None and st.shared is not None:
            groups[id(st.shared)] = st.shared
    n = 0
    for grp in groups.values():
        if grp.fused is not None or len(grp.members) < 2:
            continue
        fused = _concat_states(grp.members)
        if fused is None:
            continue
        grp.fused, grp.offsets, off = fused, [], 0
        for m in grp.members:
            grp.offsets.append(off)
            off += m.out_features
        n += 1
    return n


def release_shared_activations(transformer, classes=None) -> int:
    """Drop the input tensors that sibling groups still hold (call between denoising steps, or when a pipeline is
    parked, if activation memory matters); the next forward simply rotates and quantises again."""
    classes = tuple(classes or _wrapper_classes())
    groups = {}
    for _, mod in transformer.named_modules():
        st = getattr(mod, "_b200_state", None) if isinstance(mod, classes) else None
        if st is not None and st.shared is not None:
            groups[id(st.shared)] = st.shared
    for grp in groups.values():
        grp.release()
    return len(groups)


def fuse_gelu_modules(transformer, classes=None) -> int:
    """Fuse the activation that follows a wrapped linear into its GEMM epilogue.

    Looks for modules shaped like diffusers' GELU feed-forward head (attributes `proj` -- a prepared wrapped
    linear -- and `approximate == "tanh"`; forward = gelu(proj(x))), marks the linear to apply GELU (tanh
    form) on its bf16-rounded output inside the GEMM epilogue, and replaces the module's forward by a plain
    call of `proj`.  One full read + write pass over the [M, 4 * hidden] tensor disappears per block.
    Call after preconvert_rotations_to_device.  Returns the number of fused modules."""
    classes = tuple(classes or _wrapper_classes())
    n = 0
    for _, mod in transformer.named_modules():
        proj = getattr(mod, "proj", None)
        if not isinstance(proj, classes) or getattr(mod, "approximate", None) != "tanh":
            continue
        st = getattr(proj, "_b200_state", None)
        if st is None or getattr(mod, "_b200_gelu_fused", False):
            continue
        if st.folded is None and st.fmt.mode != ops.NVFP4_HW:
            continue                      # exact-integer route: no fused activation
        st.epilogue_act, st._c = 1, None
        object.__setattr__(mod, "_b200_gelu_fused", True)
        mod.forward = (lambda p: (lambda hidden_states, *a, **k: p(hidden_states)))(proj)
        n += 1
    return n


def chain_supported(up: LayerState, down: LayerState) -> bool:
    """Whether `up`'s GEMM epilogue can quantise for `down` (dirotq_linear_chain_supported of the C ABI)."""
    if up.shared is not None or down.shared is not None or down.hadamard_low_dim:
        return False
    return bool(_lib.lib().dirotq_linear_chain_supported(C.byref(up.c_struct()), C.byref(down.c_struct())))


def fuse_ffn_quantise(transformer=None, pairs=None, keep_hidden: bool = True, classes=None) -> int:
    """Let the up-projection of a feed-forward pair quantise its own output for the down-projection.

    The reference runs two ActQuantWrapper forwards with the activation between them
    (models/pixart-sigma/model_utils.py:120-127): GELU(up(x)) goes to memory as [M, inner] bf16 and the second
    wrapper reads it back to quantise it.  After this call the up-projection's GEMM epilogue (which already applies
    the GELU, fuse_gelu_modules) emits the down-projection's 4-bit codes, group scales, zero points and 16-bit
    channels directly -- bit for bit what the down-projection's own quantiser would have produced -- and the
    down-projection, recognising the tensor it is called on (storage, shape, version counter; the producer's output
    is kept referenced until then), runs only its GEMM.

    Pairs come from `transformer` (modules with a `net` container: first entry a GELU head fused by
    fuse_gelu_modules, last entry a prepared wrapped linear, only Dropout / Identity between them; and blocks with a
    fused head `proj_mlp_act` beside a split `proj_out.linears`) and / or from `pairs` (explicit
    (up_wrapper, down_wrapper) tuples).  Only pairs the
    library supports are fused (chain_supported); the others keep their two-step forward.

    keep_hidden=False additionally stops writing the [M, inner] tensor: the tensor the up-projection returns is
    then an UNWRITTEN buffer that only the down-projection may consume.  Use it only where nothing else reads the
    hidden activation (not for the reference's FLUX single block, whose split proj_out slices a concatenation).
    Returns the number of fused pairs."""
    classes = tuple(classes or _wrapper_classes())
    cand = list(pairs or [])
    if transformer is not None:
        for _, mod in transformer.named_modules():
            # a FLUX single block after the proj_out split (models/flux-schnell/split_proj_out.py:38-48) whose MLP
            # branch is handed over directly: GELU head `proj_mlp_act`, down-projection `proj_out.linears[1]`
            head, split = getattr(mod, "proj_mlp_act", None), getattr(getattr(mod, "proj_out", None), "linears", None)
            if head is not None and split is not None and getattr(head, "_b200_gelu_fused", False):
                split = list(split.children())
                if len(split) == 2 and isinstance(split[1], classes) and isinstance(getattr(head, "proj", None), classes):
                    cand.append((head.proj, split[1]))
            net = getattr(mod, "net", None)
            net = list(net.children()) if isinstance(net, torch.nn.Module) else None
            if not net or len(net) < 2 or not getattr(net[0], "_b200_gelu_fused", False):
                continue
            if not all(isinstance(m, (torch.nn.Dropout, torch.nn.Identity)) for m in net[1:-1]):
                continue
            if isinstance(net[-1], classes) and isinstance(getattr(net[0], "proj", None), classes):
                cand.append((net[0].proj, net[-1]))
    n = 0
    for up, down in cand:
        su, sd = getattr(up, "_b200_state", None), getattr(down, "_b200_state", None)
        if su is None or sd is None or su.chain_next is not None or not chain_supported(su, sd):
            continue
        su.chain_next, su.chain_keep_output = sd, bool(keep_hidden)
        sd.chain_fed = True
        n += 1
    return n


def _wrapper_classes():
    classes = [ActQuantWrapper]
    ref = sys.modules.get("utils.quant_utils")
    if ref is not None and hasattr(ref, "ActQuantWrapper"):
        classes.append(ref.ActQuantWrapper)     # drop-in use inside the reference project
    return classes


PACKED_CACHE_VERSION = 1


def save_packed_weights(transformer, path) -> int:
    """Write the packed weights of every prepared wrapped linear (codes, group scales, group sums, 16-bit tail,
    bias, tensor scale, and the activation format they were packed for) to ``path``; returns the number of
    layers written.  The reference keeps its quantised model as a state_dict of DEQUANTISED bf16 weights
    (apply_dirotq.py:231-257, 317-349), from which every start-up would have to recover the 4-bit grid and
    pack again; this file sits next to that cache and can always be rebuilt from it (load the reference cache,
    preconvert_rotations_to_device, save_packed_weights).  Rotations, permutations and sign flips are not
    stored: they come from the wrapper's own attributes at load time."""
    classes = tuple(_wrapper_classes())
    layers = {}
    cpu = lambda v: None if v is None else v.detach().cpu()
    for name, mod in transformer.named_modules():
        if not isinstance(mod, classes):
            continue
        st = getattr(mod, "_b200_state", None)
        s16 = getattr(mod, "_b200_w4a16", None)
        if st is not None:
            layers[name] = {"kind": "w4a4", "fmt": dataclasses.asdict(st.fmt), "out_features": st.out_features,
                            "w_codes": cpu(st.w_codes), "w_scales": cpu(st.w_scales), "w_sum": cpu(st.w_sum),
                            "w_tail": cpu(st.w_tail), "bias": cpu(st.bias), "w_tensor_scale": float(st.w_tensor_scale),
                            "w_rowscale": cpu(st.w_rowscale),
                            "n_lossy_groups": int(st.n_lossy_groups)}
        elif s16 is not None:
            pk = s16.w
            e = {"kind": "w4a16", "N": pk.N, "K": pk.n_chunks * 64, "bias": cpu(s16.bias), "codes": cpu(pk.codes)}
            if isinstance(pk, ops.PackedWeightNvfp4):
                e.update(weight="nvfp4", tensor_scale=float(pk.tensor_scale), sf=cpu(pk.sf), row_scale=cpu(pk.row_scale))
            else:
                e.update(weight="int4", scales=cpu(pk.scales), wsum=cpu(pk.wsum))
            layers[name] = e
    torch.save({"version": PACKED_CACHE_VERSION, "abi": int(_lib.lib().dirotq_abi_version()), "layers": layers}, path)
    return len(layers)


def load_packed_weights(transformer, path) -> int:
    """Attach the entries of a save_packed_weights file to the wrapped linears of the same names; the next
    preconvert_rotations_to_device (or first forward) then uploads them instead of recovering and packing the
    weights again.  A layer whose quantiser configuration differs from the cached one raises at that point.
    Returns the number of layers matched; layers absent from the file are packed from their weights as usual."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    if blob.get("version") != PACKED_CACHE_VERSION or blob.get("abi") != int(_lib.lib().dirotq_abi_version()):
        raise RuntimeError(f"{path}: packed-weight cache of another layout version; rebuild it")
    classes = tuple(_wrapper_classes())
    n = 0
    for name, mod in transformer.named_modules():
        if isinstance(mod, classes) and name in blob["layers"]:
            object.__setattr__(mod, "_b200_packed", blob["layers"][name])
            n += 1
    return n


def patch_forward():
    """Monkey-patch ActQuantWrapper.forward (this package's class and, when the reference project is
    imported, its class too) with the B200 path."""
    for cls in _wrapper_classes():
        cls.forward = _fused_forward_b200
    print("Patched ActQuantWrapper.forward with the B200 (sm_100a) fused path.")


def preconvert_rotations_to_device(transformer, device="cuda", dtype=None):
    """One-time preparation of every wrapped linear: rotations to bf16 K-major on the device, weights
    quantised/packed.  Returns the number of rotation / permutation tensors converted (the value the
    reference prints and returns, dirotq_fused_unrotation_fast.py:25-53).  ``dtype`` is accepted for
    signature compatibility; the kernels always compute in bf16."""
    classes = tuple(_wrapper_classes())
    n = 0
    for _, mod in transformer.named_modules():
        if not isinstance(mod, classes):
            continue
        if mod.quantizer.bits >= 16:
            s16 = prepare_w4a16(mod, device, getattr(mod, "_b200_explicit", None))
            if s16 is not None:
                object.__setattr__(mod, "_b200_w4a16", s16)
            continue
        st = prepare_layer(mod, device, getattr(mod, "_b200_explicit", None))
        object.__setattr__(mod, "_b200_state", st)
        if st.rot_t is not None or st.perm_idx is not None:
            n += 1
    n_groups = share_sibling_activations(transformer, classes) if SHARE_SIBLING_ACTIVATIONS else 0
    if n_groups:
        print(f"{n_groups} groups of sibling layers (same input, same rotation) share one rotate+quantise pass.")
    print(f"Preconverted {n} rotation/permutation tensors to {device} (bf16, K-major) and packed the weights.")
    return n
