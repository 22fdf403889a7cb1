"""The allocation-free entry point (dirotq_linear_forward_static) against the regular one.

Some hosts give a plug-in no way to allocate device memory; for them the library carries its own
fixed scratch array.  This test drives the entry point through the C ABI and checks that it returns
exactly what dirotq_linear_forward returns with caller-provided scratch -- on two calls in a row that
use different formats and shapes, so the second call finds the first call's bytes in the array.
Collected last on purpose (file name), and self-contained so it also passes in a fresh process.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(quant, D, N, k, seed):
    from dirotq_b200 import backend, dit
    ld = dit.LayerDef("probe", D, N, tail=k)
    w = dit.make_wrapped_linear(ld, quant, seed, "cuda")
    return backend.prepare_layer(w, "cuda", w._b200_explicit)


def test_static_scratch_entry_point_matches_regular_one():
    from dirotq_b200 import _lib, backend, ops
    from dirotq_b200.synth import synth_activations
    lib = _lib.lib()
    cap = int(lib.dirotq_linear_forward_static_capacity())
    assert cap == 32 << 20
    g = torch.Generator().manual_seed(77)
    cases = [("nvfp4", 1152, 384, 144, 1000), ("int4", 320, 256, 64, 300), ("nvfp4", 1152, 384, 144, 520)]
    for i, (quant, D, N, k, M) in enumerate(cases):
        st = _layer(quant, D, N, k, 900 + i)
        x = synth_activations(M, D, g).cuda()
        y_ref = backend.linear_forward(st, x)              # caller-provided (torch) scratch
        y_a = backend.linear_forward_static(st, x)         # library scratch, first use with this shape
        y_b = backend.linear_forward_static(st, x)         # again, over its own leftovers
        ops.check_status()
        assert torch.equal(y_a, y_ref), (quant, M)
        assert torch.equal(y_b, y_ref), (quant, M)
    # a size beyond the fixed capacity is refused before anything runs
    st = _layer("int4", 1152, 128, 64, 990)
    M_big = 200000
    need = int(lib.dirotq_linear_workspace_bytes(C.byref(st.c_struct()), M_big))
    assert need > cap
    x = torch.empty(M_big, 1152, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(M_big, 128, dtype=torch.bfloat16, device="cuda")
    rc = lib.dirotq_linear_forward_static(C.byref(st.c_struct()), C.c_void_p(x.data_ptr()), M_big,
                                          C.c_void_p(y.data_ptr()),
                                          C.c_void_p(ops.status_word(x.device).data_ptr()),
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -5 and b"capacity" in lib.dirotq_error_string(rc)


def test_static_scratch_pads_never_read_leftover_bytes():
    """Shapes whose layouts have REAL padding -- a tail of 44 channels in a pitch of 48, a last INT4 group of 20 of
    64 code slots, NVFP4 rows with a partial last 64-slot chunk, M not a multiple of 128 -- run right after a larger
    call that leaves non-zero bytes over the whole carve.  The result must equal the regular entry point's on a
    zeroed workspace: pad columns and rows reach the GEMM as zeros from the copy engine's bounds handling, pad code
    slots as zero codes from the quantiser."""
    from dirotq_b200 import backend, dit, ops
    from dirotq_b200.synth import synth_activations
    g = torch.Generator().manual_seed(78)
    big = _layer("int4", 1152, 256, 64, 950)
    x_big = synth_activations(3000, 1152, g).cuda()
    for quant, D, N, k, M, sym in [("int4", 320, 136, 44, 333, False), ("nvfp4", 320, 136, 48, 333, True),
                                   ("int4", 320, 136, 44, 77, True)]:
        ld = dit.LayerDef("probe", D, N, tail=k)
        w = dit.make_wrapped_linear(ld, quant, 960, "cuda", a_sym=sym)
        st = backend.prepare_layer(w, "cuda", w._b200_explicit)
        assert st.layout.tail_pitch != st.layout.tail_total or st.layout.q_len % 64
        x = synth_activations(M, D, g).cuda()
        backend.linear_forward_static(big, x_big)           # fills the array with another layer's bytes
        y_static = backend.linear_forward_static(st, x)
        y_ref = backend.linear_forward(st, x)
        ops.check_status()
        assert bool(torch.isfinite(y_static.float()).all())
        assert torch.equal(y_static, y_ref), (quant, D, k, M)
