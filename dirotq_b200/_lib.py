"""ctypes binding of libdirotq_b200.so (the C ABI declared in include/dirotq_b200.h).

There is no fallback: if the CUDA library has not been built, importing the ops fails loudly.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DIROTQ_B200_LIB selects another build of the same ABI (A/B measurements)
LIB_PATH = os.environ.get("DIROTQ_B200_LIB") or os.path.join(_HERE, "libdirotq_b200.so")


class ActFormatC(C.Structure):
    _fields_ = [("mode", C.c_int32), ("width", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32),
                ("tail_len", C.c_int32), ("group_size", C.c_int32), ("clip_ratio", C.c_float),
                ("tensor_scale", C.c_float)]


class ActLayoutC(C.Structure):
    _fields_ = [("q_len", C.c_int32), ("group", C.c_int32), ("n_groups", C.c_int32),
                ("chunks_per_group", C.c_int32), ("n_chunks", C.c_int32), ("k_pad", C.c_int32),
                ("code_row_bytes", C.c_int32), ("tail_total", C.c_int32), ("tail_pitch", C.c_int32),
                ("n_scales", C.c_int32)]


class LinearC(C.Structure):
    _fields_ = [("fmt", ActFormatC), ("out_features", C.c_int64), ("rot_t", C.c_void_p), ("perm_idx", C.c_void_p),
                ("w_codes", C.c_void_p), ("w_scales", C.c_void_p), ("w_sum", C.c_void_p), ("w_tail", C.c_void_p),
                ("bias", C.c_void_p), ("w_tensor_scale", C.c_float), ("w_mult", C.c_void_p),
                ("w_colscale", C.c_void_p), ("w_tail_f16", C.c_void_p), ("epilogue_act", C.c_int32),
                ("w_panel_f16", C.c_void_p)]


_P, _I64, _I32, _F, _SZ = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_size_t
_FMT, _LAY = C.POINTER(ActFormatC), C.POINTER(ActLayoutC)

# name -> (restype, argtypes); mirrors include/dirotq_b200.h one to one
SIGNATURES = {
    "dirotq_abi_version": (C.c_int, []),
    "dirotq_set_wait_limit_cycles": (C.c_int, [_I64]),
    "dirotq_error_string": (C.c_char_p, [C.c_int]),
    "dirotq_status_string": (C.c_char_p, [C.c_int]),
    "dirotq_act_layout_of": (C.c_int, [_FMT, _LAY]),
    "dirotq_act_codes_bytes": (_SZ, [_LAY, _I64]),
    "dirotq_act_scales_bytes": (_SZ, [_FMT, _LAY, _I64]),
    "dirotq_act_zeros_bytes": (_SZ, [_FMT, _LAY, _I64]),
    "dirotq_act_tail_bytes": (_SZ, [_LAY, _I64]),
    "dirotq_quantize_act": (C.c_int, [_FMT, _P, _I64, _P, _I64, _P, _P, _P, _P, _P]),
    "dirotq_rotate_quantize": (C.c_int, [_FMT, _P, _P, _I64, _P, _P, _P, _P, _P, _P, _P]),
    "dirotq_pack_weight_int4": (C.c_int, [_P, _I64, _I64, _I32, _P, _I32, _P, _P, _P, _P]),
    "dirotq_pack_weight_nvfp4": (C.c_int, [_P, _I64, _I64, _F, _P, _I32, _P, _P, _P]),
    "dirotq_gemm_w4a4_int": (C.c_int, [_I32, _I64, _I64, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _I32, _I32, _P, _P,
                                        _P, _P, _P]),
    "dirotq_hadamard_low": (C.c_int, [_P, _I64, _I32, _I32, _P, _P, _P]),
    "dirotq_fold_weight_records_bytes": (_SZ, [_I32, _I64]),
    "dirotq_fold_weight_scales_f16": (C.c_int, [_I32, _I64, _P, _P, _I32, _I32, _P, _P, _P, _P]),
    "dirotq_weight_panel_bytes": (_SZ, [_I32, _I64]),
    "dirotq_expand_weight_panel_f16": (C.c_int, [_I32, _I64, _P, _P, _P, _P]),
    "dirotq_gemm_w4a4_int_f16_workspace_bytes": (_SZ, [_I64, _I64, _I32, _I32]),
    "dirotq_gemm_w4a4_int_f16": (C.c_int, [_I32, _I64, _I64, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I32, _I32, _P,
                                            _P, _P, _SZ, _P, _P]),
    "dirotq_pack_weight_nvfp4_rowscale": (C.c_int, [_P, _I64, _I64, _P, _P, _P, _P, _P]),
    "dirotq_gemm_w4a4_nvfp4": (C.c_int, [_I64, _I64, _I32, _P, _P, _P, _P, _F, _P, _P, _P, _I32, _I32, _P, _P, _P, _P]),
    "dirotq_gemm_w4a16_workspace_bytes": (_SZ, [_I64, _I64]),
    "dirotq_gemm_w4a16": (C.c_int, [_I64, _I64, _I64, _P, _P, _P, _P, _P, _P, _SZ, _P, _P]),
    "dirotq_gemm_w4a16_nvfp4": (C.c_int, [_I64, _I64, _I64, _P, _P, _P, _F, _P, _P, _P, _P, _SZ, _P, _P]),
    "dirotq_dequant_weight_nvfp4": (C.c_int, [_I64, _I64, _P, _P, _F, _P, _P, _P]),
    "dirotq_linear_workspace_bytes": (_SZ, [C.POINTER(LinearC), _I64]),
    "dirotq_linear_forward": (C.c_int, [C.POINTER(LinearC), _P, _I64, _P, _P, _SZ, _P, _P]),
    "dirotq_linear_gemm": (C.c_int, [C.POINTER(LinearC), _I64, _P, _P, _SZ, _P, _P]),
    "dirotq_expand_weight_panel_f16_layout": (C.c_int, [_I32, _I64, _P, _P, _P, _I32, _P]),
    "dirotq_linear_uses_half_chunks": (C.c_int, [C.POINTER(LinearC)]),
    "dirotq_layernorm_modulate": (C.c_int, [_P, _I64, _I32, _I64, _P, _P, _I64, _F, _P, _P]),
    "dirotq_gated_residual": (C.c_int, [_P, _P, _P, _P, _I64, _I64, _I32, _I64, _P, _P]),
    "dirotq_qkv_norm_rope": (C.c_int, [_P, _P, _P, _I64, _I64, _I64, _I32, _I32, _P, _P, _P, _P, _I64, _I64, _F, _P, _P, _P, _P]),
    "dirotq_dequant_weight_int4": (C.c_int, [_I64, _I64, _P, _P, _P, _P]),
    "dirotq_gemm_bf16": (C.c_int, [_I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "dirotq_linear_chain_supported": (C.c_int, [C.POINTER(LinearC), C.POINTER(LinearC)]),
    "dirotq_linear_forward_chain": (C.c_int, [C.POINTER(LinearC), _P, _I64, _P, _P, _SZ, C.POINTER(LinearC), _P, _SZ, _P, _P]),
    "dirotq_linear_gemm_prequantised": (C.c_int, [C.POINTER(LinearC), _I64, _P, _P, _SZ, _P, _P]),
    "dirotq_linear_forward_static_capacity": (_SZ, []),
    "dirotq_linear_forward_static": (C.c_int, [C.POINTER(LinearC), _P, _I64, _P, _P, _P]),
}

ABI_VERSION = 6
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dirotq_b200.build_ext` "
                "(there is no CPU or PyTorch fallback for the quantized-linear path)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)       # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        if l.dirotq_abi_version() != ABI_VERSION:
            raise RuntimeError("libdirotq_b200.so ABI version mismatch")
        _lib = l
    return _lib


def check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: {lib().dirotq_error_string(rc).decode()} (code {rc})")
