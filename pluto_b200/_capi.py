"""ctypes binding of the C ABI in include/pluto_b200.h.

The shared library is built in-tree by `pluto_b200.build`; if it is missing this module raises
immediately -- there is no CPU or PyTorch fallback for any operation of the engine.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpluto_b200.so")


class PlutoStatusError(RuntimeError):
    """Non-OK return of a C entry point.  `code` uses absl::StatusCode names."""

    def __init__(self, code: str, message: str, raw: int):
        super().__init__(f"{code}: {message}")
        self.code = code
        self.message = message
        self.raw = raw


_CODES = {-1: "InvalidArgument", -2: "Unimplemented", -3: "ResourceExhausted", -4: "Internal"}

_vp, _i, _sz, _fp = C.c_void_p, C.c_int, C.c_size_t, C.c_float
_SIGNATURES = {
    "pluto_last_error": (C.c_char_p, []),
    "pluto_build_info": (C.c_char_p, []),
    "pluto_kernel_status": (_i, [C.POINTER(C.c_uint32), _i]),
    "pluto_attn_fwd": (_i, [_vp] * 5 + [_i] * 5),
    "pluto_attn_bwd": (_i, [_vp] * 8 + [_i] * 5 + [_vp, _sz]),
    "pluto_attn_bwd_workspace_bytes": (_sz, [_i] * 5),
    "pluto_attn_probs": (_i, [_vp] * 5 + [_i] * 5),
    "pluto_gqa_prefill_fwd": (_i, [_vp] * 9 + [_i] * 5 + [_sz, _sz, _sz, _sz, _i, _vp, _sz]),
    "pluto_gqa_prefill_fwd_workspace_bytes": (_sz, [_i] * 4),
    "pluto_gqa_prefill_host_workspace_bytes": (_sz, [_i] * 6),
    "pluto_gqa_prefill_fwd_host": (_i, [_vp] * 6 + [_sz] + [_i] * 6),
    "pluto_linear_imported_fwd": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i]),
    "pluto_dense_workspace_bytes": (_sz, [_i] * 3),
    "pluto_dense_fwd": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _sz]),
    "pluto_dense_bwd": (_i, [_vp, _vp, _i] + [_vp] * 5 + [_i, _i, _i, _vp, _sz]),
    "pluto_block_linear_workspace_bytes": (_sz, [_i] * 3),
    "pluto_block_linear_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _sz]),
    "pluto_block_linear_bwd": (_i, [_vp] * 6 + [_i, _i, _i, _vp, _sz]),
    "pluto_dequantize_matrix": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i]),
    "pluto_gqa_gate_bwd": (_i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp, _sz, _sz, _vp] + [_i] * 5),
    "pluto_gqa_prefill_bwd": (_i, [_vp] * 4 + [_i, _sz, _sz] + [_vp] * 8 + [_sz] + [_i] * 5),
    "pluto_gqa_prefill_bwd_workspace_bytes": (_sz, [_i] * 5),
    "pluto_qk_prepare_bwd_workspace_bytes": (_sz, [_i] * 4),
    "pluto_qk_prepare_bwd": (_i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp, _sz, _sz, _vp, _vp, _sz]
                             + [_i] * 5 + [_fp, _fp, _i]),
    "pluto_gdn_out_norm_gate_bwd": (_i, [_vp, _vp, _i, _vp, _i] + [_vp] * 6 + [_sz, C.c_longlong, _i, _fp, _i]),
    "pluto_gdn_out_norm_gate_bwd_workspace_bytes": (_sz, [C.c_longlong, _i]),
    "pluto_gdn_recurrence_bwd_workspace_bytes": (_sz, [_i] * 6),
    "pluto_gdn_recurrence_bwd": (_i, [_vp] * 4 + [_i, _sz, _sz, _vp, _vp, _i] + [_vp] * 5 + [_sz, _vp, _sz]
                                 + [_vp] * 5 + [_sz] + [_i] * 7),
    "pluto_gdn_conv_silu_bwd": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp] + [_i] * 5),
    "pluto_qk_prepare": (_i, [_vp] * 4 + [_i, _sz, _sz] + [_vp] * 4 + [_i, _vp] + [_i] * 6
                         + [_fp, _fp, _i]),
    "pluto_gqa_decode_workspace_bytes": (_sz, [_i] * 5),
    "pluto_gqa_decode": (_i, [_vp, _vp, _i, _vp, _i, _sz, _sz, _vp, _vp, _i, _vp, _i, _vp, _vp,
                              _sz] + [_i] * 5),
    "pluto_gqa_decode_noalloc": (_i, [_vp, _vp, _i, _vp, _i, _sz, _sz, _vp, _vp, _i, _vp, _i, _vp]
                                 + [_i] * 5),
    "pluto_gqa_decode_builtin_scratch_bytes": (_sz, []),
    "pluto_gqa_decode_probs": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _sz, _sz] + [_i] * 4),
    "pluto_gdn_gates": (_i, [_vp] * 5 + [_i, C.c_longlong, _i, _i, _vp, _vp]),
    "pluto_gdn_conv_silu": (_i, [_vp] * 3 + [_i] * 6 + [_vp, _vp, _i]),
    "pluto_gdn_prefill": (_i, [_vp] * 4 + [_i] + [_vp] * 4 + [_i] * 7 + [_sz, _sz, _i, _fp, _i, _vp,
                                                                          _sz]),
    "pluto_gdn_prefill_workspace_bytes": (_sz, [_i] * 7),
    "pluto_gdn_step": (_i, [_vp] * 4 + [_i] + [_vp] * 4 + [_i] * 7 + [_fp, _i]),
    "pluto_interleave_heads": (_i, [_vp, _vp, _vp, _i, C.c_longlong, _sz]),
    "pluto_allgather_heads": (_i, [_vp, _vp, _vp, _vp, _vp, _i, C.c_longlong, _sz]),
    "pluto_selftest_bounded_wait": (_i, [_vp, C.c_ulonglong, _vp]),
    "pluto_gdn_out_norm_gate": (_i, [_vp, _vp, _i, _vp, _i, _vp, C.c_longlong, _i, _fp, _i, _i,
                                     _vp, _i]),
}


class KvCacheStruct(C.Structure):
    """struct pluto_kv_cache of include/pluto_b200.h."""
    _fields_ = [("k_base", _vp), ("v_base", _vp), ("block_table", _vp), ("max_blocks", _i),
                ("page_size", _i), ("page_stride", _sz), ("token_stride", _sz), ("dtype", _i),
                ("num_pages", _i), ("k_bases", _vp), ("v_bases", _vp)]

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA engine with `python -m pluto_b200.build` "
                "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def check(code: int) -> None:
    if code == 0:
        return
    message = lib().pluto_last_error().decode()
    if code < 0:
        raise PlutoStatusError(_CODES.get(code, "Unknown"), message, code)
    raise PlutoStatusError("Internal", message, code)


def kernel_status(clear: bool = True) -> int:
    value = C.c_uint32(0)
    check(lib().pluto_kernel_status(C.byref(value), int(clear)))
    return value.value
