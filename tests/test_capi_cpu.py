"""CPU-only checks of the boundary: the shared library loads, exports every function the header
declares, and rejects bad arguments before any GPU work (so these calls need no device)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pluto_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pluto_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(engine):
    declared = declared_functions()
    assert declared, "no declarations found"
    assert declared == engine.exported_symbols()


def test_library_exports_every_declared_symbol(engine):
    handle = C.CDLL(engine.LIB_PATH)
    for name in declared_functions():
        assert hasattr(handle, name), name
    assert b"sm_100a" in engine.lib().pluto_build_info()


def test_header_cites_the_reference_for_every_entry_point():
    text = open(HEADER).read()
    for name in declared_functions():
        if name in ("pluto_last_error", "pluto_build_info", "pluto_kernel_status",
                    "pluto_gqa_decode_workspace_bytes", "pluto_gdn_prefill_workspace_bytes",
                    "pluto_attn_bwd_workspace_bytes",
                    "pluto_gqa_decode_noalloc", "pluto_selftest_bounded_wait",
                    "pluto_gqa_decode_builtin_scratch_bytes"):
            continue
        start = text.index(name + "(")
        comment = text[text.rfind("/*", 0, start):start]
        assert re.search(r"\.(cc|h):\d+", comment), f"{name} lacks a reference citation"


def _code(engine, fn, *args):
    try:
        engine.check(fn(*args))
    except engine.PlutoStatusError as error:
        return error.code, error.message
    return "Ok", ""


def test_attention_argument_validation_happens_before_gpu_work(engine):
    L = engine.lib()
    one = 16  # a non-null "device pointer" that is never dereferenced on a failed validation
    assert _code(engine, L.pluto_attn_fwd, None, one, one, one, one, 1, 0, 2, 64, 0)[0] == "InvalidArgument"
    assert _code(engine, L.pluto_attn_fwd, None, one, one, one, one, 1, 8, 2, 64, 7)[0] == "Unimplemented"
    assert _code(engine, L.pluto_attn_fwd, None, one, one, one, one, 1, 8, 2, 300, 0)[0] == "Unimplemented"
    assert _code(engine, L.pluto_attn_fwd, None, None, one, one, one, 1, 8, 2, 64, 0)[0] == "InvalidArgument"
    code, message = _code(engine, L.pluto_attn_bwd, None, one, one, one, None, one, one, one, 1, 8, 2, 64, 0, None, 0)
    assert code == "InvalidArgument" and "saved maxima" in message
    code, message = _code(engine, L.pluto_attn_bwd, None, one, one, one, one, None, one, one, 1, 8, 2, 64, 0, None, 0)
    assert code == "InvalidArgument" and "saved normalizers" in message


def test_cached_attention_argument_validation(engine):
    L = engine.lib()
    cache = engine.KvCacheStruct()
    cache.k_base = cache.v_base = 16
    cache.page_size, cache.page_stride, cache.token_stride, cache.dtype = 8, 8 * 2 * 4, 2 * 4, 1
    ref = C.cast(C.pointer(cache), C.c_void_p)
    bad_heads = _code(engine, L.pluto_gqa_decode, None, 16, 1, None, 0, 0, 0, ref, 16, 8, 16, 1, None,
                      16, 1 << 20, 1, 3, 2, 4, 1)
    assert bad_heads[0] == "InvalidArgument" and "full-attention" in bad_heads[1]
    too_wide = _code(engine, L.pluto_gqa_decode, None, 16, 1, None, 0, 0, 0, ref, 16, 8, 16, 1, None,
                     16, 1 << 20, 1, 4, 2, 260, 1)
    assert too_wide[0] == "InvalidArgument"
    cache.token_stride = 4  # smaller than kv_heads * head_dim
    mismatch = _code(engine, L.pluto_gqa_decode, None, 16, 1, None, 0, 0, 0, ref, 16, 8, 16, 1, None,
                     16, 1 << 20, 1, 4, 2, 4, 1)
    assert mismatch[0] == "InvalidArgument" and "cache shape" in mismatch[1]
    # 16 chunks of 2048 tokens, the first of them as four short ones: 19 partials per head
    assert L.pluto_gqa_decode_workspace_bytes(64, 40, 8, 128, 32768) == 64 * 40 * 19 * 130 * 4
    odd_rotary = _code(engine, L.pluto_qk_prepare, None, 16, 16, 16, 0, 8, 4, 16, 16, None, 16, 0, ref,
                       1, 1, 2, 1, 4, 3, 1e-6, 1e4, 1)
    assert odd_rotary[0] == "InvalidArgument"


def test_delta_net_argument_validation(engine):
    L = engine.lib()
    args = [None, 16, 16, 16, 0, 16, 16, 16, 16, 0, 1, 4]
    assert _code(engine, L.pluto_gdn_prefill, *args, 2, 3, 8, 8, 0, 0, 1, 1.0, 1, None, 0)[0] == "InvalidArgument"  # 3 % 2
    assert _code(engine, L.pluto_gdn_prefill, *args, 2, 4, 129, 8, 0, 0, 1, 1.0, 1, None, 0)[0] == "InvalidArgument"
    assert _code(engine, L.pluto_gdn_prefill, *args, 2, 4, 8, 257, 0, 0, 1, 1.0, 1, None, 0)[0] == "InvalidArgument"
    null_state = [None, 16, 16, 16, 0, 16, 16, None, 16, 0, 1, 4]
    code, message = _code(engine, L.pluto_gdn_prefill, *null_state, 2, 4, 8, 8, 0, 0, 1, 1.0, 1, None, 0)
    assert code == "InvalidArgument" and "non-null" in message
    # a workspace for a shape without a chunked path, and a workspace that is too small
    assert _code(engine, L.pluto_gdn_prefill, *args, 2, 4, 8, 8, 0, 0, 1, 1.0, 1, 256, 1 << 30)[0] == "InvalidArgument"
    big = [None, 16, 16, 16, 1, 16, 16, 16, 16, 1, 1, 128]
    assert _code(engine, L.pluto_gdn_prefill, *big, 2, 4, 128, 128, 0, 0, 1, 1.0, 1, 256, 1024)[0] == "InvalidArgument"
    units = 2 * 16 * 256   # (sequence, head, chunk) records
    assert L.pluto_gdn_prefill_workspace_bytes(2, 16384, 16, 16, 128, 128, 1) == units * 91136 + 1024
    assert L.pluto_gdn_prefill_workspace_bytes(2, 16384, 16, 16, 64, 128, 1) == 0
    assert _code(engine, L.pluto_gdn_conv_silu, None, 16, 16, 0, 1, 1, 8, 33, 1, 16, 16, 0)[0] == "InvalidArgument"
