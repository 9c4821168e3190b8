"""The allocation-free decode entry point (pluto_gqa_decode_noalloc).

Collected last on purpose (the file name sorts after every other test file): should it fail, a
run that stops at the first failure has already exercised everything else.

Who needs it: hosts that cannot allocate device memory when attention runs -- a server whose HBM
plan is fixed and fully committed at start-up, a sandbox that forbids cudaMalloc to loaded
plugins, a decode loop that must not wait on an allocator lock.  The entry point keeps its
split-KV scratch in a 32 MiB area inside the library; the test drives it through the C ABI and
requires the same bytes as pluto_gqa_decode with a caller workspace, on two calls in a row whose
shapes differ (so anything left in the area by the first call would show in the second).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from pluto_b200 import PlutoStatusError, _capi
from pluto_b200.layers import gqa_decode, gqa_decode_noalloc, kv_layout, C_byref

pytestmark = pytest.mark.gpu


def make_case(seed, batch, q_heads, kv_heads, dim, max_len):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    k = (torch.randn(batch, max_len, kv_heads, dim, device="cuda", generator=gen) * 0.5).bfloat16()
    v = (torch.randn(batch, max_len, kv_heads, dim, device="cuda", generator=gen) * 0.5).bfloat16()
    q = (torch.randn(batch, q_heads, dim, device="cuda", generator=gen) * 0.5).bfloat16()
    lens = torch.randint(1, max_len + 1, (batch,), device="cuda", generator=gen, dtype=torch.int32)
    lens[0] = max_len
    return q, k, v, lens


def test_noalloc_decode_matches_workspace_decode_twice_in_a_row():
    assert _capi.lib().pluto_gqa_decode_builtin_scratch_bytes() == 32 << 20
    # two different shapes back to back: long ragged sequences, then short ones with other heads
    for seed, shape in ((1, (3, 40, 8, 128, 5000)), (2, (5, 10, 2, 128, 700))):
        q, k, v, lens = make_case(seed, *shape)
        want = gqa_decode(q, k, v, lens, shape[4])
        got = torch.full_like(q, float("nan"))
        gqa_decode_noalloc(q, k, v, lens, shape[4], got)
        torch.cuda.synchronize()
        assert torch.equal(got, want), shape
    assert _capi.kernel_status() == 0


def test_noalloc_decode_other_paths_and_shorter_lengths_after_longer_ones():
    """The shared area keeps the previous call's partials.  Same shape twice, the second time with
    much shorter sequences (so most slots of the area still hold the first call's numbers and must
    not be read), with a gate and the log-sum-exp output; then the exact fp32 kernel (fp32 cache,
    head width 6) and a paged bf16 cache.  Each against the caller-workspace entry point, bit
    for bit."""
    q, k, v, lens = make_case(4, 4, 40, 8, 128, 6000)
    gate = torch.randn_like(q)
    for lengths in (lens, torch.clamp(lens // 7, min=1)):
        want, want_lse = gqa_decode(q, k, v, lengths, 6000, gate=gate, want_lse=True)
        got = torch.full_like(q, float("nan"))
        lse = torch.full((4, 40), float("nan"), device="cuda")
        gqa_decode_noalloc(q, k, v, lengths, 6000, got, gate=gate, lse=lse)
        torch.cuda.synchronize()
        assert torch.equal(got, want) and torch.equal(lse, want_lse)
    # exact fp32 kernel: fp32 cache, a head width no tensor-core path takes
    gen = torch.Generator(device="cuda").manual_seed(5)
    k32 = torch.randn(3, 90, 2, 6, device="cuda", generator=gen)
    v32 = torch.randn(3, 90, 2, 6, device="cuda", generator=gen)
    q32 = torch.randn(3, 4, 6, device="cuda", generator=gen)
    l32 = torch.tensor([90, 1, 37], dtype=torch.int32, device="cuda")
    want = gqa_decode(q32, k32, v32, l32, 90, round_to_bfloat16=False)
    got = torch.full_like(q32, float("nan"))
    gqa_decode_noalloc(q32, k32, v32, l32, 90, got, round_to_bfloat16=False)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # paged bf16 cache: 16-token pages in shuffled order
    q, k, v, lens = make_case(6, 2, 10, 2, 128, 640)
    pages = 2 * 40
    table = torch.randperm(pages, device="cuda", dtype=torch.int32).view(2, 40)
    pool_k = torch.zeros(pages, 16, 2, 128, dtype=torch.bfloat16, device="cuda")
    pool_v = torch.zeros_like(pool_k)
    pool_k[table.reshape(-1).long()] = k.view(pages, 16, 2, 128)
    pool_v[table.reshape(-1).long()] = v.view(pages, 16, 2, 128)
    want = gqa_decode(q, pool_k, pool_v, lens, 640, block_table=table)
    got = torch.full_like(q, float("nan"))
    gqa_decode_noalloc(q, pool_k, pool_v, lens, 640, got, block_table=table)
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(got, gqa_decode(q, k, v, lens, 640))
    assert _capi.kernel_status() == 0


def test_noalloc_decode_rejects_shapes_beyond_the_built_in_area():
    q, k, v, lens = make_case(3, 2, 40, 8, 128, 64)
    out = torch.zeros_like(q)
    before = out.clone()
    layout = kv_layout(k, v, None, k.shape[1], k.stride(0), k.stride(1))
    L = _capi.lib()
    # claim a batch/context whose partials need more than 32 MiB; rejected before any launch
    need = L.pluto_gqa_decode_workspace_bytes(64, 40, 8, 128, 1 << 20)
    assert need > 32 << 20
    with pytest.raises(PlutoStatusError) as info:
        _capi.check(L.pluto_gqa_decode_noalloc(
            torch.cuda.current_stream().cuda_stream, q.data_ptr(), 1, None, 0, 0, 0,
            C_byref(layout), lens.data_ptr(), 1 << 20, out.data_ptr(), 1, None, 64, 40, 8, 128, 1))
    assert info.value.code == "ResourceExhausted"
    assert str(need) in info.value.message and str(32 << 20) in info.value.message
    torch.cuda.synchronize()
    assert torch.equal(out, before)
