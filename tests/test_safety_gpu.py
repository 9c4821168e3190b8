"""Bounds and hang safety evidence that does not need a sanitizer.

* Guard bands: every output and workspace of a call sits between two bands of a fixed byte
  pattern inside a larger allocation; ragged shapes (lengths and widths that are not multiples of
  any tile) run through the C ABI and the bands must come back untouched.
* Bounded waits: a self-test kernel waits on a barrier nobody arrives at; the wait must give up
  after its limit, report through the status word, and leave the context usable.
"""
import numpy as np
import pytest
import torch

from pluto_b200 import _capi
from pluto_b200.layers import (AttentionLayer, DataType, gdn_prefill, gdn_step, gqa_decode, kv_layout, C_byref)

pytestmark = pytest.mark.gpu

BAND = 4096
PATTERN = 0xA5


class Guarded:
    """A device buffer of `nbytes` (256-byte aligned) with a pattern band either side."""

    def __init__(self, nbytes):
        self.nbytes = nbytes
        padded = (nbytes + 255) // 256 * 256
        self.raw = torch.full((BAND + padded + BAND + 256,), PATTERN, dtype=torch.uint8, device="cuda")
        self.offset = (-self.raw.data_ptr()) % 256 + BAND
        self.ptr = self.raw.data_ptr() + self.offset

    def tensor(self, shape, dtype):
        count = int(np.prod(shape))
        return self.raw[self.offset:self.offset + count * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)

    def intact(self):
        before = self.raw[:self.offset]
        after = self.raw[self.offset + self.nbytes:]
        return bool((before == PATTERN).all()) and bool((after == PATTERN).all())


def guarded_like(shape, dtype):
    g = Guarded(int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size())
    return g, g.tensor(shape, dtype)


@pytest.mark.parametrize("shape", [(3, 10, 2, 128, 333), (2, 6, 3, 20, 90), (2, 3, 1, 5, 41), (1, 8, 8, 64, 1000)])
def test_decode_stays_inside_its_output_and_workspace(shape):
    b, hq, hkv, d, lmax = shape
    gen = torch.Generator(device="cuda").manual_seed(4)
    k = (torch.randn(b, lmax, hkv, d, device="cuda", generator=gen) * 0.5).bfloat16()
    v = (torch.randn(b, lmax, hkv, d, device="cuda", generator=gen) * 0.5).bfloat16()
    q = (torch.randn(b, hq, d, device="cuda", generator=gen) * 0.5).bfloat16()
    lens = torch.tensor([lmax] + [max(1, lmax // (i + 2)) for i in range(b - 1)], dtype=torch.int32, device="cuda")
    L = _capi.lib()
    g_out, out = guarded_like((b, hq, d), torch.bfloat16)
    g_lse, lse = guarded_like((b, hq), torch.float32)
    need = L.pluto_gqa_decode_workspace_bytes(b, hq, hkv, d, lmax)
    g_ws = Guarded(need)
    layout = kv_layout(k, v, None, lmax, k.stride(0), k.stride(1))
    _capi.check(L.pluto_gqa_decode(torch.cuda.current_stream().cuda_stream, q.data_ptr(), 1, None, 0, 0, 0,
                                   C_byref(layout), lens.data_ptr(), lmax, g_out.ptr, 1, g_lse.ptr, g_ws.ptr, need,
                                   b, hq, hkv, d, 1))
    torch.cuda.synchronize()
    assert g_out.intact() and g_lse.intact() and g_ws.intact()
    want = gqa_decode(q, k, v, lens, lmax)
    assert torch.equal(out, want) and torch.isfinite(lse).all()
    assert _capi.kernel_status() == 0


@pytest.mark.parametrize("shape", [(1, 333, 6, 2, 128), (2, 77, 4, 4, 64), (1, 50, 4, 2, 24)])
def test_prefill_stays_inside_its_outputs(shape):
    b, t, hq, hkv, d = shape
    gen = torch.Generator(device="cuda").manual_seed(6)
    q = (torch.randn(b, t, hq, d, device="cuda", generator=gen) * 0.5).bfloat16()
    k = (torch.randn(b, t, hkv, d, device="cuda", generator=gen) * 0.5).bfloat16()
    v = (torch.randn(b, t, hkv, d, device="cuda", generator=gen) * 0.5).bfloat16()
    g_out, out = guarded_like((b, t, hq, d), torch.bfloat16)
    g_core, core = guarded_like((b, t, hq, d), torch.float32)
    g_max, maxima = guarded_like((b * hq * t,), torch.float32)
    g_norm, normalizers = guarded_like((b * hq * t,), torch.float32)
    _capi.check(_capi.lib().pluto_gqa_prefill_fwd(
        torch.cuda.current_stream().cuda_stream, q.data_ptr(), None, k.data_ptr(), v.data_ptr(), g_out.ptr,
        g_core.ptr, g_max.ptr, g_norm.ptr, b, t, hq, hkv, d, hq * d, d, 0, 0, 1, None, 0))
    torch.cuda.synchronize()
    assert g_out.intact() and g_core.intact() and g_max.intact() and g_norm.intact()
    assert torch.isfinite(out.float()).all() and torch.isfinite(core).all()
    assert (normalizers >= 1.0 - 1e-5).all()
    assert _capi.kernel_status() == 0


@pytest.mark.parametrize("shape,dtype", [((2, 100, 3, 64), DataType.BF16), ((1, 65, 2, 80), DataType.BF16),
                                         ((3, 33, 2, 24), DataType.FP16)])
def test_attention_layer_kernels_stay_inside_their_buffers(shape, dtype):
    batch, seq, heads, d = shape
    e = heads * d
    bf16 = dtype == DataType.BF16
    act = torch.bfloat16 if bf16 else torch.float32
    qkv = torch.randn(batch * seq, 3 * e, device="cuda").to(act)
    d_out = torch.randn(batch * seq, e, device="cuda")
    L, stream = _capi.lib(), torch.cuda.current_stream().cuda_stream
    code = 1 if bf16 else 0
    g_out, out = guarded_like((batch * seq, e), act)
    g_max, maxima = guarded_like((batch * heads * seq,), torch.float32)
    g_norm, normalizers = guarded_like((batch * heads * seq,), torch.float32)
    _capi.check(L.pluto_attn_fwd(stream, qkv.data_ptr(), g_out.ptr, g_max.ptr, g_norm.ptr, batch, seq, heads, d, code))
    g_grad, grad = guarded_like((batch * seq, 3 * e), torch.float32)
    g_delta, _ = guarded_like((batch * heads * seq,), torch.float32)
    need = L.pluto_attn_bwd_workspace_bytes(batch, seq, heads, d, code)
    g_ws = Guarded(need) if need else None
    _capi.check(L.pluto_attn_bwd(stream, qkv.data_ptr(), g_out.ptr, d_out.data_ptr(), g_max.ptr, g_norm.ptr,
                                 g_grad.ptr, g_delta.ptr, batch, seq, heads, d, code,
                                 g_ws.ptr if g_ws else None, need))
    torch.cuda.synchronize()
    for guard in (g_out, g_max, g_norm, g_grad, g_delta) + ((g_ws,) if g_ws else ()):
        assert guard.intact()
    assert torch.isfinite(grad).all() and torch.isfinite(out.float()).all()
    layer = AttentionLayer.Create(seq, heads, e, dtype)
    assert torch.equal(layer.fwd([qkv]).outputs[0], out)
    assert _capi.kernel_status() == 0


@pytest.mark.parametrize("shape", [(1, 200, 1, 2, 128), (2, 65, 2, 2, 32), (1, 130, 1, 1, 224)])
def test_delta_net_prefill_stays_inside_its_output_and_workspace(shape):
    b, t, hk, hv, dv = shape
    dk = 128
    gen = torch.Generator(device="cuda").manual_seed(8)
    q = torch.randn(b, t, hk, dk, device="cuda", generator=gen).bfloat16()
    k = torch.randn(b, t, hk, dk, device="cuda", generator=gen).bfloat16()
    v = torch.randn(b, t, hv, dv, device="cuda", generator=gen).bfloat16()
    g = torch.sigmoid(torch.randn(b, t, hv, device="cuda", generator=gen) * 2 + 2)
    beta = torch.sigmoid(torch.randn(b, t, hv, device="cuda", generator=gen))
    L = _capi.lib()
    need = L.pluto_gdn_prefill_workspace_bytes(b, t, hk, hv, dk, dv, 1)
    assert need > 0
    g_ws = Guarded(need)
    g_out, out = guarded_like((b, t, hv, dv), torch.bfloat16)
    g_state, state = guarded_like((b, hv, dk, dv), torch.float32)
    state.zero_()
    _capi.check(L.pluto_gdn_prefill(torch.cuda.current_stream().cuda_stream, q.data_ptr(), k.data_ptr(), v.data_ptr(), 1,
                                    g.data_ptr(), beta.data_ptr(), g_state.ptr, g_out.ptr, 1, b, t, hk, hv, dk, dv,
                                    0, 0, 1, 1.0, 1, g_ws.ptr, need))
    torch.cuda.synchronize()
    assert g_ws.intact() and g_out.intact() and g_state.intact()
    plain_state = torch.zeros(b, hv, dk, dv, device="cuda")
    want = gdn_prefill(q, k, v, g, beta, plain_state, chunked=True)
    assert torch.equal(out, want) and torch.equal(state, plain_state)
    # one more token through the single-step kernel, output and state guarded
    g_one, one = guarded_like((b, hv, dv), torch.bfloat16)
    _capi.check(L.pluto_gdn_step(torch.cuda.current_stream().cuda_stream, q[:, 0].contiguous().data_ptr(),
                                 k[:, 0].contiguous().data_ptr(), v[:, 0].contiguous().data_ptr(), 1,
                                 g[:, 0].contiguous().data_ptr(), beta[:, 0].contiguous().data_ptr(), g_state.ptr,
                                 g_one.ptr, 1, b, hk, hv, dk, dv, 1, 1.0, 1))
    torch.cuda.synchronize()
    assert g_one.intact() and g_state.intact() and torch.isfinite(one.float()).all()
    assert _capi.kernel_status() == 0


def test_a_bounded_wait_runs_out_and_the_context_stays_usable():
    """The wait helper every pipeline kernel uses, driven to its limit: nobody arrives at the
    barrier, so after 1 ms the kernel records (site << 8) | 1 and returns; the word clears; the
    next real kernel runs and is healthy."""
    L, stream = _capi.lib(), torch.cuda.current_stream().cuda_stream
    assert _capi.kernel_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _capi.check(L.pluto_selftest_bounded_wait(stream, 1_000_000, flag.data_ptr()))
    stop.record()
    torch.cuda.synchronize()
    assert flag.item() == 1
    assert 0.9 <= start.elapsed_time(stop) <= 50.0   # gave up after about 1 ms, not after the 2 s default
    assert _capi.kernel_status(clear=False) == (63 << 8) | 1
    assert _capi.kernel_status(clear=True) == (63 << 8) | 1
    assert _capi.kernel_status() == 0
    # a real pipeline kernel (TMA ring + mbarriers) afterwards
    k = (torch.randn(2, 512, 2, 128, device="cuda") * 0.5).bfloat16()
    q = (torch.randn(2, 10, 128, device="cuda") * 0.5).bfloat16()
    out = gqa_decode(q, k, torch.ones_like(k), torch.tensor([512, 100], dtype=torch.int32, device="cuda"), 512)
    assert (out.float() - 1.0).abs().max().item() <= 2 ** -8
    assert _capi.kernel_status() == 0
    with pytest.raises(_capi.PlutoStatusError):
        _capi.check(L.pluto_selftest_bounded_wait(stream, 10 ** 12, flag.data_ptr()))


def test_decode_reports_a_length_beyond_the_declared_maximum():
    """seq_lens is device data the host never reads back: a value above max_seq_len must not walk
    the merge kernel out of the workspace.  The kernels clamp, report kind 2 through the status
    word, and still produce finite output."""
    b, hq, hkv, d, lmax = 2, 4, 2, 64, 256
    k = (torch.randn(b, 1024, hkv, d, device="cuda") * 0.5).bfloat16()
    q = (torch.randn(b, hq, d, device="cuda") * 0.5).bfloat16()
    lens = torch.tensor([1000, 0], dtype=torch.int32, device="cuda")   # declared maximum is 256
    out = gqa_decode(q, k, torch.ones_like(k), lens, lmax)
    torch.cuda.synchronize()
    status = _capi.kernel_status()
    assert status & 0xff == 2, hex(status)
    assert (out[0].float() - 1.0).abs().max().item() <= 2 ** -8    # attended to the first 256 tokens
    assert (out[1].float() == 0).all()                            # empty sequence: zeros, not NaN
    assert _capi.kernel_status() == 0
