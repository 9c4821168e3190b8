"""Gated delta-net on the GPU against the CPU oracle: the recurrence over sequences and single
steps, DeltaNetState.Step (conv + recurrence + output stage), in the patterns of
cached_attention_ops_test.cc:400-470 and sequence_delta_net_test.cc:241-297."""
import numpy as np
import pytest
import torch

import oracle
from conftest import sine_values
from gpu_util import bf16_bits, near, to_device_bf16
from pluto_b200.layers import DeltaNetParameters, DeltaNetState, gdn_prefill, gdn_step

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def make_inputs(rng, b, t, hk, hv, dk, dv, normalised=False):
    q = rng.standard_normal((b, t, hk, dk), dtype=np.float32)
    k = rng.standard_normal((b, t, hk, dk), dtype=np.float32)
    if normalised:
        q /= np.linalg.norm(q, axis=-1, keepdims=True)
        k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((b, t, hv, dv), dtype=np.float32)
    g = (1 / (1 + np.exp(-(rng.standard_normal((b, t, hv)) * 2 + 2)))).astype(np.float32)
    beta = (1 / (1 + np.exp(-rng.standard_normal((b, t, hv))))).astype(np.float32)
    return q, k, v, g, beta


@pytest.mark.parametrize("shape", [(1, 3, 1, 2, 3, 5, False), (1, 3, 2, 4, 5, 35, False),
                                   (1, 3, 16, 48, 128, 128, True), (2, 70, 2, 4, 128, 128, True),
                                   (1, 130, 2, 2, 64, 256, True)])
def test_recurrence_matches_oracle(shape):
    b, t, hk, hv, dk, dv, bf16 = shape
    q, k, v, g, beta = make_inputs(np.random.default_rng(5), b, t, hk, hv, dk, dv)
    if bf16:
        qi, ki, vi = map(oracle.to_bf16_bits, (q, k, v))
        tq, tk, tv = map(to_device_bf16, (qi, ki, vi))
    else:
        qi, ki, vi = q, k, v
        tq, tk, tv = map(dev, (q, k, v))
    state = np.zeros((b, hv, dk, dv), np.float32)
    ts = torch.zeros(b, hv, dk, dv, device="cuda")
    want = oracle.gdn_recurrence(qi, ki, vi, g, beta, state, True, 1.0, bf16, threads=8)
    got = gdn_prefill(tq, tk, tv, dev(g), dev(beta), ts, True, 1.0, bf16, chunked=False)
    torch.cuda.synchronize()
    got_f = oracle.from_bf16_bits(bf16_bits(got)) if bf16 else got.cpu().numpy()
    want_f = oracle.from_bf16_bits(want) if bf16 else want
    assert np.all(np.abs(got_f - want_f) <= 1.5e-4 + 0.015 * np.abs(want_f) + 2.0 ** -7 * np.abs(want_f).max())
    assert np.abs(got_f - want_f).max() <= (2e-2 if bf16 else 1e-4)
    assert np.abs(ts.cpu().numpy() - state).max() <= 1e-4


def test_prefill_then_single_steps_from_the_final_state():
    """Chunk of the benchmark flow at reduced length: prefill T tokens, then single-token steps
    from the final state; both against the token-recurrent oracle (fp32 state)."""
    b, t, h, d, steps = 2, 192, 4, 128, 8
    rng = np.random.default_rng(12)
    q, k, v, g, beta = make_inputs(rng, b, t + steps, h, h, d, d, normalised=True)
    qi, ki, vi = map(oracle.to_bf16_bits, (q, k, v))
    state = np.zeros((b, h, d, d), np.float32)
    want = oracle.gdn_recurrence(qi, ki, vi, g, beta, state, True, 1.0, True, threads=8)
    tq, tk, tv, tg, tb = to_device_bf16(qi), to_device_bf16(ki), to_device_bf16(vi), dev(g), dev(beta)
    ts = torch.zeros(b, h, d, d, device="cuda")
    got = gdn_prefill(tq[:, :t], tk[:, :t], tv[:, :t], tg[:, :t].contiguous(), tb[:, :t].contiguous(), ts)
    got_f, want_f = oracle.from_bf16_bits(bf16_bits(got)), oracle.from_bf16_bits(want[:, :t])
    assert np.abs(got_f - want_f).max() <= 2e-2
    assert np.all(np.abs(got_f - want_f) <= 1.5e-4 + 0.015 * np.abs(want_f) + 2.0 ** -7 * np.abs(want_f).max())
    for s in range(steps):
        i = t + s
        out = gdn_step(tq[:, i].contiguous(), tk[:, i].contiguous(), tv[:, i].contiguous(),
                       tg[:, i].contiguous(), tb[:, i].contiguous(), ts)
        assert np.abs(oracle.from_bf16_bits(bf16_bits(out)) - oracle.from_bf16_bits(want[:, i])).max() <= 2e-2
    assert np.abs(ts.cpu().numpy() - state).max() <= 1e-2  # chunked prefill: bf16 operands


@pytest.mark.parametrize("rnd", [False, True])
@pytest.mark.parametrize("dim", [5, 128])
def test_delta_net_state_step_and_reset(rnd, dim):
    """cached_attention_ops_test.cc:400-470: Hk2/Hv6, dims (5,7) and (128,128), kernel 4, softplus
    extremes a = +-100, Reset replays the first step bit for bit."""
    p = DeltaNetParameters(key_heads=2, value_heads=6, key_head_dim=dim,
                           value_head_dim=7 if dim == 5 else 128, conv_kernel_dim=4, round_to_bfloat16=rnd)
    ch = 2 * p.key_heads * p.key_head_dim + p.value_heads * p.value_head_dim
    st = DeltaNetState.Create(p)
    w = sine_values(ch * 4, 0.73, 0.6).reshape(ch, 4)
    alog, dt = sine_values(6, 0.18, 0.5), sine_values(6, -0.7, 0.3)
    norm = sine_values(p.value_head_dim, 0.5, 0.6)
    conv_state = np.zeros((ch, 4), np.float32)
    rec_state = np.zeros((1, 6, dim, p.value_head_dim), np.float32)
    out = torch.zeros(6, p.value_head_dim, device="cuda")
    first = None
    for step in range(7):
        t = 0 if step == 6 else step
        if step == 6:
            st.Reset()
        qkv = sine_values(ch, 0.3 + t * 0.71)
        z = sine_values(6 * p.value_head_dim, -0.6 + t * 0.27).reshape(6, -1)
        a, b = sine_values(6, 0.1 + t * 0.1), sine_values(6, -0.7 + t * 0.3)
        a[0], a[1] = 100.0, -100.0
        st.Step(dev(qkv), dev(z), dev(a), dev(b), dev(w), dev(alog), dev(dt), dev(norm), out)
        got = out.cpu().numpy().copy()
        if step < 6:
            conv = oracle.gdn_conv_step(qkv, w, conv_state, rnd)
            kq = p.key_heads * dim
            core = oracle.gdn_recurrence(conv[:kq].reshape(1, 1, 2, dim), conv[kq:2 * kq].reshape(1, 1, 2, dim),
                                         conv[2 * kq:].reshape(1, 1, 6, -1),
                                         oracle.gdn_decay(a, dt, alog).reshape(1, 1, 6),
                                         oracle.gdn_beta(b, rnd).reshape(1, 1, 6), rec_state, True, 1.0, rnd)
            want = oracle.gdn_output(core.reshape(6, -1), z, norm, p.rms_norm_epsilon, rnd, True)
            tol = (2e-4, 8e-3) if rnd else (3e-5, 1e-4)
            assert np.all(np.abs(got - want) <= tol[0] + tol[1] * np.abs(want)), step
            assert np.isfinite(got).all()
        if step == 0:
            first = got
        if step == 6:
            assert np.array_equal(got, first)


def test_long_sequence_state_property():
    """Full benchmark head shape (d_k = d_v = 128) over 4096 tokens: the fp32 state written by one
    launch must equal the state after the same tokens fed as two launches (prefill is a pure
    function of (state, tokens)), and outputs must agree bit for bit."""
    b, t, h, d = 1, 4096, 2, 128
    q, k, v, g, beta = make_inputs(np.random.default_rng(31), b, t, h, h, d, d, normalised=True)
    tq, tk, tv = (to_device_bf16(oracle.to_bf16_bits(x)) for x in (q, k, v))
    tg, tb = dev(g), dev(beta)
    s1 = torch.zeros(b, h, d, d, device="cuda")
    one = gdn_prefill(tq, tk, tv, tg, tb, s1, chunked=False)
    s2 = torch.zeros(b, h, d, d, device="cuda")
    cut = 1000
    a = gdn_prefill(tq[:, :cut], tk[:, :cut], tv[:, :cut], tg[:, :cut].contiguous(), tb[:, :cut].contiguous(), s2,
                    chunked=False)
    c = gdn_prefill(tq[:, cut:], tk[:, cut:], tv[:, cut:], tg[:, cut:].contiguous(), tb[:, cut:].contiguous(), s2,
                    chunked=False)
    assert torch.equal(torch.cat([a, c], 1), one) and torch.equal(s1, s2)
    assert torch.isfinite(s1).all()
    # the chunked tensor-core form from the same inputs: same function within bf16 operand rounding,
    # also when the sequence is cut at a chunk boundary and continued from the carried state
    s3 = torch.zeros(b, h, d, d, device="cuda")
    chunked = gdn_prefill(tq, tk, tv, tg, tb, s3, chunked=True)
    assert (chunked.float() - one.float()).abs().max().item() <= 2e-3
    assert (s3 - s1).abs().max().item() <= 2e-2
    s4 = torch.zeros(b, h, d, d, device="cuda")
    cut = 1024
    a = gdn_prefill(tq[:, :cut], tk[:, :cut], tv[:, :cut], tg[:, :cut].contiguous(), tb[:, :cut].contiguous(), s4,
                    chunked=True)
    c = gdn_prefill(tq[:, cut:], tk[:, cut:], tv[:, cut:], tg[:, cut:].contiguous(), tb[:, cut:].contiguous(), s4,
                    chunked=True)
    assert torch.equal(torch.cat([a, c], 1), chunked) and torch.equal(s3, s4)
    again = torch.zeros(b, h, d, d, device="cuda")
    assert torch.equal(gdn_prefill(tq, tk, tv, tg, tb, again, chunked=True), chunked)  # deterministic


@pytest.mark.parametrize("shape", [(1, 64, 1, 1, 32, True), (1, 128, 1, 2, 128, True), (2, 200, 2, 4, 128, True),
                                   (1, 1000, 2, 2, 64, False), (1, 2048, 1, 1, 256, False)])
def test_chunked_prefill_matches_token_recurrent_oracle(shape):
    """The 64-token chunked form (key width 128) against the token-recurrent oracle: ragged
    lengths (tail chunk), grouped heads, value widths 32..256, normalised or raw q/k."""
    b, t, hk, hv, dv, raw = shape
    q, k, v, g, beta = make_inputs(np.random.default_rng(55), b, t, hk, hv, 128, dv, normalised=not raw)
    qi, ki, vi = map(oracle.to_bf16_bits, (q, k, v))
    state = np.zeros((b, hv, 128, dv), np.float32)
    want = oracle.from_bf16_bits(oracle.gdn_recurrence(qi, ki, vi, g, beta, state, True, 1.0, True, threads=8))
    ts = torch.zeros(b, hv, 128, dv, device="cuda")
    got = gdn_prefill(to_device_bf16(qi), to_device_bf16(ki), to_device_bf16(vi), dev(g), dev(beta), ts,
                      True, 1.0, True, chunked=True)
    torch.cuda.synchronize()
    got_f = oracle.from_bf16_bits(bf16_bits(got))
    assert np.abs(got_f - want).max() <= 2e-2
    # relative form of the reference's sequence tests (1.5e-4 + 1.5 %), with two bf16 ulps of the
    # largest output added for the chunked path's bf16 operands
    assert np.all(np.abs(got_f - want) <= 1.5e-4 + 0.015 * np.abs(want) + 2.0 ** -7 * np.abs(want).max())
    assert np.abs(ts.cpu().numpy() - state).max() <= 2e-2
    from pluto_b200 import _capi
    assert _capi.kernel_status() == 0
