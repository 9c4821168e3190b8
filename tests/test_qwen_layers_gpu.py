"""Layer objects of the Qwen decoder on the GPU: QwenAttentionLayer (cached and sequence form),
DeltaNetLayer and SequenceDeltaNetLayer, against compositions of the CPU oracle, following
qwen_attention_test.cc, cached_attention_test.cc and sequence_delta_net_test.cc."""
import numpy as np
import pytest
import torch

import oracle
from conftest import sine_values
from gpu_util import bf16_bits, near, to_device_bf16
from pluto_b200 import PlutoStatusError
from pluto_b200.layers import (DataType, DeltaNetLayer, DeltaNetParameters, FullAttentionParameters,
                               KeyValueCache, LayerHooks, QwenAttentionLayer, SequenceDeltaNetLayer)

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf(x):
    return oracle.to_bf16_bits(np.asarray(x, np.float32))


def oracle_sequence_attention(qg, k, v, q_norm, k_norm, p):
    """PrepareKernel + ForwardKernel of the reference, from oracle pieces: token by token prepare
    into an fp32 cache, then the causal core with the gate."""
    t, hq, _, d = qg.shape
    hkv = k.shape[1]
    keys = np.zeros((t, hkv, d), np.float32)
    values = np.zeros_like(keys)
    queries = np.zeros((t, hq, d), np.float32)
    for row in range(t):
        queries[row] = oracle.qk_prepare(qg[row], k[row], v[row], q_norm, k_norm, row, p.rotary_dim,
                                         p.rms_norm_epsilon, p.rope_theta, True, keys, values)
    out = np.zeros((t, hq, d), np.float32)
    for row in range(t):
        out[row] = oracle.gqa_decode(queries[row], qg[row], keys, values, row + 1, True)
    return out, queries, keys


@pytest.mark.parametrize("shape", [(7, 4, 2, 6, 4), (40, 4, 2, 64, 32), (150, 10, 2, 128, 64), (33, 24, 4, 256, 64)])
def test_sequence_attention_layer_matches_oracle_and_cached_path(shape):
    """qwen_attention_test.cc:155-228: the sequence forward against the scalar statement and
    against the same layer run token by token through a KV cache."""
    t, hq, hkv, d, rotary = shape
    p = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=rotary,
                                capacity=t, rope_theta=1e6)
    rng = np.random.default_rng(13)
    qg = oracle.from_bf16_bits(bf(rng.standard_normal((t, hq, 2, d)) * 0.8))
    k = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d)) * 0.8))
    v = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d)) * 0.8))
    q_norm, k_norm = sine_values(d, 0.2, 0.3), sine_values(d, 0.8, 0.4)
    want, _, _ = oracle_sequence_attention(qg, k, v, q_norm, k_norm, p)
    layer = QwenAttentionLayer.Create(p, dev(q_norm), dev(k_norm), t)
    assert layer.input_types()[0].dimensions == (-2, t, 2 * hq * d)
    seen = {}
    hooks = LayerHooks(attention_probabilities_hook=lambda n, s, pr: seen.update(name=n, shape=s, probs=pr))
    inputs = [to_device_bf16(bf(qg)).view(t, -1), to_device_bf16(bf(k)).view(t, -1), to_device_bf16(bf(v)).view(t, -1)]
    fwd = layer.fwd(inputs, hooks)
    got = oracle.from_bf16_bits(bf16_bits(fwd.outputs[0])).reshape(t, hq, d)
    assert np.abs(got - want).max() <= 2e-2
    assert near(got, want, 4e-3, 1.6e-2)
    # the reference's seven saved buffers, then maxima, normalizers and the rounded value rows
    assert len(fwd.state.intermediates) == 10 and fwd.state.intermediates[6].shape == (1, t, hq, d)
    probs = seen["probs"].cpu().numpy()
    assert seen["shape"].dimensions == (1, hq, t, t) and seen["name"] == "QwenAttentionLayer"
    assert np.abs(probs.sum(-1) - 1.0).max() <= 1e-4
    assert np.all(probs[:, ~np.tril(np.ones((t, t), bool))] == 0.0)
    grads = layer.bwd([torch.zeros(t, hq * d, device="cuda")], fwd.state)   # zero upstream gradient
    assert [tuple(g.shape) for g in grads] == [(t, hq, 2, d), (t, hkv, d), (t, hkv, d)]
    assert all(float(g.abs().max()) == 0.0 for g in grads)
    # token by token through the cached form of the same layer
    cache = KeyValueCache.Create(t, hkv, d)
    cached = QwenAttentionLayer.Create(p, dev(q_norm), dev(k_norm), 1, cache)
    for row in range(t):
        out = cached.fwd([x[row:row + 1] for x in inputs]).outputs[0]
        step = oracle.from_bf16_bits(bf16_bits(out)).reshape(hq, d)
        assert np.abs(step - got[row]).max() <= 1.6e-2, row
        assert near(step, want[row], 4e-3, 1.6e-2)
    assert cache.position() == t
    with pytest.raises(PlutoStatusError) as info:
        cached.fwd([x[:1] for x in inputs])
    assert info.value.code == "ResourceExhausted"
    with pytest.raises(PlutoStatusError) as info:
        cached.bwd([torch.zeros(1, hq * d, device="cuda")], fwd.state)
    assert info.value.code in ("Unimplemented", "InvalidArgument")


def test_cached_layer_known_answer_and_hook():
    """cached_attention_test.cc:108-156: zero queries give uniform probabilities, zero gates a
    sigmoid of one half."""
    p = FullAttentionParameters(query_heads=2, key_value_heads=1, head_dim=4, rotary_dim=2, capacity=4)
    cache = KeyValueCache.Create(4, 1, 4)
    zero = dev(np.zeros(4, np.float32))
    layer = QwenAttentionLayer.Create(p, zero, zero, 1, cache)
    seen = []
    hooks = LayerHooks(attention_probabilities_hook=lambda n, s, pr: seen.append((s.dimensions, pr.cpu().numpy())))
    q = torch.zeros(1, 16, dtype=torch.bfloat16, device="cuda")
    k = torch.ones(1, 4, dtype=torch.bfloat16, device="cuda")
    for step, values in enumerate(([1, 2, -1, -2], [2, 4, 1, 2])):
        v = torch.tensor([values], dtype=torch.bfloat16, device="cuda")
        out = layer.fwd([q, k, v], hooks).outputs[0].float().cpu().numpy().reshape(2, 4)
        dims, probs = seen[-1]
        assert dims == (1, 2, 1, step + 1) and np.abs(probs - 1.0 / (step + 1)).max() <= 1e-7
        expect = np.array([[0.5, 1, -0.5, -1]] * 2) if step == 0 else np.array([[0.75, 1.5, 0, 0]] * 2)
        assert np.array_equal(out, expect)
    with pytest.raises(PlutoStatusError):
        QwenAttentionLayer.Create(p, zero, zero, 2, cache)


def oracle_delta_sequence(qkv, z, a, b, conv_w, a_log, dt_bias, norm, p, final_round):
    t, channels = qkv.shape
    kq = p.key_heads * p.key_head_dim
    conv_state = np.zeros((channels, p.conv_kernel_dim), np.float32)
    rec = np.zeros((1, p.value_heads, p.key_head_dim, p.value_head_dim), np.float32)
    out = np.zeros((t, p.value_heads * p.value_head_dim), np.float32)
    for row in range(t):
        conv = oracle.gdn_conv_step(qkv[row], conv_w, conv_state, True)
        g = oracle.gdn_decay(a[row], dt_bias, a_log).reshape(1, 1, -1)
        beta = oracle.gdn_beta(b[row], True).reshape(1, 1, -1)
        core = oracle.gdn_recurrence(conv[:kq].reshape(1, 1, p.key_heads, -1), conv[kq:2 * kq].reshape(1, 1, p.key_heads, -1),
                                     conv[2 * kq:].reshape(1, 1, p.value_heads, -1), g, beta, rec, True, 1.0, True)
        out[row] = oracle.gdn_output(core.reshape(p.value_heads, -1), z[row].reshape(p.value_heads, -1), norm,
                                     p.rms_norm_epsilon, True, final_round).reshape(-1)
    return out


@pytest.mark.parametrize("shape", [(3, 1, 2, 3, 5), (3, 2, 4, 5, 35), (3, 16, 48, 128, 128), (200, 2, 4, 128, 64)])
def test_sequence_delta_net_layer_matches_oracle(shape):
    """sequence_delta_net_test.cc:241-297 shapes (T = 3) plus a long sequence that takes the
    chunked recurrence; tolerance 1.5e-4 + 1.5 % (+ two bf16 ulps of the largest output on the
    chunked path)."""
    t, hk, hv, dk, dv = shape
    p = DeltaNetParameters(key_heads=hk, value_heads=hv, key_head_dim=dk, value_head_dim=dv, conv_kernel_dim=4)
    channels = 2 * hk * dk + hv * dv
    tensor = lambda n, i: (0.15 + 0.4 * np.sin(0.37 * np.arange(n, dtype=np.float32) + 0.41 * i)).astype(np.float32)
    qkv = oracle.from_bf16_bits(bf(tensor(t * channels, 0))).reshape(t, channels)
    z = oracle.from_bf16_bits(bf(tensor(t * hv * dv, 1))).reshape(t, hv * dv)
    a = oracle.from_bf16_bits(bf(tensor(t * hv, 2))).reshape(t, hv)
    b = oracle.from_bf16_bits(bf(tensor(t * hv, 3))).reshape(t, hv)
    conv_w = tensor(channels * 4, 4).reshape(channels, 4) * 0.5
    a_log, dt_bias, norm = tensor(hv, 5) * 0.5, tensor(hv, 6) * 0.3, tensor(dv, 7)
    want = oracle_delta_sequence(qkv, z, a, b, conv_w, a_log, dt_bias, norm, p, False)
    layer = SequenceDeltaNetLayer.Create(p, dev(conv_w), dev(a_log), dev(dt_bias), dev(norm), t)
    fwd = layer.fwd([to_device_bf16(bf(x)) for x in (qkv, z, a, b)])
    got = oracle.from_bf16_bits(bf16_bits(fwd.outputs[0]))
    slack = 2.0 ** -7 * np.abs(want).max() if t >= 64 else 0.0
    assert np.all(np.abs(got - oracle.round_bf16(want)) <= 1.5e-4 + 0.015 * np.abs(want) + slack + 2.0 ** -8 * np.abs(want))
    grads = layer.bwd([torch.zeros(t, hv * dv, device="cuda")], fwd.state)   # zero upstream gradient
    assert [tuple(g.shape) for g in grads] == [(t, channels), (t, hv * dv), (t, hv), (t, hv)]
    assert all(float(g.abs().max()) == 0.0 for g in grads)
    # the single-token layer fed the same tokens one by one gives the cached-path rounding
    # (final product rounded once more) of the same numbers
    step_layer = DeltaNetLayer.Create(p, dev(conv_w), dev(a_log), dev(dt_bias), dev(norm))
    want_step = oracle_delta_sequence(qkv, z, a, b, conv_w, a_log, dt_bias, norm, p, True)
    for row in range(min(t, 5)):
        out = step_layer.fwd([to_device_bf16(bf(x[row:row + 1])) for x in (qkv, z, a, b)]).outputs[0]
        step = oracle.from_bf16_bits(bf16_bits(out)).reshape(-1)
        assert np.all(np.abs(step - want_step[row]) <= 2e-4 + 8e-3 * np.abs(want_step[row])), row
    step_layer.Reset()
    again = step_layer.fwd([to_device_bf16(bf(x[:1])) for x in (qkv, z, a, b)]).outputs[0]
    first = oracle.from_bf16_bits(bf16_bits(again)).reshape(-1)
    assert np.all(np.abs(first - want_step[0]) <= 2e-4 + 8e-3 * np.abs(want_step[0]))
    assert step_layer.output_type() == DataType.BF16 and len(step_layer.weights()) == 4
