"""QwenAttentionLayer sequence backward on the GPU (gate -> attention core -> RoPE^-1 + RMSNorm ->
norm-weight reduction) against the CPU oracle and against central differences of the independent
double model, following qwen_attention_test.cc:230-345 and :453-490."""
import numpy as np
import pytest
import torch

import oracle
from conftest import sine_values
from gpu_util import to_device_bf16
from pluto_b200 import PlutoStatusError
from pluto_b200.layers import (BlockParameter, FullAttentionParameters, KeyValueCache,
                               QwenAttentionLayer)
from qwen_double_model import DoubleModel, wave

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf(x):
    return oracle.to_bf16_bits(np.asarray(x, np.float32))


def make_layer(p, t, q_norm, k_norm, active=(True, True)):
    qw, kw = BlockParameter.Create(dev(q_norm)), BlockParameter.Create(dev(k_norm))
    if active[0]:
        qw.Activate()
    if active[1]:
        kw.Activate()
    return QwenAttentionLayer.Create(p, qw, kw, t), qw, kw


def run(layer, qg, k, v, dy):
    t = qg.shape[0]
    inputs = [to_device_bf16(bf(qg)).view(t, -1), to_device_bf16(bf(k)).view(t, -1),
              to_device_bf16(bf(v)).view(t, -1)]
    fwd = layer.fwd(inputs)
    grads = layer.bwd([dev(dy.astype(np.float32)).view(t, -1)], fwd.state)
    torch.cuda.synchronize()
    return fwd, [g.cpu().numpy() for g in grads]


def test_backward_matches_independent_finite_difference():
    """The reference's own check (qwen_attention_test.cc:230-301) applied to this engine: same
    configuration, inputs, step and 3e-5 tolerance."""
    t, hq, hkv, d, rotary = 3, 2, 1, 3, 2
    p = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=rotary,
                                capacity=t)
    values = [wave(t * 12, .1), wave(t * 3, 1.2), wave(t * 3, 2.3), wave(3, .2), wave(3, .4)]
    upstream = wave(t * 6, .7)
    layer, qw, kw = make_layer(p, t, values[3].astype(np.float32), values[4].astype(np.float32))
    _, grads = run(layer, values[0].reshape(t, hq, 2, d), values[1].reshape(t, hkv, d),
                   values[2].reshape(t, hkv, d), upstream.reshape(t, hq, d))
    model = DoubleModel(t, hq, hkv, d, rotary, p.rms_norm_epsilon, p.rope_theta, True)
    expected = model.gradients(values, [float(u) for u in upstream])
    actual = [grads[0].ravel(), grads[1].ravel(), grads[2].ravel(),
              qw.gradient().cpu().numpy(), kw.gradient().cpu().numpy()]
    for name, a, e in zip(["dqg", "dk", "dv", "dq_norm", "dk_norm"], actual, expected):
        assert np.abs(a - e).max() < 3e-5, (name, np.abs(a - e).max())
    # shared norm gradients accumulate across backward calls; activations are overwritten
    _, again = run(layer, values[0].reshape(t, hq, 2, d), values[1].reshape(t, hkv, d),
                   values[2].reshape(t, hkv, d), upstream.reshape(t, hq, d))
    for a, b in zip(grads, again):
        assert np.array_equal(a, b)
    assert np.abs(qw.gradient().cpu().numpy() - 2 * actual[3]).max() < 1e-6
    assert np.abs(kw.gradient().cpu().numpy() - 2 * actual[4]).max() < 1e-6


# exact fp32 forward (head widths off the tensor-core path) -> tight parity with the oracle;
# widths 64 / 128 run the forward on tcgen05 with P in bf16, so their saved core and with it every
# gradient carries bf16-level differences
# (the exact path still differs from the CPU by isolated bf16 flips of R(cos), R(sin), R(core):
# device and host cosf/sinf/expf differ in the last ulp, and one flipped rounding moves a gradient
# entry by ~4e-3 of one term)
@pytest.mark.parametrize("shape,tol", [((37, 4, 2, 48, 16), 1e-3), ((70, 6, 2, 96, 32), 1e-3),
                                       ((150, 4, 2, 64, 32), 2e-2), ((200, 10, 2, 128, 64), 2e-2),
                                       ((33, 8, 4, 256, 64), 1e-3)])
def test_backward_matches_oracle(shape, tol):
    t, hq, hkv, d, rotary = shape
    p = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=rotary,
                                capacity=t, rope_theta=1e6)
    rng = np.random.default_rng(29)
    qg = oracle.from_bf16_bits(bf(rng.standard_normal((t, hq, 2, d)) * 0.8))
    k = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d)) * 0.8))
    v = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d)) * 0.8))
    dy = rng.standard_normal((t, hq, d)).astype(np.float32)
    q_norm, k_norm = sine_values(d, 0.2, 0.3), sine_values(d, 0.8, 0.4)
    dqw, dkw = np.zeros(d, np.float32), np.zeros(d, np.float32)
    want = oracle.gqa_sequence_bwd(qg, k, v, q_norm, k_norm, dy, rotary, p.rms_norm_epsilon,
                                   p.rope_theta, True, dqw, dkw)
    layer, qw, kw = make_layer(p, t, q_norm, k_norm)
    fwd, grads = run(layer, qg, k, v, dy)
    y = fwd.outputs[0].float().cpu().numpy().reshape(t, hq, d)
    assert np.abs(y - want["y"]).max() <= 2e-2
    for name, got, ref in (("dqg", grads[0], want["dqg"]), ("dk", grads[1], want["dk"]),
                           ("dv", grads[2], want["dv"]),
                           ("dq_norm", qw.gradient().cpu().numpy(), dqw),
                           ("dk_norm", kw.gradient().cpu().numpy(), dkw)):
        scale = max(1.0, float(np.abs(ref).max()))
        assert np.abs(got.reshape(ref.shape) - ref).max() <= tol * scale, \
            (name, float(np.abs(got.reshape(ref.shape) - ref).max()), scale)
    assert len(layer.gradients()) == 2


def test_tensor_core_backward_agrees_with_exact_backward_on_long_sequence():
    """Ragged length above several 128-row tiles, five query heads per KV head: the tcgen05
    passes against the exact fp32 passes on the same saved forward state."""
    t, hq, hkv, d, rotary = 700, 10, 2, 128, 64
    p = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=rotary,
                                capacity=t, rope_theta=1e6)
    rng = np.random.default_rng(41)
    qg = oracle.from_bf16_bits(bf(rng.standard_normal((t, hq, 2, d)) * 0.8))
    k = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d)) * 0.8))
    v = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d)) * 0.8))
    dy = rng.standard_normal((t, hq, d)).astype(np.float32)
    q_norm, k_norm = sine_values(d, 0.2, 0.3), sine_values(d, 0.8, 0.4)
    results = []
    for tensor_core in (True, False):
        layer, qw, kw = make_layer(p, t, q_norm, k_norm)
        layer.tensor_core_backward = tensor_core
        _, grads = run(layer, qg, k, v, dy)
        results.append(grads + [qw.gradient().cpu().numpy(), kw.gradient().cpu().numpy()])
    for name, a, b in zip(["dqg", "dk", "dv", "dq_norm", "dk_norm"], *results):
        scale = max(1.0, float(np.abs(b).max()))
        assert np.abs(a - b).max() <= 1.5e-2 * scale, (name, float(np.abs(a - b).max()), scale)
        assert np.abs(a - b).mean() <= 1e-3 * scale, name
    from pluto_b200 import _capi
    assert _capi.kernel_status() == 0


def test_frozen_norms_still_propagate_and_either_norm_may_be_active():
    """qwen_attention_test.cc:304-345, 453-490."""
    t, hq, hkv, d, rotary = 20, 4, 2, 32, 16
    p = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=rotary,
                                capacity=t)
    rng = np.random.default_rng(5)
    qg = oracle.from_bf16_bits(bf(rng.standard_normal((t, hq, 2, d))))
    k = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d))))
    v = oracle.from_bf16_bits(bf(rng.standard_normal((t, hkv, d))))
    dy = np.zeros((t, hq, d), np.float32)
    dy[-1] = rng.standard_normal((hq, d))          # only the last token has an upstream gradient
    q_norm, k_norm = sine_values(d, 0.2, 0.3), sine_values(d, 0.8, 0.4)
    results = {}
    for active in ((False, False), (True, False), (False, True)):
        layer, qw, kw = make_layer(p, t, q_norm, k_norm, active)
        _, grads = run(layer, qg, k, v, dy)
        results[active] = grads
        assert (qw.gradient() is not None) == active[0] and (kw.gradient() is not None) == active[1]
        assert len(layer.gradients()) == sum(active)
        for parameter in (qw, kw):
            if parameter.active():
                g = parameter.gradient().cpu().numpy()
                assert np.isfinite(g).all() and np.abs(g).max() > 0
    for grads in results.values():
        for a, b in zip(grads, results[(False, False)]):
            assert np.array_equal(a, b)
    # earlier tokens receive key/value gradients from the last query
    assert np.abs(results[(False, False)][1][0]).max() > 0
    assert np.abs(results[(False, False)][2][0]).max() > 0
    # queries before the last receive nothing
    assert np.abs(results[(False, False)][0][:-1]).max() == 0


def test_backward_contracts():
    t, hq, hkv, d = 4, 2, 1, 16
    p = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=8, capacity=8)
    norm = sine_values(d, 0.1, 0.1)
    layer, _, _ = make_layer(p, t, norm, norm)
    inputs = [torch.zeros((t, 2 * hq * d), dtype=torch.bfloat16, device="cuda"),
              torch.zeros((t, hkv * d), dtype=torch.bfloat16, device="cuda"),
              torch.zeros((t, hkv * d), dtype=torch.bfloat16, device="cuda")]
    fwd = layer.fwd(inputs)
    with pytest.raises(PlutoStatusError) as e:      # wrong gradient size
        layer.bwd([torch.zeros((t, hq * d - 1), dtype=torch.float32, device="cuda")], fwd.state)
    assert e.value.code == "InvalidArgument"
    other, _, _ = make_layer(p, t, norm, norm)
    with pytest.raises(PlutoStatusError):           # state of another layer
        other.bwd([torch.zeros((t, hq * d), dtype=torch.float32, device="cuda")], fwd.state)
    # a cached layer is inference only (qwen_attention.cc:364-366)
    cache = KeyValueCache.Create(8, hkv, d)
    p1 = FullAttentionParameters(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=8, capacity=8)
    cached = QwenAttentionLayer.Create(p1, dev(norm), dev(norm), 1, cache)
    step = cached.fwd([x[:1].contiguous() for x in inputs])
    with pytest.raises(PlutoStatusError) as e:
        cached.bwd([torch.zeros((1, hq * d), dtype=torch.float32, device="cuda")], step.state)
    assert e.value.code == "Unimplemented"
