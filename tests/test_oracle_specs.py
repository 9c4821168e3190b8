"""Holds the CPU oracle (oracle/pluto_oracle.c) to what the reference project's own scalar
specifications return.

tests/golden/reference_specs.npz was written by tests/golden/make_golden_specs.py from
oracle/_ref/libpluto_ref_specs.so: class AttentionReference and class DeltaReference of
cached_attention_ops_test.cc:43-220, Reference of sequence_delta_net_test.cc:66-159 and of
qwen_attention_test.cc:26-95, and those tests' numerical-gradient loops, compiled from the
reference tree and run on the tests' own shapes and inputs.  The tolerances are the ones the
reference applies between its GPU layers and these specifications.  Where the compiled
specifications are present (a machine with the reference tree, or one that received the built
library) the same comparisons also run live on seeded random inputs.
"""
import os

import numpy as np
import pytest

import oracle
import spec_cases as cases

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_specs.npz"))
live = pytest.mark.skipif(not oracle.have_ref_specs(), reason="compiled reference specifications absent")


def near(actual, expected, absolute, relative):
    actual, expected = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    return bool(np.all(np.abs(actual - expected) <= absolute + relative * np.abs(expected)))


def oracle_attention_steps(p, q, k, v, qn, kn, rnd):
    """CachedAttentionStep over all steps with the C restatement; returns outputs and
    probability rows per step."""
    steps, dim = q.shape[0], p["head_dim"]
    keys = np.zeros((steps, p["key_value_heads"], dim), np.float32)
    values = np.zeros_like(keys)
    outs, probs = [], []
    for t in range(steps):
        queries = oracle.qk_prepare(q[t], k[t], v[t], qn, kn, t, p["rotary_dim"], p["epsilon"], p["theta"], rnd,
                                    keys, values)
        outs.append(oracle.gqa_decode(queries, q[t], keys, values, t + 1, rnd))
        probs.append(oracle.gqa_probabilities(queries, keys, t + 1))
    return outs, probs


@pytest.mark.parametrize("dim,rnd", cases.ATTENTION_STEP_CASES)
def test_cached_attention_steps_match_the_reference_specification(dim, rnd):
    """cached_attention_ops_test.cc:283-362 with its tolerance (:270-274)."""
    p, q, k, v, qn, kn = cases.attention_step_inputs(dim)
    outs, probs = oracle_attention_steps(p, q, k, v, qn, kn, rnd)
    tol = (2e-4, 8e-3) if rnd else (3e-5, 1e-4)
    for t in cases.ATTENTION_KEPT_STEPS[dim]:
        tag = f"attention_d{dim}_r{int(rnd)}_t{t}"
        assert near(outs[t], GOLDEN[tag + "_out"], *tol), tag
        assert near(probs[t], GOLDEN[tag + "_probs"], *tol), tag


def oracle_delta_steps(shape, qkv, z, a, b, w, alog, dt, norm, eps, rnd):
    kh, vh, kd, vd, kernel = shape
    channels = 2 * kh * kd + vh * vd
    conv_state = np.zeros((channels, kernel), np.float32)
    state = np.zeros((1, vh, kd, vd), np.float32)
    outs = []
    for t in range(qkv.shape[0]):
        conv = oracle.gdn_conv_step(qkv[t], w, conv_state, rnd)
        kq = kh * kd
        core = oracle.gdn_recurrence(conv[:kq].reshape(1, 1, kh, kd), conv[kq:2 * kq].reshape(1, 1, kh, kd),
                                     conv[2 * kq:].reshape(1, 1, vh, vd),
                                     oracle.gdn_decay(a[t], dt, alog).reshape(1, 1, vh),
                                     oracle.gdn_beta(b[t], rnd).reshape(1, 1, vh), state, True, 1.0, rnd)
        outs.append(oracle.gdn_output(core.reshape(vh, vd), z[t].reshape(vh, vd), norm, eps, rnd, True))
    return np.stack(outs)


@pytest.mark.parametrize("dim,rnd", cases.DELTA_STEP_CASES)
def test_delta_net_steps_match_the_reference_specification(dim, rnd):
    """cached_attention_ops_test.cc:400-470: softplus extremes a = +-100 included."""
    shape, qkv, z, a, b, w, alog, dt, norm = cases.delta_step_inputs(dim)
    got = oracle_delta_steps(shape, qkv, z, a, b, w, alog, dt, norm, 1e-6, rnd)
    tol = (2e-4, 8e-3) if rnd else (3e-5, 1e-4)
    assert near(got, GOLDEN[f"delta_d{dim}_r{int(rnd)}_out"], *tol)


def oracle_sequence_delta(shape, tensors, upstream, eps, rnd, want_gradients):
    length, kh, vh, kd, vd = shape
    channels = 2 * kh * kd + vh * vd
    params = [np.zeros(channels * 3, np.float32), np.zeros(vh, np.float32), np.zeros(vh, np.float32),
              np.zeros(vd, np.float32)] if want_gradients else [None] * 4
    got = oracle.gdn_sequence_bwd(tensors[0].reshape(length, channels), tensors[1].reshape(length, vh * vd),
                                  tensors[2].reshape(length, vh), tensors[3].reshape(length, vh),
                                  tensors[4].reshape(channels, 3), tensors[5], tensors[6], tensors[7],
                                  upstream.reshape(length, vh * vd), kh, vh, kd, vd, eps, rnd, *params)
    return got, [got["dqkv"].ravel(), got["dz"].ravel(), got["da"].ravel(), got["db"].ravel()] + params


@pytest.mark.parametrize("shape", cases.SEQUENCE_DELTA_FORWARD_SHAPES)
def test_sequence_delta_net_forward_matches_the_reference_specification(shape):
    """sequence_delta_net_test.cc:241-297 (0.00015 + 1.5 %)."""
    tensors, upstream = cases.sequence_delta_example(*shape)
    got, _ = oracle_sequence_delta(shape, tensors, upstream, 0.03, True, False)
    want = GOLDEN["sequence_delta_fwd_" + "_".join(map(str, shape))]
    # the layer stores its result as bf16; the specification rounds that last product too
    assert near(oracle.round_bf16(got["y"]).reshape(want.shape), want, 1.5e-4, 0.015)


@pytest.mark.parametrize("shape,rnd", cases.SEQUENCE_DELTA_GRADIENT_CASES)
def test_sequence_delta_net_gradients_match_the_reference_numerical_bptt(shape, rnd):
    """sequence_delta_net_test.cc:299-373: every input and parameter gradient against central
    differences of the specification (tolerances :352-356: 2e-5 + 0.2 % for the small examples,
    3e-5 + 0.3 % for the large one)."""
    tensors, upstream = cases.sequence_delta_example(*shape)
    _, grads = oracle_sequence_delta(shape, tensors, upstream, 0.03, rnd, True)
    tol = (3e-5, 0.003) if shape[-1] == 35 else (2e-5, 0.002)
    for n, g in enumerate(grads):
        want = GOLDEN["sequence_delta_grad_" + "_".join(map(str, shape)) + f"_r{int(rnd)}_{n}"]
        assert near(g, want, *tol), (n, np.abs(g - want).max())


@pytest.mark.parametrize("d,length", cases.QWEN_FORWARD_CASES)
def test_qwen_sequence_forward_matches_the_reference_specification(d, length):
    """qwen_attention_test.cc:155-228 shapes against Reference(...) (:26-95)."""
    p, qg, k, v, qw, kw = cases.qwen_forward_inputs(d, length)
    hq, hkv = p["query_heads"], p["key_value_heads"]
    got = oracle.gqa_sequence_bwd(qg.reshape(length, hq, 2, d), k.reshape(length, hkv, d), v.reshape(length, hkv, d),
                                  qw, kw, np.zeros((length, hq, d), np.float32), p["rotary_dim"], p["epsilon"],
                                  p["theta"], True)
    assert near(got["y"], GOLDEN[f"qwen_fwd_d{d}"], 2e-4, 8e-3)


@pytest.mark.parametrize("rnd", [False, True])
def test_qwen_sequence_gradients_match_the_reference_finite_differences(rnd):
    """qwen_attention_test.cc:230-301: 3e-5 on every coordinate."""
    p, t, values, upstream = cases.qwen_gradient_inputs()
    hq, hkv, d = p["query_heads"], p["key_value_heads"], p["head_dim"]
    dqw, dkw = np.zeros(d, np.float32), np.zeros(d, np.float32)
    got = oracle.gqa_sequence_bwd(values[0].reshape(t, hq, 2, d), values[1].reshape(t, hkv, d),
                                  values[2].reshape(t, hkv, d), values[3], values[4], upstream.reshape(t, hq, d),
                                  p["rotary_dim"], p["epsilon"], p["theta"], rnd, dqw, dkw)
    actual = [got["dqg"].ravel(), got["dk"].ravel(), got["dv"].ravel(), dqw, dkw]
    for n, a in enumerate(actual):
        want = GOLDEN[f"qwen_grad_r{int(rnd)}_{n}"]
        assert np.abs(a - want).max() < 3e-5, (n, np.abs(a - want).max())
    assert near(got["y"], GOLDEN[f"qwen_grad_r{int(rnd)}_fwd"], *((2e-4, 8e-3) if rnd else (3e-5, 1e-4)))


# ---------------------------------------------------------------------------- live comparisons
@live
@pytest.mark.parametrize("shape", [(8, 2, 64, 16, 40), (5, 5, 20, 20, 33), (16, 4, 128, 64, 70)])
@pytest.mark.parametrize("rnd", [False, True])
def test_live_cached_attention_on_random_inputs(shape, rnd):
    hq, hkv, dim, rotary, steps = shape
    rng = np.random.default_rng(hq * 1000 + dim)
    p = dict(query_heads=hq, key_value_heads=hkv, head_dim=dim, rotary_dim=rotary, capacity=steps, epsilon=1e-6,
             theta=1e6)
    q = rng.standard_normal((steps, hq, 2, dim)).astype(np.float32)
    k = rng.standard_normal((steps, hkv, dim)).astype(np.float32)
    v = rng.standard_normal((steps, hkv, dim)).astype(np.float32)
    qn, kn = (0.2 * rng.standard_normal(dim)).astype(np.float32), (0.2 * rng.standard_normal(dim)).astype(np.float32)
    want, want_probs = oracle.spec_attention_steps(hq, hkv, dim, rotary, steps, 1e-6, 1e6, rnd, q, k, v, qn, kn)
    outs, probs = oracle_attention_steps(p, q, k, v, qn, kn, rnd)
    # Rounded mode: an intermediate that lands on a rounding tie can fall either way between a
    # float and a double evaluation and then differs by one bf16 step; the reference's own
    # tolerance (2e-4 + 0.8 %) is for smooth test inputs, random ones get 2 bf16 ulps.
    tol = (4e-3, 1.6e-2) if rnd else (3e-5, 1e-4)
    for t in range(steps):
        assert near(outs[t], want[t], *tol), t
        assert near(probs[t], want_probs[t], *tol), t


@live
@pytest.mark.parametrize("shape", [(2, 4, 16, 24, 3), (1, 3, 128, 128, 4), (4, 8, 64, 32, 2)])
@pytest.mark.parametrize("rnd", [False, True])
def test_live_delta_net_steps_on_random_inputs(shape, rnd):
    kh, vh, kd, vd, kernel = shape
    steps = 9
    rng = np.random.default_rng(kd * 7 + vd)
    channels = 2 * kh * kd + vh * vd
    qkv = rng.standard_normal((steps, channels)).astype(np.float32)
    z = rng.standard_normal((steps, vh * vd)).astype(np.float32)
    a, b = rng.standard_normal((steps, vh)).astype(np.float32), rng.standard_normal((steps, vh)).astype(np.float32)
    w = (0.5 * rng.standard_normal((channels, kernel))).astype(np.float32)
    alog, dt = (0.5 * rng.standard_normal(vh)).astype(np.float32), (0.3 * rng.standard_normal(vh)).astype(np.float32)
    norm = (1 + 0.2 * rng.standard_normal(vd)).astype(np.float32)
    want = oracle.spec_delta_steps(kh, vh, kd, vd, kernel, 1e-6, rnd, qkv, z, a, b, w, alog, dt, norm)
    got = oracle_delta_steps(shape, qkv, z, a, b, w, alog, dt, norm, 1e-6, rnd)
    tol = (4e-3, 1.6e-2) if rnd else (3e-5, 1e-4)
    assert near(got, want.reshape(got.shape), *tol)
