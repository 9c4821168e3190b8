"""Pins oracle.gqa_sequence_bwd (the restatement of the five backward kernels of
src/llm/layers/qwen_attention.cc:124-239) with the check the reference's own test applies to its
GPU layer: central differences of an independent double-precision model, tolerance 3e-5, on the
reference test's configuration and inputs (qwen_attention_test.cc:230-301)."""
import numpy as np
import pytest

import oracle
from qwen_double_model import DoubleModel, wave


@pytest.mark.parametrize("rnd", [False, True])
def test_backward_matches_finite_differences_of_double_model(rnd):
    t, hq, hkv, d, rotary = 3, 2, 1, 3, 2
    eps, theta = 1e-6, 1e7
    values = [wave(t * 12, .1), wave(t * 3, 1.2), wave(t * 3, 2.3), wave(3, .2), wave(3, .4)]
    upstream = wave(t * 6, .7)
    model = DoubleModel(t, hq, hkv, d, rotary, eps, theta, rnd)
    expected = model.gradients(values, [float(u) for u in upstream])
    dqw, dkw = np.zeros(d, np.float32), np.zeros(d, np.float32)
    got = oracle.gqa_sequence_bwd(values[0].reshape(t, hq, 2, d), values[1].reshape(t, hkv, d),
                                  values[2].reshape(t, hkv, d), values[3], values[4],
                                  upstream.reshape(t, hq, d), rotary, eps, theta, rnd, dqw, dkw)
    actual = [got["dqg"].ravel(), got["dk"].ravel(), got["dv"].ravel(), dqw, dkw]
    for name, a, e in zip(["dqg", "dk", "dv", "dq_norm", "dk_norm"], actual, expected):
        assert np.abs(a - e).max() < 3e-5, (name, np.abs(a - e).max())
    # the forward the backward differentiates is the pinned sequence forward
    y = np.array(model.forward(*[list(x) for x in values]))
    assert np.abs(got["y"].ravel() - y).max() < (8e-3 if rnd else 2e-6)
    # shared norm gradients accumulate across calls (qwen_attention_test.cc:291-300)
    first_q, first_k = dqw.copy(), dkw.copy()
    again = oracle.gqa_sequence_bwd(values[0].reshape(t, hq, 2, d), values[1].reshape(t, hkv, d),
                                    values[2].reshape(t, hkv, d), values[3], values[4],
                                    upstream.reshape(t, hq, d), rotary, eps, theta, rnd, dqw, dkw)
    assert np.array_equal(again["dqg"], got["dqg"])
    assert np.abs(dqw - 2 * first_q).max() < 1e-6 and np.abs(dkw - 2 * first_k).max() < 1e-6


def test_frozen_norms_leave_weight_gradients_untouched_and_match_active_run():
    t, hq, hkv, d, rotary = 5, 4, 2, 8, 4
    rng = np.random.default_rng(3)
    qg = oracle.round_bf16(rng.standard_normal((t, hq, 2, d)).astype(np.float32))
    k = oracle.round_bf16(rng.standard_normal((t, hkv, d)).astype(np.float32))
    v = oracle.round_bf16(rng.standard_normal((t, hkv, d)).astype(np.float32))
    qw = (0.1 * rng.standard_normal(d)).astype(np.float32)
    kw = (0.1 * rng.standard_normal(d)).astype(np.float32)
    dy = rng.standard_normal((t, hq, d)).astype(np.float32)
    frozen = oracle.gqa_sequence_bwd(qg, k, v, qw, kw, dy, rotary, 1e-6, 1e6, True)
    dqw, dkw = np.zeros(d, np.float32), np.zeros(d, np.float32)
    active = oracle.gqa_sequence_bwd(qg, k, v, qw, kw, dy, rotary, 1e-6, 1e6, True, dqw, dkw)
    for key in ("dqg", "dk", "dv"):
        assert np.array_equal(frozen[key], active[key])
    assert np.abs(dqw).max() > 0 and np.abs(dkw).max() > 0
    # gradients reach tokens before the last one (causal attention couples the rows)
    assert np.abs(frozen["dk"][0]).max() > 0 and np.abs(frozen["dv"][0]).max() > 0
