"""Pins oracle.gdn_sequence_bwd (the restatement of the backward kernels of
src/llm/layers/sequence_delta_net.cc:126-339) the way the reference pins its GPU layer: central
differences of an independent double model with frozen rounding offsets, on the reference test's
examples and tolerances (sequence_delta_net_test.cc:299-373)."""
import numpy as np
import pytest

import oracle
from gdn_double_model import DoubleModel, make_example

NAMES = ["dqkv", "dz", "da", "db", "d_conv", "d_a_log", "d_dt_bias", "d_norm"]


def run_oracle(values, upstream, length, kh, vh, kd, vd, eps, rnd):
    channels = 2 * kh * kd + vh * vd
    params = [np.zeros(channels * 3, np.float32), np.zeros(vh, np.float32), np.zeros(vh, np.float32),
              np.zeros(vd, np.float32)]
    got = oracle.gdn_sequence_bwd(values[0].reshape(length, channels), values[1].reshape(length, vh * vd),
                                  values[2].reshape(length, vh), values[3].reshape(length, vh),
                                  values[4].reshape(channels, 3), values[5], values[6], values[7],
                                  upstream.reshape(length, vh * vd), kh, vh, kd, vd, eps, rnd,
                                  params[0], params[1], params[2], params[3])
    return [got["dqkv"].ravel(), got["dz"].ravel(), got["da"].ravel(), got["db"].ravel()] + params, got


@pytest.mark.parametrize("shape,rnd,tol", [((5, 1, 2, 3, 5), False, (2e-5, 0.002)),
                                           ((5, 1, 2, 3, 5), True, (2e-5, 0.002)),
                                           ((3, 2, 4, 5, 35), True, (3e-5, 0.003))])
def test_all_gradients_match_numerical_bptt(shape, rnd, tol):
    length, kh, vh, kd, vd = shape
    eps = 0.03
    values, upstream = make_example(length, kh, vh, kd, vd)
    actual, got = run_oracle(values, upstream, length, kh, vh, kd, vd, eps, rnd)
    upstream = [float(u) for u in upstream]   # python floats: the differences need double precision
    model = DoubleModel(length, kh, vh, kd, vd, 3, eps, rnd)
    if shape[-1] == 35:   # the large example: check a strided sample of coordinates per tensor
        expected = None
        base = [list(map(float, x)) for x in values]
        model.forward(base, record=True)
        for tensor in range(8):
            for i in range(0, len(base[tensor]), max(1, len(base[tensor]) // 25)):
                original = base[tensor][i]
                base[tensor][i] = original + 1e-5
                plus = sum(p * q for p, q in zip(model.forward(base), upstream))
                base[tensor][i] = original - 1e-5
                minus = sum(p * q for p, q in zip(model.forward(base), upstream))
                base[tensor][i] = original
                e = (plus - minus) / 2e-5
                assert abs(actual[tensor][i] - e) <= tol[0] + abs(e) * tol[1], (NAMES[tensor], i)
    else:
        expected = model.gradients(values, upstream)
        for name, a, e in zip(NAMES, actual, expected):
            assert np.all(np.abs(a - e) <= tol[0] + np.abs(e) * tol[1]), (name, np.abs(a - e).max())
    # the loss sits at the last token only: the first token must still receive a gradient
    channels = 2 * kh * kd + vh * vd
    assert np.abs(actual[0][:channels]).sum() > 1e-5
    # forward of the same pass agrees with the double model
    y = np.array(model.forward([list(map(float, x)) for x in values]))
    # (the model rounds the final product to bf16 as the layer's store does; the oracle returns it
    # unrounded)
    assert np.abs(oracle.round_bf16(got["y"].ravel()) - y).max() < (8e-3 if rnd else 1e-3)
