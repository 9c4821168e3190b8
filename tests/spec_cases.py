"""Inputs of the reference's own layer tests, shared by the script that records what the
reference's scalar specifications return for them (tests/golden/make_golden_specs.py) and by the
tests that hold the CPU oracle to those records (tests/test_oracle_specs.py)."""
import numpy as np

import oracle
from conftest import sine_values
from gdn_double_model import make_example
from qwen_double_model import wave

# cached_attention_ops_test.cc:283-362: (dim) -> parameters; 35 steps crossing the 32-row tile
ATTENTION_STEP_CASES = [(dim, rnd) for dim in (6, 256) for rnd in (False, True)]
ATTENTION_KEPT_STEPS = {6: list(range(35)), 256: [0, 31, 32, 34]}


def attention_step_parameters(dim):
    return dict(query_heads=4 if dim == 6 else 24, key_value_heads=2 if dim == 6 else 4, head_dim=dim,
                rotary_dim=4 if dim == 6 else 64, capacity=35, epsilon=1e-6,
                theta=73.0 if dim == 6 else 1e7)


def attention_step_inputs(dim):
    p = attention_step_parameters(dim)
    hq, hkv = p["query_heads"], p["key_value_heads"]
    q = np.stack([sine_values(hq * 2 * dim, 0.15 + t * 0.21).reshape(hq, 2, dim) for t in range(35)])
    k = np.stack([sine_values(hkv * dim, 0.78 + t * 0.13).reshape(hkv, dim) for t in range(35)])
    v = np.stack([sine_values(hkv * dim, -0.31 + t * 0.37).reshape(hkv, dim) for t in range(35)])
    return p, q, k, v, sine_values(dim, 0.2, 0.3), sine_values(dim, 0.8, 0.4)


# cached_attention_ops_test.cc:400-470: Hk 2 / Hv 6, dims (5, 7) and (128, 128), kernel 4, 6 steps
DELTA_STEP_CASES = [(dim, rnd) for rnd in (False, True) for dim in (5, 128)]


def delta_step_inputs(dim):
    kh, vh, kd, vd, kernel = 2, 6, dim, 7 if dim == 5 else 128, 4
    channels = 2 * kh * kd + vh * vd
    qkv = np.stack([sine_values(channels, 0.3 + t * 0.71) for t in range(6)])
    z = np.stack([sine_values(vh * vd, -0.6 + t * 0.27) for t in range(6)])
    a = np.stack([sine_values(vh, 0.1 + t * 0.1) for t in range(6)])
    b = np.stack([sine_values(vh, -0.7 + t * 0.3) for t in range(6)])
    a[:, 0], a[:, 1] = 100.0, -100.0
    weights = sine_values(channels * kernel, 0.73, 0.6).reshape(channels, kernel)
    return (kh, vh, kd, vd, kernel), qkv, z, a, b, weights, sine_values(vh, 0.18, 0.5), \
        sine_values(vh, -0.7, 0.3), sine_values(vd, 0.5, 0.6)


# sequence_delta_net_test.cc:241-297 (forward, T = 3) and :299-373 (gradients)
SEQUENCE_DELTA_FORWARD_SHAPES = [(3, 1, 2, 3, 5), (3, 2, 4, 5, 35), (3, 16, 48, 128, 128)]
SEQUENCE_DELTA_GRADIENT_CASES = [((5, 1, 2, 3, 5), False), ((5, 1, 2, 3, 5), True), ((3, 2, 4, 5, 35), True)]
sequence_delta_example = make_example   # (length, kh, vh, kd, vd) -> eight tensors, upstream

# qwen_attention_test.cc:155-228 (forward) and :230-301 (gradients)
QWEN_FORWARD_CASES = [(3, 33), (256, 3)]     # (head_dim, length); Hq 2, Hkv 1, rotary 2 / 64


def qwen_forward_inputs(d, length):
    hq, hkv = 2, 1
    return dict(query_heads=hq, key_value_heads=hkv, head_dim=d, rotary_dim=2 if d == 3 else 64,
                epsilon=1e-6, theta=1e7), wave(length * 2 * hq * d, .1), wave(length * d, 1.2), \
        wave(length * d, 2.3), wave(d, .2), wave(d, .4)


def qwen_gradient_inputs():
    t = 3
    return dict(query_heads=2, key_value_heads=1, head_dim=3, rotary_dim=2, epsilon=1e-6, theta=1e7), t, \
        [wave(t * 12, .1), wave(t * 3, 1.2), wave(t * 3, 2.3), wave(3, .2), wave(3, .4)], wave(t * 6, .7)
