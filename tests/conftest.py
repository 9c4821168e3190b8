import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_lib():
    import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def engine():
    """The built CUDA engine; building is part of the product, a missing library is an error."""
    from pluto_b200 import _capi
    _capi.lib()
    return _capi


def reference_pattern(context, heads, width, sequences, score_scale=1.0):
    """Inputs of the reference's layer-vs-CPU tests (attention_reference_test.cc:35-44)."""
    rows = context * sequences
    i = np.arange(rows * 3 * width, dtype=np.float32)
    qkv = (np.float32(0.35) * np.sin(i * np.float32(0.071))
           + np.float32(0.05) * np.cos(i * np.float32(0.19))).astype(np.float32)
    qkv = qkv.reshape(rows, 3 * width)
    qkv[:, :2 * width] *= np.float32(score_scale)
    j = np.arange(rows * width, dtype=np.float32)
    d_out = (np.float32(0.2) * np.cos(j * np.float32(0.13))).astype(np.float32).reshape(rows, width)
    return qkv, d_out


def sine_values(count, phase, scale=1.0):
    """Values() of cached_attention_ops_test.cc:34-39."""
    return (np.float32(scale) * np.sin(np.float32(phase) + np.arange(count, dtype=np.float32)
                                       * np.float32(0.29))).astype(np.float32)


# (context, heads, width, sequences) of attention_reference_test.cc:148-161
REFERENCE_SHAPES = [(1, 1, 16, 3), (4, 1, 16, 2), (4, 2, 32, 2), (8, 2, 32, 1), (33, 2, 64, 2),
                    (33, 2, 128, 2), (65, 2, 64, 2), (65, 2, 128, 2), (65, 2, 160, 2),
                    (65, 2, 192, 2), (65, 2, 256, 2)]
SUBTILE_WIDTHS = [1, 3, 7, 8, 15, 24, 33]
