"""Generates tests/golden/attention_reference.npz from the reference project's own CPU layer.

Runs oracle/_ref/libpluto_ref.so (AttentionLayerReference compiled unmodified from the reference
tree by oracle/Makefile) on the inputs of the reference's own layer tests
(attention_reference_test.cc:35-44, shapes from :148-197) and stores inputs' generating
parameters plus the outputs.  Run once in a container that has the reference tree:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402
from conftest import reference_pattern  # noqa: E402

CASES = [  # context, heads, width, sequences, score_scale
    (1, 1, 16, 3, 1.0), (4, 2, 32, 2, 1.0), (8, 2, 32, 1, 1.0), (33, 2, 64, 2, 1.0),
    (33, 2, 128, 1, 1.0), (65, 2, 160, 1, 1.0), (33, 1, 256, 1, 1.0), (65, 1, 64, 2, 20.0),
    (33, 1, 7, 2, 1.0), (33, 1, 33, 2, 1.0), (65, 3, 21, 2, 1.0), (65, 3, 96, 1, 4.0),
    (200, 1, 64, 1, 1.0),
]


def main():
    oracle.build()
    assert oracle.have_ref(), "needs the reference tree to build oracle/_ref"
    store = {"cases": np.array(CASES, dtype=np.float64)}
    for n, (s, h, e, b, scale) in enumerate(CASES):
        qkv, d_out = reference_pattern(s, h, e, b, scale)
        for bf16 in (False, True):
            x = oracle.to_bf16_bits(qkv) if bf16 else qkv
            out, d_qkv = oracle.attention_fwd_bwd(x, d_out, s, h, e, bf16, use_ref=True)
            tag = f"c{n}_{'bf16' if bf16 else 'fp32'}"
            store[tag + "_out"] = out
            store[tag + "_dqkv"] = d_qkv
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_reference.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path))


if __name__ == "__main__":
    main()
