"""Generates tests/golden/reference_specs.npz: what the reference project's own scalar
specifications return on the inputs of its own layer tests.

The specifications -- class AttentionReference and class DeltaReference
(cached_attention_ops_test.cc:43-220), Reference of sequence_delta_net_test.cc:66-159 and of
qwen_attention_test.cc:26-95, with the numerical-gradient loops of those tests -- are compiled
from the reference tree where it lies into oracle/_ref/libpluto_ref_specs.so (oracle/Makefile,
oracle/ref_specs_shim.cc).  This script runs them on the shapes and closed-form inputs of those
tests (tests/spec_cases.py) and stores the outputs.  Run once in a container that has the
reference tree:
    python tests/golden/make_golden_specs.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402
import spec_cases as cases  # noqa: E402


def check_example(shape, tensors, upstream):
    """The tests' numpy restatement of the reference's MakeExample against MakeExample itself: the
    bf16 activations are identical; the fp32 parameters and the upstream gradient may differ in
    the last bit (numpy's sinf against the C library's).  The specifications below are run on
    the numpy values, so both sides of every later comparison see the same inputs."""
    theirs, their_upstream = oracle.spec_sequence_delta_example(*shape, True)
    for n, (a, b) in enumerate(zip(theirs, tensors)):
        assert np.array_equal(a, b) if n < 4 else np.abs(a - b).max() <= 6e-8, n
    assert np.abs(their_upstream - upstream).max() <= 6e-8


def main():
    oracle.build()
    assert oracle.have_ref_specs(), "needs the reference tree to build oracle/_ref/libpluto_ref_specs.so"
    store = {}
    for dim, rnd in cases.ATTENTION_STEP_CASES:
        p, q, k, v, qn, kn = cases.attention_step_inputs(dim)
        out, probs = oracle.spec_attention_steps(p["query_heads"], p["key_value_heads"], dim, p["rotary_dim"],
                                                 p["capacity"], p["epsilon"], p["theta"], rnd, q, k, v, qn, kn)
        for t in cases.ATTENTION_KEPT_STEPS[dim]:
            store[f"attention_d{dim}_r{int(rnd)}_t{t}_out"] = out[t]
            store[f"attention_d{dim}_r{int(rnd)}_t{t}_probs"] = probs[t]
    for dim, rnd in cases.DELTA_STEP_CASES:
        (kh, vh, kd, vd, kernel), qkv, z, a, b, w, alog, dt, norm = cases.delta_step_inputs(dim)
        store[f"delta_d{dim}_r{int(rnd)}_out"] = oracle.spec_delta_steps(kh, vh, kd, vd, kernel, 1e-6, rnd, qkv,
                                                                         z, a, b, w, alog, dt, norm)
    for shape in cases.SEQUENCE_DELTA_FORWARD_SHAPES:
        tensors, upstream = cases.sequence_delta_example(*shape)
        check_example(shape, tensors, upstream)
        out = oracle.spec_sequence_delta_forward(*shape, 3, 0.03, True, tensors)
        store["sequence_delta_fwd_" + "_".join(map(str, shape))] = out.astype(np.float32)
    for shape, rnd in cases.SEQUENCE_DELTA_GRADIENT_CASES:
        tensors, upstream = cases.sequence_delta_example(*shape)
        check_example(shape, tensors, upstream)
        grads = oracle.spec_sequence_delta_gradients(*shape, 3, 0.03, rnd, tensors, upstream, 1e-5)
        for n, g in enumerate(grads):
            store["sequence_delta_grad_" + "_".join(map(str, shape)) + f"_r{int(rnd)}_{n}"] = g
    for d, length in cases.QWEN_FORWARD_CASES:
        p, qg, k, v, qw, kw = cases.qwen_forward_inputs(d, length)
        store[f"qwen_fwd_d{d}"] = oracle.spec_qwen_sequence_forward(
            p["query_heads"], p["key_value_heads"], d, p["rotary_dim"], p["epsilon"], p["theta"], True, length,
            qg, k, v, qw, kw)
    for rnd in (False, True):
        p, t, values, upstream = cases.qwen_gradient_inputs()
        grads = oracle.spec_qwen_sequence_gradients(p["query_heads"], p["key_value_heads"], p["head_dim"],
                                                    p["rotary_dim"], p["epsilon"], p["theta"], rnd, t, *values,
                                                    upstream, 1e-5)
        for n, g in enumerate(grads):
            store[f"qwen_grad_r{int(rnd)}_{n}"] = g
        store[f"qwen_grad_r{int(rnd)}_fwd"] = oracle.spec_qwen_sequence_forward(
            p["query_heads"], p["key_value_heads"], p["head_dim"], p["rotary_dim"], p["epsilon"], p["theta"], rnd,
            t, *values)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_specs.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), len(store), "arrays")


if __name__ == "__main__":
    main()
