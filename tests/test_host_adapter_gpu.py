"""Runs the C++ host adapter's GPU test program (tests/cpp/host_adapter_test.cc): the reference-
shaped C++ classes (AttentionLayer, KeyValueCache, CachedAttentionStep, DeltaNetState) over the C
ABI, checked against the oracle library.  The binary is built by __graft_entry__.build()."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
EXE = os.path.join(os.path.dirname(__file__), "cpp", "_build", "host_adapter_test")


def test_cpp_host_adapter():
    assert os.path.exists(EXE), "run __graft_entry__.build() first"
    proc = subprocess.run([EXE], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "PASS" in proc.stdout
