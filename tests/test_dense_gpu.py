"""Trainable dense projection (tcgen05 GEMMs) on the GPU, following
src/llm/layers/fully_connected_test.cc and the operand-cast semantics of fully_connected.cc:97-232."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_device_bf16
from pluto_b200 import PlutoStatusError, _capi
from pluto_b200.layers import DataType, DenseLayer

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_identity_dense_layer_has_identity_forward_and_backward():
    """fully_connected_test.cc:19-81 (FP16 policy, fp32 activations, 1e-6)."""
    tokens, width = 64, 32
    index = np.arange(tokens * width)
    x = ((index % 17 - 8) / 8).astype(np.float32).reshape(tokens, width)
    dy = ((index % 9 - 4) / 8).astype(np.float32).reshape(tokens, width)
    layer = DenseLayer.Create(width, data_type=DataType.FP16)
    layer.InitializeIdentity()
    fwd = layer.fwd([dev(x)])
    dx = layer.bwd([dev(dy)], fwd.state)
    assert np.abs(fwd.outputs[0].cpu().numpy() - x).max() <= 1e-6
    assert np.abs(dx[0].cpu().numpy() - dy).max() <= 1e-6


def test_rectangular_projection_uses_distinct_input_and_output_widths():
    """fully_connected_test.cc:83-123."""
    tokens, width, out = 64, 32, 48
    layer = DenseLayer.Create(width, out, DataType.FP16)
    assert layer.input_dim() == width and layer.output_dim() == out
    layer.InitializeIdentity()
    x = (np.arange(tokens * width) % 7).astype(np.float32).reshape(tokens, width)
    y = layer.fwd([dev(x)]).outputs[0].cpu().numpy()
    assert np.array_equal(y[:, :width], x) and np.all(y[:, width:] == 0)


@pytest.mark.parametrize("rows,in_dim,out_dim,dtype", [
    (300, 200, 136, DataType.BF16), (513, 768, 2304, DataType.BF16), (100, 77, 53, DataType.FP16),
    (1024, 1024, 1024, DataType.FP16), (64, 3000, 130, DataType.BF16),
    # every product large enough for the two-SM kernel (at least 74 tiles of 256 x 256), ragged edges
    (2500, 2300, 2100, DataType.BF16), (2340, 2200, 2500, DataType.FP16)])
def test_forward_and_backward_match_oracle(rows, in_dim, out_dim, dtype):
    rng = np.random.default_rng(rows + in_dim)
    bf16 = dtype == DataType.BF16
    x = rng.standard_normal((rows, in_dim)).astype(np.float32)
    if bf16:
        x = oracle.round_bf16(x)
    w = (rng.standard_normal((in_dim, out_dim)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(out_dim).astype(np.float32)
    dy = rng.standard_normal((rows, out_dim)).astype(np.float32)
    layer = DenseLayer.Create(in_dim, out_dim, dtype)
    layer.weights()[0].copy_(dev(w))
    layer.weights()[1].copy_(dev(bias))
    xd = to_device_bf16(oracle.to_bf16_bits(x)).view(rows, in_dim) if bf16 else dev(x)
    fwd = layer.fwd([xd])
    y = fwd.outputs[0].float().cpu().numpy()
    want = oracle.dense_fwd(x, w, bias, bf16)
    tol = 1e-2 if bf16 else 2e-4        # bf16 outputs: one ulp of the stored result
    assert np.all(np.abs(y - want) <= tol * np.maximum(1.0, np.abs(want))), np.abs(y - want).max()
    dx = layer.bwd([dev(dy)], fwd.state)[0].cpu().numpy()
    ref = oracle.dense_bwd(x, w, dy, bf16)
    for name, got, exp in (("dx", dx, ref["dx"]), ("dw", layer.gradients()[0].cpu().numpy(), ref["dw"]),
                           ("db", layer.gradients()[1].cpu().numpy(), ref["db"])):
        scale = max(1.0, float(np.abs(exp).max()))
        assert np.abs(got - exp).max() <= 3e-4 * scale, (name, float(np.abs(got - exp).max()), scale)
    # gradients are overwritten, not accumulated
    first = layer.gradients()[0].clone()
    layer.bwd([dev(dy)], layer.fwd([xd]).state)
    assert torch.equal(first, layer.gradients()[0])
    assert _capi.kernel_status() == 0


def test_contracts():
    for bad in ((0, 4), (4, 0)):
        with pytest.raises(PlutoStatusError) as e:
            DenseLayer.Create(*bad)
        assert e.value.code == "InvalidArgument"
    with pytest.raises(PlutoStatusError) as e:
        DenseLayer.Create(4, 4, DataType.FP8)
    assert e.value.code == "Unimplemented"
    layer = DenseLayer.Create(8, 8, DataType.BF16)
    with pytest.raises(PlutoStatusError):
        layer.fwd([torch.zeros(7, dtype=torch.bfloat16, device="cuda")])
    with pytest.raises(PlutoStatusError):
        layer.InitializeNormal(0.0, 1)
