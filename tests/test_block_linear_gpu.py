"""BlockLinearLayer and DequantizeMatrix on the GPU (tcgen05 GEMMs on the bf16 values, fp32 dY as
hi + lo halves), following src/llm/layers/block_training_test.cc:115-164, 188-232, 329-352."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_device_bf16
from pluto_b200 import PlutoStatusError, _capi
from pluto_b200.layers import BlockLinearLayer, BlockParameter, DataType, DequantizeMatrix, MatrixStorage

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf16_dev(x):
    return to_device_bf16(oracle.to_bf16_bits(np.asarray(x, np.float32)))


def test_linear_matches_cpu_forward_and_both_gradients():
    x = np.array([[1, 2, -3], [4, -2, 1]], np.float32)
    w = np.array([[0.25, -1, 2], [-0.5, 0.75, 1]], np.float32)
    dy = np.array([[2, -1], [-0.5, 3]], np.float32)
    y, dx, dw = x @ w.T, dy @ w, dy.T @ x
    weight = BlockParameter.Create(bf16_dev(w).view(2, 3))
    for float_output in (False, True):
        layer = BlockLinearLayer.Create(weight, 3, 2, 2, float_output)
        assert layer.output_types()[0].data_type == (DataType.FP32 if float_output else DataType.BF16)
        result = layer.fwd([bf16_dev(x).view(2, 3)])
        want = y if float_output else oracle.round_bf16(y)
        assert np.array_equal(result.outputs[0].float().cpu().numpy(), want)
        back = layer.bwd([dev(dy)], result.state)          # frozen: dx only, no optimizer storage
        assert np.array_equal(back[0].cpu().numpy(), dx) and not weight.active()
        weight.Activate()
        for accumulated in (1, 2):
            back = layer.bwd([dev(dy)], result.state)
            assert np.array_equal(back[0].cpu().numpy(), dx)
            assert np.array_equal(weight.gradient().cpu().numpy(), dw * accumulated)
        weight.Deactivate()


def test_linear_masks_tail_tiles_and_produces_repeatable_gradients():
    cols, rows, tokens = 131, 35, 3
    x = ((np.arange(tokens * cols) % 13 - 6) * 0.125).astype(np.float32).reshape(tokens, cols)
    w = ((np.arange(rows * cols) % 7 - 3) * 0.125).astype(np.float32).reshape(rows, cols)
    dy = ((np.arange(tokens * rows) % 5 - 2) * 0.0625).astype(np.float32).reshape(tokens, rows)
    weight = BlockParameter.Create(bf16_dev(w).view(rows, cols))
    layer = BlockLinearLayer.Create(weight, cols, rows, tokens)
    result = layer.fwd([bf16_dev(x).view(tokens, cols)])
    assert np.array_equal(result.outputs[0].float().cpu().numpy(), oracle.round_bf16((x @ w.T).astype(np.float32)))
    previous = None
    for _ in range(3):
        weight.Activate()
        back = layer.bwd([dev(dy)], result.state)
        assert np.array_equal(back[0].cpu().numpy(), dy @ w)          # every value is dyadic: exact
        actual = weight.gradient().cpu().numpy()
        assert np.array_equal(actual, dy.T @ x)
        if previous is not None:
            assert np.array_equal(actual, previous)
        previous = actual
        weight.Deactivate()


@pytest.mark.parametrize("tokens,cols,rows", [(200, 264, 136), (1000, 1024, 2304), (77, 5120, 300),
                                              (2500, 2304, 2104)])   # two-SM kernel, ragged tiles
def test_random_values_match_oracle_with_fp32_gradients(tokens, cols, rows):
    rng = np.random.default_rng(tokens)
    x = oracle.round_bf16(rng.standard_normal((tokens, cols)).astype(np.float32))
    w = oracle.round_bf16((rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    dy = rng.standard_normal((tokens, rows)).astype(np.float32)       # not bf16-representable
    weight = BlockParameter.Create(bf16_dev(w).view(rows, cols))
    weight.Activate()
    layer = BlockLinearLayer.Create(weight, cols, rows, tokens, True)
    result = layer.fwd([bf16_dev(x).view(tokens, cols)])
    want = oracle.block_linear_fwd(w, x, True)
    assert np.abs(result.outputs[0].cpu().numpy() - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    back = layer.bwd([dev(dy)], result.state)
    ref = oracle.block_linear_bwd(w, x, dy)
    # hi + lo halves of dY keep 16 mantissa bits: well inside the 1e-4 fp32 tolerance
    for name, got, exp in (("dx", back[0].cpu().numpy(), ref["dx"]),
                           ("dw", weight.gradient().cpu().numpy(), ref["dw"])):
        scale = max(1.0, float(np.abs(exp).max()))
        assert np.abs(got - exp).max() <= 1e-4 * scale, (name, float(np.abs(got - exp).max()), scale)
    assert _capi.kernel_status() == 0


def test_dequantize_respects_both_scale_block_boundaries():
    codes = np.full((129, 129), oracle.float_to_e4m3(np.array([0.5], np.float32))[0], np.uint8)
    scales = dev(np.array([1, 2, 3, 4], np.float32))
    result = DequantizeMatrix(dev(codes), MatrixStorage.kFp8E4M3, scales, 129, 129)
    actual = result.float().cpu().numpy()
    row, col = np.meshgrid(np.arange(129), np.arange(129), indexing="ij")
    assert np.array_equal(actual, (1 + 2 * (row // 128) + col // 128) * 0.5)
    shared = DequantizeMatrix(result, MatrixStorage.kBFloat16, None, 129, 129)
    assert shared.data_ptr() == result.data_ptr()
    values = np.linspace(-3, 3, 129 * 129).astype(np.float32).reshape(129, 129)
    converted = DequantizeMatrix(dev(values), MatrixStorage.kFloat32, None, 129, 129)
    assert np.array_equal(converted.float().cpu().numpy(), oracle.round_bf16(values))
    with pytest.raises(PlutoStatusError):
        DequantizeMatrix(dev(codes), MatrixStorage.kFp8E4M3, None, 129, 129)


def test_rejects_incorrect_storage_and_batch_size():
    weight = BlockParameter.Create(torch.zeros((2, 3), dtype=torch.bfloat16, device="cuda"))
    fp32 = BlockParameter.Create(torch.zeros((2, 3), dtype=torch.float32, device="cuda"))
    for args in ((fp32, 3, 2, 2), (weight, 3, 3, 2), (weight, 0, 2, 2), (weight, 3, 2, 0)):
        with pytest.raises(PlutoStatusError) as e:
            BlockLinearLayer.Create(*args)
        assert e.value.code == "InvalidArgument"
    layer = BlockLinearLayer.Create(weight, 3, 2, 2)
    with pytest.raises(PlutoStatusError):
        layer.fwd([torch.zeros((4, 3), dtype=torch.bfloat16, device="cuda")])      # two samples
