"""Imported projections (FullyConnectedLayer over frozen bf16 / fp32 / FP8 weights) on the GPU,
following src/llm/layers/fully_connected_imported_test.cc."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_device_bf16
from pluto_b200 import PlutoStatusError, _capi
from pluto_b200.layers import DataType, FullyConnectedLayer, MatrixStorage

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf(x):
    return oracle.to_bf16_bits(np.asarray(x, np.float32))


def upload(weights_fp32, storage):
    if storage == MatrixStorage.kFloat32:
        return dev(weights_fp32.astype(np.float32)), weights_fp32.astype(np.float32), "fp32"
    if storage == MatrixStorage.kBFloat16:
        bits = bf(weights_fp32)
        return to_device_bf16(bits), bits, "bf16"
    codes = oracle.float_to_e4m3(weights_fp32)
    return dev(codes), codes, "fp8"


def read(t):
    return t.float().cpu().numpy()


def test_shares_all_storage_without_masters_or_gradients():
    """fully_connected_imported_test.cc:96-140: [[1,2,3],[4,5,6]] x (1,0,-1) = (-2,-2)."""
    x = to_device_bf16(bf([1, 0, -1])).view(1, 3)
    w = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    for storage in MatrixStorage:
        weights, _, _ = upload(w, storage)
        scales = dev(np.ones(1, np.float32)) if storage == MatrixStorage.kFp8E4M3 else None
        layer = FullyConnectedLayer.Create(weights, storage, 3, 2, scales)
        assert layer.weights()[0].data_ptr() == weights.data_ptr()
        assert len(layer.weights()) == (2 if storage == MatrixStorage.kFp8E4M3 else 1)
        assert layer.gradients() == [] and layer.output_type() == DataType.BF16
        assert layer.input_types()[0].dimensions == (-2, 1, 3)
        assert layer.output_types()[0].dimensions == (-2, 1, 2)
        for init in (lambda: layer.InitializeIdentity(), lambda: layer.InitializeNormal(1, 123)):
            with pytest.raises(PlutoStatusError) as e:
                init()
            assert e.value.code == "FailedPrecondition"
        result = layer.fwd([x])
        assert read(result.outputs[0]).ravel().tolist() == [-2.0, -2.0]
        assert result.state.intermediates == []
        with pytest.raises(PlutoStatusError) as e:
            layer.bwd([], result.state)
        assert e.value.code == "Unimplemented"


@pytest.mark.parametrize("cols,rows", [(263, 259), (5120, 131), (4096, 520), (12288, 64)])
def test_block_scales_tails_and_real_width_match_scalar_projection(cols, rows):
    """fully_connected_imported_test.cc:142-211: sizes that straddle the row tiles and the
    128x128 scale blocks, its closed-form weights, inputs and scales, its tolerance against a
    double-precision dot product; plus the CPU oracle at bf16 resolution."""
    i = np.arange(cols * rows)
    source = (1.9 * np.sin((i % 1009).astype(np.float32) * np.float32(0.037))).astype(np.float32).reshape(rows, cols)
    x = oracle.round_bf16((np.cos(np.arange(cols, dtype=np.float32) * np.float32(0.123)) * 0.25).astype(np.float32))
    scale_cols, scale_rows = (cols + 127) // 128, (rows + 127) // 128
    scales = np.array([[(r + 1) * (c + 1) * 0.03125 for c in range(scale_cols)] for r in range(scale_rows)], np.float32)
    for storage in MatrixStorage:
        weights, stored, name = upload(source, storage)
        fp8 = storage == MatrixStorage.kFp8E4M3
        layer = FullyConnectedLayer.Create(weights, storage, cols, rows, dev(scales) if fp8 else None)
        got = read(layer.fwd([to_device_bf16(bf(x)).view(1, cols)]).outputs[0]).ravel()
        if name == "fp32":
            w = stored.astype(np.float64)
        elif name == "bf16":
            w = oracle.from_bf16_bits(stored).astype(np.float64)
        else:
            w = oracle.e4m3_to_float(stored).astype(np.float64) * np.repeat(np.repeat(scales, 128, 0), 128, 1)[:rows, :cols]
        xin = oracle.quantize_imported_input(x) if fp8 else x
        expected = oracle.round_bf16((w @ xin.astype(np.float64)).astype(np.float32))
        assert np.all(np.abs(got - expected) <= 5e-5 + 0.008 * np.abs(expected)), (name, np.abs(got - expected).max())
        want = oracle.linear_imported(stored, name, x, scales if fp8 else None)
        assert np.all(np.abs(got - want) <= 5e-5 + 0.008 * np.abs(want)), name


def test_dynamic_fp8_quantization_handles_zero_tiny_ties_and_tail():
    """fully_connected_imported_test.cc:213-256: an FP8 identity exposes the quantised input."""
    width = 389
    x = np.zeros(width, np.float32)
    for i in range(128, 256):
        x[i] = ((i % 31) - 15) * 0.0625
    x[128], x[129], x[130], x[131] = 448, -448, 1.0625, 1.1875
    for i in range(256, 384):
        x[i] = (i % 5 - 2) * 1e-14
    for i in range(384, width):
        x[i] = (i - 386) * 25.3
    x = oracle.round_bf16(x)
    identity = np.zeros((width, width), np.uint8)
    identity[np.arange(width), np.arange(width)] = oracle.float_to_e4m3(np.array([1.0], np.float32))[0]
    layer = FullyConnectedLayer.Create(dev(identity), MatrixStorage.kFp8E4M3, width, width,
                                       dev(np.ones(16, np.float32)))
    got = read(layer.fwd([to_device_bf16(bf(x)).view(1, width)]).outputs[0]).ravel()
    expected = oracle.quantize_imported_input(x)
    assert np.all(np.abs(got - oracle.round_bf16(expected)) <= 1e-20 + 0.008 * np.abs(expected))
    assert got[130] == 1.0 and got[131] == 1.25


def test_several_tokens_share_one_pass_and_match_single_token_calls():
    cols, rows = 1024, 300
    rng = np.random.default_rng(3)
    w = rng.standard_normal((rows, cols)).astype(np.float32)
    x = oracle.round_bf16(rng.standard_normal((11, cols)).astype(np.float32))
    for storage in MatrixStorage:
        weights, _, _ = upload(w, storage)
        scales = dev(np.full(((rows + 127) // 128) * (cols // 128), 0.5, np.float32)) \
            if storage == MatrixStorage.kFp8E4M3 else None
        layer = FullyConnectedLayer.Create(weights, storage, cols, rows, scales)
        xd = to_device_bf16(bf(x)).view(11, cols)
        batched = layer.fwd([xd]).outputs[0].float().cpu().numpy()
        for t in range(11):
            # a single token may take the FMA form and a batch the tensor-core form: same values up
            # to the summation order
            single = layer.fwd([xd[t:t + 1].contiguous()]).outputs[0].float().cpu().numpy()
            assert np.all(np.abs(single - batched[t:t + 1]) <= 5e-5 + 0.008 * np.abs(single)), t
        for n in (3, 8):
            part = layer.fwd([xd[:n].contiguous()]).outputs[0].float().cpu().numpy()
            assert np.all(np.abs(part - batched[:n]) <= 5e-5 + 0.008 * np.abs(part)), n


@pytest.mark.parametrize("cols,rows", [(1024, 2402), (2176, 2370), (5120, 2560), (8192, 2371)])
def test_streamed_weight_ring_matches_oracle_for_one_to_four_tokens(cols, rows):
    """Enough 4-row tasks for the persistent streaming kernels (a ring of bulk-copied weight
    slabs, two CTAs per SM), a last slab of fewer rows, a width that is not a multiple of 256
    (FP8 then takes the FMA form of the ring instead of the tensor-core form), slabs of two rows
    (8192 columns), and one to six tokens; bf16 and FP8 against the CPU oracle."""
    rng = np.random.default_rng(cols + rows)
    w = (rng.standard_normal((rows, cols)) * 0.5).astype(np.float32)
    x = oracle.round_bf16(rng.standard_normal((6, cols)).astype(np.float32))
    x[1, 128:256] = 0.0          # an all-zero quantisation group
    scale_cols, scale_rows = (cols + 127) // 128, (rows + 127) // 128
    scales = (0.25 + rng.random((scale_rows, scale_cols))).astype(np.float32)
    for storage in (MatrixStorage.kBFloat16, MatrixStorage.kFp8E4M3):
        weights, stored, name = upload(w, storage)
        fp8 = storage == MatrixStorage.kFp8E4M3
        layer = FullyConnectedLayer.Create(weights, storage, cols, rows, dev(scales) if fp8 else None)
        want = np.stack([oracle.linear_imported(stored, name, x[t], scales if fp8 else None) for t in range(6)])
        for n in (1, 2, 3, 4, 6):
            got = layer.fwd([to_device_bf16(bf(x[:n])).view(n, cols)]).outputs[0].float().cpu().numpy()
            assert np.all(np.abs(got - want[:n]) <= 5e-5 + 0.008 * np.abs(want[:n])), (name, n)


def test_back_to_back_projections_see_each_others_outputs():
    """The streaming kernels start copying weights while the previous kernel of the stream still
    runs; a chain in which every call's activation is the previous call's output (no host
    synchronisation in between, buffers re-used round after round) must still equal the oracle."""
    width = 2560
    rng = np.random.default_rng(11)
    x = oracle.round_bf16(rng.standard_normal((1, width)).astype(np.float32))
    scales = (0.5 + rng.random((width // 128, width // 128))).astype(np.float32)
    for storage in (MatrixStorage.kBFloat16, MatrixStorage.kFp8E4M3):
        fp8 = storage == MatrixStorage.kFp8E4M3
        layers, stored = [], []
        for i in range(3):
            w = (rng.standard_normal((width, width)) * (0.6 / np.sqrt(width) if not fp8 else 0.4)).astype(np.float32)
            weights, kept, name = upload(w, storage)
            layers.append(FullyConnectedLayer.Create(weights, storage, width, width, dev(scales) if fp8 else None))
            stored.append(kept)
        want = x[0]
        for kept in stored:
            want = oracle.linear_imported(kept, name, want, scales if fp8 else None)
        L, stream = _capi.lib(), torch.cuda.current_stream().cuda_stream
        buffers = [to_device_bf16(bf(x)).view(1, width)] + [torch.zeros(1, width, dtype=torch.bfloat16, device="cuda")
                                                           for _ in range(3)]
        results = []
        for _ in range(20):
            buffers[1].zero_(); buffers[2].zero_(); buffers[3].zero_()
            for i, layer in enumerate(layers):
                held = layer.weights()
                _capi.check(L.pluto_linear_imported_fwd(stream, held[0].data_ptr(), storage.value,
                                                        held[1].data_ptr() if fp8 else None, buffers[i].data_ptr(),
                                                        buffers[i + 1].data_ptr(), 1, width, width))
            results.append(buffers[3].clone())
        torch.cuda.synchronize()
        for got in results:
            got = got.float().cpu().numpy().ravel()
            assert np.all(np.abs(got - want) <= 2e-3 + 0.03 * np.abs(want)), name
            assert np.array_equal(got, results[0].float().cpu().numpy().ravel())   # and bit-identical every round


def test_rejects_bad_storage_dimensions_and_scales():
    w = dev(np.ones(4, np.float32))
    one = dev(np.ones(1, np.float32))
    for args in ((w, MatrixStorage.kFloat32, 0, 2, None), (w, MatrixStorage.kFloat32, 2, 1048577, None),
                 (w, MatrixStorage.kFloat32, 2, 3, None), (w, MatrixStorage.kFloat32, 2, 2, one),
                 (dev(np.zeros(4, np.uint8)), MatrixStorage.kFp8E4M3, 2, 2, None),
                 (dev(np.zeros(4, np.uint8)), MatrixStorage.kFp8E4M3, 2, 2, dev(np.ones(2, np.float32)))):
        with pytest.raises(PlutoStatusError) as e:
            FullyConnectedLayer.Create(*args)
        assert e.value.code == "InvalidArgument"
    layer = FullyConnectedLayer.Create(w, MatrixStorage.kFloat32, 2, 2)
    with pytest.raises(PlutoStatusError):
        layer.fwd([torch.zeros(3, dtype=torch.bfloat16, device="cuda")])
