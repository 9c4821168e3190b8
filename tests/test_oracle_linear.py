"""CPU checks of the imported-projection oracle: the E4M3 codec over all 256 codes, the dynamic
input quantisation cases of fully_connected_imported_test.cc:213-256, and the known answer of
:96-140."""
import numpy as np

import oracle


def test_e4m3_codec_round_trips_and_rounds_to_nearest_even():
    codes = np.arange(256, dtype=np.uint8)
    values = oracle.e4m3_to_float(codes)
    finite = ~np.isnan(values)
    assert finite.sum() == 254 and np.nanmax(values) == 448.0 and values[1] == 2.0 ** -9
    again = oracle.float_to_e4m3(values[finite])
    assert np.array_equal(oracle.e4m3_to_float(again), values[finite])
    got = oracle.e4m3_to_float(oracle.float_to_e4m3(np.array([1.0625, 1.1875, 500.0, -1e9, 2.0 ** -10], np.float32)))
    assert got.tolist() == [1.0, 1.25, 448.0, -448.0, 0.0]


def test_dynamic_quantization_groups():
    x = np.zeros(389, np.float32)
    x[128:132] = [448, -448, 1.0625, 1.1875]
    x[256:384] = oracle.round_bf16(((np.arange(256, 384) % 5 - 2) * 1e-14).astype(np.float32))
    q = oracle.quantize_imported_input(x)
    assert np.all(q[:128] == 0) and q[128] == 448 and q[129] == -448 and q[130] == 1.0 and q[131] == 1.25
    # tiny group: only the divisor is floored at 1e-12, the dequantisation keeps the real scale
    scale = np.abs(x[256:384]).max() / np.float32(448.0)
    want = oracle.e4m3_to_float(oracle.float_to_e4m3(x[256:384] / np.float32(1e-12))) * scale
    assert np.array_equal(q[256:384], want.astype(np.float32)) and np.isfinite(q).all()


def test_known_answer_in_every_storage():
    w = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    x = np.array([1, 0, -1], np.float32)
    assert oracle.linear_imported(w, "fp32", x).tolist() == [-2.0, -2.0]
    assert oracle.linear_imported(oracle.to_bf16_bits(w), "bf16", x).tolist() == [-2.0, -2.0]
    assert oracle.linear_imported(oracle.float_to_e4m3(w), "fp8", x, np.ones(1, np.float32)).tolist() == [-2.0, -2.0]
