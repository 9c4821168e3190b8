"""Parity of the CUDA AttentionLayer against the CPU oracle (the reference's own scalar layer),
in the pattern of the reference's layer-vs-reference tests (attention_reference_test.cc)."""
import math
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import REFERENCE_SHAPES, SUBTILE_WIDTHS, reference_pattern
from gpu_util import bf16_bits, near, to_device_bf16
from pluto_b200 import PlutoStatusError, _capi
from pluto_b200.layers import AttentionLayer, DataType, LayerHooks

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "attention_reference.npz")


def run_layer(qkv, d_out, context, heads, width, bf16, hooks=None):
    layer = AttentionLayer.Create(context, heads, width, DataType.BF16 if bf16 else DataType.FP16)
    x = to_device_bf16(oracle.to_bf16_bits(qkv)) if bf16 else torch.from_numpy(qkv).cuda()
    fwd = layer.fwd([x], hooks)
    grad = layer.bwd([torch.from_numpy(d_out).cuda()], fwd.state)[0]
    torch.cuda.synchronize()
    out = fwd.outputs[0]
    out_f = oracle.from_bf16_bits(bf16_bits(out)) if bf16 else out.cpu().numpy()
    return out_f, grad.cpu().numpy(), fwd


def oracle_layer(qkv, d_out, context, heads, width, bf16):
    x = oracle.to_bf16_bits(qkv) if bf16 else qkv
    out, d_qkv = oracle.attention_fwd_bwd(x, d_out, context, heads, width, bf16, threads=8)
    return (oracle.from_bf16_bits(out) if bf16 else out), d_qkv


def check(context, heads, width, sequences, bf16, scale=1.0, fwd_tol=None, bwd_tol=None):
    qkv, d_out = reference_pattern(context, heads, width, sequences, scale)
    got_o, got_g, _ = run_layer(qkv, d_out, context, heads, width, bf16)
    ref_o, ref_g = oracle_layer(qkv, d_out, context, heads, width, bf16)
    # fp32 policy: the 1e-4 max-abs bar; bf16: max-abs 2e-2 and the reference tests' 2e-3/3e-3 form
    if not bf16:
        assert np.abs(got_o - ref_o).max() <= 1e-4, (context, heads, width)
        assert np.abs(got_g - ref_g).max() <= 1e-4, (context, heads, width)
    else:
        assert np.abs(got_o - ref_o).max() <= 2e-2 and np.abs(got_g - ref_g).max() <= 2e-2
        assert near(got_o, ref_o, *(fwd_tol or (2e-3, 8e-3))), (context, heads, width)
        assert near(got_g, ref_g, *(bwd_tol or (3e-3, 3e-3))), (context, heads, width)
    assert _capi.kernel_status() == 0


@pytest.mark.parametrize("bf16", [False, True])
def test_reference_configurations(bf16):
    """attention_reference_test.cc:148-161."""
    for shape in REFERENCE_SHAPES:
        check(*shape, bf16)


@pytest.mark.parametrize("bf16", [False, True])
def test_peaked_scores_and_production_context(bf16):
    """attention_reference_test.cc:163-176: x20 scores across partial tiles; S=1024."""
    check(65, 1, 64, 2, bf16, 20.0, fwd_tol=(4e-3, 8e-3), bwd_tol=(3e-3, 3e-3))
    check(1024, 1, 64, 1, bf16)


@pytest.mark.parametrize("bf16", [False, True])
def test_subtile_head_widths(bf16):
    """attention_reference_test.cc:178-205."""
    for width in SUBTILE_WIDTHS:
        check(33, 1, width, 2, bf16)
    check(65, 3, 21, 2, bf16)
    if bf16:
        check(1024, 1, 8, 1, True)
        for head_dim in (16, 32):
            check(1024, 1, head_dim, 1, True, 4.0)
        check(65, 3, 96, 2, True, 4.0)


def test_many_heads_ragged_length_takes_the_two_tile_kernel():
    """Enough (sequence, head) units for the two-tile ping-pong forward kernel at a length that
    is not a multiple of its tiles (300 = 2 tiles + 44 rows: the last CTA has a lone tile), for
    both head widths; smaller shapes elsewhere in this file exercise the single-tile kernel."""
    check(300, 16, 1024, 10, True)     # head width 64
    check(300, 10, 1280, 16, True)     # head width 128


def test_golden_vectors_through_the_c_abi():
    """The committed outputs of the reference's CPU layer (tests/golden) against the CUDA path."""
    data = np.load(GOLDEN)
    for n, (s, h, e, b, scale) in enumerate(data["cases"]):
        s, h, e, b = int(s), int(h), int(e), int(b)
        qkv, d_out = reference_pattern(s, h, e, b, scale)
        for bf16 in (False, True):
            tag = f"c{n}_{'bf16' if bf16 else 'fp32'}"
            got_o, got_g, _ = run_layer(qkv, d_out, s, h, e, bf16)
            want_o = oracle.from_bf16_bits(data[tag + "_out"]) if bf16 else data[tag + "_out"]
            tol = 2e-2 if bf16 else 1e-4
            assert np.abs(got_o - want_o).max() <= tol, tag
            assert np.abs(got_g - data[tag + "_dqkv"]).max() <= tol, tag


def test_hand_computable_case():
    """attention_test.cc:282-360."""
    context, heads, width = 4, 2, 32
    x = np.zeros((4, 3 * width), np.float32)
    x[0, 0] = x[0, width] = x[0, 2 * width] = 1.0
    x[1, 0] = x[1, width] = x[1, 2 * width] = 2.0
    x[2, 2 * width] = 4.0
    d_out = np.zeros((4, width), np.float32)
    d_out[0, 0] = 1.0
    out, grad, _ = run_layer(x, d_out, context, heads, width, False)
    scale = 1.0 / math.sqrt(width / heads)
    w1, w2 = math.exp(2 * scale), math.exp(4 * scale)
    assert abs(out[0, 0] - 1.0) < 1e-6
    assert abs(out[1, 0] - (w1 + 2 * w2) / (w1 + w2)) < 1e-5
    assert abs(grad[0, 0]) < 1e-6 and abs(grad[0, width]) < 1e-6
    assert abs(grad[0, 2 * width] - 1.0) < 1e-6 and abs(grad[1, 0]) < 1e-6


@pytest.mark.parametrize("bf16", [False, True])
def test_probability_hook(bf16):
    """attention_test.cc:27-150: probabilities vs double softmax (3e-5), zeros above the diagonal,
    rows sum to one; the hook sees the [B,H,S,S] fp32 tensor before the output is published."""
    for (s, h, e, b) in [(1, 1, 7, 2), (5, 2, 14, 2), (33, 2, 160, 2), (65, 3, 21, 1)]:
        for uniform in (False, True):
            idx = np.arange(s * b * 3 * e)
            qkv = ((idx % 19 - 9) / 8.0).astype(np.float32).reshape(s * b, 3 * e)
            if uniform:
                qkv[:, :2 * e] = 0.0
            seen = {}

            def hook(name, shape, probs):
                seen["name"], seen["shape"], seen["probs"] = name, shape, probs

            out, _, fwd = run_layer(qkv, np.zeros((s * b, e), np.float32), s, h, e, bf16,
                                    LayerHooks(attention_probabilities_hook=hook))
            assert seen["name"] == "AttentionLayer"
            assert seen["shape"].dimensions == (b, h, s, s) and seen["shape"].data_type == DataType.FP32
            probs = seen["probs"].cpu().numpy()
            ref = oracle.attention_fwd(qkv if not bf16 else oracle.to_bf16_bits(qkv), s, h, e, bf16,
                                       want_probs=True)["probs"]
            assert np.abs(probs - ref).max() <= 3e-5
            mask = np.tril(np.ones((s, s), bool))
            assert np.all(probs[..., ~mask] == 0.0)
            assert np.abs(probs.sum(-1) - 1.0).max() <= 3e-5
            if uniform:
                expect = np.where(mask, 1.0 / np.arange(1, s + 1)[:, None], 0.0)
                assert np.abs(probs - expect).max() <= 1e-6


def test_hook_failure_cancels_forward():
    """attention_test.cc:246-280: an error from the hook propagates; nothing is published."""
    def hook(name, shape, probs):
        raise PlutoStatusError("Cancelled", "stop", 1)
    layer = AttentionLayer.Create(4, 2, 32, DataType.FP16)
    with pytest.raises(PlutoStatusError) as info:
        layer.fwd([torch.zeros(4, 96, device="cuda")], LayerHooks(attention_probabilities_hook=hook))
    assert info.value.code == "Cancelled"


@pytest.mark.parametrize("bf16,shape", [(False, (65, 2, 64, 2)), (True, (65, 2, 128, 2)),
                                        (True, (300, 2, 128, 1)), (True, (33, 1, 24, 2))])
def test_bitwise_repeatable(bf16, shape):
    """attention_test.cc:362-475 / attention_reference_test.cc:80-100: fresh layers and buffers
    reproduce every output and gradient bit."""
    qkv, d_out = reference_pattern(*shape)
    first = None
    for _ in range(4):
        layer = AttentionLayer.Create(shape[0], shape[1], shape[2], DataType.BF16 if bf16 else DataType.FP16)
        x = to_device_bf16(oracle.to_bf16_bits(qkv)) if bf16 else torch.from_numpy(qkv).cuda()
        fwd = layer.fwd([x.clone()])
        grad = layer.bwd([torch.from_numpy(d_out).cuda()], fwd.state)[0]
        torch.cuda.synchronize()
        now = (fwd.outputs[0].view(torch.uint8).cpu().numpy().tobytes(), grad.cpu().numpy().tobytes())
        first = first or now
        assert now == first


@pytest.mark.parametrize("bf16", [False, True])
def test_future_tokens_and_other_sequences_cannot_matter(bf16):
    """attention_reference_test.cc:207-308: perturbing invisible tokens leaves visible outputs and
    gradients bit-identical; gradients of invisible positions are exactly zero."""
    context, heads, width, sequences = 65, 2, 128, 2
    qkv, d_out = reference_pattern(context, heads, width, sequences)
    cut = 40  # tokens >= cut of sequence 0 get no upstream gradient and are perturbed
    d_out[cut:context] = 0.0
    d_out[context:] = 0.0
    base_o, base_g, _ = run_layer(qkv, d_out, context, heads, width, bf16)
    changed = qkv.copy()
    changed[cut:context] += 0.37
    changed[context:] -= 0.21
    new_o, new_g, _ = run_layer(changed, d_out, context, heads, width, bf16)
    assert np.array_equal(base_o[:cut], new_o[:cut])
    assert np.array_equal(base_g[:cut], new_g[:cut])
    assert np.all(new_g[cut:] == 0.0)


@pytest.mark.parametrize("shape", [(300, 2, 128, 2), (1024, 2, 256, 1), (65, 3, 192, 2),
                                   # head width 128 in one, three and five 128-row steps, several sequences
                                   (100, 1, 128, 3), (330, 2, 256, 2), (640, 1, 128, 2)])
def test_tensor_core_backward_matches_exact_backward(shape):
    """bf16, head width 64/128: the tcgen05 backward against the exact fp32 backward kernels on
    the same saved state (max-abs 2e-2), and bit-identical across repeated runs."""
    context, heads, width, sequences = shape
    rng = np.random.default_rng(77)
    qkv = to_device_bf16(oracle.to_bf16_bits(rng.standard_normal((context * sequences, 3 * width), dtype=np.float32)))
    d_out = torch.from_numpy(rng.standard_normal((context * sequences, width), dtype=np.float32)).cuda()
    layer = AttentionLayer.Create(context, heads, width, DataType.BF16)
    fwd = layer.fwd([qkv])
    fast = layer.bwd([d_out], fwd.state)[0]
    again = layer.bwd([d_out], fwd.state)[0]
    layer.tensor_core_backward = False
    exact = layer.bwd([d_out], fwd.state)[0]
    torch.cuda.synchronize()
    assert torch.equal(fast, again)
    assert (fast - exact).abs().max().item() <= 2e-2
    assert torch.isfinite(fast).all()
    assert _capi.kernel_status() == 0


def test_validation_errors_launch_nothing():
    """attention_test.cc:549-626."""
    layer = AttentionLayer.Create(8, 2, 32, DataType.FP16)
    with pytest.raises(PlutoStatusError) as info:
        layer.fwd([torch.zeros(12, 96, device="cuda")])
    assert "divisible by context_length" in info.value.message
    fwd = layer.fwd([torch.zeros(8, 96, device="cuda")])
    state = fwd.state
    state.intermediates[2] = torch.zeros(3, device="cuda")
    with pytest.raises(PlutoStatusError) as info:
        layer.bwd([torch.zeros(8, 32, device="cuda")], state)
    assert "saved maxima" in info.value.message
    fwd = layer.fwd([torch.zeros(8, 96, device="cuda")])
    fwd.state.intermediates[3] = torch.zeros(3, device="cuda")
    with pytest.raises(PlutoStatusError) as info:
        layer.bwd([torch.zeros(8, 32, device="cuda")], fwd.state)
    assert "saved normalizers" in info.value.message


def test_training_shape_seeded_gaussians():
    """The two training configurations on seeded N(0,1) inputs, reduced in batch so the scalar
    oracle finishes in seconds: fp32 B4 H6 S256 D64 (1e-4) and bf16 B1 H12 S1024 D64 (2e-2)."""
    rng = np.random.default_rng(2024)
    for (b, h, s, d, bf16, tol) in [(4, 6, 256, 64, False, 1e-4), (1, 12, 1024, 64, True, 2e-2)]:
        e = h * d
        qkv = rng.standard_normal((b * s, 3 * e), dtype=np.float32)
        d_out = rng.standard_normal((b * s, e), dtype=np.float32)
        if bf16:
            qkv = oracle.round_bf16(qkv)
        got_o, got_g, _ = run_layer(qkv, d_out, s, h, e, bf16)
        ref_o, ref_g = oracle_layer(qkv, d_out, s, h, e, bf16)
        assert np.abs(got_o - ref_o).max() <= tol
        assert np.abs(got_g - ref_g).max() <= tol
        assert np.isfinite(got_g).all()


def test_full_size_training_config_properties():
    """bf16 B8 H12 S1024 D64 at full size: size-independent properties instead of the scalar
    oracle -- row 0 of every sequence attends only to itself (O == V), and sum_s dV equals
    sum_s dO per sequence/channel because every probability row sums to one."""
    b, h, s, d = 8, 12, 1024, 64
    e = h * d
    torch.manual_seed(5)
    qkv = torch.randn(b * s, 3 * e, device="cuda").bfloat16()
    d_out = torch.randn(b * s, e, device="cuda")
    layer = AttentionLayer.Create(s, h, e, DataType.BF16)
    fwd = layer.fwd([qkv])
    grad = layer.bwd([d_out], fwd.state)[0]
    torch.cuda.synchronize()
    out = fwd.outputs[0].float().view(b, s, e)
    v = qkv.float().view(b, s, 3 * e)[:, :, 2 * e:]
    assert torch.equal(out[:, 0], v[:, 0])
    dv_sum = grad.view(b, s, 3 * e)[:, :, 2 * e:].double().sum(1)
    do_sum = d_out.view(b, s, e).double().sum(1)
    # the tensor-core backward rounds dO and P to bf16 (2^-9 each): allow 1 % of the summed magnitude
    scale = d_out.view(b, s, e).abs().double().sum(1)
    assert ((dv_sum - do_sum).abs() <= 2e-2 + 0.01 * scale).all()
    assert torch.isfinite(grad).all()
    assert _capi.kernel_status() == 0
