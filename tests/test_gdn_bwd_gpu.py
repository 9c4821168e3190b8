"""SequenceDeltaNetLayer backward on the GPU (output norm/gate -> recurrence BPTT with chunk
checkpoints -> gathers -> convolution) against numerical BPTT of the independent double model and
against the CPU oracle, following sequence_delta_net_test.cc:299-404."""
import numpy as np
import pytest
import torch

import oracle
from gdn_double_model import DoubleModel, make_example
from gpu_util import to_device_bf16
from pluto_b200 import PlutoStatusError
from pluto_b200.layers import BlockParameter, DeltaNetParameters, SequenceDeltaNetLayer

pytestmark = pytest.mark.gpu
NAMES = ["dqkv", "dz", "da", "db", "d_conv", "d_a_log", "d_dt_bias", "d_norm"]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf(x):
    return oracle.to_bf16_bits(np.asarray(x, np.float32))


def make_layer(p, t, params, active=True):
    owned = [BlockParameter.Create(dev(np.asarray(x, np.float32))) for x in params]
    if active:
        for parameter in owned:
            parameter.Activate()
    return SequenceDeltaNetLayer.Create(p, *owned, t), owned


def run(layer, acts, dy, t):
    inputs = [to_device_bf16(bf(x)).view(t, -1) for x in acts]
    fwd = layer.fwd(inputs)
    grads = layer.bwd([dev(np.asarray(dy, np.float32)).view(t, -1)], fwd.state)
    torch.cuda.synchronize()
    return fwd, [g.cpu().numpy().ravel() for g in grads]


@pytest.mark.parametrize("shape,tol", [((5, 1, 2, 3, 5), (2e-5, 0.002)), ((3, 2, 4, 5, 35), (3e-5, 0.003))])
def test_all_gradients_match_numerical_bptt(shape, tol):
    """The reference's own check (sequence_delta_net_test.cc:299-373): its examples, step and
    tolerances; the large example is sampled."""
    length, kh, vh, kd, vd = shape
    eps = 0.03
    values, upstream = make_example(length, kh, vh, kd, vd)
    p = DeltaNetParameters(key_heads=kh, value_heads=vh, key_head_dim=kd, value_head_dim=vd,
                           conv_kernel_dim=3, rms_norm_epsilon=eps, round_to_bfloat16=True)
    channels = 2 * kh * kd + vh * vd
    layer, owned = make_layer(p, length, [values[4].reshape(channels, 3), values[5], values[6], values[7]])
    acts = [values[0].reshape(length, channels), values[1].reshape(length, vh * vd),
            values[2].reshape(length, vh), values[3].reshape(length, vh)]
    _, grads = run(layer, acts, upstream, length)
    actual = grads + [o.gradient().cpu().numpy().ravel() for o in owned]
    model = DoubleModel(length, kh, vh, kd, vd, 3, eps, True)
    base = [list(map(float, x)) for x in values]
    up = [float(u) for u in upstream]
    model.forward(base, record=True)
    for tensor in range(8):
        n = len(base[tensor])
        for i in range(0, n, max(1, n // 40)):
            original = base[tensor][i]
            base[tensor][i] = original + 1e-5
            plus = sum(x * y for x, y in zip(model.forward(base), up))
            base[tensor][i] = original - 1e-5
            minus = sum(x * y for x, y in zip(model.forward(base), up))
            base[tensor][i] = original
            e = (plus - minus) / 2e-5
            assert abs(actual[tensor][i] - e) <= tol[0] + abs(e) * tol[1], (NAMES[tensor], i, actual[tensor][i], e)
    assert np.abs(actual[0][:channels]).sum() > 1e-5      # the first token still gets a gradient


@pytest.mark.parametrize("shape", [(40, 2, 4, 32, 48, 4), (150, 2, 4, 128, 128, 4), (97, 1, 2, 64, 40, 3),
                                   (333, 1, 2, 128, 128, 4), (512, 2, 2, 128, 128, 4)])
def test_backward_matches_oracle_across_chunk_boundaries(shape):
    """Sequences longer than one 64-token chunk (state recompute from checkpoints), grouped value
    heads, partial value tiles; against the CPU restatement that stores every state.  The last two
    shapes (256 tokens or more at width 128) take the chunk-parallel backward: two tensor-core
    scans and one CTA per chunk, with a ragged last chunk in the first of them."""
    t, kh, vh, kd, vd, kernel = shape
    channels = 2 * kh * kd + vh * vd
    rng = np.random.default_rng(17)
    r = lambda *s: oracle.round_bf16((rng.standard_normal(s) * 0.5).astype(np.float32))
    qkv, z, a, b = r(t, channels), r(t, vh * vd), r(t, vh), r(t, vh)
    conv = (rng.standard_normal((channels, kernel)) * 0.4).astype(np.float32)
    a_log = (rng.standard_normal(vh) * 0.3 - 0.7).astype(np.float32)
    dt_bias = (rng.standard_normal(vh) * 0.3).astype(np.float32)
    norm = (1.0 + 0.2 * rng.standard_normal(vd)).astype(np.float32)
    dy = rng.standard_normal((t, vh * vd)).astype(np.float32)
    eps = 1e-6
    want_p = [np.zeros_like(conv), np.zeros_like(a_log), np.zeros_like(dt_bias), np.zeros_like(norm)]
    want = oracle.gdn_sequence_bwd(qkv, z, a, b, conv, a_log, dt_bias, norm, dy, kh, vh, kd, vd, eps,
                                   True, *want_p)
    p = DeltaNetParameters(key_heads=kh, value_heads=vh, key_head_dim=kd, value_head_dim=vd,
                           conv_kernel_dim=kernel, rms_norm_epsilon=eps, round_to_bfloat16=True)
    layer, owned = make_layer(p, t, [conv, a_log, dt_bias, norm])
    _, grads = run(layer, [qkv, z, a, b], dy, t)
    got = grads + [o.gradient().cpu().numpy().ravel() for o in owned]
    ref = [want["dqkv"].ravel(), want["dz"].ravel(), want["da"].ravel(), want["db"].ravel()] + \
          [x.ravel() for x in want_p]
    for name, g, w in zip(NAMES, got, ref):
        scale = max(1.0, float(np.abs(w).max()))
        # the forward core comes from the chunked tensor-core recurrence (bf16 operands): its
        # rounded values, and through them every gradient, differ from the CPU at bf16 level
        assert np.abs(g - w).max() <= 3e-2 * scale, (name, float(np.abs(g - w).max()), scale)
    # bitwise repeatable, parameter gradients accumulate
    first = [o.gradient().clone() for o in owned]
    _, again = run(layer, [qkv, z, a, b], dy, t)
    for x, y in zip(grads, again):
        assert np.array_equal(x, y)
    for o, f in zip(owned, first):
        assert torch.allclose(o.gradient(), 2 * f, rtol=1e-6, atol=1e-6)


def test_frozen_parameters_and_contracts():
    t, kh, vh, kd, vd = 20, 1, 2, 16, 24
    channels = 2 * kh * kd + vh * vd
    rng = np.random.default_rng(2)
    p = DeltaNetParameters(key_heads=kh, value_heads=vh, key_head_dim=kd, value_head_dim=vd,
                           conv_kernel_dim=4, rms_norm_epsilon=1e-6, round_to_bfloat16=True)
    params = [rng.standard_normal((channels, 4)).astype(np.float32) * 0.3,
              np.full(vh, -0.5, np.float32), np.zeros(vh, np.float32), np.ones(vd, np.float32)]
    acts = [oracle.round_bf16(rng.standard_normal(s).astype(np.float32) * 0.5)
            for s in ((t, channels), (t, vh * vd), (t, vh), (t, vh))]
    dy = rng.standard_normal((t, vh * vd)).astype(np.float32)
    frozen, owned_f = make_layer(p, t, params, active=False)
    active, owned_a = make_layer(p, t, params, active=True)
    _, g_frozen = run(frozen, acts, dy, t)
    _, g_active = run(active, acts, dy, t)
    for x, y in zip(g_frozen, g_active):
        assert np.array_equal(x, y)
    assert frozen.gradients() == [] and len(active.gradients()) == 4
    assert all(o.gradient() is None for o in owned_f)
    inputs = [to_device_bf16(bf(x)).view(t, -1) for x in acts]
    fwd = active.fwd(inputs)
    with pytest.raises(PlutoStatusError) as e:
        active.bwd([torch.zeros((t, vh * vd + 1), dtype=torch.float32, device="cuda")], fwd.state)
    assert e.value.code == "InvalidArgument"
    with pytest.raises(PlutoStatusError):
        frozen.bwd([torch.zeros((t, vh * vd), dtype=torch.float32, device="cuda")], fwd.state)


@pytest.mark.parametrize("shape", [(1, 320, 1, 2), (2, 333, 2, 4), (1, 1100, 1, 1), (1, 256, 1, 1), (3, 257, 1, 2)])
def test_chunk_parallel_recurrence_backward_matches_the_token_sequential_kernel(shape):
    """pluto_gdn_recurrence_bwd takes the chunk-parallel path for bf16 activations at width 128 from
    256 tokens on, the token-sequential kernel otherwise.  The same values given once as bf16 and
    once as fp32 therefore run both; every gradient within 5e-3 of its largest magnitude (the
    chunked scans round their operands to bf16), and the chunked path bitwise repeatable."""
    import ctypes

    from pluto_b200 import _capi
    L = _capi.lib()
    P = lambda x: ctypes.c_void_p(x.data_ptr())
    bsz, t, kh, vh = shape
    d = 128
    ch, kq = 2 * kh * d + vh * d, kh * d

    def run(as_bf16):
        g = torch.Generator(device="cuda").manual_seed(5)
        post = (torch.randn(bsz, t, ch, device="cuda", generator=g) * 0.5).bfloat16()
        a = (torch.randn(bsz, t, vh, device="cuda", generator=g) * 0.5).bfloat16()
        b = (torch.randn(bsz, t, vh, device="cuda", generator=g) * 0.5).bfloat16()
        a_log = torch.randn(vh, device="cuda", generator=g) * 0.3 - 0.7
        dt_bias = torch.randn(vh, device="cuda", generator=g) * 0.3
        dcore = torch.randn(bsz, t, vh, d, device="cuda", generator=g)
        if not as_bf16:
            post, a, b = post.float(), a.float(), b.float()
        dtype = 1 if as_bf16 else 0
        dpost = torch.zeros(bsz, t, ch, device="cuda")
        da, db = torch.zeros(bsz, t, vh, device="cuda"), torch.zeros(bsz, t, vh, device="cuda")
        d_a_log, d_dt = torch.zeros(vh, device="cuda"), torch.zeros(vh, device="cuda")
        size = L.pluto_gdn_recurrence_bwd_workspace_bytes(bsz, t, kh, vh, d, d)
        ws = torch.empty(size, dtype=torch.uint8, device="cuda")
        flat, dflat = post.view(-1), dpost.view(-1)
        _capi.check(L.pluto_gdn_recurrence_bwd(
            None, P(flat), P(flat[kq:]), P(flat[2 * kq:]), dtype, ch, ch, P(a), P(b), dtype, P(a_log), P(dt_bias),
            P(dcore), P(dflat), P(dflat[kq:]), ch, P(dflat[2 * kq:]), ch, P(da), P(db), P(d_a_log), P(d_dt),
            P(ws), size, bsz, t, kh, vh, d, d, 1))
        torch.cuda.synchronize()
        assert _capi.kernel_status() == 0
        return [dpost, da, db, d_a_log, d_dt]

    chunked, again, sequential = run(True), run(True), run(False)
    for name, x, y, z in zip(["dpost", "da", "db", "d_a_log", "d_dt_bias"], chunked, again, sequential):
        assert torch.equal(x, y), name
        assert torch.isfinite(x).all(), name
        assert (x - z).abs().max().item() <= 5e-3 * z.abs().max().item(), name
