"""The benchmark configurations at their own sizes, each against the CPU oracle.

The smaller parity suites cover every code path on shapes the scalar oracle finishes at once;
these cases run the workloads the throughput figures are quoted on -- same shapes, same seeded
length distribution -- and compare as much of each result with the oracle as a few CPU seconds
buy: whole (sequence, head) units for decode and delta-net, rows at every tile boundary for the
prefill.
"""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import bf16_bits
from pluto_b200 import _capi
from pluto_b200.layers import gdn_prefill, gdn_step, gqa_decode, gqa_prefill

pytestmark = pytest.mark.gpu

BENCH_SEED = 20240611  # the seed bench.py draws the decode lengths from


def bits_to_float(bits):
    return oracle.from_bf16_bits(bits)


def prefill_sample_rows(seq, extra, seed):
    """Query rows either side of every 128-row tile boundary (and so of every 256-row tile-pair
    boundary), the first and last rows, plus `extra` random ones."""
    rows = {0, 1, seq - 2, seq - 1}
    for edge in range(128, seq, 128):
        rows.update((edge - 1, edge))
    rng = np.random.default_rng(seed)
    rows.update(int(r) for r in rng.integers(0, seq, size=extra))
    return sorted(rows)


@pytest.mark.parametrize("q_heads,kv_heads", [(40, 8), (5, 1)])
def test_prefill_8192_rows_at_every_tile_boundary(q_heads, kv_heads):
    """GQA causal prefill at the headline shape (prompt 8192, head width 128): the full 40/8-head
    problem one GPU runs, and the 5/1-head shard each GPU holds in an 8-way head split (which
    takes the one-tile-per-CTA kernel).  More than 256 query rows against the oracle."""
    t, d = 8192, 128
    gen = torch.Generator(device="cuda").manual_seed(3 + q_heads)
    q = (torch.randn(1, t, q_heads, d, device="cuda", generator=gen) * 0.5).bfloat16()
    k = (torch.randn(1, t, kv_heads, d, device="cuda", generator=gen) * 0.5).bfloat16()
    v = (torch.randn(1, t, kv_heads, d, device="cuda", generator=gen) * 0.5).bfloat16()
    out = gqa_prefill(q, k, v)["out"][0]
    torch.cuda.synchronize()
    rows = prefill_sample_rows(t, 140, q_heads)
    assert len(rows) >= 256
    want = oracle.gqa_prefill_rows(bf16_bits(q[0]), bf16_bits(k[0]), bf16_bits(v[0]), rows, threads=8)
    got = bf16_bits(out[torch.tensor(rows, device="cuda")])
    error = np.abs(bits_to_float(got) - bits_to_float(want))
    assert error.max() <= 2e-2, (rows[int(error.reshape(len(rows), -1).max(1).argmax())], error.max())
    assert _capi.kernel_status() == 0


def test_decode_batch_64_with_the_benchmark_lengths():
    """Decode at the benchmark's batch: 64 sequences, 40/8 heads, head width 128, cached lengths
    drawn as bench.py draws them (U[4096, 32768] from its seed), bf16 cache of capacity 32768.
    Every head of nine sequences -- the longest, the shortest and seven in between -- against
    the oracle, and every output finite."""
    batch, hq, hkv, d, cap = 64, 40, 8, 128, 32768
    lens = np.random.default_rng(BENCH_SEED).integers(4096, 32769, size=batch).astype(np.int32)
    gen = torch.Generator(device="cuda").manual_seed(17)
    k_pool = torch.empty((batch, cap, hkv, d), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.empty_like(k_pool)
    for pool in (k_pool, v_pool):
        for b in range(batch):  # per sequence: keeps the fp32 staging buffer small
            pool[b] = (torch.randn(cap, hkv, d, device="cuda", generator=gen) * 0.5).bfloat16()
    q = (torch.randn(batch, hq, d, device="cuda", generator=gen) * 0.5).bfloat16()
    out = gqa_decode(q, k_pool, v_pool, torch.from_numpy(lens).cuda(), cap)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    order = np.argsort(lens)
    picked = sorted({int(order[0]), int(order[-1]), *(int(i) for i in order[4:60:8])})
    assert len(picked) >= 8
    keys = [bf16_bits(k_pool[b, :lens[b]]) for b in picked]
    values = [bf16_bits(v_pool[b, :lens[b]]) for b in picked]
    want = oracle.gqa_decode_batch(bf16_bits(q[picked]), keys, values, lens[picked], threads=8)
    got = bits_to_float(bf16_bits(out[picked]))
    want = bits_to_float(want)
    assert np.abs(got - want).max() <= 2e-2
    # the reference's relative form for rounded outputs (cached_attention_ops_test.cc:270-274)
    assert np.all(np.abs(got - want) <= 2e-4 + 8e-3 * np.abs(want))
    assert _capi.kernel_status() == 0


def test_delta_net_16384_prefill_then_256_steps():
    """Gated delta-net at the benchmark shape: batch 2, 16 heads, key and value width 128, 16384
    tokens through the chunked prefill from a zero state, then 256 single-token steps from the
    final state.  Two (sequence, head) units are followed through all 16640 tokens by the
    token-recurrent oracle (sequence_delta_net.cc:55-102): outputs within 2e-2 and the
    reference's relative form, fp32 state after the prefill and after the steps within 2e-2."""
    b, t, h, d, steps = 2, 16384, 16, 128, 256
    gen = torch.Generator(device="cuda").manual_seed(29)
    total = t + steps

    def unit(shape):
        return torch.nn.functional.normalize(torch.randn(*shape, device="cuda", generator=gen), dim=-1)

    q = unit((b, total, h, d)).bfloat16()
    k = unit((b, total, h, d)).bfloat16()
    v = torch.randn(b, total, h, d, device="cuda", generator=gen).bfloat16()
    g = torch.sigmoid(torch.randn(b, total, h, device="cuda", generator=gen) * 2 + 2)
    beta = torch.sigmoid(torch.randn(b, total, h, device="cuda", generator=gen))
    state = torch.zeros(b, h, d, d, device="cuda")
    out = torch.empty(b, total, h, d, dtype=torch.bfloat16, device="cuda")
    out[:, :t] = gdn_prefill(q[:, :t], k[:, :t], v[:, :t], g[:, :t].contiguous(), beta[:, :t].contiguous(),
                             state, chunked=True)
    after_prefill = state.clone()
    for i in range(t, total):
        out[:, i] = gdn_step(q[:, i].contiguous(), k[:, i].contiguous(), v[:, i].contiguous(),
                             g[:, i].contiguous(), beta[:, i].contiguous(), state)
    torch.cuda.synchronize()
    assert _capi.kernel_status() == 0
    assert torch.isfinite(out.float()).all() and torch.isfinite(state).all()
    for (bi, hi) in ((0, 3), (1, 12)):
        one = lambda x: bf16_bits(x[bi:bi + 1, :, hi:hi + 1])
        gs = g[bi:bi + 1, :, hi:hi + 1].cpu().numpy()
        bs = beta[bi:bi + 1, :, hi:hi + 1].cpu().numpy()
        ref_state = np.zeros((1, 1, d, d), np.float32)
        qi, ki, vi = one(q), one(k), one(v)
        head = lambda x, lo, hi_: np.ascontiguousarray(x[:, lo:hi_])
        want_pre = oracle.gdn_recurrence(head(qi, 0, t), head(ki, 0, t), head(vi, 0, t), head(gs, 0, t),
                                         head(bs, 0, t), ref_state, True, 1.0, True)
        state_error = np.abs(after_prefill[bi, hi].cpu().numpy() - ref_state[0, 0]).max()
        assert state_error <= 2e-2, ("state after prefill", bi, hi, state_error)
        want_steps = oracle.gdn_recurrence(head(qi, t, total), head(ki, t, total), head(vi, t, total),
                                           head(gs, t, total), head(bs, t, total), ref_state, True, 1.0, True)
        want = bits_to_float(np.concatenate([want_pre, want_steps], axis=1))[0, :, 0]
        got = bits_to_float(bf16_bits(out[bi, :, hi]))
        error = np.abs(got - want)
        assert error.max() <= 2e-2, (bi, hi, int(error.max(1).argmax()), error.max())
        # sequence_delta_net_test.cc:241-297 form, plus two bf16 ulps of the largest output for the
        # chunked path's bf16 operands
        assert np.all(error <= 1.5e-4 + 0.015 * np.abs(want) + 2.0 ** -7 * np.abs(want).max())
        state_error = np.abs(state[bi, hi].cpu().numpy() - ref_state[0, 0]).max()
        assert state_error <= 2e-2, ("state after the steps", bi, hi, state_error)


def test_delta_net_pieces_with_a_ragged_tail():
    """A sequence long enough that the prefill runs as overlapping pieces (prepare of one piece
    beside the scan of the one before, on two streams) whose last piece is short and ends in an
    odd chunk count and a partial chunk: 9001 tokens = 140 chunks + 41 tokens, from a non-zero
    state, called twice back to back on the same workspace.  One (sequence, head) unit against the
    token-recurrent oracle, and the second call's output identical to the first's."""
    b, t, h, d = 2, 9001, 16, 128
    gen = torch.Generator(device="cuda").manual_seed(31)

    def unit(shape):
        return torch.nn.functional.normalize(torch.randn(*shape, device="cuda", generator=gen), dim=-1)

    q, k = unit((b, t, h, d)).bfloat16(), unit((b, t, h, d)).bfloat16()
    v = torch.randn(b, t, h, d, device="cuda", generator=gen).bfloat16()
    g = torch.sigmoid(torch.randn(b, t, h, device="cuda", generator=gen) * 2 + 2)
    beta = torch.sigmoid(torch.randn(b, t, h, device="cuda", generator=gen))
    start = torch.randn(b, h, d, d, device="cuda", generator=gen) * 0.1
    state, again = start.clone(), start.clone()
    out = gdn_prefill(q, k, v, g, beta, state, chunked=True)
    out_again = gdn_prefill(q, k, v, g, beta, again, chunked=True)
    torch.cuda.synchronize()
    assert _capi.kernel_status() == 0
    assert torch.equal(out, out_again) and torch.equal(state, again)
    bi, hi = 1, 5
    one = lambda x: bf16_bits(x[bi:bi + 1, :, hi:hi + 1])
    ref_state = start[bi:bi + 1, hi:hi + 1].cpu().numpy().copy()
    want = oracle.gdn_recurrence(one(q), one(k), one(v), g[bi:bi + 1, :, hi:hi + 1].cpu().numpy(),
                                 beta[bi:bi + 1, :, hi:hi + 1].cpu().numpy(), ref_state, True, 1.0, True)
    want = bits_to_float(want)[0, :, 0]
    got = bits_to_float(bf16_bits(out[bi, :, hi]))
    error = np.abs(got - want)
    assert error.max() <= 2e-2, (int(error.max(1).argmax()), error.max())
    assert np.abs(state[bi, hi].cpu().numpy() - ref_state[0, 0]).max() <= 2e-2
