"""Headline benchmark: Qwen-style grouped-query causal attention prefill on B200.

One "step" is one pass of the attention hot path over the prefill workload (batch 1, 40 query
heads / 8 KV heads, head width 128, prompt 8192, bf16, causal): 4 * D * S(S+1)/2 * Hq =
687.28 GFLOP per step.  With N GPUs the KV heads (and the query heads that read them) are split
across ranks with no communication; `value` is whole-job TFLOP/s = total FLOP / max-over-ranks
device time.

    python bench.py [--gpus N] [--steps K] [--warmup W]          our CUDA engine
    python bench.py --impl reference [...]                       the reference's CPU layer

The JSON line also carries: `roofline` for the dominant kernel (tensor-core bound), `e2e` (the
same metric through the public API from pinned host buffers, copies inside the timed region)
with `e2e_copy_floor_ms` (the same chunked copies with no kernels) beside it, `parity_max_abs`
(sampled rows of this run's own output against the CPU oracle, outside the timed region),
`clocks` sampled during the timed region, and at every N the other half of the metric:
`decode` (batch-64 GQA decode sharded by KV head, KV GB/s against the HBM roofline), `gdn` (gated
delta-net sharded by head: chunked prefill, single steps, a fused 256-token launch) and
`allgather_ms` (the optional NCCL gather of the head-sharded outputs, reported separately).  At
N = 1 it adds `sustained` (seconds of back-to-back headline launches with sampled clocks),
`cpu_baseline` (the reference's own CPU attention layer timed on a bounded sample on the host
cores) and `other_workloads` (training forward/backward, projections).
Inputs are seeded synthetic tensors with the configuration's shapes and distributions.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEQ, Q_HEADS, KV_HEADS, HEAD_DIM = 8192, 40, 8, 128
PAIRS = SEQ * (SEQ + 1) // 2
FLOP_PER_STEP = 4.0 * HEAD_DIM * PAIRS * Q_HEADS          # 687.28 GFLOP
WORKLOAD = ("Qwen-style GQA causal prefill, bf16: batch 1, 40 query heads / 8 KV heads, "
            "head_dim 128, prompt 8192")
SEED = 20240611


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            peaks = json.load(fh)
        return {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                "bf16_tflops_sustained": peaks.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.file = None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.device_index)], stdout=self.file,
                stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if self.file is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.file.flush()
        rows = []
        with open(self.file.name) as fh:
            for line in fh:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 9 and parts[1].replace(".", "").isdigit():
                    rows.append(parts)
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        clocks = sorted(float(r[1]) for r in rows)
        busy = [c for c in clocks if c >= 0.5 * clocks[-1]] or clocks
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[5 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": float(rows[0][2]),
                "power_w_max": max(float(r[3]) for r in rows if r[3].replace(".", "").isdigit()),
                "samples": len(rows), "reasons": reasons}


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own AttentionLayerReference on the host cores
# --------------------------------------------------------------------------------------------
def cpu_reference_sample(context: int, heads: int, threads: int):
    """Runs the reference CPU layer (oracle/_ref when built, else the C port) on a bounded sample
    of the prefill workload: `heads` query heads (each expanded with its KV head into an
    independent single-head sequence, as the layer has no grouped heads), first `context` prompt
    tokens.  Returns (seconds, flop, kind)."""
    import numpy as np

    import oracle
    rng = np.random.default_rng(SEED)
    q = oracle.to_bf16_bits(rng.standard_normal((context, heads, HEAD_DIM), dtype=np.float32) * 0.5)
    kv_heads = max(1, heads // (Q_HEADS // KV_HEADS))
    k = oracle.to_bf16_bits(rng.standard_normal((context, kv_heads, HEAD_DIM), dtype=np.float32) * 0.5)
    v = oracle.to_bf16_bits(rng.standard_normal((context, kv_heads, HEAD_DIM), dtype=np.float32) * 0.5)
    packed = np.empty((heads, context, 3 * HEAD_DIM), np.uint16)
    for h in range(heads):
        kv = min(h // (Q_HEADS // KV_HEADS), kv_heads - 1)
        packed[h, :, :HEAD_DIM] = q[:, h]
        packed[h, :, HEAD_DIM:2 * HEAD_DIM] = k[:, kv]
        packed[h, :, 2 * HEAD_DIM:] = v[:, kv]
    packed = packed.reshape(heads * context, 3 * HEAD_DIM)
    kind = "reference" if oracle.have_ref() else "port"
    start = time.perf_counter()
    oracle.attention_fwd(packed, context, 1, HEAD_DIM, True, threads=threads,
                         use_ref=(kind == "reference"))
    seconds = time.perf_counter() - start
    flop = heads * 4.0 * HEAD_DIM * (context * (context + 1) // 2)
    return seconds, flop, kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    heads = min(Q_HEADS, cores)
    context = 1024
    times, flop, kind = [], 0.0, "port"
    for i in range(args.warmup + args.steps):
        seconds, flop, kind = cpu_reference_sample(context, heads, cores)
        if i >= args.warmup:
            times.append(seconds)
    per_step = sum(times) / len(times)
    value = flop / per_step / 1e12
    sample = (f"{heads} of {Q_HEADS} query heads x first {context} of {SEQ} prompt tokens per step "
              f"({flop / 1e9:.2f} GFLOP), one single-head instance of the CPU layer per thread")
    line = {
        "impl": "reference", "metric": "attn_prefill_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "seed": SEED, "timed": "bounded sample per step: " + sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
class Ranks:
    """The process group as the timed legs need it: barriers and max-over-ranks device times."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB L2

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, warmup, flush=True, hold=True):
        """Mean device time per step in ms: CUDA events around each step, L2 flushed between
        steps (outside the events), barrier + synchronize either side, max over ranks.

        With `hold` the stream is first occupied by a sleep kernel while the host enqueues the
        steps, so the events bracket device work only: a step of two short launches is otherwise
        stretched by whatever the host needs between them (measured: 99 against 104 us on an idle
        host, far more with eight ranks sharing its cores).  Calls that synchronise inside
        (the end-to-end leg) or meet other ranks (the gather) are timed without it."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        self.barrier()
        sleep = getattr(torch.cuda, "_sleep", None)
        if hold and sleep is not None:
            sleep(min(steps * 400_000, 400_000_000))   # ~0.2 ms of device time per step
        for i in range(steps):
            if flush:
                self.flush.fill_(i & 0xFF)
            starts[i].record()
            fn()
            stops[i].record()
        self.barrier()
        total = sum(s.elapsed_time(e) for s, e in zip(starts, stops))
        return self.max_over_ranks(total) / steps

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def prefill_parity(out, q, k, v, count=24):
    """max |engine - oracle| over `count` sampled query rows (all heads of this rank) of the
    step's own output; the oracle runs outside every timed region."""
    import numpy as np

    import oracle
    seq = out.shape[1]
    rows = sorted({0, 127, 128, 255, 256, seq // 2 - 1, seq // 2, seq - 129, seq - 128, seq - 1,
                   *(int(r) for r in np.random.default_rng(SEED).integers(0, seq, size=count))})
    import torch
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.gqa_prefill_rows(bits(q[0]), bits(k[0]), bits(v[0]), rows, threads=os.cpu_count() or 1)
    got = bits(out[0][rows])
    return float(np.abs(oracle.from_bf16_bits(got) - oracle.from_bf16_bits(want)).max()), len(rows)


def copy_floor_ms(ranks, q_host, k_host, v_host, out_host, steps=5):
    """The end-to-end call's transfers with no kernels: the same token chunks (pluto_b200/csrc/
    host_pipeline.cu: 1024 tokens, grown to 4 MB of input, tapering at the end), input copies on
    one stream and output copies on another, so both PCIe directions are busy as in the real
    call.  What the link delivers is the floor of `e2e`."""
    torch = ranks.torch
    seq = q_host.shape[1]
    token_bytes = (q_host.shape[2] + 2 * k_host.shape[2]) * HEAD_DIM * 2
    full = max(1, ((4 << 20) // token_bytes + 1023) // 1024) * 1024
    chunks, t0 = [], 0
    while t0 < seq:
        left = seq - t0
        count = min(left, full if left > 2 * full else (full // 2 if left > full else full // 4))
        chunks.append((t0, count))
        t0 += count
    q_dev, k_dev, v_dev = (torch.empty_like(t, device="cuda") for t in (q_host, k_host, v_host))
    out_dev = torch.zeros_like(out_host, device="cuda")
    h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()

    def step():
        main = torch.cuda.current_stream()
        h2d.wait_stream(main)
        d2h.wait_stream(main)
        for (t0, count) in chunks:
            with torch.cuda.stream(h2d):
                for dev, host in ((k_dev, k_host), (v_dev, v_host), (q_dev, q_host)):
                    dev[:, t0:t0 + count].copy_(host[:, t0:t0 + count], non_blocking=True)
            d2h.wait_stream(h2d)
            with torch.cuda.stream(d2h):
                out_host[:, t0:t0 + count].copy_(out_dev[:, t0:t0 + count], non_blocking=True)
        main.wait_stream(d2h)

    return ranks.timed(step, steps, 2, hold=False)


def decode_leg(ranks, peaks, steps=20, batch=64, capacity=32768):
    """BASELINE config 4: one query token per sequence, 40/8 heads, head width 128, bf16 cache,
    cached lengths U[4096, 32768] from the seed, sharded by KV head (rank r holds KV heads
    [r*8/N, (r+1)*8/N) of every sequence and their query heads).  One step = one pluto_gqa_decode
    call (chunk kernel + merge kernel).  KV GB/s = algorithmic bytes of all ranks / max-over-ranks
    device time; the roofline fraction is one GPU's share against the measured HBM copy peak."""
    import numpy as np
    torch = ranks.torch

    import oracle
    from pluto_b200.layers import gqa_decode
    from pluto_b200.sharding import shard_heads

    shard = shard_heads(Q_HEADS, KV_HEADS, ranks.world, ranks.rank)
    lens = np.random.default_rng(SEED).integers(4096, capacity + 1, size=batch).astype(np.int32)
    gen = torch.Generator(device="cuda").manual_seed(SEED + 101 * ranks.rank)
    k_pool = torch.empty((batch, capacity, shard.kv_heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.empty_like(k_pool)
    for pool in (k_pool, v_pool):
        for b in range(batch):
            pool[b] = (torch.randn(capacity, shard.kv_heads, HEAD_DIM, device="cuda", generator=gen) * 0.5).bfloat16()
    q = (torch.randn(batch, shard.q_heads, HEAD_DIM, device="cuda", generator=gen) * 0.5).bfloat16()
    tl = torch.from_numpy(lens).cuda()
    out = torch.empty_like(q)
    ms = ranks.timed(lambda: gqa_decode(q, k_pool, v_pool, tl, capacity, out=out), steps, 3)
    per_rank_bytes = 512.0 * shard.kv_heads * float(lens.sum()) + 2 * q.numel() * 2
    total_bytes = 512.0 * KV_HEADS * float(lens.sum()) + 2 * batch * Q_HEADS * HEAD_DIM * 2
    # parity: every head of this rank for the shortest and the median sequence
    order = np.argsort(lens)
    picked = [int(order[0]), int(order[batch // 2])]
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.gqa_decode_batch(bits(q[picked]), [bits(k_pool[b, :lens[b]]) for b in picked],
                                   [bits(v_pool[b, :lens[b]]) for b in picked], lens[picked],
                                   threads=os.cpu_count() or 1)
    parity = float(np.abs(oracle.from_bf16_bits(bits(out[picked])) - oracle.from_bf16_bits(want)).max())
    parity = ranks.max_over_ranks(parity)
    per_gpu = per_rank_bytes / (ms * 1e-3) / 1e9
    result = {
        "workload": f"batch {batch}, 40/8 heads, head_dim 128, cached lengths U[4096,32768], bf16 cache, "
                    f"{shard.kv_heads} KV head(s) per GPU",
        "ms": ms, "kv_gbs": total_bytes / (ms * 1e-3) / 1e9, "kv_gbs_per_gpu": per_gpu,
        "sum_lengths": int(lens.sum()), "algorithmic_bytes": total_bytes,
        "algorithmic_bytes_per_gpu": per_rank_bytes, "steps": steps, "gpu_launches": 2 * steps,
        "parity_max_abs": parity, "parity_sample": "all heads of the shortest and the median sequence",
        "roofline": {"bound": "hbm", "kernel": "gqa_decode_tc<128> + gqa_decode_merge", "achieved": per_gpu,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
                     "frac_of_nominal_8TBs": per_gpu / 8000.0, "peak_source": peaks["source"] + " (copy)"}}
    return result, out


def gdn_leg(ranks, peaks, batch=2, tokens=16384, heads=16, dim=128):
    """BASELINE config 5 sharded by head: chunked prefill from a zero state, then single-token
    steps from the final state (256 of them replayed as one CUDA graph: the device cost without
    the per-call host cost), and the same 256 tokens as ONE launch of the token-sequential kernel
    (state on chip for all of them)."""
    import numpy as np
    torch = ranks.torch

    import oracle
    from pluto_b200.layers import gdn_prefill, gdn_step

    local = heads // ranks.world
    gen = torch.Generator(device="cuda").manual_seed(SEED + 7 * ranks.rank)
    total = tokens + 256
    unit = lambda: torch.nn.functional.normalize(torch.randn(batch, total, local, dim, device="cuda", generator=gen), dim=-1).bfloat16()
    q, k = unit(), unit()
    v = torch.randn(batch, total, local, dim, device="cuda", generator=gen).bfloat16()
    g = torch.sigmoid(torch.randn(batch, total, local, device="cuda", generator=gen) * 2 + 2)
    beta = torch.sigmoid(torch.randn(batch, total, local, device="cuda", generator=gen))
    qp, kp, vp = (t[:, :tokens].contiguous() for t in (q, k, v))
    gp, bp = g[:, :tokens].contiguous(), beta[:, :tokens].contiguous()
    state = torch.zeros(batch, local, dim, dim, device="cuda")
    out = torch.empty_like(vp)

    def prefill():
        state.zero_()
        gdn_prefill(qp, kp, vp, gp, bp, state, out=out)

    prefill_ms = ranks.timed(prefill, 5, 2)
    final = state.clone()
    # parity: one (sequence, head) unit of this rank over its first 2048 tokens
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    n = 2048
    ref_state = np.zeros((1, 1, dim, dim), np.float32)
    want = oracle.gdn_recurrence(bits(qp[1:2, :n, :1]), bits(kp[1:2, :n, :1]), bits(vp[1:2, :n, :1]),
                                 gp[1:2, :n, :1].cpu().numpy(), bp[1:2, :n, :1].cpu().numpy(), ref_state,
                                 True, 1.0, True)
    parity = float(np.abs(oracle.from_bf16_bits(bits(out[1:2, :n, :1])) - oracle.from_bf16_bits(want)).max())
    parity = ranks.max_over_ranks(parity)

    # single steps: 256 fresh tokens from the final state, replayed as one CUDA graph
    steps_in = [tuple(t[:, tokens + i].contiguous() for t in (q, k, v, g, beta)) for i in range(256)]
    o1 = torch.empty_like(v[:, 0])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        gdn_step(*steps_in[0], state, out=o1)
        with torch.cuda.graph(graph, stream=side):
            for item in steps_in:
                gdn_step(*item, state, out=o1)
    torch.cuda.current_stream().wait_stream(side)
    graph_ms = ranks.timed(graph.replay, 5, 2, flush=False)
    # the same 256 tokens as one launch (token-sequential kernel, state held on chip throughout)
    qs, ks, vs = (t[:, tokens:].contiguous() for t in (q, k, v))
    gs, bs = g[:, tokens:].contiguous(), beta[:, tokens:].contiguous()
    fused_out = torch.empty_like(vs)

    def fused():
        state.copy_(final)
        gdn_prefill(qs, ks, vs, gs, bs, state, out=fused_out, chunked=False)

    fused_ms = ranks.timed(fused, 5, 2, flush=False)
    state_bytes = 2.0 * batch * local * dim * dim * 4
    flop = 94.49e9 * (batch * local * tokens) / (2 * 16 * 16384)
    tflops = flop / (prefill_ms * 1e-3) / 1e12
    return {
        "workload": f"batch {batch}, {local} of {heads} heads per GPU, d_k = d_v = {dim}, {tokens}-token chunked "
                    "prefill from a zero state, then 256 single-token steps",
        "prefill_ms": prefill_ms, "prefill_tflops_chunked_count": tflops * ranks.world,
        "prefill_tflops_per_gpu": tflops,
        "prefill_roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": tflops / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                             "note": "dense chunked count (11.53 MFLOP per chunk and head); the kernels are bound "
                                     "by latency inside the chunk-parallel prepare CTA and by the chain of "
                                     "dependent chunk steps, not by the tensor pipe"},
        # the memory view: q, k, v in and the output out are the algorithmic bytes; the chunk records
        # (91136 B per chunk and head, written by the prepare kernel and read by the scan) are traffic
        # of this design
        "prefill_hbm": {"algorithmic_bytes_per_gpu": 4 * batch * tokens * local * dim * 2,
                        "algorithmic_gbs": 4 * batch * tokens * local * dim * 2 / (prefill_ms * 1e-3) / 1e9,
                        "with_records_bytes_per_gpu": (4 * batch * tokens * local * dim * 2 +
                                                       2 * batch * local * ((tokens + 63) // 64) * 91136),
                        "with_records_gbs": (4 * batch * tokens * local * dim * 2 +
                                             2 * batch * local * ((tokens + 63) // 64) * 91136) /
                                            (prefill_ms * 1e-3) / 1e9,
                        "frac_of_measured_hbm": (4 * batch * tokens * local * dim * 2 +
                                                 2 * batch * local * ((tokens + 63) // 64) * 91136) /
                                                (prefill_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
        "step_in_cuda_graph_us": graph_ms * 1e3 / 256,
        "step_state_gbs_per_gpu": state_bytes / (graph_ms * 1e-3 / 256) / 1e9,
        "fused_256_step_launch_us": fused_ms * 1e3, "fused_us_per_token": fused_ms * 1e3 / 256,
        "fused_note": "one launch, state read and written once: not bound by per-step state traffic",
        "parity_max_abs": parity, "parity_sample": "one (sequence, head) unit per rank, first 2048 prefill tokens",
    }


def allgather_leg(ranks, prefill_out, decode_out):
    """The optional gather of the head-sharded outputs into the [rows, E] layout (outside `value`):
    ncclAllGather over NVLink + local interleave through the C entry point pluto_allgather_heads,
    for the headline's 84 MB output and the decode step's 0.66 MB output."""
    torch = ranks.torch
    from pluto_b200.sharding import NcclCommunicator, allgather_heads
    comm = NcclCommunicator()
    result = {}
    for name, local in (("prefill_out", prefill_out.reshape(SEQ, -1)), ("decode_out", decode_out.reshape(decode_out.shape[0], -1))):
        rows, cols = local.shape
        scratch = torch.empty((ranks.world * rows, cols), dtype=local.dtype, device="cuda")
        full = torch.empty((rows, ranks.world * cols), dtype=local.dtype, device="cuda")
        ms = ranks.timed(lambda: allgather_heads(local, comm=comm, out=full, scratch=scratch), 10, 3, hold=False)
        # check: this rank's own columns come back where they belong
        mine = full[:, ranks.rank * cols:(ranks.rank + 1) * cols]
        if not torch.equal(mine, local):
            raise SystemExit("all-gather returned this rank's heads in the wrong place")
        result[name] = {"ms": ms, "bytes_gathered": rows * cols * ranks.world * local.element_size()}
    comm.close()
    return result


def sustained_leg(ranks, step, peaks, seconds=2.5):
    """Back-to-back headline launches for a few seconds (no L2 flush, no pauses) with the clocks
    sampled: the regime of a long job under the power cap, against the sustained cuBLAS figure."""
    torch = ranks.torch
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    with ClockSampler(ranks.local_rank) as sampler:
        begin = time.perf_counter()
        a.record()
        while time.perf_counter() - begin < seconds:
            for _ in range(50):
                step()
            launches += 50
            torch.cuda.synchronize()
        b.record()
        torch.cuda.synchronize()
    clocks = sampler.summary()
    ms = a.elapsed_time(b) / launches
    tflops = FLOP_PER_STEP / (ms * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
    return {"seconds": a.elapsed_time(b) / 1e3, "launches": launches, "ms_per_step": ms, "tflops": tflops,
            "sm_mhz_median": clocks.get("sm_mhz"), "ms_times_mhz": ms * (clocks.get("sm_mhz") or 0.0),
            "power_w_max": clocks.get("power_w_max"), "reasons": clocks.get("reasons"),
            "frac_of_sustained_peak": tflops / peak, "sustained_peak": peak}


def run_engine(args):
    import numpy as np
    import torch

    from pluto_b200 import _capi
    from pluto_b200.layers import gqa_prefill, gqa_prefill_host
    from pluto_b200.sharding import shard_heads

    if int(os.environ.get("WORLD_SIZE", "1")) == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    ranks = Ranks()
    world, rank = ranks.world, ranks.rank
    _capi.lib()
    shard = shard_heads(Q_HEADS, KV_HEADS, world, rank)

    # Seeded inputs, identical for every GPU count: generate the full tensors, keep this rank's heads.
    gen = torch.Generator(device="cpu").manual_seed(SEED)
    q_host = (torch.randn(1, SEQ, Q_HEADS, HEAD_DIM, generator=gen) * 0.5).bfloat16()
    k_host = (torch.randn(1, SEQ, KV_HEADS, HEAD_DIM, generator=gen) * 0.5).bfloat16()
    v_host = (torch.randn(1, SEQ, KV_HEADS, HEAD_DIM, generator=gen) * 0.5).bfloat16()
    q_host = q_host[:, :, shard.q_begin:shard.q_end].contiguous().pin_memory()
    k_host = k_host[:, :, shard.kv_begin:shard.kv_end].contiguous().pin_memory()
    v_host = v_host[:, :, shard.kv_begin:shard.kv_end].contiguous().pin_memory()
    q, k, v = q_host.cuda(), k_host.cuda(), v_host.cuda()
    out_host = torch.empty((1, SEQ, shard.q_heads, HEAD_DIM), dtype=torch.bfloat16).pin_memory()

    step_state = {"workspace": None, "out": None}

    def step():
        # (with few heads per GPU the kernel cuts the key range of every query-tile pair into parts
        # and needs scratch for the partials; it is allocated once and handed back in)
        result = gqa_prefill(q, k, v, workspace=step_state["workspace"])
        step_state["workspace"] = result.get("workspace")
        step_state["out"] = result["out"]

    e2e_state = {"workspace": None}

    def e2e_step():
        # host-resident activations in, host-resident result out: the prompt goes in by chunks of
        # 1024 tokens (contiguous copies); a chunk's copy in, its kernel (its queries against all
        # keys copied so far) and its copy out overlap those of its neighbours
        e2e_state["workspace"] = gqa_prefill_host(q_host, k_host, v_host, out_host,
                                                  kv_heads_per_group=0,
                                                  workspace=e2e_state["workspace"])

    with ClockSampler(ranks.local_rank) as sampler:
        time.sleep(0.3)  # let the sampler take its first readings before the timed region
        ms = ranks.timed(step, args.steps, max(args.warmup, 3))
        e2e_ms = ranks.timed(e2e_step, max(3, min(args.steps, 10)), 3, hold=False)
    clocks = sampler.summary()
    status = _capi.kernel_status()
    if status != 0:
        raise SystemExit(f"kernel status word = {status:#x}")

    # parity of what was just timed (outside the timed region): sampled rows of the device-resident
    # step's output and of the end-to-end call's host output, against the CPU oracle
    parity, parity_rows = prefill_parity(step_state["out"], q, k, v)
    e2e_parity, _ = prefill_parity(out_host.cuda(), q, k, v)
    parity = ranks.max_over_ranks(max(parity, e2e_parity))

    peaks = measured_peaks()
    floor_ms = copy_floor_ms(ranks, q_host, k_host, v_host, out_host)
    extras = {}
    if not args.no_extras:
        decode, decode_out = decode_leg(ranks, peaks)
        extras["decode"] = decode
        torch.cuda.empty_cache()
        extras["gdn"] = gdn_leg(ranks, peaks)
        torch.cuda.empty_cache()
        if world > 1:
            extras["allgather_ms"] = allgather_leg(ranks, step_state["out"], decode_out)
        status = _capi.kernel_status()
        if status != 0:
            raise SystemExit(f"kernel status word = {status:#x}")

    value = FLOP_PER_STEP / (ms * 1e-3) / 1e12
    elements = 2  # bf16
    h2d = (q_host.numel() + k_host.numel() + v_host.numel()) * elements
    d2h = out_host.numel() * elements
    line = {
        "metric": "attn_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "seed": SEED, "batch": 1, "seq_len": SEQ,
                   "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
                   "parallelism": f"kv-head shard x{world} (no collective)",
                   "l2": "256 MiB buffer written between timed steps",
                   "timing": "CUDA events around each step; a sleep kernel holds the stream while the host "
                             "enqueues the steps, so host launch gaps are outside the events (not for e2e)",
                   "flop_per_step": FLOP_PER_STEP},
        "e2e": {"value": FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "pluto_b200.layers.gqa_prefill_host (pluto_gqa_prefill_fwd_host): pinned host buffers in and out, copies and kernels pipelined per chunk of 1024 prompt tokens"},
        "e2e_copy_floor_ms": floor_ms,
        "parity_max_abs": parity,
        "parity_sample": f"{parity_rows} query rows x all heads of every rank, device-resident and end-to-end outputs",
        # one attention kernel per step, plus the merge kernel when the key/value split is active
        "gpu_launches": args.steps * (2 if step_state["workspace"] is not None else 1),
        "clocks": clocks,
    }
    line.update(extras)
    if rank == 0:
        # roofline of the one kernel in the step: bf16 tensor-core bound, timed as isolated launches
        # with an L2 flush between them, hence against the burst figure
        per_rank_flop = FLOP_PER_STEP / world
        achieved = per_rank_flop / (ms * 1e-3) / 1e12
        # which kernel the launch plan picks: cut tile pairs + merge when a workspace is in use, whole
        # pairs from two pairs per SM on, single tiles below that
        pairs_per_sm = shard.q_heads * (SEQ // 256) / 148.0
        kernel = ("attn_fwd_sm100_pair<128> + attn_fwd_merge<128>" if step_state["workspace"] is not None
                  else "attn_fwd_sm100_pair<128>" if pairs_per_sm >= 2 else "attn_fwd_sm100<128>")
        line["roofline"] = {
            "bound": "tensor",
            "kernel": kernel,
            "achieved": achieved,
            "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
            "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
            "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
            "algorithmic_flop_per_launch": per_rank_flop,
        }
        if world == 1 and not args.no_extras:
            # (the seconds-long leg last: it leaves the GPU hot and power-capped, which would colour the
            # burst-timed secondary figures)
            line["other_workloads"] = other_workloads(peaks, skip=("decode", "gdn"))
            line["sustained"] = sustained_leg(ranks, step, peaks)
            cores = os.cpu_count() or 1
            heads = min(Q_HEADS, cores)
            seconds, flop, kind = cpu_reference_sample(4096, heads, cores)
            line["cpu_baseline"] = {
                "value": flop / seconds / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                "seconds": seconds,
                "sample": f"{heads} of {Q_HEADS} query heads x first 4096 of {SEQ} prompt tokens "
                          f"({flop / 1e9:.2f} GFLOP), one single-head CPU-layer instance per thread"}
        print(json.dumps(line))
    ranks.close()


# dram__bytes_read.sum + dram__bytes_write.sum of one attn_fwd_sm100_pair<128> launch on this
# workload, from the ncu captures summarised in profiles/attn_fwd_sm100_pair_d128_gqa_prefill_8192.md
# (117.5 + 47 MB in the first, 117.7 + 49.8 MB in the latest: part of the output is still in L2 when
# the launch ends).
TRAFFIC_BYTES_PER_LAUNCH = 167.5e6


def other_workloads(peaks, only=None, decode_batch=64, steps_scale=1.0, skip=()):
    """Secondary figures of the same run (one GPU): decode against the HBM roofline, the GPT-2
    training forward/backward, and the delta-net prefill + step.  `only` restricts the run to one
    of them (used by --profile-case, with a smaller decode batch so an ncu capture stays small)."""
    import numpy as np
    import torch

    from pluto_b200.layers import AttentionLayer, DataType, gdn_prefill, gdn_step, gqa_decode

    def time_ms(fn, steps=10, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    result = {}
    if only not in (None, "decode"):
        return _other_rest(peaks, only, time_ms, skip)
    if "decode" in skip:
        return _other_rest(peaks, only, time_ms, skip)
    # decode: batch 64, L ~ U[4096, 32768]; cache 8.6 GB >> L2
    rng = np.random.default_rng(SEED)
    batch, cap = decode_batch, 32768
    lens = rng.integers(4096, 32769, size=batch).astype(np.int32)
    k_pool = torch.empty((batch, cap, KV_HEADS, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.empty_like(k_pool)
    for t in (k_pool, v_pool):
        t.view(-1)[:].normal_(0, 0.5)
    qd = (torch.randn(batch, Q_HEADS, HEAD_DIM, device="cuda") * 0.5).bfloat16()
    tl = torch.from_numpy(lens).cuda()
    out = torch.empty_like(qd)
    ms = time_ms(lambda: gqa_decode(qd, k_pool, v_pool, tl, cap, out=out), steps=20)
    nbytes = 4096.0 * float(lens.sum()) + 2 * qd.numel() * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    result["gqa_decode"] = {
        "workload": f"batch {batch}, 40/8 heads, head_dim 128, cached lengths U[4096,32768], bf16 cache",
        "ms": ms, "kv_gbs": gbs, "sum_lengths": int(lens.sum()), "algorithmic_bytes": nbytes,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal_8TBs": gbs / 8000.0,
                     "peak_source": peaks["source"]}}
    del k_pool, v_pool
    if only == "decode":
        return result
    result.update(_other_rest(peaks, only, time_ms, skip))
    return result


def _other_rest(peaks, only, time_ms, skip=()):
    import torch

    from pluto_b200.layers import AttentionLayer, DataType, gdn_prefill, gdn_step

    result = {}
    if only == "gdn":
        return _gdn_workload(time_ms)
    if only == "gdn_bptt":
        return _gdn_bptt_only(time_ms)
    if only == "gdn_prefill":
        return _gdn_prefill_only(time_ms)
    if only == "gqa_bwd":
        return _gqa_bwd_workload(time_ms)
    if only == "linear":
        return _linear_workload(time_ms, peaks)
    if only == "dense":
        return _dense_workload(time_ms, peaks)
    # GPT-2 small training forward + backward, bf16
    b, h, s, d = 8, 12, 1024, 64
    e = h * d
    qkv = torch.randn(b * s, 3 * e, device="cuda").bfloat16()
    d_out = torch.randn(b * s, e, device="cuda")
    layer = AttentionLayer.Create(s, h, e, DataType.BF16)
    fwd_ms = time_ms(lambda: layer.fwd([qkv]), steps=20)
    state = layer.fwd([qkv]).state
    bwd_ms = time_ms(lambda: layer.bwd([d_out], state), steps=5)
    pairs = s * (s + 1) // 2
    result["mha_train_bf16"] = {
        "workload": "batch 8, 12 heads, seq 1024, head_dim 64, forward + backward",
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "fwd_tflops": 4.0 * d * pairs * b * h / (fwd_ms * 1e-3) / 1e12,
        "bwd_tflops": 10.0 * d * pairs * b * h / (bwd_ms * 1e-3) / 1e12}
    # BASELINE config 1 (the reference's CPU-runnable case): fp32 activations, exact fp32 kernels
    b1, h1, s1, d1 = 16, 6, 256, 64
    qkv1 = torch.randn(b1 * s1, 3 * h1 * d1, device="cuda")
    dout1 = torch.randn(b1 * s1, h1 * d1, device="cuda")
    layer1 = AttentionLayer.Create(s1, h1, h1 * d1, DataType.FP16)
    f1 = time_ms(lambda: layer1.fwd([qkv1]), steps=20)
    state1 = layer1.fwd([qkv1]).state
    g1 = time_ms(lambda: layer1.bwd([dout1], state1), steps=10)
    pairs1 = s1 * (s1 + 1) // 2
    result["mha_fp32_config1"] = {
        "workload": "batch 16, 6 heads, seq 256, head_dim 64, fp32 activations (exact fp32 FFMA kernels)",
        "fwd_ms": f1, "bwd_ms": g1,
        "fwd_tflops": 4.0 * d1 * pairs1 * b1 * h1 / (f1 * 1e-3) / 1e12,
        "bwd_tflops": 10.0 * d1 * pairs1 * b1 * h1 / (g1 * 1e-3) / 1e12}
    if only == "mha_train":
        return result
    result.update(_gqa_bwd_workload(time_ms))
    result.update(_linear_workload(time_ms, peaks))
    result.update(_dense_workload(time_ms, peaks))
    result.update(_gdn_workload(time_ms, bptt_only="gdn" in skip))
    return result


def _linear_workload(time_ms, peaks):
    """Imported projection of the Qwen decoder (hidden 5120 -> 2*40*128 query/gate columns), one
    token, bf16 and FP8 weights: a weight stream against the HBM roofline.  Calls rotate over
    enough distinct weight matrices (> 3x the 126 MB L2) that every call streams from HBM, as the
    layers of a decoder do."""
    import torch

    from pluto_b200.layers import FullyConnectedLayer, MatrixStorage

    cols, rows = 5120, 10240
    x = torch.randn(1, cols, device="cuda").bfloat16()
    out = {}
    for name, storage, elem in (("bf16", MatrixStorage.kBFloat16, 2), ("fp8_e4m3", MatrixStorage.kFp8E4M3, 1)):
        copies = (420 << 20) // (rows * cols * elem) + 1
        layers = []
        for _ in range(copies):
            if elem == 2:
                w, scales = (torch.randn(rows, cols, device="cuda") * 0.02).bfloat16(), None
            else:
                w = torch.randint(0, 120, (rows, cols), dtype=torch.uint8, device="cuda")
                scales = torch.full((rows // 128 * (cols // 128),), 0.01, device="cuda")
            layers.append(FullyConnectedLayer.Create(w, storage, cols, rows, scales))
        # the C entry point directly with a preallocated output: the kernel runs ~20 us, less
        # than the Python layer object spends per call
        from pluto_b200 import _capi
        L, stream = _capi.lib(), torch.cuda.current_stream().cuda_stream
        y = torch.empty(1, rows, dtype=torch.bfloat16, device="cuda")
        args = [(l.weights()[0].data_ptr(), l.weights()[1].data_ptr() if elem == 1 else None) for l in layers]
        state = {"i": 0}

        def call():
            w_ptr, s_ptr = args[state["i"] % copies]
            L.pluto_linear_imported_fwd(stream, w_ptr, storage.value, s_ptr, x.data_ptr(), y.data_ptr(),
                                        1, cols, rows)
            state["i"] += 1

        ms = time_ms(call, steps=4 * copies, warmup=copies)
        nbytes = rows * cols * elem + (0 if elem == 2 else rows // 128 * (cols // 128) * 4) + cols * 2 + rows * 2
        out[name] = {"ms": ms, "weight_gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    return {"imported_linear": {"workload": "one token, [10240 x 5120] frozen weights, calls rotate over "
                                            "> 420 MB of distinct matrices; back-to-back calls in one "
                                            "stream (programmatic dependent launch lets a call's weight "
                                            "copies start under the previous call's tail)", **out}}


def _dense_workload(time_ms, peaks):
    """Trainable dense projection (tcgen05 GEMMs incl. the operand casts): the GPT-2 QKV projection
    of 8192 tokens, and a square 8192 problem against the measured cuBLAS bf16 peak."""
    import torch

    from pluto_b200.layers import DataType, DenseLayer

    out = {}
    for name, (rows, i, o) in (("gpt2_qkv_8192x768x2304", (8192, 768, 2304)), ("square_8192", (8192, 8192, 8192))):
        layer = DenseLayer.Create(i, o, DataType.BF16)
        layer.InitializeNormal(0.02, 1)
        x = torch.randn(rows, i, device="cuda").bfloat16()
        dy = torch.randn(rows, o, device="cuda")
        fwd_ms = time_ms(lambda: layer.fwd([x]), steps=10)
        state = layer.fwd([x]).state
        bwd_ms = time_ms(lambda: layer.bwd([dy], state), steps=5)
        flop = 2.0 * rows * i * o
        out[name] = {"fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_tflops": flop / (fwd_ms * 1e-3) / 1e12,
                     "bwd_tflops": 2 * flop / (bwd_ms * 1e-3) / 1e12,
                     "fwd_frac_of_measured_bf16": flop / (fwd_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    return {"dense_projection": {"workload": "bf16 activations, fp32 master weights, casts included", **out}}


def _gqa_bwd_workload(time_ms):
    """Backward of the attention core at the headline prefill shape (gate pass + the two tcgen05
    passes of pluto_gqa_prefill_bwd); 10*D*S(S+1)/2 FLOP per query head."""
    import torch

    from pluto_b200 import _capi
    from pluto_b200.layers import gqa_prefill

    L = _capi.lib()
    t, hq, hkv, d = SEQ, Q_HEADS, KV_HEADS, HEAD_DIM
    q = (torch.randn(1, t, hq, d, device="cuda") * 0.5).bfloat16()
    k = (torch.randn(1, t, hkv, d, device="cuda") * 0.5).bfloat16()
    v = (torch.randn(1, t, hkv, d, device="cuda") * 0.5).bfloat16()
    gate = torch.randn(1, t, hq, d, device="cuda").bfloat16()
    fwd = gqa_prefill(q, k, v, gate=gate, want_core=True, want_stats=True)
    dy = torch.randn(t, hq, d, device="cuda")
    dc, dgate, dq = (torch.empty(t, hq, d, device="cuda") for _ in range(3))
    dk, dv = torch.empty(t, hkv, d, device="cuda"), torch.empty(t, hkv, d, device="cuda")
    deltas = torch.empty(hq * t, device="cuda")
    size = L.pluto_gqa_prefill_bwd_workspace_bytes(1, t, hq, d, 1)
    ws = torch.empty(size, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def bwd():
        _capi.check(L.pluto_gqa_gate_bwd(stream, gate.data_ptr(), hq * d, d, fwd["core"].data_ptr(),
                                         dy.data_ptr(), dc.data_ptr(), dgate.data_ptr(), hq * d, d,
                                         deltas.data_ptr(), 1, t, hq, d, 1))
        _capi.check(L.pluto_gqa_prefill_bwd(stream, q.data_ptr(), k.data_ptr(), v.data_ptr(), 1, hq * d, d,
                                            dc.data_ptr(), fwd["maxima"].data_ptr(),
                                            fwd["normalizers"].data_ptr(), deltas.data_ptr(),
                                            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), size,
                                            1, t, hq, hkv, d))

    ms = time_ms(bwd, steps=5, warmup=2)
    flop = 10.0 * d * (t * (t + 1) // 2) * hq
    return {"gqa_prefill_bwd": {
        "workload": "backward of the headline prefill shape: gate pass + attention core (tcgen05)",
        "ms": ms, "tflops": flop / (ms * 1e-3) / 1e12}}


def _gdn_prefill_only(time_ms):
    """The chunked delta-net prefill alone at the benchmark shape (the two tcgen05 kernels): the
    case the ncu captures of gdn_prepare_sm100 / gdn_scan_sm100 are taken on."""
    import torch

    from pluto_b200.layers import gdn_prefill
    bb, tt, hh, dd = 2, 16384, 16, 128
    qn = torch.nn.functional.normalize(torch.randn(bb, tt, hh, dd, device="cuda"), dim=-1).bfloat16()
    kn = torch.nn.functional.normalize(torch.randn(bb, tt, hh, dd, device="cuda"), dim=-1).bfloat16()
    vn = torch.randn(bb, tt, hh, dd, device="cuda").bfloat16()
    g = torch.sigmoid(torch.randn(bb, tt, hh, device="cuda") * 2 + 2)
    beta = torch.sigmoid(torch.randn(bb, tt, hh, device="cuda"))
    st = torch.zeros(bb, hh, dd, dd, device="cuda")
    og = torch.empty_like(vn)

    def prefill():
        gdn_prefill(qn, kn, vn, g, beta, st, out=og)

    ms = time_ms(prefill, steps=5, warmup=2)
    return {"gated_delta_net_prefill": {"workload": "batch 2, 16 heads, d_k = d_v = 128, seq 16384", "ms": ms,
                                        "tflops_chunked_count": 94.49e9 / (ms * 1e-3) / 1e12}}


def _gdn_workload(time_ms, bptt_only=False):
    import torch

    from pluto_b200 import _capi
    from pluto_b200.layers import gdn_prefill, gdn_step

    result = {}
    # gated delta-net prefill + single steps
    bb, tt, hh, dd = 2, 16384, 16, 128
    qn = torch.nn.functional.normalize(torch.randn(bb, tt, hh, dd, device="cuda"), dim=-1).bfloat16()
    kn = torch.nn.functional.normalize(torch.randn(bb, tt, hh, dd, device="cuda"), dim=-1).bfloat16()
    vn = torch.randn(bb, tt, hh, dd, device="cuda").bfloat16()
    g = torch.sigmoid(torch.randn(bb, tt, hh, device="cuda") * 2 + 2)
    beta = torch.sigmoid(torch.randn(bb, tt, hh, device="cuda"))
    st = torch.zeros(bb, hh, dd, dd, device="cuda")
    og = torch.empty_like(vn)

    def prefill():
        st.zero_()
        gdn_prefill(qn, kn, vn, g, beta, st, out=og)

    pre_ms = step_ms = graph_ms = None
    if not bptt_only:
        pre_ms, step_ms, graph_ms = _gdn_forward_times(time_ms, prefill, qn, kn, vn, g, beta, st)
    result.update(_gdn_bptt(time_ms, qn, kn, vn, bb, tt, hh, dd, pre_ms, step_ms, graph_ms))
    return result


def _gdn_bptt_only(time_ms):
    """The chunk-parallel delta-net BPTT alone on a quarter-size shape (batch 1, 8 heads, 4096 tokens:
    512 chunk CTAs, under 1 GB on the device): the case the ncu captures of gdn_scan_bwd_sm100 and
    gdn_bwd_chunk_local are taken on."""
    import torch
    bb, tt, hh, dd = 1, 4096, 8, 128
    qn = torch.nn.functional.normalize(torch.randn(bb, tt, hh, dd, device="cuda"), dim=-1).bfloat16()
    kn = torch.nn.functional.normalize(torch.randn(bb, tt, hh, dd, device="cuda"), dim=-1).bfloat16()
    vn = torch.randn(bb, tt, hh, dd, device="cuda").bfloat16()
    out = _gdn_bptt(time_ms, qn, kn, vn, bb, tt, hh, dd, None, None, None)
    out["gated_delta_net"]["workload"] = "batch 1, 8 heads, d_k = d_v = 128, seq 4096"
    del out["gated_delta_net"]["recurrence_bwd_tflops"]
    return out


def _gdn_forward_times(time_ms, prefill, qn, kn, vn, g, beta, st):
    import torch

    from pluto_b200.layers import gdn_step
    pre_ms = time_ms(prefill, steps=3, warmup=1)
    q1, k1, v1 = qn[:, 0].contiguous(), kn[:, 0].contiguous(), vn[:, 0].contiguous()
    g1, b1, o1 = g[:, 0].contiguous(), beta[:, 0].contiguous(), torch.empty_like(vn[:, 0])
    step_ms = time_ms(lambda: gdn_step(q1, k1, v1, g1, b1, st, out=o1), steps=256)
    # the same 256 steps as one CUDA graph: the entry point neither allocates nor synchronises,
    # so a serving loop can capture it, and the replay shows the device cost without the ~10 us
    # a Python call spends per launch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        gdn_step(q1, k1, v1, g1, b1, st, out=o1)
        with torch.cuda.graph(graph, stream=side):
            for _ in range(256):
                gdn_step(q1, k1, v1, g1, b1, st, out=o1)
    torch.cuda.current_stream().wait_stream(side)
    graph_ms = time_ms(graph.replay, steps=5, warmup=3) / 256
    return pre_ms, step_ms, graph_ms


def _gdn_bptt(time_ms, qn, kn, vn, bb, tt, hh, dd, pre_ms, step_ms, graph_ms):
    """BPTT through the recurrence at the benchmark shape (the chunk-parallel path: forward prefill
    with the state kept per chunk, reverse tcgen05 scan, one CTA per chunk), q/k normalisation
    included."""
    import torch

    from pluto_b200 import _capi
    result = {}
    L = _capi.lib()
    a_raw = torch.randn(bb, tt, hh, device="cuda").bfloat16()
    b_raw = torch.randn(bb, tt, hh, device="cuda").bfloat16()
    a_log = torch.full((hh,), -0.7, device="cuda")
    dt_bias = torch.zeros(hh, device="cuda")
    dcore = torch.randn(bb, tt, hh, dd, device="cuda")
    dq, dk2, dv2 = (torch.empty(bb, tt, hh, dd, device="cuda") for _ in range(3))
    da, db = torch.empty(bb, tt, hh, device="cuda"), torch.empty(bb, tt, hh, device="cuda")
    ws_bytes = L.pluto_gdn_recurrence_bwd_workspace_bytes(bb, tt, hh, hh, dd, dd)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def bptt():
        _capi.check(L.pluto_gdn_recurrence_bwd(
            stream, qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), 1, hh * dd, hh * dd,
            a_raw.data_ptr(), b_raw.data_ptr(), 1, a_log.data_ptr(), dt_bias.data_ptr(),
            dcore.data_ptr(), dq.data_ptr(), dk2.data_ptr(), hh * dd, dv2.data_ptr(), hh * dd,
            da.data_ptr(), db.data_ptr(), None, None, ws.data_ptr(), ws_bytes, bb, tt, hh, hh, dd, dd, 1))

    bptt_ms = time_ms(bptt, steps=3, warmup=2)
    entry = {"workload": "batch 2, 16 heads, d_k = d_v = 128, seq 16384",
             "recurrence_bwd_ms": bptt_ms, "recurrence_bwd_workspace_gb": ws_bytes / 1e9,
             "recurrence_bwd_note": "chunk-parallel: two tcgen05 scans + one CTA per 64-token chunk (about 215 GFLOP "
                                    "of products at fp32-level accuracy: mma.sync on bf16 high part + remainder "
                                    "for the long ones, fp32 FMAs for the short ones)",
             "recurrence_bwd_tflops": 215.0e9 / (bptt_ms * 1e-3) / 1e12}
    if pre_ms is not None:
        entry.update({
            "prefill_ms": pre_ms, "prefill_tflops_chunked_count": 94.49e9 / (pre_ms * 1e-3) / 1e12,
            "step_us": step_ms * 1e3, "step_state_gbs": 4.19e6 / (step_ms * 1e-3) / 1e9,
            "step_in_cuda_graph_us": graph_ms * 1e3,
            "step_in_cuda_graph_state_gbs": 4.19e6 / (graph_ms * 1e-3) / 1e9})
    result["gated_delta_net"] = entry
    return result


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["engine", "reference"], default="engine")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the secondary workloads and the CPU baseline (profiling runs)")
    parser.add_argument("--profile-case", choices=["decode", "mha_train", "gdn", "gdn_prefill", "gdn_bptt", "gqa_bwd", "linear", "dense"], default=None,
                        help="run only one secondary workload at a capture-friendly size and exit")
    args = parser.parse_args()
    if args.profile_case:
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(other_workloads(measured_peaks(), only=args.profile_case, decode_batch=8)))
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_engine(args)


if __name__ == "__main__":
    main()
