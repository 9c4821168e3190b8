"""Headline benchmark: Qwen-style grouped-query causal attention prefill on B200.

One "step" is one pass of the attention hot path over the prefill workload (batch 1, 40 query
heads / 8 KV heads, head width 128, prompt 8192, bf16, causal): 4 * D * S(S+1)/2 * Hq =
687.28 GFLOP per step.  With N GPUs the KV heads (and the query heads that read them) are split
across ranks with no communication; `value` is whole-job TFLOP/s = total FLOP / max-over-ranks
device time.

    python bench.py [--gpus N] [--steps K] [--warmup W]          our CUDA engine
    python bench.py --impl reference [...]                       the reference's CPU layer

The JSON line also carries: `roofline` for the dominant kernel (tensor-core bound), `e2e` (the
same metric through the public API from pinned host buffers, copies inside the timed region),
`cpu_baseline` (the reference's own CPU attention layer timed on a bounded sample on the host
cores), `clocks` sampled during the timed region, and `other_workloads` with the decode (HBM
roofline), training forward/backward and delta-net figures measured in the same run (N = 1 only).
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
def run_engine(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from pluto_b200 import _capi
    from pluto_b200.layers import gqa_prefill, gqa_prefill_host
    from pluto_b200.sharding import shard_heads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
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
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB L2
    out_host = torch.empty((1, SEQ, shard.q_heads, HEAD_DIM), dtype=torch.bfloat16).pin_memory()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step_state = {"workspace": None}

    def step():
        # (with few heads per GPU the kernel cuts the key range of every query-tile pair into parts
        # and needs scratch for the partials; it is allocated once and handed back in)
        result = gqa_prefill(q, k, v, workspace=step_state["workspace"])
        step_state["workspace"] = result.get("workspace")
        return result["out"]

    e2e_state = {"workspace": None}

    def e2e_step():
        # host-resident activations in, host-resident result out: the prompt goes in by chunks of
        # 1024 tokens (contiguous copies); a chunk's copy in, its kernel (its queries against all
        # keys copied so far) and its copy out overlap those of its neighbours
        e2e_state["workspace"] = gqa_prefill_host(q_host, k_host, v_host, out_host,
                                                  kv_heads_per_group=0,
                                                  workspace=e2e_state["workspace"])

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        barrier()
        for i in range(steps):
            flush.fill_(i & 0xFF)          # evict L2 between timed iterations (outside the events)
            starts[i].record()
            fn()
            stops[i].record()
        barrier()
        total = sum(s.elapsed_time(e) for s, e in zip(starts, stops))
        t = torch.tensor([total], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    with ClockSampler(local_rank) as sampler:
        time.sleep(0.3)  # let the sampler take its first readings before the timed region
        ms = timed(step, args.steps, max(args.warmup, 3))
        e2e_ms = timed(e2e_step, max(3, min(args.steps, 10)), 3)
    clocks = sampler.summary()
    status = _capi.kernel_status()
    if status != 0:
        raise SystemExit(f"kernel status word = {status:#x}")

    peaks = measured_peaks()
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
                   "flop_per_step": FLOP_PER_STEP},
        "e2e": {"value": FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "pluto_b200.layers.gqa_prefill_host (pluto_gqa_prefill_fwd_host): pinned host buffers in and out, copies and kernels pipelined per chunk of 1024 prompt tokens"},
        # one attention kernel per step, plus the merge kernel when the key/value split is active
        "gpu_launches": args.steps * (2 if step_state["workspace"] is not None else 1),
        "clocks": clocks,
    }
    if rank == 0:
        # roofline of the one kernel in the step (attn_fwd_sm100_pair<128>): bf16 tensor-core bound.
        per_rank_flop = FLOP_PER_STEP / world
        achieved = per_rank_flop / (ms * 1e-3) / 1e12
        line["roofline"] = {
            "bound": "tensor", "kernel": "attn_fwd_sm100_pair<128>", "achieved": achieved,
            "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
            "frac_of_sustained": (achieved / peaks["bf16_tflops_sustained"]
                                  if peaks.get("bf16_tflops_sustained") else None),
            "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
            "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
            "algorithmic_flop_per_launch": per_rank_flop,
        }
        if world == 1 and not args.no_extras:
            line["other_workloads"] = other_workloads(peaks)
            cores = os.cpu_count() or 1
            heads = min(Q_HEADS, cores)
            seconds, flop, kind = cpu_reference_sample(4096, heads, cores)
            line["cpu_baseline"] = {
                "value": flop / seconds / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                "seconds": seconds,
                "sample": f"{heads} of {Q_HEADS} query heads x first 4096 of {SEQ} prompt tokens "
                          f"({flop / 1e9:.2f} GFLOP), one single-head CPU-layer instance per thread"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one attn_fwd_sm100_pair<128> launch on this
# workload, from the ncu capture summarised in profiles/attn_fwd_sm100_pair_d128_gqa_prefill_8192.md.
TRAFFIC_BYTES_PER_LAUNCH = 164.5e6


def other_workloads(peaks, only=None, decode_batch=64, steps_scale=1.0):
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
        return _other_rest(peaks, only, time_ms)
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
    result.update(_other_rest(peaks, only, time_ms))
    return result


def _other_rest(peaks, only, time_ms):
    import torch

    from pluto_b200.layers import AttentionLayer, DataType, gdn_prefill, gdn_step

    result = {}
    if only == "gdn":
        return _gdn_workload(time_ms)
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
    result.update(_gdn_workload(time_ms))
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


def _gdn_workload(time_ms):
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
    # BPTT through the recurrence (checkpointed every 64 tokens), q/k normalisation included
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

    bptt_ms = time_ms(bptt, steps=2, warmup=1)
    result["gated_delta_net"] = {
        "workload": "batch 2, 16 heads, d_k = d_v = 128, seq 16384 prefill then single-token steps",
        "prefill_ms": pre_ms, "prefill_tflops_chunked_count": 94.49e9 / (pre_ms * 1e-3) / 1e12,
        "step_us": step_ms * 1e3, "step_state_gbs": 4.19e6 / (step_ms * 1e-3) / 1e9,
        "step_in_cuda_graph_us": graph_ms * 1e3, "step_in_cuda_graph_state_gbs": 4.19e6 / (graph_ms * 1e-3) / 1e9,
        "recurrence_bwd_ms": bptt_ms, "recurrence_bwd_workspace_gb": ws_bytes / 1e9}
    return result


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["engine", "reference"], default="engine")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the secondary workloads and the CPU baseline (profiling runs)")
    parser.add_argument("--profile-case", choices=["decode", "mha_train", "gdn", "gqa_bwd", "linear", "dense"], default=None,
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
