"""Benchmark of the paged-decode hot path on N GPUs of one node.

One step = one decode step of a serving batch: the fused RoPE + paged-KV write
of the batch's new tokens, then paged decode attention over every cached token
(partition kernel + log-sum-exp merge kernel). The workload is a seeded
synthetic stand-in for the named attention geometry (default: the
Qwen2.5-1.5B-shaped BF16 case, 64 sequences of 512..4096 tokens); no dataset or
model weight is involved.

    python bench.py --gpus 1 --steps 200 --warmup 20
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference            # CPU oracle on the host cores

Rank 0 prints one JSON line. `value` is the whole-job KV-read bandwidth with all
inputs resident in HBM (CUDA-graph replay of exactly K steps, device timed,
max over ranks); `e2e` is the same metric through the public operator API with
the step's inputs coming from pinned host memory and its output read back.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "paged_decode_kv_read_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of one decode partition-kernel
# launch, from the ncu captures summarised under profiles/ (bytes per launch for
# the default workload); None until a capture exists for the workload.
NCU_DRAM_TRAFFIC_BYTES = {"cfg2": 154_178_048 + 3_579_648, "kv-move": 537_019_136 + 486_040_832,
                          "kv-swap": 1_073_888_512 + 1_016_135_680}


def reference_kernels_baseline(case, config, cache_views, steps):
    """Times the reference's own CUDA kernels (compiled for sm_100a by
    oracle/build_reference_cuda.py, where that was possible) on the same decode
    inputs, CUDA events over `steps` back-to-back launches after a warm-up. Only
    for workloads inside their envelope: contexts up to 1024 tokens, NHD, native
    cache. A baseline beside the number, never part of the measured path."""
    from oracle import launch_abi

    if not os.path.exists(launch_abi.REFERENCE):
        return None
    import torch

    key_cache, value_cache = cache_views
    query = case.query.contiguous()
    arguments = (query, key_cache, value_cache, case.block_tables, case.sequence_lengths)
    options = dict(max_sequence_length=case.max_sequence_length, scale=case.scale)

    def time_launch(launch):
        for _ in range(5):
            launch()
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(steps):
                    launch()
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps * 1e3

    def time_library(path):
        library = launch_abi.LaunchLibrary(path)
        decode_us = time_launch(library.prepared_decode(*arguments, **options)[0])
        view = case.qkv.clone().view(config.batch, config.query_heads + 2 * config.kv_heads, config.head_size)
        write_us = time_launch(library.prepared_rope_write(
            view[:, :config.query_heads], view[:, config.query_heads:config.query_heads + config.kv_heads],
            view[:, config.query_heads + config.kv_heads:], case.positions, case.cos_sin_cache, key_cache, value_cache,
            case.key_scales, case.value_scales, case.slot_mapping, is_neox=config.rope_style == "neox"))
        return decode_us, write_us

    reference_us, reference_write_us = time_library(launch_abi.REFERENCE)
    ours_us, ours_write_us = time_library(launch_abi.OURS)
    return {"kernel": "reference paged_decode_attention.cu recompiled for sm_100a",
            "protocol": "decode only through the shared launch ABI (each library's split-K entry when its sizing "
                        "function asks for it), a CUDA graph of the K launches on one cache copy, CUDA events",
            "us_per_launch": reference_us, "value": case.kv_bytes / (reference_us * 1e-6) / 1e9, "unit": UNIT,
            "this_library_same_protocol_us": ours_us,
            "rope_kv_write_us": {"reference": reference_write_us, "this_library": ours_write_us}}


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", choices=["b200", "reference"], default="b200")
    parser.add_argument("--workload", default="cfg2", help="cfg2 (default), cfg3, cfg4, cfg5, cfg1; kv-move / kv-swap time KV block movement")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--batch", type=int, default=0,
                        help="override the workload's batch size (smaller cases for profiler captures)")
    parser.add_argument("--copies", type=int, default=0, help="cache copies rotated between steps (0 = auto)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--programmatic-launch", type=int, choices=[0, 1], default=None,
                        help="programmatic dependent launch mode of the library (default: the library's, 1)")
    parser.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU work per baseline sample")
    parser.add_argument("--query-tokens", type=int, default=1,
                        help="> 1 times ops.paged_multi_token_decode_attention on the workload (decode only)")
    parser.add_argument("--expanded", action="store_true",
                        help="with --query-tokens: the B x Tq single-token form instead of the one-pass form")
    return parser.parse_args()


def host_threads() -> int:
    """Host cores this process may use. Not OMP_NUM_THREADS: torchrun sets that to 1
    for every rank, which would make the CPU arm single-threaded at N > 1."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines: list[str] = []
        self.process = None
        self.thread = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._drain, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _drain(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self):
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima),
                "reasons": sorted(reasons), "samples": len(clocks)}


# ------------------------------------------------------------------ CPU arm

_HOST_ARRAYS = {}


def _host_arrays(case):
    """Host copies of a case in the oracle's storage convention (made once)."""
    key = id(case)
    if key not in _HOST_ARRAYS:
        from oracle import torch_glue as glue

        key_view, value_view = case.cache_views()
        _HOST_ARRAYS.clear()
        _HOST_ARRAYS[key] = dict(
            query=glue.bits(case.query), key=glue.bits(case.key), value=glue.bits(case.value),
            key_cache=glue.bits(key_view), value_cache=glue.bits(value_view),
            positions=glue.bits(case.positions), slots=glue.bits(case.slot_mapping),
            cos_sin=glue.bits(case.cos_sin_cache), tables=glue.bits(case.block_tables),
            lengths=glue.bits(case.sequence_lengths),
            key_scales=case.key_scales.cpu().numpy(), value_scales=case.value_scales.cpu().numpy())
    return _HOST_ARRAYS[key]


def oracle_step_seconds(case, sequences, threads):
    """Times the CPU oracle (RoPE + paged-KV write, then decode) on the first
    `sequences` rows of the batch; only the two oracle calls are inside the timer."""
    from oracle import binding as ob
    from oracle import torch_glue as glue

    c = case.config
    host = _host_arrays(case)
    dtype = glue.ORACLE_DTYPE[c.torch_dtype]
    fp8 = c.cache == "fp8"
    width = c.head_size
    query = host["query"][: sequences * c.query_heads * width].copy()
    key = host["key"][: sequences * c.kv_heads * width].copy()
    value = host["value"][: sequences * c.kv_heads * width]
    max_blocks = case.block_tables.shape[1]
    tables = host["tables"][: sequences * max_blocks]
    lengths = host["lengths"][:sequences]
    if fp8:
        encoding = ob.CACHE_FP8_PER_TENSOR if host["key_scales"].size == 1 else ob.CACHE_FP8_PER_HEAD
    else:
        encoding = ob.CACHE_NATIVE
    rotary = ob.RotarySpec(sequences, c.query_heads, c.kv_heads, width, width, case.cos_sin_cache.shape[0],
                           dtype, c.rope_style == "neox")
    rope_spec = ob.RopeKvSpec(rotary, width, case.num_blocks, c.block_size, encoding)
    decode_spec = ob.DecodeSpec(sequences, c.query_heads, c.kv_heads, width, width, case.num_blocks,
                                c.block_size, max_blocks, case.max_sequence_length, case.scale, dtype)
    output = np.zeros(sequences * c.query_heads * width, dtype=query.dtype)
    started = time.perf_counter()
    if fp8:
        ob.rope_paged_kv_write_fp8(dtype, query, key, value, host["positions"][:sequences], host["cos_sin"],
                                   host["key_cache"], host["value_cache"], host["slots"][:sequences],
                                   host["key_scales"], host["value_scales"], rope_spec)
        ob.paged_decode_attention_fp8(dtype, query, host["key_cache"], host["value_cache"], host["key_scales"],
                                      host["value_scales"], 0 if host["key_scales"].size == 1 else 1, tables,
                                      lengths, output, decode_spec, threads)
    else:
        ob.rope_paged_kv_write(dtype, query, key, value, host["positions"][:sequences], host["cos_sin"],
                               host["key_cache"], host["value_cache"], host["slots"][:sequences], rope_spec)
        ob.paged_decode_attention(dtype, query, host["key_cache"], host["value_cache"], tables, lengths, output,
                                  decode_spec, threads)
    elapsed = time.perf_counter() - started
    tokens = int(case.lengths[:sequences].sum())
    return elapsed, tokens * c.kv_bytes_per_token


def cpu_baseline(case, budget_seconds, threads):
    """Oracle throughput on a bounded sample: as many sequences as fit the budget."""
    probe = min(2, case.config.batch)
    elapsed, sample_bytes = oracle_step_seconds(case, probe, threads)
    per_byte = elapsed / max(sample_bytes, 1)
    total_bytes = case.kv_bytes
    sequences = case.config.batch
    if per_byte * total_bytes > budget_seconds:
        cumulative = np.cumsum(case.lengths) * case.config.kv_bytes_per_token
        sequences = int(max(1, np.searchsorted(cumulative * per_byte, budget_seconds)))
    elapsed, sample_bytes = oracle_step_seconds(case, sequences, threads)
    repeats = int(max(1, min(50, budget_seconds / max(elapsed, 1e-6))))
    total = 0.0
    for _ in range(repeats):
        total += oracle_step_seconds(case, sequences, threads)[0]
    elapsed = total / repeats
    single, single_bytes = oracle_step_seconds(case, min(sequences, 4), 1)
    return {
        "value": sample_bytes / elapsed / 1e9,
        "unit": UNIT,
        "cores": threads,
        "kind": "port",
        "sample": f"{repeats} steps over the first {sequences} of {case.config.batch} sequences "
                  f"({sample_bytes / 1e6:.1f} MB of KV per step, {elapsed:.3f} s per step)",
        "seconds_per_step": elapsed,
        "sequences": sequences,
        "single_thread_value": single_bytes / single / 1e9,
    }


def run_reference(args):
    """The reference arm: the reference's CPU implementation (this repo's C++
    restatement of it; the Rust original cannot be built here) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from attnarc_b200 import workloads
    from oracle import binding as ob

    config = workloads.CONFIGS[args.workload]
    if args.batch:
        config = workloads.scaled(config, batch=args.batch, name=f"{config.name}-batch{args.batch}")
    case = workloads.build_case(config, "cpu", seed=args.seed)
    threads = host_threads()
    steps_total = max(1, args.steps + args.warmup)
    budget = max(0.02, min(args.cpu_seconds, 150.0 / steps_total))
    probe_elapsed, probe_bytes = oracle_step_seconds(case, min(2, config.batch), threads)
    per_byte = probe_elapsed / max(probe_bytes, 1)
    cumulative = np.cumsum(case.lengths) * config.kv_bytes_per_token
    sequences = int(min(config.batch, max(1, np.searchsorted(cumulative * per_byte, budget))))
    for _ in range(args.warmup):
        oracle_step_seconds(case, sequences, threads)
    started = time.perf_counter()
    total_bytes = 0
    for _ in range(args.steps):
        _, step_bytes = oracle_step_seconds(case, sequences, threads)
        total_bytes += step_bytes
    elapsed = time.perf_counter() - started
    value = total_bytes / elapsed / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": config.dtype if config.cache == "native" else "u8", "data": "synthetic",
        "config": {"workload": f"{config.name}: {config.description}", "batch": config.batch,
                   "query_heads": config.query_heads, "kv_heads": config.kv_heads,
                   "head_size": config.head_size, "block_size": config.block_size},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"each step = RoPE+write and decode of the first {sequences} of "
                                   f"{config.batch} sequences on the host"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm

def run_b200(args):
    import torch
    import torch.distributed as dist

    from attnarc_b200 import ops, workloads

    if args.programmatic_launch is not None:
        ops.set_programmatic_launch(args.programmatic_launch)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    config = workloads.CONFIGS[args.workload]
    if args.batch:
        config = workloads.scaled(config, batch=args.batch, name=f"{config.name}-batch{args.batch}")
    # Weak scaling: every rank serves its own batch of the named shape. The
    # path needs no exchange between ranks (sequences are independent).
    case = workloads.build_case(config, device, seed=args.seed + rank, fast_device_fill=True)
    is_neox = config.rope_style == "neox"
    fp8 = config.cache == "fp8"
    kv_bytes = case.kv_bytes

    # Rotate over several copies of the cache so that a step never finds its
    # KV in the 126 MB L2 left there by the previous step.
    cache_bytes = case.kv_cache.numel() * case.kv_cache.element_size()
    copies = args.copies or int(min(8, max(2, (4 << 30) // max(cache_bytes, 1))))
    caches = [case.kv_cache] + [case.kv_cache.clone() for _ in range(copies - 1)]
    views = [workloads.logical_cache_views(c, config.layout) for c in caches]
    rope_views = [c if config.layout == "NHD" else c.permute(0, 1, 3, 2, 4) for c in caches]
    qkv_steps = [case.qkv.clone() for _ in range(copies)]
    pristine_qkv = case.qkv.clone()

    sequences, query_heads, kv_heads = config.batch, config.query_heads, config.kv_heads
    needed, partition = ops.decode_workspace_elements_ex(sequences, query_heads, kv_heads, config.head_size,
                                                         case.max_sequence_length, config.partition_tokens)
    split = case.max_sequence_length > partition
    workspace = torch.empty(needed, device=device, dtype=torch.float32) if split else None
    output = torch.empty((sequences, query_heads, config.head_size), device=device, dtype=config.torch_dtype)
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if fp8 else {}

    def qkv_views(buffer):
        view = buffer.view(sequences, query_heads + 2 * kv_heads, config.head_size)
        return (view[:, :query_heads], view[:, query_heads:query_heads + kv_heads],
                view[:, query_heads + kv_heads:])

    def write_step(index):
        q, k, v = qkv_views(qkv_steps[index])
        ops.rope_paged_kv_write_(q, k, v, case.positions, case.cos_sin_cache, rope_views[index],
                                 case.key_scales, case.value_scales, case.slot_mapping, is_neox=is_neox)
        return q

    def decode_step(index, q):
        # The rotated Q is read in place from the packed QKV row (strided view).
        key_cache, value_cache = views[index]
        ops.paged_decode_attention_ex(q, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                      max_sequence_length=case.max_sequence_length, scale=case.scale,
                                      workspace=workspace, partition_tokens=partition, split=split,
                                      output=output, **scales)

    def step(index):
        # RoPE rotates Q/K in place, so a buffer that is reused keeps turning by
        # the same angle each time it comes round; rotations preserve the norm,
        # so the values stay N(0,1)-like and the work per step is unchanged.
        decode_step(index, write_step(index))

    launches_per_step = 2 + (1 if split else 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for w in range(max(args.warmup, 3)):
        step(w % copies)
    barrier()

    # ---- device-resident timing: one CUDA graph holding exactly K steps ------
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for w in range(3):
            step(w % copies)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for k in range(args.steps):
                step(k % copies)
    barrier()
    graph.replay()  # one untimed replay to settle the graph upload
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        barrier()
        start.record()
        graph.replay()
        stop.record()
        barrier()
        # keep the GPU under the same load a little longer so the sampler sees it
        deadline = time.time() + 0.6
        while time.time() < deadline:
            graph.replay()
        torch.cuda.synchronize()
    graph_ms = start.elapsed_time(stop)

    # ---- the decode operator on its own, for the roofline ---------------------
    # A second graph with only the K decode calls (partition kernel + merge
    # kernel each), timed by CUDA events on the stream that launches it.
    decode_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        queries = [qkv_views(qkv_steps[index])[0] for index in range(copies)]
        with torch.cuda.graph(decode_graph, stream=stream):
            for k in range(args.steps):
                decode_step(k % copies, queries[k % copies])
    barrier()
    decode_graph.replay()
    barrier()
    decode_start, decode_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    decode_start.record()
    decode_graph.replay()
    decode_stop.record()
    barrier()
    decode_ms = decode_start.elapsed_time(decode_stop) / args.steps

    # ---- end to end through the public API with host buffers ----------------
    # attnarc_b200.decode_step.CapturedDecodeStep: the step's inputs (packed QKV
    # rows, positions, slots, block tables, lengths) sit in one pinned host buffer;
    # one graph launch copies them in, runs RoPE + KV write and the decode, and
    # copies the attention rows back to pinned memory; the host waits for them
    # before it starts the next step. The same sequence issued call by call is
    # timed beside it (`eager_us_per_step`).
    from attnarc_b200.decode_step import CapturedDecodeStep

    host_rows = pristine_qkv.cpu().view(sequences, query_heads + 2 * kv_heads, config.head_size)
    captured = []
    for index in range(copies):
        one = CapturedDecodeStep(
            rope_views[index], case.cos_sin_cache, sequences=sequences, query_heads=query_heads,
            max_blocks_per_sequence=case.block_tables.shape[1], max_sequence_length=case.max_sequence_length,
            dtype=config.torch_dtype, scale=case.scale, is_neox=is_neox,
            key_scales=case.key_scales if fp8 else None, value_scales=case.value_scales if fp8 else None,
            partition_tokens=config.partition_tokens)
        one.host_qkv.copy_(host_rows)
        one.host_positions.copy_(case.positions.cpu())
        one.host_slot_mapping.copy_(case.slot_mapping.cpu())
        one.host_block_tables.copy_(case.block_tables.cpu())
        one.host_sequence_lengths.copy_(case.sequence_lengths.cpu())
        captured.append(one.capture())
    h2d, d2h = captured[0].h2d_bytes, captured[0].d2h_bytes

    def timed_steps(run_step):
        for w in range(3):
            run_step(w % copies)
        barrier()
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        for k in range(args.steps):
            run_step(k % copies)  # each waits for its result: the next step depends on it
        last.record()
        barrier()
        return first.elapsed_time(last)

    e2e_ms = timed_steps(lambda index: captured[index].run())
    eager_ms = timed_steps(lambda index: captured[index].run_eager())

    # ---- reduce over ranks: the slowest rank sets the time -------------------
    times = torch.tensor([graph_ms, e2e_ms, decode_ms, eager_ms], device=device, dtype=torch.float64)
    total_bytes = torch.tensor([float(kv_bytes)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    graph_ms, e2e_ms, decode_ms_max, eager_ms_max = (float(x) for x in times.tolist())
    job_bytes = float(total_bytes.item())

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        value = job_bytes * args.steps / (graph_ms * 1e-3) / 1e9
        e2e_value = job_bytes * args.steps / (e2e_ms * 1e-3) / 1e9
        achieved = kv_bytes / (decode_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": graph_ms / args.steps,
            "us_per_step": graph_ms / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8" if fp8 else config.dtype, "data": "synthetic",
            "config": {
                "workload": f"{config.name}: {config.description}", "batch_per_gpu": config.batch,
                "query_heads": query_heads, "kv_heads": kv_heads, "head_size": config.head_size,
                "block_size": config.block_size, "layout": config.layout, "cache": config.cache,
                "context_tokens_rank0": int(case.lengths.sum()), "partition_tokens": partition if split else 0,
                "kv_bytes_per_step_rank0": kv_bytes, "parallelism": f"sequence-sharded x{world}, no collective",
                "launch": "cuda_graph of K steps (value); one captured step per launch, host waits for each (e2e)",
                "programmatic_launch": 1 if args.programmatic_launch is None else args.programmatic_launch,
                "l2": f"inputs rotate over {copies} cache copies of {cache_bytes / 1e6:.0f} MB (> 126 MB L2 in total)",
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "us_per_step": e2e_ms / args.steps * 1e3,
                    "eager_us_per_step": eager_ms_max / args.steps * 1e3,
                    "api": "attnarc_b200.decode_step.CapturedDecodeStep.run"},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                "peak_source": f"{peak_kind} copy bandwidth", "frac_of_nominal_8TBps": achieved / 8000.0,
                "kernel": "decode partition kernel + merge kernel (one operator call)",
                "us_per_launch": decode_ms * 1e3, "algorithmic_bytes_per_launch": kv_bytes,
                "traffic": NCU_DRAM_TRAFFIC_BYTES.get(config.name),
            },
            "clocks": sampler.summary(),
            "decode_route": ops.last_decode_route(),
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle import binding as ob

            line["cpu_baseline"] = cpu_baseline(case, args.cpu_seconds, host_threads())
        if world == 1 and case.max_sequence_length <= 1024 and config.layout == "NHD" and not fp8:
            reference_gpu = reference_kernels_baseline(case, config, views[0], args.steps)
            if reference_gpu is not None:
                line["reference_gpu_baseline"] = reference_gpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------ KV block movement

KV_MOVE = dict(blocks=32768, block_size=16, kv_heads=8, head_size=128, fraction=4)


def run_kv_move(args):
    """`--workload kv-move`: a quarter of the blocks of a 2 GB BF16 cache move to free blocks.

    One step = one `kv_block_move_` launch over 8192 pairs of 64 KB blocks
    (0.5 GB read + 0.5 GB written, scattered; far beyond L2). `value` counts
    bytes read plus bytes written, like the copy bandwidth it is compared with.
    """
    import numpy as np
    import torch

    from attnarc_b200 import ops

    shape = KV_MOVE
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    blocks, count = shape["blocks"], shape["blocks"] // shape["fraction"]
    cache = torch.empty((blocks, 2, shape["block_size"], shape["kv_heads"], shape["head_size"]),
                        dtype=torch.bfloat16, device=device)
    cache.view(torch.int16).random_(generator=torch.Generator(device=device).manual_seed(args.seed))
    order = np.random.default_rng(args.seed).permutation(blocks)
    host_pairs = torch.from_numpy(np.stack([order[:count], order[count:2 * count]], axis=1)).pin_memory()
    pairs = host_pairs.to(device)
    block_bytes = 2 * shape["block_size"] * shape["kv_heads"] * shape["head_size"] * 2  # K + V
    swap = args.workload == "kv-swap"
    moved = (4 if swap else 2) * count * block_bytes  # read + written (a swap reads and writes both blocks)

    def operate():
        if swap:
            ops.kv_block_swap_(cache, pairs)
        else:
            ops.kv_block_move_(cache, cache, pairs)

    for _ in range(max(args.warmup, 3)):
        operate()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        operate()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(args.steps):
                operate()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        deadline = time.time() + 0.6
        while time.time() < deadline:
            graph.replay()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop)

    # end to end: the pairs come from pinned host memory, the host waits for the move
    def e2e_step():
        pairs.copy_(host_pairs, non_blocking=True)
        operate()
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first.record()
    for _ in range(args.steps):
        e2e_step()
    last.record()
    torch.cuda.synchronize()
    e2e_ms = first.elapsed_time(last)

    peak, source = measured_peak_gbs()
    achieved = moved / (ms / args.steps * 1e-3) / 1e9
    line = {
        "metric": "kv_block_swap_bandwidth" if swap else "kv_block_move_bandwidth", "value": achieved, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "%s: %d of %d blocks of %d KB (K+V) %s inside a %.1f GB BF16 cache"
                               % (args.workload, count, blocks, block_bytes // 1024,
                                  "swap with as many others" if swap else "move", blocks * block_bytes / 1e9),
                   "bytes_read_plus_written_per_step": moved, "l2": "1.07 GB touched per step (> 126 MB L2)"},
        "e2e": {"value": moved * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": host_pairs.numel() * 8, "d2h_bytes_per_step": 0,
                "us_per_step": e2e_ms / args.steps * 1e3},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                     "peak_source": f"{source} copy bandwidth (also bytes read plus written)",
                     "kernel": "kv_block_swap_bulk_kernel" if swap else "kv_block_move_bulk_kernel", "us_per_launch": ms / args.steps * 1e3,
                     "algorithmic_bytes_per_launch": moved, "traffic": NCU_DRAM_TRAFFIC_BYTES.get(args.workload)},
        "clocks": sampler.summary(),
    }
    if not args.no_cpu_baseline:
        from oracle import kv_blocks

        sample = 512  # blocks of the same size on the host
        host_cache = np.random.default_rng(1).integers(0, 256, size=(4 * sample, 2, block_bytes // 2), dtype=np.uint8)
        host_order = np.random.default_rng(2).permutation(4 * sample)
        sample_pairs = np.stack([host_order[:sample], host_order[sample:2 * sample]], axis=1)
        begin = time.perf_counter()
        repeats = 0
        while time.perf_counter() - begin < min(args.cpu_seconds, 5.0):
            kv_blocks.kv_block_move(host_cache, host_cache, sample_pairs)
            repeats += 1
        seconds = (time.perf_counter() - begin) / repeats
        line["cpu_baseline"] = {"value": 2 * sample * block_bytes / seconds / 1e9, "unit": UNIT, "cores": 1,
                                "kind": "port", "sample": f"{sample} pairs of {block_bytes // 1024} KB blocks, numpy"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ multi-token queries

def run_multi_token(args):
    """`--query-tokens N`: causal attention of N new tokens per sequence on the named workload.

    One step = one `ops.paged_multi_token_decode_attention` call (pack, decode over the common
    prefix, finish; or the expanded form). `value` = distinct KV bytes of the batch / time.
    """
    import torch

    from attnarc_b200 import ops, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    config = workloads.CONFIGS[args.workload]
    if args.batch:
        config = workloads.scaled(config, batch=args.batch, name=f"{config.name}-batch{args.batch}")
    case = workloads.build_case(config, device, seed=args.seed, fast_device_fill=True)
    key_cache, value_cache = case.cache_views()
    fp8 = config.cache == "fp8"
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if fp8 else {}
    query = torch.randn((config.batch, args.query_tokens, config.query_heads, config.head_size),
                        device=device, generator=torch.Generator(device=device).manual_seed(args.seed))
    query = query.to(config.torch_dtype)

    def step():
        return ops.paged_multi_token_decode_attention(
            query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
            max_sequence_length=case.max_sequence_length, scale=case.scale, one_pass=not args.expanded, **scales)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / args.steps
    peak, source = measured_peak_gbs()
    achieved = case.kv_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "multi_token_decode_kv_read_bandwidth", "value": achieved, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": config.dtype if not fp8 else "u8", "data": "synthetic",
        "config": {"workload": f"{config.name}: {config.description}", "query_tokens": args.query_tokens,
                   "form": "expanded" if args.expanded else "one pass", "distinct_kv_bytes_per_step": case.kv_bytes,
                   "launch": "eager operator calls, CUDA events around K steps",
                   "l2": "KV of %.2f GB per step" % (case.kv_bytes / 1e9)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                     "peak_source": f"{source} copy bandwidth", "algorithmic_bytes_per_launch": case.kv_bytes,
                     "traffic": None},
        "decode_route": ops.last_decode_route(), "clocks": sampler.summary(),
    }), flush=True)


def main():
    args = parse_args()
    if args.workload in ("kv-move", "kv-swap") and args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": "the reference lists KV block movement as planned and has no code for it"}))
    elif args.workload in ("kv-move", "kv-swap"):
        run_kv_move(args)
    elif args.query_tokens > 1 and args.impl != "reference":
        run_multi_token(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
