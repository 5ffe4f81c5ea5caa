"""Benchmark of the paged-decode hot path on N GPUs of one node.

One step = one decode step of a serving batch: the fused RoPE + paged-KV write
of the batch's new tokens, then paged decode attention over every cached token
(partition kernel + log-sum-exp merge kernel). The workload is a seeded
synthetic stand-in for the named attention geometry; no dataset or model weight
is involved. The headline is the largest single-GPU configuration (Llama-3-8B
shape, BF16, 256 sequences of 1024..8192 tokens, HND cache, 512-token
partitions); the other configurations are measured beside it and reported under
`configs`. With N GPUs ONE global batch is spread over the ranks (strong
scaling): by sequence, by KV head (FP8 workload) or, for the long-context
workload, by block ranges of the long sequence with an NCCL all-gather of the
partial states and a merge inside the step. Each rank holds only its share's
pages and checks its rows against its own single-GPU decode of the global
batch before anything is timed (`parity_max_abs_err`).

    python bench.py --gpus 1 --steps 200 --warmup 20
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference            # CPU oracle on the host cores

Rank 0 prints one JSON line. `value` is the whole-job KV-read bandwidth with all
inputs resident in HBM (CUDA-graph replay of exactly K steps, device timed,
max over ranks); `e2e` is the same metric through the public step API with
the step's inputs coming from pinned host memory and its rows read back.
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

# stdout carries the one JSON line and nothing else. Libraries write to it too (NCCL prints its
# version line there at the first communicator), so a multi-rank run moves file descriptor 1 over
# to stderr for its lifetime and keeps the real stdout for emit().
_REAL_STDOUT = None


def keep_stdout_for_the_json_line():
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict):
    text = json.dumps(line) + "\n"
    if _REAL_STDOUT is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, text.encode())

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "paged_decode_kv_read_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of one decode partition-kernel
# launch, from the ncu captures summarised under profiles/ (bytes per launch for
# the default workload); None until a capture exists for the workload.
NCU_DRAM_TRAFFIC_BYTES = {"kv-move": 537_019_136 + 486_040_832, "kv-swap": 1_073_888_512 + 1_016_135_680}
# DRAM bytes (read + written) per algorithmic KV byte of the decode kernel, from one-launch ncu
# captures (dram__bytes_read.sum + dram__bytes_write.sum of the first captured launch) on a
# 24-sequence cut of cfg3 and cfg4 and on the whole of cfg2 and cfg5; traffic grows with the
# token count, so a full launch is this ratio times its KV bytes
# (profiles/decode_dram_traffic_all_configs.md).
NCU_DRAM_TRAFFIC_PER_KV_BYTE = {"cfg2": 1.0267, "cfg3": 1.0170, "cfg4": 1.0137, "cfg5": 1.0056}
# The kernel that copies a block of eight KV heads per tile (cfg4 on one GPU): reads 1.0056 x the KV
# bytes plus 9.1 MB of partial states per launch, whatever the size (profiles/decode_block_tile_fp8_cfg4.md).
NCU_BLOCK_TILE_READ_PER_KV_BYTE, NCU_BLOCK_TILE_WRITTEN_BYTES = 1.0056, 9_123_072


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
    parser.add_argument("--workload", default="cfg3",
                        help="cfg3 (default: the largest single-GPU configuration), cfg2, cfg4, cfg5, cfg1; "
                             "kv-move / kv-swap time KV block movement")
    parser.add_argument("--sub-configs", default="cfg2,cfg4,cfg5",
                        help="workloads measured beside the headline and reported under `configs` (\"none\" = skip)")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--batch", type=int, default=0,
                        help="override the workload's batch size (smaller cases for profiler captures)")
    parser.add_argument("--copies", type=int, default=0, help="cache copies rotated between steps (0 = auto)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--copy-engine", choices=["tma", "cp_async", "tma-mma", "tma-umma", "tma-head"], default=None,
                        help="how the balanced decode kernel is fed (default: the library's choice)")
    parser.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                        help="long-context mode at N > 1: this library's push/merge kernels over peer memory "
                             "(default) or an NCCL all-gather followed by the merge kernel")
    parser.add_argument("--rows-by-copy", action="store_true",
                        help="end-to-end step: copy the attention rows to the host after the last kernel instead "
                             "of letting that kernel store them into pinned host memory itself")
    parser.add_argument("--late-metadata", action="store_true",
                        help="do not promise stable metadata: the decode kernel plans after the grid dependency wait")
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


# ------------------------------------------------------------------ workloads and sharding

# How each workload is spread over N > 1 GPUs: the sharding BASELINE's configs name.
SHARDING = {"cfg1": "by sequence", "cfg2": "by sequence", "cfg2-1024": "by sequence", "ref-b8-ctx1024": "by sequence",
            "cfg3": "by sequence", "cfg4": "by KV head", "cfg5": "long context"}
COLLECTIVE = {"by sequence": "no collective", "by KV head": "no collective",
              "long context": "(O, max, sum) states exchanged inside the step (push + merge kernels over NVLink peer "
                              "memory; --exchange nccl: NCCL all-gather + merge kernel)",
              "single GPU": "no collective"}


def workload_config(args, name):
    from attnarc_b200 import workloads

    config = workloads.CONFIGS[name]
    if args.batch:
        config = workloads.scaled(config, batch=args.batch, name=f"{config.name}-batch{args.batch}")
    return config


def config_record(config, lengths, world):
    """The `config` object of a line: what is computed, identical for both arms."""
    mode = SHARDING.get(config.name.split("-batch")[0], "by sequence") if world > 1 else "single GPU"
    return {
        "workload": f"{config.name}: {config.description}", "global_batch": config.batch,
        "query_heads": config.query_heads, "kv_heads": config.kv_heads, "head_size": config.head_size,
        "block_size": config.block_size, "layout": config.layout, "cache": config.cache,
        "context_tokens": int(lengths.sum()), "longest_context": int(lengths.max()),
        "kv_bytes_per_step": int(lengths.sum()) * config.kv_bytes_per_token,
        "partition_tokens": config.partition_tokens,
        "parallelism": ("one GPU, no collective" if world == 1 else
                        f"one global batch {mode} over {world} GPUs, {COLLECTIVE[mode]}"),
        "step": "fused RoPE + paged-KV write of one new token per sequence, then paged decode attention",
    }


# ------------------------------------------------------------------ CPU arm

CPU_SAMPLE_KV_BYTES = 512 << 20  # a CPU sample step never reads more KV than this


def oracle_step_seconds(case, sequences, threads):
    """Times the CPU oracle (RoPE + paged-KV write, then decode) on the first
    `sequences` rows of a host-resident case; only the two oracle calls are timed."""
    from oracle import binding as ob
    from oracle import torch_glue as glue

    c = case.config
    host = case.extras.get("host_arrays")
    if host is None:
        key_view, value_view = case.cache_views()
        host = dict(
            query=glue.bits(case.query), key=glue.bits(case.key), value=glue.bits(case.value),
            key_cache=glue.bits(key_view), value_cache=glue.bits(value_view),
            positions=glue.bits(case.positions), slots=glue.bits(case.slot_mapping),
            cos_sin=glue.bits(case.cos_sin_cache), tables=glue.bits(case.block_tables),
            lengths=glue.bits(case.sequence_lengths),
            key_scales=case.key_scales.cpu().numpy(), value_scales=case.value_scales.cpu().numpy())
        case.extras["host_arrays"] = host
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


def cpu_sample_case(config, seed):
    """A host-resident case holding the first sequences of the global batch (the batch's own
    lengths, drawn with the bench seed; at most CPU_SAMPLE_KV_BYTES of KV), so that a CPU
    sample never has to materialise a multi-GB cache on the host. Returns (case, global lengths)."""
    from attnarc_b200 import workloads

    lengths = workloads.sample_lengths(config, np.random.default_rng(seed))
    cumulative = np.cumsum(lengths) * config.kv_bytes_per_token
    sequences = int(max(1, np.searchsorted(cumulative, CPU_SAMPLE_KV_BYTES, side="right")))
    sequences = min(sequences, config.batch)
    sample = workloads.scaled(config, batch=sequences, lengths=("fixed", lengths[:sequences].tolist()))
    return workloads.build_case(sample, "cpu", seed=seed), lengths


def sequences_within(case, seconds, threads):
    """How many of the sample's sequences one CPU step can cover in about `seconds`."""
    probe = min(2, case.config.batch)
    elapsed, sample_bytes = oracle_step_seconds(case, probe, threads)
    per_byte = elapsed / max(sample_bytes, 1)
    cumulative = np.cumsum(case.lengths) * case.config.kv_bytes_per_token
    return int(min(case.config.batch, max(1, np.searchsorted(cumulative * per_byte, seconds))))


def cpu_baseline(config, seed, budget_seconds, threads):
    """Oracle throughput on a bounded sample of the workload (about `budget_seconds` of CPU work)."""
    case, lengths = cpu_sample_case(config, seed)
    sequences = sequences_within(case, min(2.0, budget_seconds / 4), threads)
    elapsed, sample_bytes = oracle_step_seconds(case, sequences, threads)
    repeats = int(max(1, min(50, budget_seconds / max(elapsed, 1e-6))))
    total = 0.0
    for _ in range(repeats):
        total += oracle_step_seconds(case, sequences, threads)[0]
    elapsed = total / repeats
    single, single_bytes = oracle_step_seconds(case, min(sequences, 2), 1)
    return {
        "value": sample_bytes / elapsed / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
        "sample": f"{repeats} steps (RoPE + KV write, then decode) over the first {sequences} of the global batch's "
                  f"{config.batch} sequences ({sample_bytes / 1e6:.1f} MB of KV per step, {elapsed:.3f} s per step)",
        "seconds_per_step": elapsed, "sequences": sequences,
        "single_thread_value": single_bytes / single / 1e9,
    }


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path (this repo's C++
    restatement of its Rust oracle; the original cannot be built here) on all host cores, on
    the same global batch at every N. Rank 0 alone works and prints."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    config = workload_config(args, args.workload)
    case, lengths = cpu_sample_case(config, args.seed)
    threads = host_threads()
    steps_total = max(1, args.steps + args.warmup)
    budget = max(0.02, min(args.cpu_seconds, 150.0 / steps_total))
    sequences = sequences_within(case, budget, threads)
    for _ in range(args.warmup):
        oracle_step_seconds(case, sequences, threads)
    started = time.perf_counter()
    total_bytes = 0
    for _ in range(args.steps):
        _, step_bytes = oracle_step_seconds(case, sequences, threads)
        total_bytes += step_bytes
    elapsed = time.perf_counter() - started
    value = total_bytes / elapsed / 1e9
    sample = (f"each step = RoPE + KV write and decode of the first {sequences} of the global batch's "
              f"{config.batch} sequences on the host ({total_bytes / max(args.steps, 1) / 1e6:.1f} MB of KV)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / max(args.steps, 1) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": config.dtype if config.cache == "native" else "u8", "data": "synthetic",
        "config": config_record(config, lengths, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------ GPU arm

class Ranks:
    """Process-group plumbing of one bench process."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            keep_stdout_for_the_json_line()
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        import torch
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        """MAX or SUM over ranks of a list of floats."""
        import torch
        import torch.distributed as dist

        tensor = torch.tensor(values, device=self.device, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(tensor, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return [float(x) for x in tensor.tolist()]

    def close(self):
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
            dist.destroy_process_group()


def single_gpu_rows(case):
    """Attention rows of the whole batch from one GPU (this rank's), through the same operators:
    the reference the sharded step is compared with, outside any timed region."""
    import torch

    from attnarc_b200 import ops

    c = case.config
    rows = case.qkv.clone().view(c.batch, c.query_heads + 2 * c.kv_heads, c.head_size)
    query = rows[:, :c.query_heads]
    ops.rope_paged_kv_write_(query, rows[:, c.query_heads:c.query_heads + c.kv_heads],
                             rows[:, c.query_heads + c.kv_heads:], case.positions, case.cos_sin_cache,
                             case.rope_cache_argument(), case.key_scales, case.value_scales, case.slot_mapping,
                             is_neox=c.rope_style == "neox")
    key_cache, value_cache = case.cache_views()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if c.cache == "fp8" else {}
    out = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                        max_sequence_length=case.max_sequence_length, scale=case.scale, **scales)
    torch.cuda.synchronize()
    return out


def reference_abi_single_pass_us(case, launches=5):
    """Times `loom_cuda_paged_decode_attention_bf16` / `_f16`, the reference-shaped entry point WITHOUT
    a workspace (one CTA walks a whole context), on a dense-inner NHD native cache. On long contexts
    and small batches this uses a handful of SMs: the figure is on record so that callers of the
    reference ABI know to use its split-K entry (or the `_ex` entry) with a workspace there."""
    import torch

    from attnarc_b200 import _native

    c = case.config
    if c.layout != "NHD" or c.cache != "native" or c.dtype not in ("bf16", "f16"):
        return None
    lib = _native.library()
    entry = getattr(lib, f"loom_cuda_paged_decode_attention_{c.dtype}")
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    output = torch.empty_like(query)
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        status = entry(query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), case.block_tables.data_ptr(),
                       case.sequence_lengths.data_ptr(), output.data_ptr(), c.batch, c.query_heads, c.kv_heads,
                       c.head_size, c.head_size, case.num_blocks, c.block_size, key_cache.stride(0),
                       value_cache.stride(0), case.block_tables.shape[1], case.max_sequence_length, case.scale,
                       stream)
        if status != 0:
            raise SystemExit(f"reference-shaped decode entry failed with status {status}")

    launch()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(launches):
        launch()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / launches * 1e3


def measure_workload(args, ranks, name, steps, headline):
    """Builds the workload's global batch, shards it over the ranks, times it; returns rank-local
    figures already reduced over ranks (every rank gets the same record)."""
    import torch

    from attnarc_b200 import ops, sharded_step, workloads

    config = workload_config(args, name)
    world, rank, device = ranks.world, ranks.rank, ranks.device
    is_neox = config.rope_style == "neox"
    fp8 = config.cache == "fp8"
    # every rank draws the same global batch (same seed), then keeps its share
    case = workloads.build_case(config, device, seed=args.seed, fast_device_fill=True)
    global_bytes = case.kv_bytes
    mode = SHARDING.get(name, "by sequence") if world > 1 else "single GPU"
    parity = None
    if world > 1:
        shard = sharded_step.SHARDERS[mode](case, rank, world)
        reference_rows = single_gpu_rows(case)  # [B, Hq, D] on this rank's own copy of the global batch
        first, count = shard.query_heads
        index = torch.tensor(shard.rows, dtype=torch.int64, device=device)
        reference_rows = reference_rows[index][:, first:first + count].clone()
        cos_sin = case.cos_sin_cache
        lengths = case.lengths
        del case
        torch.cuda.empty_cache()
    else:
        shard = sharded_step.whole_case(case)
        cos_sin, lengths = case.cos_sin_cache, case.lengths

    def make_step(rope_cache, rows_to_host=False):
        return sharded_step.ShardedDecodeStep(shard, cos_sin, rope_cache=rope_cache, dtype=config.torch_dtype,
                                              scale=1.0 / float(np.sqrt(config.head_size)), is_neox=is_neox,
                                              partition_tokens=config.partition_tokens,
                                              early_metadata=not args.late_metadata, exchange=args.exchange,
                                              rows_to_host=rows_to_host)

    # Rotate over several copies of the local cache so that a step never finds its KV in the
    # 126 MB L2 left there by the previous step.
    cache_bytes = shard.kv_cache.numel() * shard.kv_cache.element_size()
    copies = args.copies or int(min(8, max(2, -(-(1 << 30) // max(cache_bytes, 1)))))
    caches = [shard.kv_cache] + [shard.kv_cache.clone() for _ in range(copies - 1)]
    layout_view = (lambda c: c) if config.layout == "NHD" else (lambda c: c.permute(0, 1, 3, 2, 4))
    step = make_step(layout_view(caches[0]))
    rope_views = [layout_view(c) for c in caches]
    step.upload()
    torch.cuda.synchronize()

    if world > 1:
        got = step.run_eager().to(device)
        parity = float((got.float() - reference_rows.float()).abs().max()) if got.numel() else 0.0
        tolerance = 1e-2
        limit = tolerance + tolerance * float(reference_rows.float().abs().max()) if got.numel() else tolerance
        if not parity <= limit:
            raise SystemExit(f"{name}: rank {rank}'s sharded rows differ from the single-GPU decode by {parity}")
        step.upload()  # fresh, unrotated inputs for the timed runs
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for w in range(warmup):
        step.enqueue_kernels(rope_views[w % copies])
    ranks.barrier()

    def timed_graph(body):
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            body(0)
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                for k in range(steps):
                    body(k % copies)
        ranks.barrier()
        graph.replay()  # one untimed replay to settle the graph upload
        ranks.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(ranks.local_rank) as sampler:
            ranks.barrier()
            start.record()
            graph.replay()
            stop.record()
            ranks.barrier()
            elapsed_ms = start.elapsed_time(stop)
            # Keep the GPU under the same load a little longer so that the sampler sees it. Every rank
            # replays the SAME number of times (derived from the slowest rank's time): a step that
            # exchanges states needs every rank in every step.
            slowest_ms = ranks.reduce([elapsed_ms])[0]
            for _ in range(int(min(5000, max(1, (600.0 if headline else 350.0) / max(slowest_ms, 1e-3))))):
                graph.replay()
            ranks.barrier()
        return elapsed_ms, sampler.summary()

    # ---- device-resident timing: one CUDA graph holding exactly `steps` steps ----------------
    step_ms, clocks = timed_graph(lambda index: step.enqueue_kernels(rope_views[index]))
    route = ops.last_decode_route() if shard.sequences else "none"
    # ---- the decode operator alone (decode + merge kernels), for the roofline ----------------
    decode_ms, _ = timed_graph(lambda index: step.enqueue_kernels(rope_views[index], rope=False, exchange=False))

    record = {}
    e2e_ms = eager_ms = None
    if headline:
        # ---- end to end through the public step API with host buffers ------------------------
        # (the end-to-end step lets its last kernel store the rows into the pinned buffer itself, unless
        # --rows-by-copy asks for the device-to-host copy after it; the resident steps above write to HBM)
        captured = [make_step(view, rows_to_host=not args.rows_by_copy).capture() for view in rope_views]

        def timed_steps(run_step):
            for w in range(3):
                run_step(w % copies)
            ranks.barrier()
            first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            first.record()
            for k in range(steps):
                run_step(k % copies)  # each waits for its rows: the next step depends on them
            last.record()
            ranks.barrier()
            return first.elapsed_time(last)

        e2e_ms = timed_steps(lambda index: captured[index].run())
        eager_ms = timed_steps(lambda index: captured[index].run_eager())

    if (headline and world == 1 and shard.max_sequence_length <= 1024 and config.layout == "NHD" and not fp8):
        reference_gpu = reference_kernels_baseline(case, config, case.cache_views(), steps)
        if reference_gpu is not None:
            record["reference_gpu_baseline"] = reference_gpu

    if world == 1 and name == "cfg5":
        single_pass_us = reference_abi_single_pass_us(case)
        if single_pass_us is not None:
            record["reference_abi_without_workspace"] = {
                "us_per_launch": single_pass_us,
                "note": "loom_cuda_paged_decode_attention_bf16 without a workspace: one CTA per (sequence, KV head) "
                        "walks the whole context; with a workspace (split-K entry) the same call takes the "
                        "decode time of this record"}

    launches = step.kernel_launches if shard.sequences else 0
    step_ms, decode_ms_max = ranks.reduce([step_ms, decode_ms])
    sums = ranks.reduce([float(shard.kv_bytes), float(step.h2d_bytes), float(step.d2h_bytes), float(launches)], "sum")
    peak, peak_kind = measured_peak_gbs()
    us = step_ms / steps * 1e3
    local_decode_us = decode_ms / steps * 1e3
    achieved = shard.kv_bytes / (local_decode_us * 1e-6) / 1e9 if shard.kv_bytes else 0.0
    traffic = NCU_DRAM_TRAFFIC_PER_KV_BYTE.get(name)
    if traffic is not None and "block" in route and shard.kv_bytes:
        traffic = NCU_BLOCK_TILE_READ_PER_KV_BYTE + NCU_BLOCK_TILE_WRITTEN_BYTES / shard.kv_bytes
    record.update({
        "workload": f"{config.name}: {config.description}", "sharding": mode, "n_gpus": world, "steps": steps,
        "us_per_step": us, "value": global_bytes / (us * 1e-6) / 1e9, "unit": UNIT,
        "kv_bytes_per_step": global_bytes, "kv_bytes_all_ranks": sums[0],
        "decode_us_max_over_ranks": decode_ms_max / steps * 1e3,
        "frac_of_measured_peak_all_gpus": global_bytes / (us * 1e-6) / 1e9 / (peak * world),
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
            "peak_source": f"{peak_kind} copy bandwidth", "frac_of_nominal_8TBps": achieved / 8000.0,
            "kernel": "decode kernel + merge kernel of rank 0 (one operator call), its own CUDA graph",
            "us_per_launch": local_decode_us, "algorithmic_bytes_per_launch": shard.kv_bytes,
            "traffic": None if traffic is None else int(traffic * shard.kv_bytes),
            "traffic_source": None if traffic is None else
            "ncu dram__bytes_read.sum + dram__bytes_write.sum of one decode launch on a cut of the workload, "
            "scaled by KV bytes (profiles/decode_dram_traffic_all_configs.md, profiles/decode_block_tile_fp8_cfg4.md)",
        },
        "exchange": (None if not shard.exchange else
                     "push + merge kernels over NVLink peer memory" if step.peer_exchange is not None else
                     "NCCL all-gather + merge kernel"),
        "decode_route": route, "clocks": clocks, "parity_max_abs_err": parity,
        "parity_against": None if parity is None else "this rank's single-GPU decode of the global batch",
        "l2": f"steps rotate over {copies} copies of the rank's {cache_bytes / 1e6:.0f} MB cache",
        "gpu_launches": int(sums[3]) * steps,
    })
    if parity is not None:
        record["parity_max_abs_err"] = ranks.reduce([parity])[0]
    if headline:
        e2e_ms, eager_ms = ranks.reduce([e2e_ms, eager_ms])
        record["e2e"] = {"value": global_bytes * steps / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                         "h2d_bytes_per_step": int(sums[1]), "d2h_bytes_per_step": int(sums[2]),
                         "us_per_step": e2e_ms / steps * 1e3, "eager_us_per_step": eager_ms / steps * 1e3,
                         "api": "attnarc_b200.sharded_step.ShardedDecodeStep.run (one per rank)"}
        record["config"] = config_record(config, lengths, world)
    del caches, step
    torch.cuda.empty_cache()
    return record, config


def run_b200(args):
    from attnarc_b200 import ops

    if args.programmatic_launch is not None:
        ops.set_programmatic_launch(args.programmatic_launch)
    if args.copy_engine is not None:
        ops.set_decode_copy_engine(args.copy_engine)
    ranks = Ranks()
    head, config = measure_workload(args, ranks, args.workload, args.steps, headline=True)
    others = {}
    if args.sub_configs != "none":
        names = [n for n in args.sub_configs.split(",") if n and n != args.workload]
        for name in names:
            others[name], _ = measure_workload(args, ranks, name, max(args.steps, 50), headline=False)
            others[name].pop("gpu_launches", None)
    if ranks.rank == 0:
        line = {
            "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": ranks.world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": head["us_per_step"] / 1e3,
            "us_per_step": head["us_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u8" if config.cache == "fp8" else config.dtype, "data": "synthetic",
            "config": head["config"],
            "protocol": {"value": "one CUDA graph of exactly K steps per rank, inputs resident, CUDA events, "
                                  "barrier on both sides, max over ranks",
                         "e2e": "one captured step per launch: inputs copied from one pinned host buffer, rows stored "
                                "into pinned host memory by the step's last kernel, host waits for each",
                         "l2": head["l2"],
                         "programmatic_launch": 1 if args.programmatic_launch is None else args.programmatic_launch},
            "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "roofline": head["roofline"],
            "clocks": head["clocks"], "decode_route": head["decode_route"], "sharding": head["sharding"],
            "parity_max_abs_err": head["parity_max_abs_err"], "parity_against": head["parity_against"],
            "decode_us_max_over_ranks": head["decode_us_max_over_ranks"],
            "frac_of_measured_peak_all_gpus": head["frac_of_measured_peak_all_gpus"],
            "configs": others,
        }
        if "reference_gpu_baseline" in head:
            line["reference_gpu_baseline"] = head["reference_gpu_baseline"]
        if ranks.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(config, args.seed, args.cpu_seconds, host_threads())
        emit(line)
    ranks.close()


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
    emit(line)


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
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    eager_ms = start.elapsed_time(stop) / args.steps
    # the same K steps as one CUDA graph, like the single-token benchmark
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(args.steps):
                step()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as sampler:
        start.record()
        graph.replay()
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
                   "launch": "one CUDA graph of K operator calls, CUDA events around its replay",
                   "eager_ms_per_step": eager_ms,
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
