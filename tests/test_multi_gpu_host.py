"""Host-side logic of the multi-GPU sharding, on CPU.

The partitioner is plain host arithmetic; the long-context exchange is run as
two ``gloo`` ranks on CPU tensors. The attention arithmetic of those ranks is a
float64 numpy restatement that lives in this file (a checker, injected through
the ``decode_states``/``merge_states`` hooks); the merged result is compared
with the pinned oracle's decode of the unsplit sequences. The CUDA operators
themselves are covered by the ``gpu`` tests.
"""

import os
import socket

import numpy as np
import pytest
import torch

from attnarc_b200 import build, multi_gpu
from tests.helpers import assert_close, oracle_decode


@pytest.fixture(scope="module", autouse=True)
def built_library():
    build.build()


# --------------------------------------------------------------- partitioner

def test_by_sequence_balances_and_is_deterministic():
    rng = np.random.default_rng(7)
    lengths = rng.integers(1, 9000, size=257).tolist()
    owners, tokens = multi_gpu.partition_by_sequence(lengths, 8)
    assert len(owners) == len(lengths) and set(owners) <= set(range(8))
    recount = [0] * 8
    for length, owner in zip(lengths, owners):
        recount[owner] += length
    assert recount == tokens and sum(tokens) == sum(lengths)
    # greedy longest-first keeps the spread below the longest sequence
    assert max(tokens) - min(tokens) <= max(lengths)
    assert multi_gpu.partition_by_sequence(lengths, 8) == (owners, tokens)


def test_by_sequence_ties_go_to_the_lower_rank_and_index():
    owners, tokens = multi_gpu.partition_by_sequence([5, 5, 5, 5], 2)
    assert owners == [0, 1, 0, 1] and tokens == [10, 10]
    owners, _ = multi_gpu.partition_by_sequence([0, 0, 3], 4)
    assert owners[2] == 0  # the longest goes first, to rank 0
    owners, tokens = multi_gpu.partition_by_sequence([4], 3)
    assert owners == [0] and tokens == [4, 0, 0]


@pytest.mark.parametrize("call", [
    lambda: multi_gpu.partition_by_sequence([], 2),
    lambda: multi_gpu.partition_by_sequence([1, -1], 2),
    lambda: multi_gpu.partition_by_sequence([1], 0),
    lambda: multi_gpu.partition_by_kv_head(0, 2),
    lambda: multi_gpu.partition_long_context([1], 2, 0),
    lambda: multi_gpu.partition_long_context([], 2, 16),
])
def test_partitioner_rejects_bad_arguments(call):
    with pytest.raises(ValueError):
        call()


def test_by_kv_head_ranges_are_contiguous_and_even():
    assert multi_gpu.partition_by_kv_head(8, 8) == [(i, 1) for i in range(8)]
    assert multi_gpu.partition_by_kv_head(8, 2) == [(0, 4), (4, 4)]
    assert multi_gpu.partition_by_kv_head(2, 4) == [(0, 1), (1, 1), (2, 0), (2, 0)]
    ranges = multi_gpu.partition_by_kv_head(10, 4)
    assert ranges == [(0, 3), (3, 3), (6, 2), (8, 2)]


@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
def test_long_context_shards_cover_every_token_once(ranks):
    lengths = [131072, 17, 4096, 0, 70000, 33]
    block = 16
    shards, tokens = multi_gpu.partition_long_context(lengths, ranks, block)
    assert sum(tokens) == sum(lengths)
    for sequence, length in enumerate(lengths):
        mine = [s for s in shards if s.sequence == sequence]
        assert mine, "every sequence has an owner, even an empty one"
        if len(mine) == 1 and not mine[0].split:
            assert mine[0].first_block == 0 and mine[0].token_count == length
            continue
        assert all(s.split for s in mine)
        assert [s.rank for s in mine] == sorted(s.rank for s in mine)
        cursor = 0
        for shard in mine:
            assert shard.first_block * block == shard.first_token == cursor
            assert 0 < shard.token_count <= shard.block_count * block
            cursor += shard.block_count * block
        assert sum(s.token_count for s in mine) == length
    if ranks > 1:
        assert any(s.split for s in shards)
        # whole sequences are placed greedily: the spread stays below the longest of them
        whole = [lengths[s.sequence] for s in shards if not s.split]
        assert max(tokens) - min(tokens) <= max(whole) + block * ranks
    else:
        assert not any(s.split for s in shards)


def test_long_context_threshold_is_respected():
    shards, _ = multi_gpu.partition_long_context([1000, 1000, 1000], 2, 16, split_threshold_tokens=4096)
    assert not any(s.split for s in shards)
    shards, _ = multi_gpu.partition_long_context([1000, 5000], 2, 16, split_threshold_tokens=4096)
    assert [s.split for s in shards] == [False, True, True]


def test_local_inputs_shift_the_block_table_of_a_split_row():
    plan = multi_gpu.RankBatch(rank=1, rows=[2, 0], first_blocks=[3, 0], lengths=[40, 20], split_rows=[True, False])
    query = torch.arange(3 * 2 * 4, dtype=torch.float32).reshape(3, 2, 4)
    tables = torch.arange(3 * 6, dtype=torch.int32).reshape(3, 6)
    local_query, local_tables, lengths = multi_gpu.local_decode_inputs(plan, query, tables)
    assert torch.equal(local_query, query[[2, 0]])
    assert local_tables[0].tolist() == [15, 16, 17, 17, 17, 17]  # row 2 from block 3 on, tail clamped
    assert local_tables[1].tolist() == [0, 1, 2, 3, 4, 5]
    assert lengths.tolist() == [40, 20] and lengths.dtype == torch.int32


# ------------------------------------------------- two gloo ranks, long context

def numpy_states(query, key_cache, value_cache, block_tables, lengths, *, max_sequence_length, scale, **_):
    """Float64 partial states [B, Hq, Dv + 2] of the given block ranges."""
    q = query.to(torch.float64).numpy()
    keys = key_cache.to(torch.float64).numpy()
    values = value_cache.to(torch.float64).numpy()
    batch, query_heads, _ = q.shape
    _, block_size, kv_heads, _ = keys.shape
    value_dim = values.shape[3]
    group = query_heads // kv_heads
    out = np.zeros((batch, query_heads, value_dim + 2))
    for b in range(batch):
        n = int(lengths[b])
        blocks = block_tables[b].numpy()
        token_block = blocks[np.arange(n) // block_size]
        token_page = np.arange(n) % block_size
        for h in range(query_heads):
            if n == 0:
                out[b, h, value_dim] = -np.inf
                continue
            k = keys[token_block, token_page, h // group]
            v = values[token_block, token_page, h // group]
            scores = (k @ q[b, h]) * scale
            top = scores.max()
            weights = np.exp(scores - top)
            out[b, h, :value_dim] = weights @ v
            out[b, h, value_dim] = top
            out[b, h, value_dim + 1] = weights.sum()
    return torch.from_numpy(out).to(torch.float32)


def numpy_merge(states, dtype):
    s = states.to(torch.float64).numpy()
    value_dim = s.shape[2] - 2
    top = s[:, :, value_dim].max(axis=0)
    safe_top = np.where(np.isfinite(top), top, 0.0)
    factor = np.exp(s[:, :, value_dim] - safe_top[None, :])
    total = (s[:, :, value_dim + 1] * factor).sum(axis=0)
    acc = (s[:, :, :value_dim] * factor[:, :, None]).sum(axis=0)
    merged = np.where(total[:, None] > 0, acc / np.where(total > 0, total, 1.0)[:, None], 0.0)
    return torch.from_numpy(merged).to(dtype)


def build_case(seed):
    gen = torch.Generator().manual_seed(seed)
    lengths = [700, 9, 0, 333]
    block, kv_heads, query_heads, dim = 16, 2, 4, 32
    max_blocks = (max(lengths) + block - 1) // block
    num_blocks = len(lengths) * max_blocks + 3
    keys = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(torch.bfloat16)
    values = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(torch.bfloat16)
    query = torch.randn((len(lengths), query_heads, dim), generator=gen).to(torch.bfloat16)
    order = torch.randperm(num_blocks, generator=gen)[: len(lengths) * max_blocks]
    tables = order.reshape(len(lengths), max_blocks).to(torch.int32)
    return query, keys, values, tables, lengths, block, dim ** -0.5


def _long_context_rank(rank, world, port, results):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        query, keys, values, tables, lengths, block, scale = build_case(11)
        merged = multi_gpu.decode_long_context(
            query, keys, values, tables, lengths, scale=scale, block_size=block,
            split_threshold_tokens=256, decode_states=numpy_states, merge_states=numpy_merge)
        plan = multi_gpu.plan_long_context(lengths, world, block, 256)[rank]
        results[rank] = (merged, plan.rows, plan.split_rows)
    finally:
        dist.destroy_process_group()


def test_long_context_exchange_over_two_gloo_ranks():
    import torch.multiprocessing as mp

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_long_context_rank, args=(2, port, results), nprocs=2, join=True)
    assert set(results.keys()) == {0, 1}
    query, keys, values, tables, lengths, block, scale = build_case(11)
    # the reference contract has no empty sequences: the oracle sees the others, the empty one gives zeros
    live = [i for i, n in enumerate(lengths) if n > 0]
    expected = torch.zeros((len(lengths), query.shape[1], values.shape[3]), dtype=torch.bfloat16)
    expected[live] = oracle_decode(query[live], keys, values, tables[live],
                                   torch.tensor([lengths[i] for i in live], dtype=torch.int32),
                                   scale=scale, max_sequence_length=max(lengths))
    for rank in (0, 1):
        merged, rows, split_rows = results[rank]
        assert_close(merged, expected, torch.bfloat16, f"rank {rank}")
    # sequences 0 and 3 exceed the threshold: both ranks hold a range of each
    assert sorted(r for r, s in zip(results[0][1], results[0][2]) if s) == [0, 3]
    assert sorted(r for r, s in zip(results[1][1], results[1][2]) if s) == [0, 3]
    # the short and the empty sequence have exactly one owner
    owners = [rank for rank in (0, 1) for r in results[rank][1] if r in (1, 2)]
    assert len(owners) == 2


def test_by_sequence_decode_keeps_rows_local():
    query, keys, values, tables, lengths, block, scale = build_case(5)
    covered = []
    for rank in range(2):
        def states_as_output(q, k, v, t, n, **kwargs):
            return numpy_merge(numpy_states(q, k, v, t, n, **kwargs).unsqueeze(0).reshape(1, -1, v.shape[3] + 2),
                               torch.bfloat16).reshape(q.shape[0], q.shape[1], v.shape[3])
        rows, output = multi_gpu.decode_by_sequence(query, keys, values, tables, lengths, scale=scale,
                                                    rank=rank, ranks=2, decode=states_as_output)
        covered += rows
        live = [i for i, r in enumerate(rows) if lengths[r] > 0]
        live_rows = [rows[i] for i in live]
        expected = oracle_decode(query[live_rows], keys, values, tables[live_rows],
                                 torch.tensor([lengths[r] for r in live_rows], dtype=torch.int32),
                                 scale=scale, max_sequence_length=max(lengths))
        assert_close(output[live], expected, torch.bfloat16, f"rank {rank}")
        assert all(float(output[i].abs().max()) == 0.0 for i in range(len(rows)) if i not in live)
    assert sorted(covered) == [0, 1, 2, 3]


# ------------------------------------------------- KV-head sharding (no exchange)

def test_by_kv_head_decode_covers_disjoint_column_slices():
    query, keys, values, tables, lengths, block, scale = build_case(13)
    live = [i for i, n in enumerate(lengths) if n > 0]
    query, tables = query[live], tables[live]
    lengths = torch.tensor([lengths[i] for i in live], dtype=torch.int32)

    def states_as_output(q, k, v, t, n, **kwargs):
        return numpy_merge(numpy_states(q, k, v, t, n, **kwargs).reshape(1, -1, v.shape[3] + 2),
                           torch.bfloat16).reshape(q.shape[0], q.shape[1], v.shape[3])

    expected = oracle_decode(query, keys, values, tables, lengths, scale=scale, max_sequence_length=int(lengths.max()))
    result = torch.zeros_like(expected)
    covered = []
    for rank in range(2):
        (first, count), rows = multi_gpu.decode_by_kv_head(
            query, keys, values, tables, lengths, scale=scale, max_sequence_length=int(lengths.max()),
            rank=rank, ranks=2, decode=states_as_output)
        result[:, first:first + count] = rows
        covered += list(range(first, first + count))
    assert covered == list(range(query.shape[1]))
    assert_close(result, expected, torch.bfloat16, "by KV head")
    # more ranks than KV heads: the surplus ranks get an empty slice and launch nothing
    (first, count), rows = multi_gpu.decode_by_kv_head(
        query, keys, values, tables, lengths, scale=scale, max_sequence_length=int(lengths.max()),
        rank=3, ranks=4, decode=lambda *a, **k: pytest.fail("an empty share must not decode"))
    assert count == 0 and rows.shape[1] == 0


# ------------------------------------------------- failure detection on CPU ranks

def test_rank_health_reports_a_peer_that_left_or_went_silent():
    import torch.distributed as dist

    store = dist.HashStore()
    now = [0.0]
    mine = multi_gpu.RankHealth(store, 0, 2, stale_after=5.0, clock=lambda: now[0])
    peer = multi_gpu.RankHealth(store, 1, 2, stale_after=5.0, clock=lambda: now[0])
    assert mine.before_launch() == multi_gpu.STATUS_SUCCESS
    peer.beat(1)
    now[0] = 4.0
    assert mine.before_launch() == multi_gpu.STATUS_SUCCESS
    now[0] = 8.0  # 4 s since the last change: still fresh
    assert mine.before_launch() == multi_gpu.STATUS_SUCCESS
    now[0] = 9.5  # no beat for more than 5 s
    assert mine.before_launch() == multi_gpu.STATUS_UNAVAILABLE and "not reported" in mine.last_error
    peer.beat(2)
    assert mine.before_launch() == multi_gpu.STATUS_SUCCESS
    peer.leave()
    assert mine.before_launch() == multi_gpu.STATUS_UNAVAILABLE and "left" in mine.last_error


def _late_or_leaving_rank(rank, world, port, results):
    """Rank 1 first arrives late at an exchange, then leaves between steps."""
    import datetime
    import time

    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    store = dist.distributed_c10d._get_default_store()
    health = multi_gpu.RankHealth(store, rank, world, stale_after=30.0)
    try:
        query, keys, values, tables, lengths, block, scale = build_case(11)
        decoder = multi_gpu.LongContextDecoder(
            lengths, tables, query_heads=query.shape[1], value_head_size=values.shape[3], block_size=block,
            dtype=query.dtype, split_threshold_tokens=256, decode_states=numpy_states, merge_states=numpy_merge,
            timeout_seconds=1.0, health=health)
        # step 1: both ranks on time
        first = decoder.decode(query, keys, values, scale=scale)
        health.beat(1)
        # step 2: rank 1 arrives three seconds late; rank 0 gives up after one second
        if rank == 1:
            time.sleep(3.0)
        started = time.monotonic()
        second = decoder.decode(query, keys, values, scale=scale)
        waited = time.monotonic() - started
        results[rank] = dict(first_ok=torch.is_tensor(first), second=second if isinstance(second, int) else "rows",
                             waited=waited, error=decoder.last_error)
        # step 3: rank 1 leaves between steps; rank 0 learns of it before it launches anything
        if rank == 1:
            health.leave()
            store.set("loom/test/left", "1")
        else:
            store.wait(["loom/test/left"], datetime.timedelta(seconds=30))
            calls = []
            decoder.decode_states = lambda *a, **k: calls.append(1)
            third = decoder.decode(query, keys, values, scale=scale)
            entry = results[rank]
            entry.update(third=third, launched=len(calls), third_error=decoder.last_error)
            results[rank] = entry
    finally:
        # the late exchange left this group's collectives out of step: no barrier, no orderly shutdown
        results[f"done{rank}"] = True


def test_long_context_exchange_reports_a_late_and_a_departed_rank():
    import torch.multiprocessing as mp

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    context = mp.get_context("spawn")
    workers = [context.Process(target=_late_or_leaving_rank, args=(rank, 2, port, results)) for rank in range(2)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(120)
    for worker in workers:
        if worker.is_alive():
            worker.kill()
    assert results.get("done0") and results.get("done1")
    zero = results[0]
    assert zero["first_ok"]
    # the late peer: a status within about the timeout, not a hang until it shows up
    assert zero["second"] == multi_gpu.STATUS_UNAVAILABLE, zero
    assert zero["waited"] < 2.5 and zero["error"]
    # the departed peer: refused on the host, nothing launched
    assert zero["third"] == multi_gpu.STATUS_UNAVAILABLE and zero["launched"] == 0
    assert "left" in zero["third_error"]


# ------------------------------------------------- peer exchange: host-side arithmetic and refusals

def test_peer_exchange_sizes_and_argument_checks_need_no_device():
    import ctypes

    from attnarc_b200 import _native

    lib = _native.library()
    header = 192  # step counter, ticket, error word, 16 arrival counters, reserve
    assert lib.loom_cuda_peer_exchange_bytes(8, 256, 128) == header + 2 * 8 * 256 * 130 * 4
    assert lib.loom_cuda_peer_exchange_bytes(1, 2, 126) == header + 2 * 1 * 2 * 128 * 4
    for world, rows, dim in ((0, 8, 128), (17, 8, 128), (2, 0, 128), (2, 8, 0), (2, 1, 129)):
        assert lib.loom_cuda_peer_exchange_bytes(world, rows, dim) == 0  # too many ranks, empty, or not 16-byte rows
    fake = 0x100000
    buffers = (ctypes.c_void_p * 2)(fake, fake)
    # refused before any CUDA call: misaligned states, rank outside the world, a missing peer buffer, bad dtype
    assert lib.loom_cuda_peer_exchange_push(fake + 4, buffers, 0, 2, 8, 128, None) == 1
    assert lib.loom_cuda_peer_exchange_push(fake, buffers, 2, 2, 8, 128, None) == 1
    assert lib.loom_cuda_peer_exchange_push(fake, (ctypes.c_void_p * 2)(fake, None), 0, 2, 8, 128, None) == 1
    assert lib.loom_cuda_peer_exchange_merge(fake, 2, 8, 128, 3, fake, None) == 1
    assert lib.loom_cuda_peer_exchange_merge(None, 2, 8, 128, 2, fake, None) == 1
    handle = ctypes.create_string_buffer(64)
    out = ctypes.c_void_p()
    assert lib.loom_cuda_peer_exchange_create(16, ctypes.byref(out), handle, 64) == 1   # smaller than the header
    assert lib.loom_cuda_peer_exchange_create(4096, ctypes.byref(out), handle, 8) == 1  # no room for the handle
    assert lib.loom_cuda_peer_exchange_open(handle, 8, ctypes.byref(out)) == 1
