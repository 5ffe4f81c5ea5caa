"""The sharding plans of ``attnarc_b200.multi_gpu`` driven through the CUDA
operators on one device: every rank's part is decoded in turn, the partial
states are stacked as an all-gather would deliver them, and the merged result
is compared with the oracle's decode of the unsplit batch.
"""

import pytest
import torch

from attnarc_b200 import multi_gpu
from tests.helpers import assert_close, oracle_decode
from tests.test_multi_gpu_host import build_case

pytestmark = pytest.mark.gpu


def expected_output(query, keys, values, tables, lengths, scale):
    live = [i for i, n in enumerate(lengths) if n > 0]
    expected = torch.zeros((len(lengths), query.shape[1], values.shape[3]), dtype=query.dtype)
    expected[live] = oracle_decode(query[live], keys, values, tables[live],
                                   torch.tensor([lengths[i] for i in live], dtype=torch.int32),
                                   scale=scale, max_sequence_length=max(lengths))
    return expected


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_long_context_plan_merges_to_the_unsplit_result(ranks):
    from attnarc_b200 import ops

    query, keys, values, tables, lengths, block, scale = build_case(23)
    device = torch.device("cuda:0")
    q, k, v, t = (x.to(device) for x in (query, keys, values, tables))
    batch, heads, dim = q.shape
    stacked = torch.zeros((ranks, batch, heads, dim + 2), dtype=torch.float32, device=device)
    stacked[:, :, :, dim] = float("-inf")
    plans = multi_gpu.plan_long_context(lengths, ranks, block, split_threshold_tokens=256)
    assert sum(p.tokens for p in plans) == sum(lengths)
    for plan in plans:
        if not plan.rows:
            continue
        local_q, local_t, local_n = multi_gpu.local_decode_inputs(plan, q, t)
        states = ops.paged_decode_attention_ex(local_q, k, v, local_t, local_n,
                                               max_sequence_length=max(plan.lengths + [1]), scale=scale,
                                               emit_state=True)
        stacked[plan.rank].index_copy_(0, torch.tensor(plan.rows, device=device), states)
    merged = ops.merge_decode_states(stacked.reshape(ranks, batch * heads, dim + 2).contiguous(), torch.bfloat16)
    assert_close(merged.reshape(batch, heads, dim).cpu(), expected_output(query, keys, values, tables, lengths, scale),
                 torch.bfloat16, f"{ranks} ranks")


def test_by_sequence_plan_covers_the_batch():
    query, keys, values, tables, lengths, block, scale = build_case(29)
    device = torch.device("cuda:0")
    q, k, v, t = (x.to(device) for x in (query, keys, values, tables))
    result = torch.zeros((len(lengths), q.shape[1], v.shape[3]), dtype=torch.bfloat16)
    for rank in range(3):
        rows, output = multi_gpu.decode_by_sequence(q, k, v, t, lengths, scale=scale, rank=rank, ranks=3)
        if rows:
            result[rows] = output.cpu()
    assert_close(result, expected_output(query, keys, values, tables, lengths, scale), torch.bfloat16, "by sequence")


# ---- the rank steps of attnarc_b200.sharded_step, one rank after the other on one GPU ----------

def _small_case(name, batch, lengths, seed):
    from attnarc_b200 import workloads

    config = workloads.scaled(workloads.CONFIGS[name], batch=batch, lengths=("fixed", lengths))
    return config, workloads.build_case(config, torch.device("cuda:0"), seed=seed)


def _oracle_rows(case):
    """Oracle attention rows of the global batch after the oracle's own RoPE + KV write."""
    from tests.helpers import oracle_rope_write

    config = case.config
    key_view, value_view = case.cache_views()
    fp8 = config.cache == "fp8"
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if fp8 else {}
    query, _, key_cache, value_cache = oracle_rope_write(
        case.query, case.key, case.value, case.positions, case.cos_sin_cache, key_view, value_view,
        case.slot_mapping, is_neox=config.rope_style == "neox", key_scales=case.key_scales,
        value_scales=case.value_scales)
    return oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                         scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)


def _step(shard, case):
    from attnarc_b200 import sharded_step

    config = case.config
    # one process emulates the ranks here: no process group exists, so the exchange buffers of the NCCL
    # form (plain tensors) are asked for; the exchange itself is not run by these tests
    return sharded_step.ShardedDecodeStep(shard, case.cos_sin_cache, dtype=config.torch_dtype, scale=case.scale,
                                          is_neox=config.rope_style == "neox",
                                          partition_tokens=config.partition_tokens, exchange="nccl")


@pytest.mark.parametrize("name,mode,ranks", [("cfg3", "by sequence", 4), ("cfg2", "by sequence", 8),
                                             ("cfg4", "by KV head", 8), ("cfg4", "by KV head", 2)])
def test_rank_steps_without_exchange_cover_the_batch(name, mode, ranks):
    from attnarc_b200 import sharded_step

    config, case = _small_case(name, 6, [700, 33, 1500, 16, 257, 1024], seed=31)
    expected = _oracle_rows(case)
    result = torch.zeros_like(expected)
    seen = torch.zeros(expected.shape[:2], dtype=torch.int32)
    local_bytes = 0
    for rank in range(ranks):
        shard = sharded_step.SHARDERS[mode](case, rank, ranks)
        local_bytes += shard.kv_bytes
        assert shard.kv_cache.data_ptr() != case.kv_cache.data_ptr()  # the rank holds its own pages only
        step = _step(shard, case)
        eager = step.run_eager().clone()
        rows = step.capture().run()  # the captured step repeats the eager one bit for bit
        assert torch.equal(rows.view(torch.int16), eager.view(torch.int16))
        placed = sharded_step.gather_rows(shard, rows, expected.shape)
        first, count = shard.query_heads
        if shard.rows:
            result[shard.rows, first:first + count] = placed[shard.rows, first:first + count]
            seen[shard.rows, first:first + count] += 1
    assert bool((seen == 1).all()), "every (sequence, query head) row belongs to exactly one rank"
    assert local_bytes == case.kv_bytes
    assert_close(result, expected, config.torch_dtype, f"{name} {mode} x{ranks}")


@pytest.mark.parametrize("ranks", [2, 8])
def test_long_context_rank_steps_merge_to_the_oracle(ranks):
    from attnarc_b200 import ops, sharded_step

    config, case = _small_case("cfg5", 4, [9000, 40, 700, 16], seed=37)
    expected = _oracle_rows(case)
    batch, heads, dim = expected.shape
    stacked = torch.zeros((ranks, batch * heads, dim + 2), dtype=torch.float32, device="cuda:0")
    writers = 0
    for rank in range(ranks):
        shard = sharded_step.shard_long_context(case, rank, ranks)
        assert shard.exchange and shard.sequences == batch
        writers += int((shard.slot_mapping >= 0).sum())
        step = _step(shard, case)
        step.upload()
        step.enqueue_kernels(exchange=False)  # this rank's states of every row (empty where it holds nothing)
        stacked[rank] = step._states.view(batch * heads, dim + 2)
    assert writers == batch, "the new token of every sequence is written by exactly one rank"
    merged = ops.merge_decode_states(stacked, config.torch_dtype).view(batch, heads, dim)
    assert_close(merged.cpu(), expected, config.torch_dtype, f"long context x{ranks}")


# ---- the merge of partial states itself: few parts (eight per round trip) and many (four groups of
# 32 threads, from 17 parts on), against the log-sum-exp merge written out in F64 ------------------------

@pytest.mark.parametrize("parts", [1, 3, 16, 17, 40, 131])
@pytest.mark.parametrize("dim", [64, 128, 256])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_merge_of_states_matches_the_log_sum_exp_merge(parts, dim, out_dtype):
    from attnarc_b200 import ops

    rows = 37
    generator = torch.Generator(device="cuda:0").manual_seed(parts * 1000 + dim)
    states = torch.randn((parts, rows, dim + 2), device="cuda:0", generator=generator)
    states[..., dim] = states[..., dim] * 6.0                       # maxima in natural-log units
    states[..., dim + 1] = states[..., dim + 1].abs() + 0.1         # sums of exponentials
    if parts > 2:
        # parts that saw no token: sum 0, maximum -inf, whatever in O (must not matter)
        states[1, ::3, dim + 1] = 0.0
        states[1, ::3, dim] = float("-inf")
        states[parts - 1, 5, dim + 1] = 0.0
    merged = ops.merge_decode_states(states.contiguous(), out_dtype)
    wide = states.double().cpu()
    live = wide[..., dim + 1] > 0
    maxima = torch.where(live, wide[..., dim], torch.full_like(wide[..., dim], float("-inf")))
    top = maxima.max(dim=0).values
    factor = torch.where(live, torch.exp(maxima - top), torch.zeros_like(maxima))
    total = (wide[..., dim + 1] * factor).sum(dim=0)
    expected = (wide[..., :dim] * factor.unsqueeze(-1)).sum(dim=0) / total.unsqueeze(-1)
    assert_close(merged.cpu(), expected.float(), out_dtype, f"{parts} parts, Dv {dim}")


# ---- the exchange over peer memory (multi_gpu.PeerExchange), ranks emulated on one GPU ---------------
#
# Kernels that wait for each other must not run as separate launches on one device. The emulation
# therefore enqueues every rank's push before the first merge: each merge finds all parts in place
# and never waits for a later launch.

def _emulated_exchanges(world, rows, dim):
    import ctypes

    from attnarc_b200 import _native

    lib = _native.library()
    size = lib.loom_cuda_peer_exchange_bytes(world, rows, dim)
    assert size > 0
    buffers = [torch.zeros(size, dtype=torch.uint8, device="cuda:0") for _ in range(world)]
    pointers = [b.data_ptr() for b in buffers]
    return buffers, [multi_gpu.PeerExchange(rows, dim, rank=r, world=world, buffers=pointers) for r in range(world)]


@pytest.mark.parametrize("world", [1, 2, 8])
def test_peer_exchange_merges_like_the_merge_operator_step_after_step(world):
    from attnarc_b200 import ops

    rows, dim = 64, 128
    buffers, exchanges = _emulated_exchanges(world, rows, dim)
    generator = torch.Generator(device="cuda:0").manual_seed(world)
    for step in range(5):  # both generations of the buffers, counters that keep growing
        states = torch.randn((world, rows, dim + 2), device="cuda:0", generator=generator)
        states[:, :, dim + 1] = states[:, :, dim + 1].abs() + 0.1       # sums of exponentials are positive
        if world > 1:
            states[1, ::3, dim + 1] = 0.0                                # rank 1 holds nothing of every third row
            states[1, ::3, dim] = float("-inf")
        expected = ops.merge_decode_states(states.contiguous(), torch.float32)
        for rank, exchange in enumerate(exchanges):
            exchange.push(states[rank].contiguous())
        outputs = [exchange.merge(torch.empty((rows, dim), dtype=torch.float32, device="cuda:0"))
                   for exchange in exchanges]
        torch.cuda.synchronize()
        for rank, output in enumerate(outputs):
            # the same log-sum-exp merge, folded in another order
            assert torch.allclose(output, expected, rtol=1e-5, atol=1e-5), f"step {step} rank {rank}"
    assert all(exchange.status() == (5, 0) for exchange in exchanges)


def test_peer_exchange_reports_a_part_that_never_arrives():
    from attnarc_b200 import ops

    rows, dim = 8, 64
    buffers, exchanges = _emulated_exchanges(2, rows, dim)
    states = torch.rand((rows, dim + 2), device="cuda:0") + 0.5
    ops.set_wait_policy(attempts=2000)
    try:
        exchanges[0].push(states)  # rank 1 never pushes: rank 0's wait for it must run out, not hang
        output = exchanges[0].merge(torch.full((rows, dim), 7.0, dtype=torch.float32, device="cuda:0"))
        torch.cuda.synchronize()
    finally:
        ops.set_wait_policy()
    steps, error = exchanges[0].status()
    assert error == 1 and steps == 1
    assert bool((output == 0).all()), "rows of a step with a missing part are zeroed, never half merged"
    # after an error every rank resets its buffer; the next step is clean
    for exchange in exchanges:
        exchange.reset()
    for exchange in exchanges:
        exchange.push(states)
    merged = exchanges[1].merge(torch.empty((rows, dim), dtype=torch.float32, device="cuda:0"))
    exchanges[0].merge(torch.empty((rows, dim), dtype=torch.float32, device="cuda:0"))
    torch.cuda.synchronize()
    assert exchanges[1].status() == (1, 0)
    twice = torch.stack([states, states]).contiguous()
    assert torch.allclose(merged, ops.merge_decode_states(twice, torch.float32), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg4"])
def test_rows_stored_into_pinned_memory_by_the_last_kernel_equal_the_copied_rows(name):
    # rows_to_host: the pinned buffer is the kernels' output; no device-to-host copy follows them
    from attnarc_b200 import sharded_step

    config, case = _small_case(name, 5, [700, 33, 1500, 16, 4000], seed=41)
    shard = sharded_step.whole_case(case)
    common = dict(dtype=config.torch_dtype, scale=case.scale, is_neox=config.rope_style == "neox",
                  partition_tokens=config.partition_tokens)
    copied = sharded_step.ShardedDecodeStep(shard, case.cos_sin_cache, rope_cache=shard.rope_cache.clone(), **common)
    stored = sharded_step.ShardedDecodeStep(shard, case.cos_sin_cache, rope_cache=shard.rope_cache.clone(),
                                            rows_to_host=True, **common)
    assert stored.output.is_pinned() and stored.output.data_ptr() == stored.host_output.data_ptr()
    want = copied.run_eager().clone()
    assert torch.equal(stored.run_eager().view(torch.int16), want.view(torch.int16))
    stored.host_output.zero_()
    assert torch.equal(stored.capture().run().view(torch.int16), want.view(torch.int16))
    assert_close(want, _oracle_rows(case), config.torch_dtype, f"{name} rows to host")
