"""KV block movement on the GPU against the numpy oracle, bit for bit.

The reference has no implementation of these operators (it lists them as its
next ones), so parity is against ``oracle/kv_blocks.py`` and against
properties: gather -> scatter restores a cache, a swap is its own inverse, and
decode attention is unchanged by a compaction of the cache it reads.
"""

import numpy as np
import pytest
import torch

from oracle import kv_blocks
from tests import helpers

pytestmark = pytest.mark.gpu

DEVICE = torch.device("cuda:0")
DTYPES = {"bf16": torch.bfloat16, "f32": torch.float32, "fp8": torch.uint8}


def make_cache(rng, blocks, block_size, heads, dim, dtype, layout):
    """A packed allocation of random bytes and the [blocks, 2, ...] argument the operators take."""
    inner = (block_size, heads, dim) if layout == "NHD" else (heads, block_size, dim)
    width = torch.empty((), dtype=dtype).element_size()
    raw = torch.from_numpy(rng.integers(0, 256, size=(blocks, 2) + inner + (width,), dtype=np.uint8))
    allocation = raw.view(dtype).reshape((blocks, 2) + inner).to(DEVICE)
    argument = allocation if layout == "NHD" else allocation.permute(0, 1, 3, 2, 4)
    return allocation, argument


def block_bytes_of(allocation):
    """[blocks, 2, block_bytes] uint8 on the host, in memory order."""
    return allocation.contiguous().view(torch.uint8).reshape(allocation.shape[0], 2, -1).cpu().numpy()


@pytest.fixture(params=["bulk", "vector"])
def engine(request):
    """Both ways the move kernel moves bytes; the default is restored afterwards."""
    from attnarc_b200 import ops

    ops.set_kv_block_move_engine(request.param)
    yield request.param
    ops.set_kv_block_move_engine("bulk")
    assert ops.kv_block_move_timeout_flag() == 0


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("dtype", ["bf16", "f32", "fp8"])
@pytest.mark.parametrize("same_cache", [True, False])
def test_move_matches_the_oracle(layout, dtype, same_cache, engine):
    from attnarc_b200 import ops

    rng = np.random.default_rng(sum(map(ord, layout + dtype)) + int(same_cache))
    blocks = 37
    source_allocation, source = make_cache(rng, blocks, 16, 3, 64, DTYPES[dtype], layout)
    if same_cache:
        destination_allocation, destination = source_allocation, source
        order = rng.permutation(blocks)
        from_ids, to_ids = order[:15], order[15:30]           # disjoint: nothing both read and written
    else:
        destination_allocation, destination = make_cache(rng, 29, 16, 3, 64, DTYPES[dtype], layout)
        from_ids, to_ids = rng.integers(0, blocks, size=15), rng.permutation(29)[:15]
    pairs = np.stack([from_ids, to_ids], axis=1).astype(np.int64)
    pairs = np.concatenate([pairs, [[-1, to_ids[0]], [from_ids[0], 10_000], [blocks, 2]]]).astype(np.int64)
    want = kv_blocks.kv_block_move(block_bytes_of(destination_allocation), block_bytes_of(source_allocation), pairs)
    before = ops.kv_block_movement_launches()
    ops.kv_block_move_(destination, source, torch.from_numpy(pairs).to(DEVICE))
    torch.cuda.synchronize()
    assert np.array_equal(block_bytes_of(destination_allocation), want)
    assert ops.kv_block_movement_launches() == before + 1


@pytest.mark.parametrize("block_size,heads,dim", [(16, 8, 128), (32, 1, 64), (16, 5, 80), (1, 1, 16), (16, 9, 120)])
def test_move_covers_block_sizes_around_the_chunk_size(block_size, heads, dim, engine):
    from attnarc_b200 import ops

    rng = np.random.default_rng(block_size * 1000 + heads * 10 + dim)
    allocation, cache = make_cache(rng, 21, block_size, heads, dim, torch.bfloat16, "NHD")
    order = rng.permutation(21)
    pairs = np.stack([order[:10], order[10:20]], axis=1).astype(np.int64)
    want = kv_blocks.kv_block_move(block_bytes_of(allocation), block_bytes_of(allocation), pairs)
    ops.kv_block_move_(cache, cache, torch.from_numpy(pairs).to(DEVICE))
    torch.cuda.synchronize()
    assert np.array_equal(block_bytes_of(allocation), want)


@pytest.mark.parametrize("layout", ["NHD", "HND"])
def test_swap_matches_the_oracle_and_undoes_itself(layout, engine):
    from attnarc_b200 import ops

    rng = np.random.default_rng(7)
    allocation, cache = make_cache(rng, 33, 16, 4, 128, torch.bfloat16, layout)
    original = block_bytes_of(allocation)
    order = rng.permutation(33)
    pairs = np.stack([order[:12], order[12:24]], axis=1).astype(np.int64)
    pairs = np.concatenate([pairs, [[order[30], order[30]], [-3, order[31]], [order[32], 33]]]).astype(np.int64)
    device_pairs = torch.from_numpy(pairs).to(DEVICE)
    ops.kv_block_swap_(cache, device_pairs)
    torch.cuda.synchronize()
    assert np.array_equal(block_bytes_of(allocation), kv_blocks.kv_block_swap(original, pairs))
    ops.kv_block_swap_(cache, device_pairs)
    torch.cuda.synchronize()
    assert np.array_equal(block_bytes_of(allocation), original)


def test_table_remap_matches_the_oracle():
    from attnarc_b200 import ops

    rng = np.random.default_rng(9)
    blocks = 500
    tables = rng.integers(-2, blocks + 3, size=(64, 257)).astype(np.int32)
    new_ids = rng.permutation(blocks).astype(np.int32)
    device_tables = torch.from_numpy(tables).to(DEVICE)
    ops.block_table_remap_(device_tables, torch.from_numpy(new_ids).to(DEVICE))
    assert np.array_equal(device_tables.cpu().numpy(), kv_blocks.block_table_remap(tables, new_ids))


def test_empty_calls_and_rejected_shapes():
    from attnarc_b200 import BridgeError, ops

    rng = np.random.default_rng(11)
    allocation, cache = make_cache(rng, 5, 16, 2, 64, torch.bfloat16, "NHD")
    original = block_bytes_of(allocation)
    empty = torch.zeros((0, 2), dtype=torch.int64, device=DEVICE)
    ops.kv_block_move_(cache, cache, empty)
    ops.kv_block_swap_(cache, empty)
    torch.cuda.synchronize()
    assert np.array_equal(block_bytes_of(allocation), original)
    with pytest.raises(RuntimeError, match=r"int64 \[pairs, 2\]"):
        ops.kv_block_move_(cache, cache, torch.zeros((3, 2), dtype=torch.int32, device=DEVICE))
    with pytest.raises(RuntimeError, match="dense in memory"):
        ops.kv_block_move_(cache[:, :, :, :1], cache[:, :, :, :1], empty)   # one head of two: gaps inside a block
    odd = torch.zeros((4, 2, 3, 1, 5), dtype=torch.uint8, device=DEVICE)     # 15-byte blocks
    with pytest.raises(BridgeError, match="16 bytes"):
        ops.kv_block_move_(odd, odd, torch.tensor([[0, 1]], dtype=torch.int64, device=DEVICE))


def test_decode_is_unchanged_by_a_compaction_of_its_cache():
    """Pack the live blocks to the front, rewrite the tables, and attend again."""
    from attnarc_b200 import ops, workloads

    config = workloads.scaled(workloads.CONFIGS["cfg2"], batch=6)
    case = workloads.build_case(config, DEVICE, seed=3)
    key_cache, value_cache = case.cache_views()

    def attend(tables):
        return ops.paged_decode_attention_ex(case.query, key_cache, value_cache, tables, case.sequence_lengths,
                                             max_sequence_length=case.max_sequence_length, scale=case.scale)

    before = attend(case.block_tables).clone()
    tables = case.block_tables.cpu().numpy()
    lengths = case.sequence_lengths.cpu().numpy()
    live = np.zeros(case.num_blocks, dtype=bool)
    for row, length in zip(tables, lengths):
        live[row[: (length + config.block_size - 1) // config.block_size]] = True
    pairs, new_ids = kv_blocks.compaction_plan(live)
    assert len(pairs) > 0  # the seeded tables scatter blocks over the pool
    ops.kv_block_move_(case.rope_cache_argument(), case.rope_cache_argument(), torch.from_numpy(pairs).to(DEVICE))
    new_tables = case.block_tables.clone()
    ops.block_table_remap_(new_tables, torch.from_numpy(new_ids).to(DEVICE))
    assert int(new_tables.max()) < int(live.sum())
    # the blocks that moved away no longer matter: poison them
    freed = torch.from_numpy(pairs[:, 0]).to(DEVICE)
    case.kv_cache[freed] = float("nan")
    after = attend(new_tables)
    assert helpers.same_bits(before, after)


def test_gather_then_scatter_restores_a_gigabyte_cache(engine):
    from attnarc_b200 import ops

    blocks, block_size, heads, dim = 2048, 16, 8, 128   # 2048 x 2 x 32 KB x 2 B = 0.27 GB per cache
    generator = torch.Generator(device=DEVICE).manual_seed(5)
    cache = torch.randint(-32768, 32767, (blocks, 2, block_size, heads, dim), device=DEVICE, dtype=torch.int16,
                          generator=generator).view(torch.bfloat16)
    original = cache.clone()
    staging = torch.zeros_like(cache)
    order = torch.randperm(blocks, device=DEVICE, generator=generator)
    gather = torch.stack([order, torch.arange(blocks, device=DEVICE)], dim=1).contiguous()
    ops.kv_block_move_(staging, cache, gather)
    assert helpers.same_bits(staging[7], original[int(order[7])])
    cache.zero_()
    ops.kv_block_move_(cache, staging, gather.flip(1).contiguous())
    assert helpers.same_bits(cache, original)


def test_blocks_swap_out_to_pinned_host_memory_and_back_in():
    """Preemption and resume: device cache -> pinned host cache -> other blocks of the device cache."""
    from attnarc_b200 import ops

    rng = np.random.default_rng(21)
    allocation, cache = make_cache(rng, 40, 16, 4, 128, torch.bfloat16, "NHD")
    original = block_bytes_of(allocation)
    host_cache = torch.zeros((12, 2, 16, 4, 128), dtype=torch.bfloat16).pin_memory()
    order = rng.permutation(40)
    out_pairs = np.stack([order[:10], np.arange(10)], axis=1).astype(np.int64)      # device block -> host slot
    ops.kv_block_move_(host_cache, cache, torch.from_numpy(out_pairs).to(DEVICE))
    torch.cuda.synchronize()
    want_host = kv_blocks.kv_block_move(np.zeros((12, 2, original.shape[2]), dtype=np.uint8), original, out_pairs)
    assert np.array_equal(host_cache.view(torch.uint8).reshape(12, 2, -1).numpy(), want_host)

    allocation[torch.from_numpy(order[:10]).to(DEVICE)] = 0                           # the blocks are given away
    in_pairs = np.stack([np.arange(10), order[10:20]], axis=1).astype(np.int64)      # host slot -> other blocks
    ops.kv_block_move_(cache, host_cache, torch.from_numpy(in_pairs).to(DEVICE))
    torch.cuda.synchronize()
    after = block_bytes_of(allocation)
    for slot in range(10):
        assert np.array_equal(after[order[10 + slot]], original[order[slot]])
        assert not after[order[slot]].any()
    assert ops.kv_block_move_timeout_flag() == 0

    pageable = torch.zeros((12, 2, 16, 4, 128), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="pinned host memory"):
        ops.kv_block_move_(pageable, cache, torch.from_numpy(out_pairs).to(DEVICE))
