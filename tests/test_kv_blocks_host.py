"""KV block movement without a GPU: the numpy oracle's own properties and the
bridge's argument checks (which run before anything touches CUDA)."""

import ctypes

import numpy as np
import pytest

from oracle import kv_blocks


def random_cache(rng, blocks=12, block_bytes=48):
    return rng.integers(0, 256, size=(blocks, 2, block_bytes), dtype=np.uint8)


def test_move_copies_named_blocks_and_skips_ids_outside_the_cache():
    rng = np.random.default_rng(0)
    cache = random_cache(rng)
    pairs = np.array([[0, 7], [3, 8], [-1, 9], [4, 12], [99, 10]], dtype=np.int64)
    moved = kv_blocks.kv_block_move(cache, cache, pairs)
    assert np.array_equal(moved[7], cache[0]) and np.array_equal(moved[8], cache[3])
    untouched = [b for b in range(12) if b not in (7, 8)]
    assert np.array_equal(moved[untouched], cache[untouched])


def test_gather_then_scatter_restores_the_cache():
    rng = np.random.default_rng(1)
    cache = random_cache(rng)
    order = rng.permutation(12)
    gather = np.stack([order, np.arange(12)], axis=1)
    staged = kv_blocks.kv_block_move(np.zeros_like(cache), cache, gather)
    back = kv_blocks.kv_block_move(np.zeros_like(cache), staged, gather[:, ::-1])
    assert np.array_equal(back, cache)


def test_swap_is_its_own_inverse():
    rng = np.random.default_rng(2)
    cache = random_cache(rng)
    pairs = np.array([[0, 5], [2, 2], [3, 11], [4, 40]], dtype=np.int64)
    once = kv_blocks.kv_block_swap(cache, pairs)
    assert np.array_equal(once[0], cache[5]) and np.array_equal(once[5], cache[0])
    assert np.array_equal(once[2], cache[2]) and np.array_equal(once[4], cache[4])
    assert np.array_equal(kv_blocks.kv_block_swap(once, pairs), cache)


def test_compaction_plan_keeps_every_live_block_reachable():
    rng = np.random.default_rng(3)
    for _ in range(20):
        blocks = int(rng.integers(1, 40))
        live = rng.random(blocks) < 0.5
        cache = random_cache(rng, blocks=blocks)
        pairs, new_ids = kv_blocks.compaction_plan(live)
        assert not set(pairs[:, 0]) & set(pairs[:, 1])           # nothing both read and written
        assert len(set(pairs[:, 1])) == len(pairs)               # no destination twice
        compacted = kv_blocks.kv_block_move(cache, cache, pairs)
        count = int(live.sum())
        for block in np.flatnonzero(live):
            assert new_ids[block] < count
            assert np.array_equal(compacted[new_ids[block]], cache[block])
        tables = np.where(rng.random((3, 7)) < 0.3, -1,
                          rng.choice(np.flatnonzero(live), size=(3, 7)) if count else -1).astype(np.int32)
        remapped = kv_blocks.block_table_remap(tables, new_ids)
        assert np.array_equal(remapped[tables < 0], tables[tables < 0])
        for old, new in zip(tables[tables >= 0], remapped[tables >= 0]):
            assert np.array_equal(compacted[new], cache[old])


# ---- bridge argument checks ----------------------------------------------------------------

@pytest.fixture(scope="module")
def lib():
    from attnarc_b200 import _native

    return _native.library()


def last_error(lib):
    return lib.loom_cuda_bridge_last_error_message().decode()


def test_move_rejects_bad_arguments_before_any_launch(lib):
    buffer = (ctypes.c_uint8 * 4096)()
    base = (ctypes.addressof(buffer) + 15) // 16 * 16
    pairs = (ctypes.c_int64 * 4)(0, 1, 1, 2)
    ok = dict(block=64, stride=128, blocks=4, span=4 * 128)

    def call(source=base, span=ok["span"], pair_elements=4, block=ok["block"], stride=ok["stride"], pair_pointer=None):
        return lib.loom_cuda_bridge_kv_block_move(
            source, span, base + 64, span, base + 2048, span, base + 2048 + 64, span,
            pair_pointer if pair_pointer is not None else ctypes.addressof(pairs), pair_elements, ok["blocks"],
            ok["blocks"], block, stride, stride, stride, stride, None)

    assert call(source=None) == 1 and "source key cache pointer is null" in last_error(lib)
    assert call(source=base + 8) == 1 and "not aligned to 16 bytes" in last_error(lib)
    assert call(pair_elements=3) == 1 and "two ids per pair" in last_error(lib)
    assert call(span=3 * 128) == 1 and "shorter than its 4 blocks need" in last_error(lib)
    assert call(block=256) == 1 and "smaller than a block" in last_error(lib)
    assert call(block=40, stride=120) == 1 and "multiples of 16 bytes" in last_error(lib)
    assert call(pair_pointer=base + 2048) == 1 and "must not overlap" in last_error(lib)


def test_swap_and_remap_reject_bad_arguments(lib):
    buffer = (ctypes.c_uint8 * 2048)()
    base = (ctypes.addressof(buffer) + 15) // 16 * 16
    pairs = (ctypes.c_int64 * 2)(0, 1)
    assert lib.loom_cuda_bridge_kv_block_swap(None, 512, base + 64, 512, ctypes.addressof(pairs), 2, 4, 64, 128, 128,
                                              None) == 1
    assert "key cache pointer is null" in last_error(lib)
    assert lib.loom_cuda_bridge_kv_block_swap(base, 512, base + 64, 512, ctypes.addressof(pairs), 1, 4, 64, 128, 128,
                                              None) == 1
    assert "two ids per pair" in last_error(lib)
    ids = (ctypes.c_int32 * 4)(0, 1, 2, 3)
    assert lib.loom_cuda_bridge_block_table_remap(base, 16, None, 4, None) == 1
    assert "new block ids pointer is null" in last_error(lib)
    assert lib.loom_cuda_bridge_block_table_remap(ctypes.addressof(ids), 4, ctypes.addressof(ids), 4, None) == 1
    assert "must not overlap" in last_error(lib)


def test_zero_counts_succeed_without_a_device(lib):
    buffer = (ctypes.c_uint8 * 2048)()
    base = (ctypes.addressof(buffer) + 15) // 16 * 16
    assert lib.loom_cuda_bridge_kv_block_move(base, 512, base + 64, 512, base + 1024, 512, base + 1088, 512, None, 0,
                                              4, 4, 64, 128, 128, 128, 128, None) == 0
    assert lib.loom_cuda_bridge_kv_block_swap(base, 512, base + 64, 512, None, 0, 4, 64, 128, 128, None) == 0
    ids = (ctypes.c_int32 * 4)(0, 1, 2, 3)
    assert lib.loom_cuda_bridge_block_table_remap(None, 0, ctypes.addressof(ids), 4, None) == 0
