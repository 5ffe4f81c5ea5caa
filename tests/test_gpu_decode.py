"""GPU parity of the paged decode against the CPU oracle, through the C ABI.

Every case runs the CUDA path (``attnarc_b200.ops`` -> bridge ABI ->
dispatch -> launch ABI -> kernels) and compares with the oracle on identical
seeded inputs. Tolerances: rtol = atol = 1e-4 for F32 and 1e-2 for F16/BF16.
The shape matrix is the one the reference's Python tests use
(python/tests/test_paged_decode_attention.py:110-137); the two fixtures of its
Rust wrapper tests (crates/loom-cuda/src/attention_dispatch.rs:487-606) are
replayed as well.
"""

import math

import numpy as np
import pytest
import torch

from tests import helpers
from attnarc_b200 import workloads

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


@pytest.fixture(scope="module")
def ops():
    from attnarc_b200 import ops as module

    return module


def make_case(dtype, sequences, query_heads, kv_heads, head_size, value_head_size, block_size, lengths,
              seed, interleaved=False):
    generator = torch.Generator().manual_seed(seed)
    max_blocks = math.ceil(max(lengths) / block_size)
    num_blocks = sequences * max_blocks + 7
    query = torch.randn((sequences, query_heads, head_size), generator=generator).to(dtype)
    if interleaved:
        kv = torch.randn((num_blocks, 2, block_size, kv_heads, head_size), generator=generator).to(dtype)
        kv = kv.to(DEVICE)
        key_cache, value_cache = kv[:, 0], kv[:, 1]
    else:
        key_cache = torch.randn((num_blocks, block_size, kv_heads, head_size), generator=generator).to(dtype).to(DEVICE)
        value_cache = torch.randn((num_blocks, block_size, kv_heads, value_head_size), generator=generator).to(dtype).to(DEVICE)
    tables = torch.randperm(num_blocks, generator=generator)[: sequences * max_blocks]
    tables = tables.reshape(sequences, max_blocks).to(torch.int32)
    return (query.to(DEVICE), key_cache, value_cache, tables.to(DEVICE),
            torch.tensor(lengths, dtype=torch.int32, device=DEVICE))


REFERENCE_SHAPES = [
    (3, 8, 1, 32, 24, 16, [1, 17, 31]),
    (4, 8, 2, 64, 64, 16, [16, 33, 64, 7]),
    (3, 12, 4, 80, 48, 32, [63, 129, 255]),
    (2, 8, 2, 128, 96, 32, [257, 511]),
    (16, 32, 8, 32, 24, 16, list(range(17, 33))),
    (2, 8, 2, 33, 17, 8, [17, 23]),
    (2, 14, 2, 64, 64, 16, [17, 32]),
    (64, 14, 2, 64, 64, 16, list(range(17, 33)) * 4),
    (1, 32, 8, 128, 128, 16, [128]),
    (4, 32, 8, 128, 128, 16, [512, 501, 489, 477]),
    (8, 32, 8, 128, 128, 32, list(range(491, 499))),
    (2, 14, 2, 128, 128, 16, [129, 256]),
    (1, 8, 8, 128, 128, 16, [257]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", REFERENCE_SHAPES, ids=[str(i) for i in range(len(REFERENCE_SHAPES))])
def test_reference_shape_matrix(ops, dtype, shape):
    sequences, query_heads, kv_heads, head_size, value_head_size, block_size, lengths = shape
    query, key_cache, value_cache, tables, seq_lens = make_case(
        dtype, sequences, query_heads, kv_heads, head_size, value_head_size, block_size, lengths, seed=len(lengths))
    scale = head_size ** -0.5
    expected = helpers.oracle_decode(query, key_cache, value_cache, tables, seq_lens, scale=scale,
                                     max_sequence_length=max(lengths))
    assert ops.supports_paged_decode_attention(query, key_cache, value_cache, tables, seq_lens,
                                               max_sequence_length=max(lengths))
    actual = ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens,
                                        max_sequence_length=max(lengths), scale=scale)
    helpers.assert_close(actual, expected, dtype, "reference-shaped entry point")
    # the same case through the partitioned path with a small partition
    split = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, seq_lens,
                                          max_sequence_length=max(lengths), scale=scale,
                                          partition_tokens=64, split=True)
    helpers.assert_close(split, expected, dtype, "partitioned path")
    # and through the library's own choice of partitioned kernel (balanced where it applies)
    balanced = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, seq_lens,
                                             max_sequence_length=max(lengths), scale=scale, split=True)
    helpers.assert_close(balanced, expected, dtype, "balanced path")


def test_expected_kernel_routes(ops):
    query, key_cache, value_cache, tables, seq_lens = make_case(torch.bfloat16, 2, 8, 2, 128, 128, 16, [40, 70], 1)
    ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=70)
    assert ops.last_decode_route() == "mma16"
    ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=70,
                                  split=True)
    assert ops.last_decode_route() == "mma16-balanced-tma"
    ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=70,
                                  split=True, partition_tokens=32)
    assert ops.last_decode_route() == "mma16"
    query, key_cache, value_cache, tables, seq_lens = make_case(torch.float32, 2, 8, 2, 128, 128, 16, [40, 70], 1)
    ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=70)
    assert ops.last_decode_route() == "scalar"
    query, key_cache, value_cache, tables, seq_lens = make_case(torch.float16, 2, 8, 2, 80, 48, 16, [40, 70], 1)
    ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=70)
    assert ops.last_decode_route() == "scalar"


def test_rust_wrapper_fixture_base(ops):
    # attention_dispatch.rs:487-540, tolerance 2e-5 there.
    q = torch.tensor([(i - 9.0) * 0.07 for i in range(32)], dtype=torch.float32).reshape(2, 4, 4)
    k = torch.tensor([(np.float32(i) % np.float32(13.0) - 6.0) * 0.11 for i in range(64)], dtype=torch.float32)
    v = torch.tensor([(np.float32(i) % np.float32(17.0) - 8.0) * 0.09 for i in range(48)], dtype=torch.float32)
    k, v = k.reshape(4, 2, 2, 4).to(DEVICE), v.reshape(4, 2, 2, 3).to(DEVICE)
    tables = torch.tensor([[2, 0], [1, 3]], dtype=torch.int32, device=DEVICE)
    lens = torch.tensor([3, 2], dtype=torch.int32, device=DEVICE)
    expected = helpers.oracle_decode(q, k, v, tables, lens, scale=0.5, max_sequence_length=4)
    actual = ops.paged_decode_attention(q.to(DEVICE), k, v, tables, lens, max_sequence_length=4, scale=0.5)
    assert (actual.cpu() - expected).abs().max().item() <= 2.0e-5


def test_rust_wrapper_fixture_split_k(ops):
    # attention_dispatch.rs:542-606, tolerance 2e-4 there.
    q = torch.tensor([(i % 29 - 14.0) * 0.013 for i in range(512)], dtype=torch.float32).reshape(1, 4, 128)
    k = torch.tensor([(i % 37 - 18.0) * 0.011 for i in range(8 * 16 * 128)], dtype=torch.float32)
    v = torch.tensor([(i % 41 - 20.0) * 0.009 for i in range(8 * 16 * 128)], dtype=torch.float32)
    k, v = k.reshape(8, 16, 1, 128).to(DEVICE), v.reshape(8, 16, 1, 128).to(DEVICE)
    tables = torch.arange(8, dtype=torch.int32, device=DEVICE).reshape(1, 8)
    lens = torch.tensor([128], dtype=torch.int32, device=DEVICE)
    expected = helpers.oracle_decode(q, k, v, tables, lens, scale=0.125, max_sequence_length=128)
    actual = ops.paged_decode_attention_ex(q.to(DEVICE), k, v, tables, lens, max_sequence_length=128,
                                           scale=0.125, partition_tokens=32, split=True)
    assert (actual.cpu() - expected).abs().max().item() <= 2.0e-4


def test_vllm_interleaved_cache_views(ops):
    # K and V are views of one [blocks, 2, block, heads, D] allocation
    # (python/tests/test_paged_decode_attention.py:186-230).
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        query, key_cache, value_cache, tables, seq_lens = make_case(
            dtype, 3, 8, 2, 128, 128, 16, [5, 130, 300], seed=9, interleaved=True)
        expected = helpers.oracle_decode(query, key_cache, value_cache, tables, seq_lens, scale=0.09,
                                         max_sequence_length=300)
        actual = ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens,
                                            max_sequence_length=300, scale=0.09)
        helpers.assert_close(actual, expected, dtype, "interleaved K/V views")


def test_runs_on_a_caller_stream(ops):
    query, key_cache, value_cache, tables, seq_lens = make_case(torch.bfloat16, 2, 8, 2, 128, 128, 16, [100, 200], 2)
    expected = helpers.oracle_decode(query, key_cache, value_cache, tables, seq_lens, scale=0.1,
                                     max_sequence_length=200)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        actual = ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens,
                                            max_sequence_length=200, scale=0.1)
    stream.synchronize()
    helpers.assert_close(actual, expected, torch.bfloat16, "side stream")


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("group", [(8, 8), (12, 2), (32, 8), (64, 8), (32, 2), (4, 4)])
def test_layouts_groups_and_partitions(ops, layout, dtype, group):
    query_heads, kv_heads = group
    config = workloads.DecodeConfig("t", 5, query_heads, kv_heads, dtype=dtype, layout=layout,
                                    lengths=("fixed", [1, 16, 257, 512, 700]))
    case = workloads.build_case(config, DEVICE, seed=query_heads + kv_heads)
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length)
    for partition, split in ((0, False), (0, True), (128, True), (256, True)):
        actual = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths,
                                               max_sequence_length=case.max_sequence_length, scale=case.scale,
                                               partition_tokens=partition, split=split)
        helpers.assert_close(actual, expected, config.torch_dtype, f"{layout} partition={partition} split={split}")


@pytest.mark.parametrize("granularity", ["tensor", "head"])
@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
def test_fp8_cache_dequantised_on_load(ops, granularity, dtype, layout):
    config = workloads.DecodeConfig("t", 4, 16, 2, dtype=dtype, cache="fp8", fp8_granularity=granularity,
                                    layout=layout, lengths=("fixed", [3, 64, 300, 1000]))
    case = workloads.build_case(config, DEVICE, seed=4)
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length,
                                     key_scales=case.key_scales, value_scales=case.value_scales)
    for partition, split in ((0, False), (0, True), (256, True)):
        actual = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths,
                                               max_sequence_length=case.max_sequence_length, scale=case.scale,
                                               key_scales=case.key_scales, value_scales=case.value_scales,
                                               partition_tokens=partition, split=split)
        helpers.assert_close(actual, expected, config.torch_dtype,
                             f"fp8 {granularity} partition={partition} split={split}")
    expected_route = "scalar-fp8" if dtype == "f32" else "mma16-fp8"
    assert ops.last_decode_route() == expected_route


@pytest.mark.parametrize("head_size", [64, 128])
@pytest.mark.parametrize("block_size", [8, 16, 32, 48])
def test_block_sizes_and_head_sizes(ops, head_size, block_size):
    lengths = [block_size - 1, block_size, block_size + 1, 5 * block_size + 3, 333]
    query, key_cache, value_cache, tables, seq_lens = make_case(
        torch.bfloat16, 5, 8, 2, head_size, head_size, block_size, lengths, seed=block_size)
    expected = helpers.oracle_decode(query, key_cache, value_cache, tables, seq_lens, scale=0.1,
                                     max_sequence_length=max(lengths))
    actual = ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens,
                                        max_sequence_length=max(lengths), scale=0.1)
    # blocks of a multiple of 16 tokens take the balanced kernel, others fixed partitions
    assert ops.last_decode_route() == ("mma16-balanced-tma" if block_size % 16 == 0 else "mma16")
    helpers.assert_close(actual, expected, torch.bfloat16, f"block_size={block_size}")


def test_unused_cache_slots_do_not_leak(ops):
    # Slots past the sequence length hold NaN; they must never reach the output.
    query, key_cache, value_cache, tables, seq_lens = make_case(torch.bfloat16, 3, 8, 2, 128, 128, 16, [1, 17, 40], 3)
    expected = helpers.oracle_decode(query, key_cache, value_cache, tables, seq_lens, scale=0.1,
                                     max_sequence_length=40)
    poisoned_k, poisoned_v = key_cache.clone(), value_cache.clone()
    for s, length in enumerate([1, 17, 40]):
        block = int(tables[s, (length - 1) // 16])
        poisoned_k[block, length % 16 if length % 16 else 16:] = float("nan")
        poisoned_v[block, length % 16 if length % 16 else 16:] = float("nan")
    actual = ops.paged_decode_attention(query, poisoned_k, poisoned_v, tables, seq_lens,
                                        max_sequence_length=40, scale=0.1)
    helpers.assert_close(actual, expected, torch.bfloat16, "poisoned tail slots")


def test_partial_states_merge_to_the_same_answer(ops):
    # Split a batch's context into two block ranges, decode each range to
    # (O, max, sum) states, merge: must equal the single-shot decode. This is
    # the arithmetic of the multi-GPU long-context mode on one device.
    config = workloads.DecodeConfig("t", 3, 32, 8, dtype="bf16", lengths=("fixed", [2048, 900, 4096]))
    case = workloads.build_case(config, DEVICE, seed=12)
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length)
    tables = case.block_tables
    half_blocks = tables.shape[1] // 2
    lengths = case.sequence_lengths
    first_len = torch.clamp(lengths, max=half_blocks * 16)
    second_len = torch.clamp(lengths - half_blocks * 16, min=0)
    states = []
    for sub_tables, sub_len in ((tables[:, :half_blocks].contiguous(), first_len),
                                (tables[:, half_blocks:].contiguous(), second_len)):
        states.append(ops.paged_decode_attention_ex(
            query, key_cache, value_cache, sub_tables, sub_len.to(torch.int32),
            max_sequence_length=sub_tables.shape[1] * 16, scale=case.scale, emit_state=True,
            partition_tokens=256, split=True))
    stacked = torch.stack([s.reshape(-1, s.shape[-1]) for s in states]).contiguous()
    merged = ops.merge_decode_states(stacked, torch.bfloat16).reshape(expected.shape)
    helpers.assert_close(merged, expected, torch.bfloat16, "merged states")
    # single-pass state emission agrees too
    whole = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, lengths,
                                          max_sequence_length=case.max_sequence_length, scale=case.scale,
                                          emit_state=True, split=False)
    merged_one = ops.merge_decode_states(whole.reshape(1, -1, whole.shape[-1]).contiguous(), torch.bfloat16)
    helpers.assert_close(merged_one.reshape(expected.shape), expected, torch.bfloat16, "single state")
    balanced = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, lengths,
                                             max_sequence_length=case.max_sequence_length, scale=case.scale,
                                             emit_state=True, split=True)
    merged_two = ops.merge_decode_states(balanced.reshape(1, -1, balanced.shape[-1]).contiguous(), torch.bfloat16)
    helpers.assert_close(merged_two.reshape(expected.shape), expected, torch.bfloat16, "balanced state")


def test_cfg1_f32_oracle_case(ops):
    case = workloads.build_case(workloads.CONFIGS["cfg1"], DEVICE, seed=1)
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length)
    actual = ops.paged_decode_attention(query, key_cache, value_cache, case.block_tables,
                                        case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                        scale=case.scale)
    helpers.assert_close(actual, expected, torch.float32, "cfg1")


def test_cfg2_full_size_against_the_oracle(ops):
    # The benchmark workload itself: 64 sequences of 512..4096 tokens, BF16.
    case = workloads.build_case(workloads.CONFIGS["cfg2"], DEVICE, seed=2)
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length)
    for split in (False, True):
        actual = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths,
                                               max_sequence_length=case.max_sequence_length, scale=case.scale,
                                               split=split)
        helpers.assert_close(actual, expected, torch.bfloat16, f"cfg2 split={split}")


@pytest.mark.parametrize("name", ["cfg3", "cfg4", "cfg5"])
def test_large_configs_at_full_size_against_the_oracle(ops, name):
    # The whole batch of each large configuration (256 sequences in an HND cache; 128 sequences
    # over a per-head FP8 cache; the skewed batch with its 131072-token row) against the F64
    # oracle on all host cores: the balanced schedule with items split across many CTAs, and the
    # caller-fixed 512-token partitions the Llama-3-8B-shaped configuration names.
    import os

    config = workloads.CONFIGS[name]
    case = workloads.build_case(config, DEVICE, seed=6, fast_device_fill=True)
    assert case.config.batch == config.batch and int(case.lengths.max()) == case.max_sequence_length
    if name == "cfg5":
        assert case.max_sequence_length == 131072
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if config.cache == "fp8" else {}
    threads = max(1, len(os.sched_getaffinity(0)))
    expected = helpers.oracle_decode(query, key_cache.contiguous(), value_cache.contiguous(), case.block_tables,
                                     case.sequence_lengths, scale=case.scale,
                                     max_sequence_length=case.max_sequence_length, threads=threads, **scales)
    routes = []
    for partition in (0, 512):
        actual = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths,
                                               max_sequence_length=case.max_sequence_length, scale=case.scale,
                                               partition_tokens=partition, split=True, **scales)
        routes.append(ops.last_decode_route())
        helpers.assert_close(actual, expected, config.torch_dtype, f"{name} partition_tokens={partition}")
    assert "balanced" in routes[0] and "balanced" not in routes[1], routes
    assert ops.decode_timeout_flag() == 0


def test_long_context_properties_at_full_length(ops):
    # 131072 tokens, size-independent checks: (1) if every V row equals one
    # vector the output is that vector whatever the scores; (2) the split path
    # equals the single pass; (3) permuting which physical blocks hold the
    # tokens (with the table following) changes nothing.
    length, heads, kv_heads, dim = 131072, 32, 8, 128
    blocks = length // 16
    generator = torch.Generator(device=DEVICE).manual_seed(7)
    key_cache = torch.randn((blocks + 3, 16, kv_heads, dim), device=DEVICE, dtype=torch.bfloat16, generator=generator)
    constant = torch.randn((kv_heads, dim), device=DEVICE, dtype=torch.bfloat16, generator=generator)
    value_cache = constant.expand(blocks + 3, 16, kv_heads, dim).contiguous()
    query = torch.randn((1, heads, dim), device=DEVICE, dtype=torch.bfloat16, generator=generator)
    tables = torch.randperm(blocks + 3, device=DEVICE)[:blocks].to(torch.int32).reshape(1, blocks)
    lens = torch.tensor([length], dtype=torch.int32, device=DEVICE)
    out = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, lens, max_sequence_length=length,
                                        partition_tokens=512, split=True)
    want = constant.repeat_interleave(heads // kv_heads, dim=0).unsqueeze(0)
    helpers.assert_close(out, want, torch.bfloat16, "constant V")

    value_cache = torch.randn((blocks + 3, 16, kv_heads, dim), device=DEVICE, dtype=torch.bfloat16, generator=generator)
    split = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, lens, max_sequence_length=length,
                                          partition_tokens=512, split=True)
    single = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, lens, max_sequence_length=length,
                                           split=False)
    helpers.assert_close(split, single, torch.bfloat16, "split vs single pass")
    balanced = ops.paged_decode_attention_ex(query, key_cache, value_cache, tables, lens,
                                             max_sequence_length=length, split=True)
    assert ops.last_decode_route() == "mma16-balanced-tma"
    helpers.assert_close(balanced, single, torch.bfloat16, "balanced vs single pass")

    shuffle = torch.randperm(blocks + 3, device=DEVICE)
    moved_k, moved_v = torch.empty_like(key_cache), torch.empty_like(value_cache)
    moved_k[shuffle] = key_cache
    moved_v[shuffle] = value_cache
    moved_tables = shuffle[tables.long()].to(torch.int32)
    moved = ops.paged_decode_attention_ex(query, moved_k, moved_v, moved_tables, lens, max_sequence_length=length,
                                          partition_tokens=512, split=True)
    assert torch.equal(moved, split), "block placement must not change the result"


def test_launch_counter_and_error_text(ops):
    query, key_cache, value_cache, tables, seq_lens = make_case(torch.bfloat16, 2, 8, 2, 128, 128, 16, [100, 200], 2)
    ops.reset_launch_count(ops.Operator.PAGED_DECODE_ATTENTION)
    ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=200)
    assert ops.launch_count(ops.Operator.PAGED_DECODE_ATTENTION) == 1
    with pytest.raises(RuntimeError, match="maximum sequence length 100000 exceeds block-table capacity"):
        ops.paged_decode_attention(query, key_cache, value_cache, tables, seq_lens, max_sequence_length=100000)
    with pytest.raises(RuntimeError, match="query head count 8 must be divisible by KV head count 3"):
        ops.paged_decode_attention(query, key_cache[:, :, :1].repeat(1, 1, 3, 1), value_cache[:, :, :1].repeat(1, 1, 3, 1),
                                   tables, seq_lens, max_sequence_length=200)
    with pytest.raises(RuntimeError, match="regions output and query must not overlap"):
        ops.paged_decode_attention_out(query, key_cache, value_cache, tables, seq_lens, query,
                                       max_sequence_length=200)
    assert ops.launch_count(ops.Operator.PAGED_DECODE_ATTENTION) == 1  # failures are not counted


@pytest.mark.parametrize("engine", ["cp_async", "tma", "tma-mma", "tma-umma"])
@pytest.mark.parametrize("cache", ["native", "fp8"])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("head_size", [64, 128])
def test_both_copy_engines_of_the_balanced_kernel(ops, engine, cache, layout, head_size):
    # ragged lengths: partial last pages, tiles with idle warps, items split over CTAs
    config = workloads.DecodeConfig("t", 7, 16, 2, head_size=head_size, dtype="bf16", cache=cache, layout=layout,
                                    lengths=("fixed", [1, 15, 16, 17, 63, 65, 3000]))
    case = workloads.build_case(config, DEVICE, seed=31)
    key_cache, value_cache = case.cache_views()
    query = case.query  # strided view of the packed QKV row
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if cache == "fp8" else {}
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    # stale contents after the end of each sequence must not matter to either engine
    poisoned_k, poisoned_v = key_cache.clone(), value_cache.clone()
    for s, length in enumerate(case.lengths.tolist()):
        if length % 16:
            block = int(case.block_tables[s, (length - 1) // 16])
            # NaN in the cache's own encoding (0x7f is the E4M3 NaN)
            poisoned_k[block, length % 16:] = float("nan") if cache == "native" else 0x7F
            poisoned_v[block, length % 16:] = float("nan") if cache == "native" else 0x7F
    ops.set_decode_copy_engine(engine)
    try:
        actual = ops.paged_decode_attention_ex(query, poisoned_k, poisoned_v, case.block_tables,
                                               case.sequence_lengths,
                                               max_sequence_length=case.max_sequence_length, scale=case.scale,
                                               split=True, **scales)
        route = ops.last_decode_route()
    finally:
        ops.set_decode_copy_engine("tma")
    assert route.endswith("-tma") == (engine != "cp_async")
    # the tcgen05 kernel covers FP8 caches with head size 128 and up to 8 query heads per KV head
    assert route.startswith("umma") == (engine == "tma-umma" and cache == "fp8" and head_size == 128)
    # over an FP8 cache the default engine's copies are issued by a warp of their own
    assert ("producer" in route) == (engine in ("tma", "tma-umma") and cache == "fp8" and not route.startswith("umma"))
    helpers.assert_close(actual, expected, torch.bfloat16, f"{engine} {cache} {layout} D={head_size}")
    assert ops.decode_timeout_flag() == 0


@pytest.mark.parametrize("sequences,route", [(1500, "mma16-balanced"), (2500, "mma16")])
def test_large_batches_fall_back_to_the_kernels_without_a_sequence_limit(ops, sequences, route):
    # the TMA-fed kernel keeps 1024 tile counts in shared memory, the cp.async one 2048
    lengths = [1 + (7 * i) % 90 for i in range(sequences)]
    config = workloads.DecodeConfig("many", sequences, 4, 2, head_size=64, dtype="bf16", lengths=("fixed", lengths))
    case = workloads.build_case(config, DEVICE, seed=3)
    key_cache, value_cache = case.cache_views()
    expected = helpers.oracle_decode(case.query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length)
    actual = ops.paged_decode_attention_ex(case.query, key_cache, value_cache, case.block_tables,
                                           case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                           scale=case.scale, split=True)
    assert ops.last_decode_route() == route
    helpers.assert_close(actual, expected, torch.bfloat16, f"{sequences} sequences")


def test_tcgen05_kernel_emits_states_that_merge(ops):
    config = workloads.DecodeConfig("t", 5, 16, 2, head_size=128, dtype="bf16", cache="fp8", fp8_granularity="head",
                                    lengths=("fixed", [3, 128, 129, 700, 2100]))
    case = workloads.build_case(config, DEVICE, seed=17)
    key_cache, value_cache = case.cache_views()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales)
    expected = helpers.oracle_decode(case.query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    ops.set_decode_copy_engine("tma-umma")
    try:
        states = ops.paged_decode_attention_ex(case.query, key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                               scale=case.scale, split=True, emit_state=True, **scales)
        route = ops.last_decode_route()
    finally:
        ops.set_decode_copy_engine("tma")
    assert route == "umma-fp8-balanced-tma" and states.dtype == torch.float32
    merged = ops.merge_decode_states(states.reshape(1, -1, states.shape[-1]).contiguous(), torch.bfloat16)
    helpers.assert_close(merged.reshape(expected.shape), expected, torch.bfloat16, "tcgen05 states")
    assert ops.decode_timeout_flag() == 0


# ---- the kernel whose tile is one 16-token block of eight KV heads (FP8 caches, KV heads in eights) ----

@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("query_heads,kv_heads", [(64, 8), (32, 16), (8, 8)])
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_block_of_eight_heads_per_tile(ops, layout, query_heads, kv_heads, dtype):
    # one token, partial last blocks, whole blocks, items split over CTAs
    config = workloads.DecodeConfig("t", 9, query_heads, kv_heads, head_size=128, dtype=dtype, cache="fp8",
                                    fp8_granularity="head", layout=layout,
                                    lengths=("fixed", [1, 15, 16, 17, 33, 3000, 4097, 640, 48]))
    case = workloads.build_case(config, DEVICE, seed=41)
    key_cache, value_cache = case.cache_views()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales)
    torch_dtype = config.torch_dtype
    expected = helpers.oracle_decode(case.query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    # stale contents after the end of each sequence must not matter (0x7f is the E4M3 NaN)
    poisoned_k, poisoned_v = key_cache.clone(), value_cache.clone()
    for s, length in enumerate(case.lengths.tolist()):
        if length % 16:
            block = int(case.block_tables[s, (length - 1) // 16])
            poisoned_k[block, length % 16:] = 0x7F
            poisoned_v[block, length % 16:] = 0x7F
    outputs = {}
    for engine in ("tma", "tma-head"):
        ops.set_decode_copy_engine(engine)
        try:
            outputs[engine] = ops.paged_decode_attention_ex(
                case.query, poisoned_k, poisoned_v, case.block_tables, case.sequence_lengths,
                max_sequence_length=case.max_sequence_length, scale=case.scale, split=True, **scales)
            route = ops.last_decode_route()
        finally:
            ops.set_decode_copy_engine("tma")
        assert route == ("mma16-fp8-balanced-block-tma" if engine == "tma" else "mma16-fp8-balanced-producer-tma")
        helpers.assert_close(outputs[engine], expected, torch_dtype, f"{engine} {layout} {query_heads}/{kv_heads}")
    assert ops.decode_timeout_flag() == 0


@pytest.mark.parametrize("block_size", [32, 64])
def test_block_of_eight_heads_with_larger_cache_blocks(ops, block_size):
    # a tile is 16 tokens, so a cache block of 32 or 64 tokens is copied in two or four pieces
    config = workloads.DecodeConfig("t", 5, 40, 8, head_size=128, block_size=block_size, dtype="bf16", cache="fp8",
                                    fp8_granularity="head", lengths=("fixed", [block_size - 1, block_size + 17, 1000, 16, 2500]))
    case = workloads.build_case(config, DEVICE, seed=47)
    key_cache, value_cache = case.cache_views()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales)
    expected = helpers.oracle_decode(case.query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    actual = ops.paged_decode_attention_ex(case.query, key_cache, value_cache, case.block_tables,
                                           case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                           scale=case.scale, split=True, **scales)
    assert ops.last_decode_route() == "mma16-fp8-balanced-block-tma"
    helpers.assert_close(actual, expected, torch.bfloat16, f"block size {block_size}")
    assert ops.decode_timeout_flag() == 0


def test_block_of_eight_heads_emits_states_that_merge(ops):
    config = workloads.DecodeConfig("t", 6, 48, 8, head_size=128, dtype="bf16", cache="fp8", fp8_granularity="tensor",
                                    lengths=("fixed", [3, 128, 129, 64, 700, 2100]))
    case = workloads.build_case(config, DEVICE, seed=43)
    key_cache, value_cache = case.cache_views()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales)
    expected = helpers.oracle_decode(case.query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    states = ops.paged_decode_attention_ex(case.query, key_cache, value_cache, case.block_tables,
                                           case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                           scale=case.scale, split=True, emit_state=True, **scales)
    assert ops.last_decode_route() == "mma16-fp8-balanced-block-tma" and states.dtype == torch.float32
    merged = ops.merge_decode_states(states.reshape(1, -1, states.shape[-1]).contiguous(), torch.bfloat16)
    helpers.assert_close(merged.reshape(expected.shape), expected, torch.bfloat16, "states of the block-tile kernel")
    assert ops.decode_timeout_flag() == 0


# ---- sliding window and logits soft cap (options beyond the reference's contract; parity unpinned:
# the expectation is the oracle's F64 attention restricted to the window / with capped scores) -------

@pytest.mark.parametrize("name,batch,lengths", [
    ("cfg2", 5, [1, 63, 200, 1100, 4096]),
    ("cfg3", 4, [64, 1000, 2049, 5000]),
    ("cfg4", 4, [17, 900, 3000, 6000]),
    ("cfg1", 3, [5, 130, 512]),
])
@pytest.mark.parametrize("window,cap", [(0, 30.0), (128, 0.0), (1000, 0.0), (333, 20.0)])
def test_sliding_window_and_soft_cap_against_the_oracle(ops, name, batch, lengths, window, cap):
    config = workloads.scaled(workloads.CONFIGS[name], batch=batch, lengths=("fixed", lengths))
    case = workloads.build_case(config, DEVICE, seed=13)
    key_cache, value_cache = case.cache_views()
    query = (case.query * 3.0).contiguous()  # scores large enough for the cap to bend them
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if config.cache == "fp8" else {}
    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length,
                                     sliding_window=window, logits_soft_cap=cap, **scales)
    plain = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                  scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    if cap or window < max(lengths):
        assert not torch.allclose(expected.float(), plain.float(), atol=2e-2), "the options must matter in this case"
    else:  # a window wider than every context changes nothing
        assert torch.equal(expected, plain)
    routes = set()
    for split, partition in ((False, 0), (True, 0), (True, 256)):
        actual = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths,
                                               max_sequence_length=case.max_sequence_length, scale=case.scale,
                                               split=split, partition_tokens=partition,
                                               sliding_window=window, logits_soft_cap=cap, **scales)
        routes.add(ops.last_decode_route())
        helpers.assert_close(actual, expected, config.torch_dtype,
                             f"{name} window={window} cap={cap} split={split} partition={partition}")
    if name != "cfg1":
        assert any("balanced" in route for route in routes), routes


def test_options_are_refused_where_they_do_not_apply(ops):
    config = workloads.scaled(workloads.CONFIGS["cfg2"], batch=2, lengths=("fixed", [40, 300]))
    case = workloads.build_case(config, DEVICE, seed=3)
    key_cache, value_cache = case.cache_views()
    with pytest.raises(helpers_bridge_error()):
        ops.paged_decode_attention_ex(case.query.contiguous(), key_cache, value_cache, case.block_tables,
                                      case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                      scale=case.scale, logits_soft_cap=float("nan"))
    with pytest.raises(helpers_bridge_error()):
        ops.paged_decode_attention_ex(case.query.contiguous(), key_cache, value_cache, case.block_tables,
                                      case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                      scale=case.scale, logits_soft_cap=-1.0)


def helpers_bridge_error():
    from attnarc_b200 import BridgeError

    return BridgeError


# ---- the caller's promise of stable metadata: the kernel plans its work before the preceding kernel
# has completed; results must not change ------------------------------------------------------------

@pytest.mark.parametrize("name,lengths", [
    ("cfg2", [1, 0, 700, 4096, 64, 2049, 0, 333]),
    ("cfg4", [5000, 16, 0, 1200]),
    ("cfg5", [40000, 300, 0, 7]),
])
def test_stable_metadata_changes_nothing_but_the_timing(ops, name, lengths):
    config = workloads.scaled(workloads.CONFIGS[name], batch=len(lengths), lengths=("fixed", [max(n, 1) for n in lengths]))
    case = workloads.build_case(config, DEVICE, seed=17)
    case.sequence_lengths.copy_(torch.tensor(lengths, dtype=torch.int32))  # empty sequences included
    key_cache, value_cache = case.cache_views()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if config.cache == "fp8" else {}
    rows = case.qkv.view(len(lengths), config.query_heads + 2 * config.kv_heads, config.head_size)
    outputs = []
    for stable in (False, True):
        qkv = rows.clone()
        query = qkv[:, :config.query_heads]
        # a RoPE launch directly before the decode, as in a serving step: with the promise the decode
        # kernel starts planning while this one is still rotating
        ops.rope_paged_kv_write_(query, qkv[:, config.query_heads:config.query_heads + config.kv_heads],
                                 qkv[:, config.query_heads + config.kv_heads:], case.positions, case.cos_sin_cache,
                                 case.rope_cache_argument(), case.key_scales, case.value_scales, case.slot_mapping,
                                 is_neox=config.rope_style == "neox")
        outputs.append(ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables,
                                                     case.sequence_lengths,
                                                     max_sequence_length=case.max_sequence_length, scale=case.scale,
                                                     split=True, stable_metadata=stable, **scales))
        assert "balanced" in ops.last_decode_route() and ops.last_decode_route().endswith("-tma")
    assert torch.equal(outputs[0], outputs[1])
    assert ops.decode_timeout_flag() == 0


def test_unknown_decode_flags_are_refused(ops):
    import ctypes

    from attnarc_b200 import _native

    args = _native.LoomDecodeArgs()
    args.struct_size = ctypes.sizeof(_native.LoomDecodeArgs)
    args.flags = 1
    assert _native.library().loom_cuda_paged_decode_attention_ex(ctypes.byref(args)) == 1
