"""GPU parity of the fused RoPE + paged-KV write: bit-exact against the oracle.

Q, K and every byte of both caches (written slots, untouched slots with their
canary pattern, FP8 codes) must equal the CPU oracle's, as the reference
demands of itself (python/tests/test_rope_paged_kv.py:164-247 compares the
whole packed allocation with torch.equal). The two fixtures of its Rust wrapper
tests (crates/loom-cuda/src/rope_kv_dispatch.rs:596-741) are replayed too.
"""

import numpy as np
import pytest
import torch

from tests import helpers
from attnarc_b200 import workloads

pytestmark = pytest.mark.gpu

DEVICE = "cuda"
CANARY = 0xA5


@pytest.fixture(scope="module")
def ops():
    from attnarc_b200 import ops as module

    return module


def canary_cache(shape, dtype):
    """A cache pre-filled with the byte 0xA5, as the reference's tests do."""
    element = torch.empty((), dtype=dtype).element_size()
    raw = torch.full((int(np.prod(shape)) * element,), CANARY, dtype=torch.uint8, device=DEVICE)
    return raw.view(dtype).reshape(shape)


def run_and_compare(ops, *, dtype, tokens, query_heads, kv_heads, head_size, rotary_dim, block_size,
                    num_blocks, is_neox, layout="NHD", cache="native", granularity="tensor", packed=True,
                    padding=0, negative_slots=(), seed=0, max_position=64):
    generator = torch.Generator().manual_seed(seed)
    width = (query_heads + 2 * kv_heads) * head_size
    if packed:
        qkv = torch.randn((tokens, width), generator=generator).to(dtype).to(DEVICE)
        view = qkv.view(tokens, query_heads + 2 * kv_heads, head_size)
        query, key = view[:, :query_heads], view[:, query_heads:query_heads + kv_heads]
        value = view[:, query_heads + kv_heads:]
    else:
        query = torch.randn((tokens, query_heads, head_size), generator=generator).to(dtype).to(DEVICE)
        key = torch.randn((tokens, kv_heads, head_size), generator=generator).to(dtype).to(DEVICE)
        value = torch.randn((tokens, kv_heads, head_size), generator=generator).to(dtype).to(DEVICE)
    positions = torch.randint(0, max_position, (tokens,), generator=generator)
    cos_sin = workloads.rope_table(max_position, rotary_dim, 10000.0, dtype)
    slots = torch.randperm(num_blocks * block_size, generator=generator)[: tokens - padding]
    for index in negative_slots:
        slots[index] = -1
    fp8 = cache == "fp8"
    cache_dtype = torch.uint8 if fp8 else dtype
    inner = (block_size, kv_heads, head_size) if layout == "NHD" else (kv_heads, block_size, head_size)
    kv_cache = canary_cache((num_blocks, 2, *inner), cache_dtype)
    rope_view = kv_cache if layout == "NHD" else kv_cache.permute(0, 1, 3, 2, 4)
    if fp8:
        count = 1 if granularity == "tensor" else kv_heads
        key_scales = (torch.rand(count, generator=generator) * 0.05 + 0.005).to(DEVICE)
        value_scales = (torch.rand(count, generator=generator) * 0.05 + 0.005).to(DEVICE)
    else:
        key_scales = torch.ones(1, device=DEVICE)
        value_scales = torch.ones(1, device=DEVICE)
    key_view, value_view = workloads.logical_cache_views(kv_cache, layout)

    expected_q, expected_k, expected_kc, expected_vc = helpers.oracle_rope_write(
        query, key, value, positions, cos_sin, key_view, value_view, slots, is_neox=is_neox,
        key_scales=key_scales, value_scales=value_scales)

    args = (query, key, value, positions.to(DEVICE), cos_sin.to(DEVICE), rope_view, key_scales, value_scales,
            slots.to(DEVICE))
    assert ops.supports_rope_paged_kv_write(*args)
    ops.rope_paged_kv_write_(*args, is_neox=is_neox)
    torch.cuda.synchronize()

    assert helpers.same_bits(query, expected_q), "rotated Q differs"
    assert helpers.same_bits(key, expected_k), "rotated K differs"
    assert helpers.same_bits(key_view, expected_kc), "key cache bytes differ"
    assert helpers.same_bits(value_view, expected_vc), "value cache bytes differ"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("cache,granularity", [("native", "tensor"), ("fp8", "tensor"), ("fp8", "head")])
def test_vector_path_is_bit_exact(ops, dtype, is_neox, layout, cache, granularity):
    run_and_compare(ops, dtype=dtype, tokens=37, query_heads=12, kv_heads=2, head_size=128, rotary_dim=128,
                    block_size=16, num_blocks=9, is_neox=is_neox, layout=layout, cache=cache,
                    granularity=granularity, packed=True, padding=3, negative_slots=(1, 20), seed=11,
                    max_position=4096)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("cache,granularity", [("native", "tensor"), ("fp8", "head")])
def test_partial_rotary_and_separate_sources(ops, dtype, is_neox, cache, granularity):
    run_and_compare(ops, dtype=dtype, tokens=19, query_heads=14, kv_heads=2, head_size=64, rotary_dim=32,
                    block_size=16, num_blocks=5, is_neox=is_neox, cache=cache, granularity=granularity,
                    packed=False, seed=5, max_position=300)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("cache,granularity", [("native", "tensor"), ("fp8", "tensor"), ("fp8", "head")])
def test_scalar_path_for_odd_shapes(ops, dtype, is_neox, cache, granularity):
    # head size 6 with 4 rotated dims: nothing is 16-byte friendly.
    run_and_compare(ops, dtype=dtype, tokens=9, query_heads=3, kv_heads=3, head_size=6, rotary_dim=4,
                    block_size=2, num_blocks=7, is_neox=is_neox, cache=cache, granularity=granularity,
                    packed=True, padding=1, negative_slots=(0,), seed=3, max_position=50)


def test_rust_wrapper_fixture_native(ops):
    # rope_kv_dispatch.rs:606-664.
    query = torch.arange(1, 17, dtype=torch.float32, device=DEVICE).reshape(2, 2, 4)
    key = torch.arange(17, 25, dtype=torch.float32, device=DEVICE).reshape(2, 1, 4)
    value = torch.arange(25, 33, dtype=torch.float32, device=DEVICE).reshape(2, 1, 4)
    cos_sin = torch.tensor([[1, 1, 0, 0], [0, 0, 1, 1]], dtype=torch.float32, device=DEVICE)
    kv_cache = torch.full((1, 2, 4, 1, 4), -5.0, device=DEVICE)
    positions = torch.tensor([0, 1], device=DEVICE)
    slots = torch.tensor([3, -1], device=DEVICE)
    ones = torch.ones(1, device=DEVICE)
    ops.rope_paged_kv_write_(query, key, value, positions, cos_sin, kv_cache, ones, ones, slots, is_neox=True)
    assert query[0].flatten().tolist() == list(range(1, 9))
    assert query[1].flatten().tolist() == [-11.0, -12.0, 9.0, 10.0, -15.0, -16.0, 13.0, 14.0]
    assert key[1].flatten().tolist() == [-23.0, -24.0, 21.0, 22.0]
    assert kv_cache[0, 0, :3].eq(-5.0).all() and kv_cache[0, 1, :3].eq(-5.0).all()
    assert kv_cache[0, 0, 3].flatten().tolist() == [17.0, 18.0, 19.0, 20.0]
    assert kv_cache[0, 1, 3].flatten().tolist() == [25.0, 26.0, 27.0, 28.0]


def test_rust_wrapper_fixture_fp8(ops):
    # rope_kv_dispatch.rs:666-741: per-tensor scales 0.25 and 0.5.
    from oracle import binding as ob

    query = torch.arange(1, 17, dtype=torch.float32, device=DEVICE).reshape(2, 2, 4)
    key = torch.arange(17, 25, dtype=torch.float32, device=DEVICE).reshape(2, 1, 4)
    value = torch.arange(25, 33, dtype=torch.float32, device=DEVICE).reshape(2, 1, 4)
    cos_sin = torch.tensor([[1, 1, 0, 0], [0, 0, 1, 1]], dtype=torch.float32, device=DEVICE)
    kv_cache = torch.full((1, 2, 4, 1, 4), 0xAA, dtype=torch.uint8, device=DEVICE)
    ops.rope_paged_kv_write_(query, key, value, torch.tensor([0, 1], device=DEVICE), cos_sin, kv_cache,
                             torch.tensor([0.25], device=DEVICE), torch.tensor([0.5], device=DEVICE),
                             torch.tensor([3, -1], device=DEVICE), is_neox=True)
    assert kv_cache[0, :, :3].eq(0xAA).all()
    assert kv_cache[0, 0, 3].flatten().cpu().numpy().tolist() == ob.fp8_from_f32(np.float32([17, 18, 19, 20]) / 0.25).tolist()
    assert kv_cache[0, 1, 3].flatten().cpu().numpy().tolist() == ob.fp8_from_f32(np.float32([25, 26, 27, 28]) / 0.5).tolist()


@pytest.mark.parametrize("name", ["cfg2", "cfg4"])
def test_benchmark_configs_write_step_is_bit_exact(ops, name):
    # Full token count of the configuration; the cache pool is shortened (the
    # write touches one slot per sequence whatever the context length).
    config = workloads.CONFIGS[name]
    small = workloads.scaled(config, lengths=("uniform", 17, 200))
    case = workloads.build_case(small, DEVICE, seed=8)
    key_view, value_view = case.cache_views()
    expected_q, expected_k, expected_kc, expected_vc = helpers.oracle_rope_write(
        case.query, case.key, case.value, case.positions, case.cos_sin_cache, key_view, value_view,
        case.slot_mapping, is_neox=config.rope_style == "neox",
        key_scales=case.key_scales, value_scales=case.value_scales)
    ops.rope_paged_kv_write_(case.query, case.key, case.value, case.positions, case.cos_sin_cache,
                             case.rope_cache_argument(), case.key_scales, case.value_scales,
                             case.slot_mapping, is_neox=config.rope_style == "neox")
    torch.cuda.synchronize()
    assert helpers.same_bits(case.query, expected_q)
    assert helpers.same_bits(case.key, expected_k)
    assert helpers.same_bits(key_view, expected_kc)
    assert helpers.same_bits(value_view, expected_vc)


def test_write_then_decode_round_trip(ops):
    # The two halves of a step together: after the write, decoding with the
    # updated lengths must see the new token exactly as the oracle does.
    config = workloads.scaled(workloads.CONFIGS["cfg2"], batch=6, lengths=("uniform", 30, 400))
    case = workloads.build_case(config, DEVICE, seed=21)
    key_view, value_view = case.cache_views()
    expected_q, _, expected_kc, expected_vc = helpers.oracle_rope_write(
        case.query, case.key, case.value, case.positions, case.cos_sin_cache, key_view, value_view,
        case.slot_mapping, is_neox=True, key_scales=case.key_scales, value_scales=case.value_scales)
    expected = helpers.oracle_decode(expected_q, expected_kc, expected_vc, case.block_tables,
                                     case.sequence_lengths, scale=case.scale,
                                     max_sequence_length=case.max_sequence_length)
    ops.rope_paged_kv_write_(case.query, case.key, case.value, case.positions, case.cos_sin_cache,
                             case.rope_cache_argument(), case.key_scales, case.value_scales,
                             case.slot_mapping, is_neox=True)
    actual = ops.paged_decode_attention(case.query.contiguous(), key_view, value_view, case.block_tables,
                                        case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                        scale=case.scale)
    helpers.assert_close(actual, expected, torch.bfloat16, "write + decode")


def test_rope_is_idempotent_under_inverse_rotation(ops):
    # Size-independent property: rotating by +theta and then by -theta (sines
    # negated) returns Q within storage rounding; the cache is untouched when
    # every slot is padding.
    tokens, heads, dim = 256, 12, 128
    generator = torch.Generator().manual_seed(2)
    query = torch.randn((tokens, heads, dim), generator=generator).to(torch.float32).to(DEVICE)
    key = torch.randn((tokens, 2, dim), generator=generator).to(torch.float32).to(DEVICE)
    value = torch.randn((tokens, 2, dim), generator=generator).to(torch.float32).to(DEVICE)
    original = query.clone()
    table = workloads.rope_table(512, dim, 1.0e6, torch.float32).to(DEVICE)
    inverse = table.clone()
    inverse[:, dim // 2:] *= -1
    positions = torch.randint(0, 512, (tokens,), generator=generator).to(DEVICE)
    kv_cache = canary_cache((4, 2, 16, 2, dim), torch.float32)
    slots = torch.full((tokens,), -1, dtype=torch.int64, device=DEVICE)
    ones = torch.ones(1, device=DEVICE)
    ops.rope_paged_kv_write_(query, key, value, positions, table, kv_cache, ones, ones, slots)
    ops.rope_paged_kv_write_(query, key, value, positions, inverse, kv_cache, ones, ones, slots)
    assert torch.allclose(query, original, rtol=0, atol=5e-6)
    assert kv_cache.view(torch.uint8).eq(CANARY).all()


def test_launch_counter_and_rejections(ops):
    query = torch.randn((4, 8, 64), device=DEVICE, dtype=torch.float16)
    key = torch.randn((4, 2, 64), device=DEVICE, dtype=torch.float16)
    value = torch.randn((4, 2, 64), device=DEVICE, dtype=torch.float16)
    positions = torch.arange(4, device=DEVICE)
    cos_sin = workloads.rope_table(16, 64, 1e4, torch.float16).to(DEVICE)
    kv_cache = torch.zeros((3, 2, 16, 2, 64), device=DEVICE, dtype=torch.float16)
    ones = torch.ones(1, device=DEVICE)
    slots = torch.arange(4, device=DEVICE)
    ops.reset_launch_count(ops.Operator.ROPE_PAGED_KV_WRITE)
    ops.rope_paged_kv_write_(query, key, value, positions, cos_sin, kv_cache, ones, ones, slots)
    assert ops.launch_count(ops.Operator.ROPE_PAGED_KV_WRITE) == 1
    with pytest.raises(RuntimeError, match="one value or one value per KV head"):
        ops.rope_paged_kv_write_(query, key, value, positions, cos_sin, kv_cache, torch.ones(3, device=DEVICE),
                                 torch.ones(3, device=DEVICE), slots)
    with pytest.raises(RuntimeError, match="regions key cache and value must not overlap|overlap"):
        ops.rope_paged_kv_write_(query, key, kv_cache[0, 0, :4], positions, cos_sin, kv_cache, ones, ones, slots)
    # a K/V cache whose two halves overlap is refused
    overlapping = torch.as_strided(kv_cache, (3, 2, 16, 2, 64), (2 * 16 * 2 * 64, 64, 2 * 64, 64, 1))
    with pytest.raises(RuntimeError):
        ops.rope_paged_kv_write_(query, key, value, positions, cos_sin, overlapping, ones, ones, slots)
    assert ops.launch_count(ops.Operator.ROPE_PAGED_KV_WRITE) == 1
