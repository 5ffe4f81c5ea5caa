"""The reference's own, unmodified torch dispatcher on top of this bridge.

``oracle/build_reference_dispatcher.py`` compiles the reference's
``python/csrc/*.cpp`` (which registers ``torch.ops.loom_kernels.*`` and calls
the checked bridge ABI) where the sources lie and links it against
``libloom_cuda_bridge.so``. Here the decode and the RoPE/KV write are driven
through those registrations and checked against the oracle: the drop-in claim
exercised end to end. Skipped where the dispatcher has not been built (no
reference checkout on the machine that built the tree).
"""

import os

import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DISPATCHER = os.path.join(ROOT, "oracle", "_ref", "libloom_kernels_torch.so")
DEVICE = torch.device("cuda:0")


@pytest.fixture(scope="module")
def reference_ops():
    if not os.path.exists(DISPATCHER):
        pytest.skip("the reference dispatcher was not built")
    from attnarc_b200 import _native

    _native.library()  # the bridge must be the one of this tree
    torch.ops.load_library(DISPATCHER)
    return torch.ops.loom_kernels


def test_abi_version_through_the_reference_dispatcher(reference_ops):
    assert reference_ops.bridge_abi_version() == 2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("lengths", [[1, 17, 200, 64], [1024, 3, 700, 999, 512]])
def test_decode_through_the_reference_dispatcher(reference_ops, dtype, lengths):
    gen = torch.Generator().manual_seed(len(lengths))
    batch, query_heads, kv_heads, dim, block = len(lengths), 8, 2, 128, 16
    max_blocks = (max(lengths) + block - 1) // block
    num_blocks = batch * max_blocks + 5
    keys = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(dtype)
    values = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(dtype)
    query = torch.randn((batch, query_heads, dim), generator=gen).to(dtype)
    tables = torch.randperm(num_blocks, generator=gen)[: batch * max_blocks].reshape(batch, max_blocks).to(torch.int32)
    lens = torch.tensor(lengths, dtype=torch.int32)
    scale = dim ** -0.5
    expected = helpers.oracle_decode(query, keys, values, tables, lens, scale=scale, max_sequence_length=max(lengths))
    output = torch.empty((batch, query_heads, dim), dtype=dtype, device=DEVICE)
    before = reference_ops.bridge_launch_count(9)
    reference_ops.paged_decode_attention(query.to(DEVICE), keys.to(DEVICE), values.to(DEVICE), tables.to(DEVICE),
                                         lens.to(DEVICE), output, max(lengths), scale)
    torch.cuda.synchronize()
    helpers.assert_close(output, expected, dtype, f"reference dispatcher {dtype} {lengths}")
    assert reference_ops.bridge_launch_count(9) == before + 1


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("is_neox", [True, False])
def test_rope_write_through_the_reference_dispatcher(reference_ops, layout, fp8, is_neox):
    gen = torch.Generator().manual_seed(11)
    dtype = torch.bfloat16
    tokens, query_heads, kv_heads, dim, block, num_blocks = 6, 4, 2, 64, 16, 5
    qkv = torch.randn((tokens, query_heads + 2 * kv_heads, dim), generator=gen).to(dtype)
    positions = torch.randint(0, 64, (tokens,), generator=gen, dtype=torch.int64)
    slots = torch.randperm(num_blocks * block, generator=gen)[:tokens].to(torch.int64)
    inverse = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    angles = torch.arange(64, dtype=torch.float64)[:, None] * inverse[None, :]
    table = torch.cat([angles.cos(), angles.sin()], dim=1).to(dtype)
    cache_dtype = torch.uint8 if fp8 else dtype
    if layout == "NHD":
        kv_cache = torch.zeros((num_blocks, 2, block, kv_heads, dim), dtype=cache_dtype)
        logical = kv_cache
    else:
        kv_cache = torch.zeros((num_blocks, 2, kv_heads, block, dim), dtype=cache_dtype)
        logical = kv_cache.permute(0, 1, 3, 2, 4)  # [blocks, 2, block, heads, dim] view of the HND allocation
    key_scales = torch.tensor([0.02, 0.03], dtype=torch.float32) if fp8 else torch.ones(1, dtype=torch.float32)
    value_scales = torch.tensor([0.025, 0.015], dtype=torch.float32) if fp8 else torch.ones(1, dtype=torch.float32)
    q, k, v = qkv[:, :query_heads], qkv[:, query_heads:query_heads + kv_heads], qkv[:, query_heads + kv_heads:]
    scales = dict(key_scales=key_scales, value_scales=value_scales) if fp8 else {}
    want_q, want_k, want_kc, want_vc = helpers.oracle_rope_write(
        q.clone(), k.clone(), v.clone(), positions, table, logical[:, 0].clone(), logical[:, 1].clone(), slots,
        is_neox=is_neox, **scales)

    device_qkv = qkv.to(DEVICE)
    dq = device_qkv[:, :query_heads]
    dk = device_qkv[:, query_heads:query_heads + kv_heads]
    dv = device_qkv[:, query_heads + kv_heads:]
    device_cache = kv_cache.to(DEVICE)
    device_logical = device_cache if layout == "NHD" else device_cache.permute(0, 1, 3, 2, 4)
    reference_ops.rope_paged_kv_write_(dq, dk, dv, positions.to(DEVICE), table.to(DEVICE), device_logical,
                                       key_scales.to(DEVICE), value_scales.to(DEVICE), slots.to(DEVICE), is_neox)
    torch.cuda.synchronize()
    assert helpers.same_bits(dq, want_q) and helpers.same_bits(dk, want_k)
    assert helpers.same_bits(device_logical[:, 0], want_kc)
    assert helpers.same_bits(device_logical[:, 1], want_vc)
