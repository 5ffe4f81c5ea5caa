"""This library against the reference's own CUDA kernels, both through the
launch ABI they share.

``oracle/build_reference_cuda.py`` compiles the reference's
paged_decode_attention.cu and rope_paged_kv.cu for sm_100a where a reference
checkout exists; the result travels as ``oracle/_ref/libloom_cuda_reference.so``.
Skipped where it was not built. The reference kernels stop at 1024 tokens, so
these cases stay inside that envelope; larger contexts are covered against the
oracle in ``test_gpu_decode.py``.
"""

import os

import pytest
import torch

from oracle import launch_abi
from tests import helpers

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")


@pytest.fixture(scope="module")
def libraries():
    if not os.path.exists(launch_abi.REFERENCE):
        pytest.skip("the reference CUDA kernels were not built")
    from attnarc_b200 import build

    build.build()
    return launch_abi.LaunchLibrary(launch_abi.OURS), launch_abi.LaunchLibrary(launch_abi.REFERENCE)


def decode_case(seed, dtype, lengths, query_heads, kv_heads, dim, block=16):
    gen = torch.Generator().manual_seed(seed)
    batch = len(lengths)
    max_blocks = (max(lengths) + block - 1) // block
    num_blocks = batch * max_blocks + 3
    keys = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(dtype)
    values = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(dtype)
    query = torch.randn((batch, query_heads, dim), generator=gen).to(dtype)
    tables = torch.randperm(num_blocks, generator=gen)[: batch * max_blocks].reshape(batch, max_blocks).to(torch.int32)
    return query, keys, values, tables, torch.tensor(lengths, dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [
    ([1, 40, 333, 1024], 8, 2, 128),     # GQA 4, base and split-K sizes
    ([1000, 512, 77], 12, 2, 128),       # the cfg2 head geometry
    ([64, 65, 300], 4, 4, 64),           # MHA, head size 64
    ([900, 1024, 128, 640, 31], 32, 8, 128),
])
def test_decode_agrees_with_the_reference_kernels(libraries, dtype, shape):
    ours, reference = libraries
    lengths, query_heads, kv_heads, dim = shape
    query, keys, values, tables, lens = decode_case(5, dtype, lengths, query_heads, kv_heads, dim)
    scale = dim ** -0.5
    expected = helpers.oracle_decode(query, keys, values, tables, lens, scale=scale, max_sequence_length=max(lengths))
    device_args = [t.to(DEVICE) for t in (query, keys, values, tables, lens)]
    mine = ours.decode(*device_args, max_sequence_length=max(lengths), scale=scale)
    theirs = reference.decode(*device_args, max_sequence_length=max(lengths), scale=scale)
    torch.cuda.synchronize()
    helpers.assert_close(theirs, expected, dtype, "reference kernels vs oracle")
    helpers.assert_close(mine, expected, dtype, "this library vs oracle")
    helpers.assert_close(mine, theirs.cpu(), dtype, "this library vs reference kernels")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("is_neox", [True, False])
def test_rope_write_is_bit_identical_to_the_reference_kernel(libraries, dtype, layout, fp8, is_neox):
    ours, reference = libraries
    gen = torch.Generator().manual_seed(3)
    tokens, query_heads, kv_heads, dim, block, num_blocks = 9, 8, 2, 128, 16, 6
    qkv = torch.randn((tokens, query_heads + 2 * kv_heads, dim), generator=gen).to(dtype)
    positions = torch.randint(0, 256, (tokens,), generator=gen, dtype=torch.int64)
    slots = torch.randperm(num_blocks * block, generator=gen)[:tokens].to(torch.int64)
    slots[2] = -1  # rotated, not written
    inverse = 1.0 / (1.0e6 ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    angles = torch.arange(256, dtype=torch.float64)[:, None] * inverse[None, :]
    table = torch.cat([angles.cos(), angles.sin()], dim=1).to(dtype).to(DEVICE)
    key_scales = (torch.tensor([0.02, 0.03]) if fp8 else torch.ones(1)).to(torch.float32).to(DEVICE)
    value_scales = (torch.tensor([0.025, 0.015]) if fp8 else torch.ones(1)).to(torch.float32).to(DEVICE)
    results = []
    for library in (ours, reference):
        buffer = qkv.clone().to(DEVICE)
        q, k, v = buffer[:, :query_heads], buffer[:, query_heads:query_heads + kv_heads], buffer[:, query_heads + kv_heads:]
        cache_dtype = torch.uint8 if fp8 else dtype
        shape = (num_blocks, 2, block, kv_heads, dim) if layout == "NHD" else (num_blocks, 2, kv_heads, block, dim)
        cache = torch.zeros(shape, dtype=cache_dtype, device=DEVICE)
        logical = cache if layout == "NHD" else cache.permute(0, 1, 3, 2, 4)
        library.rope_write(q, k, v, positions.to(DEVICE), table, logical[:, 0], logical[:, 1], key_scales,
                           value_scales, slots.to(DEVICE), is_neox=is_neox)
        torch.cuda.synchronize()
        results.append((buffer.cpu(), cache.cpu()))
    assert results[0][1].ne(0).any()
    if dtype == torch.float32:
        # The reference's CUDA file is compiled with nvcc's default FMA contraction, so in F32 its
        # x*cos - y*sin differs from the reference's own CPU oracle (separately rounded products, which
        # this library reproduces bit for bit, see test_gpu_rope_kv.py) in the last place.
        torch.testing.assert_close(results[0][0], results[1][0], rtol=1e-6, atol=1e-6)
        if not fp8:
            torch.testing.assert_close(results[0][1], results[1][1], rtol=1e-6, atol=1e-6)
        else:
            differing = (results[0][1] != results[1][1]).float().mean().item()
            assert differing < 1e-3, f"{differing:.2e} of the FP8 bytes differ"
        return
    assert helpers.same_bits(results[0][0], results[1][0]), "rotated Q/K differ from the reference kernel"
    assert helpers.same_bits(results[0][1], results[1][1]), "cache bytes differ from the reference kernel"
