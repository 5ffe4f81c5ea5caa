"""Multi-token entry points without a GPU: argument checks run before any CUDA call."""

import ctypes

import pytest


@pytest.fixture(scope="module")
def lib():
    from attnarc_b200 import _native

    return _native.library()


def test_expand_and_prepare_reject_malformed_arguments(lib):
    buffer = (ctypes.c_int32 * 64)()
    at = ctypes.addressof(buffer)
    assert lib.loom_cuda_expand_query_tokens(None, at, at, at, 2, 2, 4, None) == 1
    assert lib.loom_cuda_expand_query_tokens(at, at, at, at, 2, 0, 4, None) == 1
    assert lib.loom_cuda_expand_query_tokens(at, at, at, at, 1 << 31, 2, 4, None) == 1   # rows overflow int32
    assert lib.loom_cuda_multi_token_prepare(at, at, at, None, 2, 2, 2, 4, 2, 8, None) == 1
    assert lib.loom_cuda_multi_token_prepare(at, at, at, at, 2, 2, 2, 5, 2, 8, None) == 1  # 5 heads over 2 KV heads
    assert lib.loom_cuda_multi_token_prepare(at, at, at, at, 3, 2, 2, 4, 2, 8, None) == 1  # unknown dtype


def test_finish_and_the_single_call_check_the_argument_struct(lib):
    from attnarc_b200 import _native

    buffer = (ctypes.c_float * 64)()
    at = ctypes.addressof(buffer)
    args = _native.LoomDecodeArgs()
    assert lib.loom_cuda_multi_token_finish(ctypes.byref(args), 2, at) == 1            # struct_size not set
    args.struct_size = ctypes.sizeof(_native.LoomDecodeArgs)
    assert lib.loom_cuda_multi_token_finish(ctypes.byref(args), 2, at) == 1            # null tensors
    assert lib.loom_cuda_multi_token_finish(None, 2, at) == 1
    assert lib.loom_cuda_paged_multi_token_decode(ctypes.byref(args), 2, None, at, at) == 1
    assert lib.loom_cuda_paged_multi_token_decode(ctypes.byref(args), 0, at, at, at) == 1
    for name in ("query", "key_cache", "value_cache", "block_tables", "sequence_lengths", "output"):
        setattr(args, name, at)
    args.sequences, args.query_heads, args.kv_heads = 1, 4, 2
    args.block_size, args.num_blocks, args.max_blocks_per_sequence = 16, 1, 1
    args.dtype, args.head_size, args.value_head_size = 2, 512, 128
    assert lib.loom_cuda_multi_token_finish(ctypes.byref(args), 2, at) == 2            # head size above 256
    args.head_size, args.dtype, args.cache_encoding = 128, 0, 1
    assert lib.loom_cuda_multi_token_finish(ctypes.byref(args), 2, at) == 1            # FP8 cache without scales
