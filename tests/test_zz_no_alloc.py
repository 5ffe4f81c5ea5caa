"""The decode entry point that works out of the library's own scratch block.

Some callers cannot give the partitioned decode a workspace, because at the
moment of the call they have no way to obtain device memory (an engine that
fixed its memory budget at start-up, a handler that must not stall the device
with an allocation, a plug-in that only ever receives input and output
buffers). `loom_cuda_paged_decode_attention_built_in_scratch` serves them from a
16 MiB block inside the library. This file checks, through the C ABI, that it
gives the same answer as the workspace-taking entry point (and as the CPU
oracle) on two calls in a row, that the device's free memory does not change
across a call, and that it refuses shapes that do not fit its block.

It is named to be collected last, so that a run stopping at the first failure
has already run every other test.
"""

import ctypes

import pytest
import torch

from attnarc_b200 import _native, workloads
from tests import helpers

u32, u64, ptr = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p
BUILT_IN_SCRATCH_FLOATS = 4 * 1024 * 1024


class LoomDecodeArgs(ctypes.Structure):
    """Mirror of LoomDecodeArgs in include/loom_launch.h."""

    _fields_ = [
        ("struct_size", u32), ("dtype", u32), ("cache_encoding", u32), ("scale_stride", u32),
        ("query", ptr), ("key_cache", ptr), ("value_cache", ptr), ("key_scales", ptr), ("value_scales", ptr),
        ("block_tables", ptr), ("sequence_lengths", ptr), ("output", ptr), ("workspace", ptr),
        ("workspace_elements", u64),
        ("sequences", u32), ("query_heads", u32), ("kv_heads", u32), ("head_size", u32), ("value_head_size", u32),
        ("num_blocks", u32), ("block_size", u32), ("max_blocks_per_sequence", u32), ("max_sequence_length", u32),
        ("partition_tokens", u32),
        ("key_block_stride", u64), ("key_page_stride", u64), ("key_head_stride", u64),
        ("value_block_stride", u64), ("value_page_stride", u64), ("value_head_stride", u64),
        ("query_token_stride", u64), ("query_head_stride", u64),
        ("scale", ctypes.c_float), ("emit_state", u32), ("stream", ptr),
    ]


def decode_args(case, query, output, partition_tokens=0):
    config = case.config
    key_cache, value_cache = case.cache_views()
    args = LoomDecodeArgs()
    args.struct_size = ctypes.sizeof(LoomDecodeArgs)
    args.dtype = {"f32": 0, "f16": 1, "bf16": 2}[config.dtype]
    args.query, args.key_cache, args.value_cache = query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr()
    args.block_tables, args.sequence_lengths = case.block_tables.data_ptr(), case.sequence_lengths.data_ptr()
    args.output = output.data_ptr()
    args.sequences, args.query_heads, args.kv_heads = config.batch, config.query_heads, config.kv_heads
    args.head_size = args.value_head_size = config.head_size
    args.num_blocks, args.block_size = case.num_blocks, config.block_size
    args.max_blocks_per_sequence = case.block_tables.shape[1]
    args.max_sequence_length = case.max_sequence_length
    args.partition_tokens = partition_tokens
    args.key_block_stride, args.key_page_stride, args.key_head_stride = key_cache.stride()[:3]
    args.value_block_stride, args.value_page_stride, args.value_head_stride = value_cache.stride()[:3]
    args.scale = case.scale
    args.stream = torch.cuda.current_stream().cuda_stream
    return args


@pytest.fixture(scope="module")
def lib():
    library = _native.library()
    # this file binds the entry points to its own (shorter, first-version) mirror of the struct;
    # the package's bindings come back afterwards whatever the order of the test files
    before = library.loom_cuda_paged_decode_attention_ex.argtypes
    library.loom_cuda_paged_decode_attention_ex.argtypes = [ctypes.POINTER(LoomDecodeArgs)]
    library.loom_cuda_paged_decode_attention_built_in_scratch.argtypes = [
        ctypes.POINTER(LoomDecodeArgs), ctypes.c_char_p, u64]
    yield library
    library.loom_cuda_paged_decode_attention_ex.argtypes = before


@pytest.mark.gpu
@pytest.mark.parametrize("partition_tokens", [0, 128])
def test_built_in_scratch_matches_the_workspace_entry_point_twice(lib, partition_tokens):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    message = ctypes.create_string_buffer(256)
    for call, seed in enumerate((41, 42)):  # two calls in a row share the scratch block
        config = workloads.DecodeConfig("t", 6, 12, 2, dtype="bf16",
                                        lengths=("fixed", [5, 64, 300, 1000, 2049, 700 + call]))
        case = workloads.build_case(config, device, seed=seed)
        query = case.query.contiguous()
        shape = (config.batch, config.query_heads, config.head_size)
        expected = torch.empty(shape, device=device, dtype=torch.bfloat16)
        actual = torch.full(shape, float("nan"), device=device, dtype=torch.bfloat16)

        needed = lib.loom_cuda_paged_decode_workspace_elements(
            config.batch, config.query_heads, config.kv_heads, config.head_size, case.max_sequence_length,
            partition_tokens)
        assert 0 < needed <= BUILT_IN_SCRATCH_FLOATS
        workspace = torch.empty(needed, device=device, dtype=torch.float32)
        reference_args = decode_args(case, query, expected, partition_tokens)
        reference_args.workspace, reference_args.workspace_elements = workspace.data_ptr(), needed
        assert lib.loom_cuda_paged_decode_attention_ex(ctypes.byref(reference_args)) == 0

        scratch_args = decode_args(case, query, actual, partition_tokens)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(device)
        status = lib.loom_cuda_paged_decode_attention_built_in_scratch(ctypes.byref(scratch_args), message, 256)
        assert status == 0, message.value.decode()
        torch.cuda.synchronize()
        if call == 1:
            # the first call on a device may make the runtime load the block's module; from then on
            # the entry point must leave the device's free memory exactly as it found it
            free_after, _ = torch.cuda.mem_get_info(device)
            assert free_after >= free_before, "the entry point must not allocate device memory"

        # same kernels, same arithmetic: the tolerance of the parity tests, in practice bit-equal
        assert torch.isfinite(actual.float()).all()
        assert torch.allclose(actual.float(), expected.float(), rtol=1e-2, atol=1e-2)
        assert torch.equal(actual, expected)
        # and a third party: the CPU oracle, so that the library is not only compared with itself
        key_cache, value_cache = case.cache_views()
        oracle = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                       scale=case.scale, max_sequence_length=case.max_sequence_length)
        helpers.assert_close(actual, oracle, torch.bfloat16, f"built-in scratch, call {call}")


@pytest.mark.gpu
def test_built_in_scratch_refuses_what_does_not_fit(lib):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    config = workloads.DecodeConfig("t", 2, 8, 2, dtype="bf16", lengths=("fixed", [40, 70]))
    case = workloads.build_case(config, device, seed=1)
    output = torch.zeros((2, 8, 128), device=device, dtype=torch.bfloat16)
    args = decode_args(case, case.query.contiguous(), output)
    # pretend the batch were far larger: the size check comes before anything is launched
    args.sequences = 4096
    args.max_sequence_length = 70
    args.partition_tokens = 16
    message = ctypes.create_string_buffer(256)
    status = lib.loom_cuda_paged_decode_attention_built_in_scratch(ctypes.byref(args), message, 256)
    assert status == 2  # LOOM_CUDA_UNSUPPORTED
    text = message.value.decode()
    assert "built-in block holds 4194304" in text and "needs" in text
    torch.cuda.synchronize()
    assert output.eq(0).all()
