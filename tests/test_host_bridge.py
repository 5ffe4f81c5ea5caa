"""Host-side checks that need no GPU: the built library loads, exports every
symbol the headers declare, and rejects bad calls before launching anything.

The rejection cases follow the reference's bridge unit tests, which also work
on fabricated addresses (crates/loom-cuda-bridge/src/cuda/tests.rs:4-12,
rope_kv_bridge.rs:484-514): nothing here dereferences device memory.
"""

import ctypes
import os
import re

import pytest

from attnarc_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from attnarc_b200 import build

    build.build()
    return _native.library()


def declared_symbols(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    names = set(re.findall(r"\b(loom_(?:cuda|partition)_[a-z0-9_]+)\s*\(", text))
    for macro, suffixes in (("loom_cuda_paged_decode_attention_##suffix", ("f32", "f16", "bf16")),
                            ("loom_cuda_paged_decode_attention_split_k_##suffix", ("f32", "f16", "bf16")),
                            ("loom_cuda_rope_paged_kv_write_##suffix", ("f32", "f16", "bf16"))):
        if macro in text:
            names |= {macro.replace("##suffix", s) for s in suffixes}
    return {n for n in names if not n.endswith("_")}


@pytest.mark.parametrize("header", ["loom_launch.h", "loom_bridge.h", "loom_partition.h"])
def test_every_declared_symbol_is_exported(lib, header):
    missing = [name for name in sorted(declared_symbols(header)) if not hasattr(lib, name)]
    assert not missing, missing
    assert len(declared_symbols(header)) >= 3


def test_abi_version_and_status_strings(lib):
    assert lib.loom_cuda_bridge_abi_version() == 2
    texts = [lib.loom_cuda_status_string(i).decode() for i in range(6)]
    assert texts == ["success", "invalid argument", "unsupported", "CUDA launch error", "CUDA unavailable",
                     "unknown Loom CUDA status"]


def test_launch_counters_reject_unknown_operators(lib):
    count = ctypes.c_uint64(99)
    assert lib.loom_cuda_bridge_launch_count(9, count) == 0
    assert lib.loom_cuda_bridge_launch_count(11, count) == 1
    assert _native.last_error() == "invalid operator contract: unknown bridge operator code 11"
    assert lib.loom_cuda_bridge_launch_count(9, None) == 1
    assert "null or misaligned" in _native.last_error()
    assert lib.loom_cuda_bridge_reset_launch_count(5) == 0


def decode_call(lib, *, dtype=0, query=0x1000, output=0x6000, workspace=None, workspace_elements=0,
                sequences=1, query_heads=2, kv_heads=1, head=4, blocks=1, block_size=2, max_blocks=1,
                max_len=2, scale=0.5, key_stride=8, lengths=0x5000, query_elements=8):
    return lib.loom_cuda_bridge_paged_decode_attention(
        dtype, query, query_elements, 0x2000, 8, 0x3000, 8, 0x4000, 1, lengths, 1, output, 8, workspace,
        workspace_elements, sequences, query_heads, kv_heads, head, head, blocks, block_size, key_stride, 8,
        max_blocks, max_len, scale, None)


def test_decode_bridge_rejections_use_the_reference_wording(lib):
    cases = [
        (dict(dtype=7), "unknown bridge dtype code 7"),
        (dict(query_heads=3, kv_heads=2), "query head count 3 must be divisible by KV head count 2"),
        (dict(scale=0.0), "attention scale must be finite and positive, got 0"),
        (dict(max_len=3), "maximum sequence length 3 exceeds block-table capacity 2"),
        (dict(sequences=0), "tensor dimensions must be non-zero"),
        (dict(key_stride=7), "paged key block stride is smaller than one dense NHD block"),
        (dict(workspace_elements=5), "paged decode workspace has 5 F32 elements, expected 0"),
        (dict(workspace=0x9000), "base paged decode requires a null workspace pointer"),
        (dict(query=None), "paged decode query pointer is null"),
        (dict(query=0x1002), "paged decode query pointer is not aligned to 4 bytes"),
        (dict(query_elements=0), "paged decode query region is empty"),
        (dict(output=0x1010), "paged decode regions output and query must not overlap"),
        (dict(query_elements=9), "paged decode query has 9 elements, expected 8"),
    ]
    for arguments, message in cases:
        assert decode_call(lib, **arguments) == 1, arguments
        assert _native.last_error() == "invalid operator contract: " + message


def test_workspace_rule_matches_the_sizing_function(lib):
    elements = ctypes.c_uint64(0)
    # a context that one partition covers needs no workspace
    assert lib.loom_cuda_bridge_paged_decode_workspace_elements(2, 1, 8, 2, 128, 128, 64, 16, 4, 64, 0.1, elements) == 0
    assert elements.value == 0
    # cfg2-shaped: 64 x 12 heads, 4096 tokens, partitions of 256 -> 16 parts of 130 floats
    assert lib.loom_cuda_bridge_paged_decode_workspace_elements(2, 64, 12, 2, 128, 128, 20000, 16, 256, 4096, 0.1, elements) == 0
    tokens = lib.loom_cuda_paged_decode_default_partition_tokens(64, 2, 4096)
    assert tokens % 16 == 0 and tokens >= 64
    assert elements.value == 64 * 12 * ((4096 + tokens - 1) // tokens) * 130
    chosen = ctypes.c_uint32(0)
    assert lib.loom_cuda_bridge_paged_decode_workspace_elements_ex(64, 12, 2, 128, 4096, 512, elements, chosen) == 0
    assert (elements.value, chosen.value) == (64 * 12 * 8 * 130, 512)
    assert lib.loom_cuda_bridge_paged_decode_workspace_elements_ex(64, 12, 2, 128, 4096, 100, elements, chosen) == 1
    assert "multiple of 16" in _native.last_error()


def test_workspace_covers_the_layout_of_the_eight_heads_per_tile_kernel(lib):
    # KV heads in eights, head size 128, up to 8 query heads per KV head: eight state slots of
    # 8 x 130 floats per (sequence + CTA), two CTAs per SM of at least 148 SMs, then two words per item
    elements = ctypes.c_uint64(0)
    assert lib.loom_cuda_bridge_paged_decode_workspace_elements(2, 128, 64, 8, 128, 128, 80000, 16, 1024, 16384, 0.1,
                                                                elements) == 0
    block_tiles = (128 * (8 // 8) + 2 * 148) * 8 * 8 * 130 + 2 * 128 * 8
    assert elements.value >= block_tiles
    # a group of 16 query heads per KV head is not served by that kernel: the other layouts alone decide
    assert lib.loom_cuda_bridge_paged_decode_workspace_elements(2, 128, 128, 8, 128, 128, 80000, 16, 1024, 16384, 0.1,
                                                                elements) == 0
    per_item_slots = (128 * 8 + 4 * 148) * 16 * 130 + 2 * 128 * 8
    tokens = lib.loom_cuda_paged_decode_default_partition_tokens(128, 8, 16384)
    fixed = 128 * 128 * ((16384 + tokens - 1) // tokens) * 130
    assert elements.value == max(per_item_slots, fixed)


def rope_call(lib, **overrides):
    a = dict(dtype=0, encoding=0, query=0x10000, query_elements=2 * 3 * 8, key=0x20000, key_elements=2 * 1 * 8,
             value=0x30000, value_elements=2 * 1 * 8, positions=0x40000, cos_sin=0x50000, cos_sin_elements=4 * 8,
             key_cache=0x60000, cache_elements=2 * 4 * 1 * 8, value_cache=0x70000, key_scales=0x80000,
             scale_elements=1, value_scales=0x80100, slots=0x90000, slot_elements=2, tokens=2, cache_tokens=2,
             query_heads=3, kv_heads=1, head=8, rotary=8, max_position=4, blocks=2, block_size=4,
             q_token=24, q_head=8, k_token=8, k_head=8, v_token=8, v_head=8, c_block=32, c_page=8, c_head=8,
             neox=1)
    a.update(overrides)
    return lib.loom_cuda_bridge_rope_paged_kv_write(
        a["dtype"], a["encoding"], a["query"], a["query_elements"], a["key"], a["key_elements"], a["value"],
        a["value_elements"], a["positions"], a["tokens"], a["cos_sin"], a["cos_sin_elements"], a["key_cache"],
        a["cache_elements"], a["value_cache"], a["cache_elements"], a["key_scales"], a["scale_elements"],
        a["value_scales"], a["scale_elements"], a["slots"], a["slot_elements"], a["tokens"], a["cache_tokens"],
        a["query_heads"], a["kv_heads"], a["head"], a["head"], a["rotary"], a["max_position"], a["blocks"],
        a["block_size"], a["q_token"], a["q_head"], a["k_token"], a["k_head"], a["v_token"], a["v_head"],
        a["c_block"], a["c_page"], a["c_head"], a["c_block"], a["c_page"], a["c_head"], a["neox"], None)


def test_rope_bridge_rejections_use_the_reference_wording(lib):
    cases = [
        (dict(neox=2), "RoPE style flag must be 0 or 1"),
        (dict(rotary=3), "rotary dimension must be non-zero, even, and no larger than head size; got rotary_dim=3, head_size=8"),
        (dict(scale_elements=3), "paged K/V cache scales must contain one value or one value per KV head"),
        (dict(encoding=2), "unsupported paged K/V cache encoding"),
        (dict(cache_tokens=3), "RoPE+paged-KV cache token count must be in [1, tokens]"),
        (dict(q_head=4), "RoPE query layout overlaps itself"),
        (dict(key=0x10000 + 4 * 8), "RoPE+paged-KV packed regions query and key must share an outer stride"),
        (dict(positions=0x10000), "RoPE+paged-KV regions query and positions must not overlap"),
        (dict(value=0x60000), "RoPE+paged-KV regions key cache and value must not overlap"),
        (dict(query_elements=47), "RoPE query has 47 elements, expected 48"),
    ]
    for arguments, message in cases:
        assert rope_call(lib, **arguments) == 1, arguments
        assert _native.last_error() == "invalid operator contract: " + message, arguments


def test_packed_qkv_views_are_accepted_up_to_the_launch(lib):
    # Q, K, V interleaved in one [tokens, (3+1+1)*8] allocation: the alias rule
    # lets the call through (rope_kv_bridge.rs:484-514 tests the same rule).
    # Sizes are then checked, so ask for one element too many to stop before a launch.
    base = 0x100000
    status = rope_call(lib, query=base, key=base + 3 * 8 * 4, value=base + 4 * 8 * 4, q_token=40, k_token=40,
                       v_token=40, query_elements=40 + 24, key_elements=40 + 8, value_elements=40 + 8 + 1)
    assert status == 1
    assert _native.last_error() == "invalid operator contract: RoPE value has 49 elements, expected 48"
    # the same views with K shifted into Q's columns are refused by the alias rule
    status = rope_call(lib, query=base, key=base + 2 * 8 * 4, value=base + 4 * 8 * 4, q_token=40, k_token=40,
                       v_token=40, query_elements=40 + 24, key_elements=40 + 8, value_elements=40 + 8)
    assert status == 1
    assert "logical elements in packed regions query and key overlap" in _native.last_error()


def test_capability_queries(lib):
    assert lib.loom_cuda_bridge_supports_paged_decode(2, 0, 64, 12, 2, 128, 128, 20000, 16, 256, 4096, 0.1) == 1
    # contexts far beyond the reference's 1024-token cap are supported
    assert lib.loom_cuda_bridge_supports_paged_decode(2, 1, 8, 32, 8, 128, 128, 70000, 16, 8192, 131072, 0.1) == 1
    assert lib.loom_cuda_bridge_supports_paged_decode(5, 0, 1, 1, 1, 8, 8, 1, 1, 1, 1, 0.1) == 0
    assert lib.loom_cuda_bridge_supports_paged_decode(0, 0, 1, 1, 1, 8, 1024, 1, 1, 1, 1, 0.1) == 0
    assert "value heads of at most 512" in _native.last_error()
    assert lib.loom_cuda_bridge_supports_rope_paged_kv_write(1, 1, 64, 12, 2, 128, 128, 128, 4096, 100, 16) == 1
    assert lib.loom_cuda_bridge_supports_rope_paged_kv_write(1, 0, 64, 12, 2, 128, 128, 130, 4096, 100, 16) == 0


def test_out_of_scope_operators_report_unavailable(lib):
    lib.loom_cuda_bridge_rms_norm.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p,
                                              ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32,
                                              ctypes.c_uint32, ctypes.c_float, ctypes.c_void_p]
    assert lib.loom_cuda_bridge_rms_norm(0, None, 0, None, 0, None, 0, 1, 1, 1e-6, None) == 3
    assert "outside the paged-decode library" in _native.last_error()


def test_reference_dispatcher_links_against_this_bridge(lib):
    """The reference's unmodified torch dispatcher, where it could be built."""
    from oracle import build_reference_dispatcher

    path = build_reference_dispatcher.build()
    if path is None:
        path = build_reference_dispatcher.OUTPUT
        if not os.path.exists(path):
            pytest.skip("no reference checkout and no prebuilt dispatcher")
    import subprocess

    import torch

    wanted = {line.split()[-1] for line in
              subprocess.run(["nm", "-D", "--undefined-only", path], capture_output=True, text=True).stdout.splitlines()
              if "loom_cuda_bridge_" in line}
    assert len(wanted) >= 10
    missing = [name for name in sorted(wanted) if not hasattr(lib, name)]
    assert not missing, missing
    torch.ops.load_library(path)
    assert torch.ops.loom_kernels.bridge_abi_version() == 2
    assert torch.ops.loom_kernels.bridge_launch_count(9) >= 0


def test_decode_args_of_both_layouts_are_read_and_others_refused():
    """LoomDecodeArgs grew at its end (sliding window, logits soft cap): a caller built against the
    shorter layout passes its own struct_size and gets both options off."""
    import ctypes

    from attnarc_b200 import _native

    lib = _native.library()
    lib.loom_cuda_read_decode_args.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    full = ctypes.sizeof(_native.LoomDecodeArgs)
    base = _native.LoomDecodeArgs.sliding_window.offset
    assert full == base + 16  # sliding window, soft cap, flags, reserved

    source = _native.LoomDecodeArgs()
    source.sequences, source.sliding_window, source.logits_soft_cap = 7, 99, 2.5
    out = _native.LoomDecodeArgs()
    source.struct_size = full
    assert lib.loom_cuda_read_decode_args(ctypes.byref(source), ctypes.byref(out)) == 1
    assert (out.sequences, out.sliding_window, out.logits_soft_cap, out.struct_size) == (7, 99, 2.5, full)
    source.struct_size = base  # the older layout: whatever follows `stream` is not read
    assert lib.loom_cuda_read_decode_args(ctypes.byref(source), ctypes.byref(out)) == 1
    assert (out.sequences, out.sliding_window, out.logits_soft_cap, out.struct_size) == (7, 0, 0.0, full)
    for bad in (0, base - 8, full + 8):
        source.struct_size = bad
        assert lib.loom_cuda_read_decode_args(ctypes.byref(source), ctypes.byref(out)) == 0
    assert lib.loom_cuda_read_decode_args(None, ctypes.byref(out)) == 0
    # launch entry points refuse an unknown layout before touching anything
    assert lib.loom_cuda_paged_decode_attention_ex(ctypes.byref(source)) == 1


def test_capability_answer_agrees_with_the_launch_for_oversized_heads():
    """`loom_cuda_supports_paged_decode` and the launch share one predicate for the general kernel's
    shared memory: a shape the query refuses is refused by the launch with LOOM_CUDA_UNSUPPORTED,
    before any CUDA call (so this runs without a device)."""
    import ctypes

    from attnarc_b200 import _native

    lib = _native.library()
    lib.loom_cuda_supports_paged_decode.argtypes = [ctypes.c_uint32] * 11 + [ctypes.POINTER(ctypes.c_char_p)]
    reason = ctypes.c_char_p()

    def supported(dtype, head_size, value_head_size):
        return lib.loom_cuda_supports_paged_decode(dtype, 0, 2, 4, 2, head_size, value_head_size, 8, 16, 4, 64,
                                                   ctypes.byref(reason))

    def launch_status(dtype, head_size, value_head_size):
        args = _native.LoomDecodeArgs()
        args.struct_size = ctypes.sizeof(_native.LoomDecodeArgs)
        args.dtype = dtype
        fake = 0x10000  # never dereferenced on the host; the refusal comes before any launch
        for name in ("query", "key_cache", "value_cache", "block_tables", "sequence_lengths", "output"):
            setattr(args, name, fake)
        args.sequences, args.query_heads, args.kv_heads = 2, 4, 2
        args.head_size, args.value_head_size = head_size, value_head_size
        args.num_blocks, args.block_size, args.max_blocks_per_sequence, args.max_sequence_length = 8, 16, 4, 64
        args.key_block_stride, args.key_page_stride, args.key_head_stride = 16 * 2 * head_size, 2 * head_size, head_size
        args.value_block_stride = 16 * 2 * value_head_size
        args.value_page_stride, args.value_head_stride = 2 * value_head_size, value_head_size
        args.scale = 0.1
        return lib.loom_cuda_paged_decode_attention_ex(ctypes.byref(args))

    assert supported(0, 128, 128) == 1 and supported(2, 256, 256) == 1
    for dtype, head_size, value_head_size in ((0, 16384, 256), (2, 20000, 64), (1, 12288, 512)):
        assert supported(dtype, head_size, value_head_size) == 0, reason.value
        assert b"shared memory" in reason.value
        assert launch_status(dtype, head_size, value_head_size) == 2  # LOOM_CUDA_UNSUPPORTED
    assert supported(0, 64, 1024) == 0 and launch_status(0, 64, 1024) == 2  # value heads beyond 512 elements
