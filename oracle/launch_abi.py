"""ctypes driver for the launch ABI of ``include/loom_launch.h`` Part 1.

The same driver loads this repository's library and, where it was built, the
reference's own CUDA kernels (``oracle/_ref/libloom_cuda_reference.so``): both
export the same symbols, which is the drop-in claim at the lowest level.
"""

from __future__ import annotations

import ctypes
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))  # repository root
OURS = os.path.join(ROOT, "attnarc_b200", "libloom_cuda_bridge.so")
REFERENCE = os.path.join(ROOT, "oracle", "_ref", "libloom_cuda_reference.so")

_SUFFIX = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}
u32, u64, ptr = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p


class LaunchLibrary:
    def __init__(self, path: str):
        self.lib = ctypes.CDLL(path)
        for suffix in _SUFFIX.values():
            base = getattr(self.lib, f"loom_cuda_paged_decode_attention_{suffix}")
            base.restype = ctypes.c_int
            base.argtypes = [ptr] * 6 + [u32] * 7 + [u64, u64, u32, u32, ctypes.c_float, ptr]
            split = getattr(self.lib, f"loom_cuda_paged_decode_attention_split_k_{suffix}")
            split.restype = ctypes.c_int
            split.argtypes = [ptr] * 7 + [u64] + [u32] * 7 + [u64, u64, u32, u32, ctypes.c_float, ptr]
            rope = getattr(self.lib, f"loom_cuda_rope_paged_kv_write_{suffix}")
            rope.restype = ctypes.c_int
            rope.argtypes = [ptr] * 10 + [u32] * 12 + [u64] * 12 + [u32, ptr]
        sizing = self.lib.loom_cuda_paged_decode_attention_split_k_workspace_elements
        sizing.restype = u64
        sizing.argtypes = [u32] * 6

    def prepared_decode(self, query, key_cache, value_cache, block_tables, lengths, *, max_sequence_length, scale,
                        split: bool | None = None):
        """Returns (launch, output): `launch()` enqueues one decode on torch's current stream and allocates
        nothing (so it can be captured in a CUDA graph); the split-K entry is used when the sizing function
        asks for it."""
        batch, query_heads, dim = query.shape
        num_blocks, block, kv_heads, _ = key_cache.shape
        value_dim = value_cache.shape[3]
        output = torch.empty((batch, query_heads, value_dim), dtype=query.dtype, device=query.device)
        elements = int(self.lib.loom_cuda_paged_decode_attention_split_k_workspace_elements(
            batch, query_heads, kv_heads, dim, value_dim, max_sequence_length))
        use_split = (elements != 0 if split is None else split) and elements != 0
        workspace = torch.empty(max(elements, 1), dtype=torch.float32, device=query.device)
        suffix = _SUFFIX[query.dtype]
        shape = (batch, query_heads, kv_heads, dim, value_dim, num_blocks, block, key_cache.stride(0),
                 value_cache.stride(0), block_tables.shape[1], max_sequence_length, float(scale))
        pointers = (query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), block_tables.data_ptr(),
                    lengths.data_ptr(), output.data_ptr())
        keep = (query, key_cache, value_cache, block_tables, lengths, workspace)
        if use_split:
            function = getattr(self.lib, f"loom_cuda_paged_decode_attention_split_k_{suffix}")
            arguments = pointers + (workspace.data_ptr(), elements) + shape
        else:
            function = getattr(self.lib, f"loom_cuda_paged_decode_attention_{suffix}")
            arguments = pointers + shape

        def launch(_keep=keep):
            status = function(*arguments, torch.cuda.current_stream(query.device).cuda_stream)
            if status != 0:
                raise RuntimeError(f"launch ABI status {status}")

        return launch, output

    def decode(self, query, key_cache, value_cache, block_tables, lengths, *, max_sequence_length, scale,
               split: bool | None = None):
        """One launch-ABI decode (dense-inner NHD caches); returns the output tensor."""
        launch, output = self.prepared_decode(query, key_cache, value_cache, block_tables, lengths,
                                              max_sequence_length=max_sequence_length, scale=scale, split=split)
        launch()
        return output

    def prepared_rope_write(self, query, key, value, positions, cos_sin_cache, key_cache, value_cache, key_scales,
                            value_scales, slot_mapping, *, is_neox: bool):
        """Returns `launch()`: one launch-ABI RoPE + paged-KV write on [tokens, heads, dim] views and logical
        [blocks, block, heads, dim] caches, on torch's current stream, without allocations."""
        tokens, query_heads, dim = query.shape
        kv_heads, value_dim = key.shape[1], value.shape[2]
        fp8 = key_cache.dtype == torch.uint8
        function = getattr(self.lib, f"loom_cuda_rope_paged_kv_write_{_SUFFIX[query.dtype]}")
        arguments = (
            query.data_ptr(), key.data_ptr(), value.data_ptr(), positions.data_ptr(), cos_sin_cache.data_ptr(),
            key_cache.data_ptr(), value_cache.data_ptr(), key_scales.data_ptr(), value_scales.data_ptr(),
            slot_mapping.data_ptr(),
            tokens, slot_mapping.numel(), query_heads, kv_heads, dim, value_dim, cos_sin_cache.shape[1],
            cos_sin_cache.shape[0], key_cache.shape[0], key_cache.shape[1], 1 if fp8 else 0,
            0 if key_scales.numel() == 1 else 1,
            query.stride(0), query.stride(1), key.stride(0), key.stride(1), value.stride(0), value.stride(1),
            key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
            value_cache.stride(0), value_cache.stride(1), value_cache.stride(2),
            1 if is_neox else 0)
        keep = (query, key, value, positions, cos_sin_cache, key_cache, value_cache, key_scales, value_scales,
                slot_mapping)

        def launch(_keep=keep):
            status = function(*arguments, torch.cuda.current_stream(query.device).cuda_stream)
            if status != 0:
                raise RuntimeError(f"launch ABI status {status}")

        return launch

    def rope_write(self, query, key, value, positions, cos_sin_cache, key_cache, value_cache, key_scales,
                   value_scales, slot_mapping, *, is_neox: bool):
        self.prepared_rope_write(query, key, value, positions, cos_sin_cache, key_cache, value_cache, key_scales,
                                 value_scales, slot_mapping, is_neox=is_neox)()
