"""Glue between torch tensors and the CPU oracle.

TEST INFRASTRUCTURE ONLY: used by the tests, the smoke check and the CPU
baseline leg of the benchmark.
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import binding as ob

ORACLE_DTYPE = {torch.float32: ob.F32, torch.float16: ob.F16, torch.bfloat16: ob.BF16}

# Tolerances of the parity gate: KV bytes bit-exact; attention outputs within
# rtol = atol = 1e-2 for BF16/FP16 and 1e-4 for F32 of the CPU oracle.
TOLERANCE = {torch.float32: 1e-4, torch.float16: 1e-2, torch.bfloat16: 1e-2}


def bits(tensor: torch.Tensor) -> np.ndarray:
    """Contiguous host copy in the oracle's storage convention."""
    tensor = tensor.detach().cpu().contiguous()
    if tensor.dtype == torch.float32:
        return tensor.numpy().reshape(-1).copy()
    if tensor.dtype in (torch.float16, torch.bfloat16):
        return tensor.view(torch.int16).numpy().view(np.uint16).reshape(-1).copy()
    if tensor.dtype == torch.uint8:
        return tensor.numpy().reshape(-1).copy()
    if tensor.dtype in (torch.int32, torch.int64):
        return tensor.numpy().astype(np.int64).reshape(-1)
    raise TypeError(tensor.dtype)


def from_bits(array: np.ndarray, dtype: torch.dtype, shape) -> torch.Tensor:
    if dtype == torch.float32:
        return torch.from_numpy(array.astype(np.float32)).reshape(shape)
    return torch.from_numpy(array.view(np.int16).copy()).view(dtype).reshape(shape)


def oracle_decode(query, key_cache, value_cache, block_tables, sequence_lengths, *, scale,
                  max_sequence_length, key_scales=None, value_scales=None, threads=8, sliding_window=0,
                  logits_soft_cap=0.0) -> torch.Tensor:
    """Reference output for logical [blocks, block, heads, D] cache views (any strides).
    ``sliding_window`` / ``logits_soft_cap`` are the unpinned extensions of ``ob.decode_options``."""
    if sliding_window or logits_soft_cap:
        with ob.decode_options(sliding_window, logits_soft_cap):
            return oracle_decode(query, key_cache, value_cache, block_tables, sequence_lengths, scale=scale,
                                 max_sequence_length=max_sequence_length, key_scales=key_scales,
                                 value_scales=value_scales, threads=threads)
    sequences, query_heads, head_size = query.shape
    num_blocks, block_size, kv_heads, _ = key_cache.shape
    value_head_size = value_cache.shape[3]
    dtype = query.dtype
    spec = ob.DecodeSpec(sequences, query_heads, kv_heads, head_size, value_head_size, num_blocks,
                         block_size, block_tables.shape[1], int(max_sequence_length), float(scale),
                         ORACLE_DTYPE[dtype])
    out = np.zeros(sequences * query_heads * value_head_size,
                   dtype=np.float32 if dtype == torch.float32 else np.uint16)
    if key_cache.dtype == torch.uint8:
        stride = 0 if key_scales.numel() == 1 else 1
        ob.paged_decode_attention_fp8(
            ORACLE_DTYPE[dtype], bits(query), bits(key_cache), bits(value_cache),
            key_scales.detach().cpu().numpy(), value_scales.detach().cpu().numpy(), stride,
            bits(block_tables), bits(sequence_lengths), out, spec, threads)
    else:
        ob.paged_decode_attention(ORACLE_DTYPE[dtype], bits(query), bits(key_cache), bits(value_cache),
                                  bits(block_tables), bits(sequence_lengths), out, spec, threads)
    return from_bits(out, dtype, (sequences, query_heads, value_head_size))


def oracle_rope_write(query, key, value, positions, cos_sin_cache, key_cache, value_cache, slot_mapping,
                      *, is_neox, key_scales=None, value_scales=None):
    """Runs the reference RoPE + paged-KV write on host copies.

    `key_cache`/`value_cache` are logical [blocks, block, heads, D] views; the
    oracle works on contiguous NHD copies. `slot_mapping` may be shorter than
    the token count (padding tokens); it is extended with -1 as the CUDA ABI
    defines. Returns (query, key, key_cache, value_cache) as torch tensors with
    the logical shapes.
    """
    tokens, query_heads, head_size = query.shape
    kv_heads, value_head_size = key.shape[1], value.shape[2]
    num_blocks, block_size = key_cache.shape[0], key_cache.shape[1]
    dtype = query.dtype
    fp8 = key_cache.dtype == torch.uint8
    if fp8:
        encoding = ob.CACHE_FP8_PER_TENSOR if key_scales.numel() == 1 else ob.CACHE_FP8_PER_HEAD
    else:
        encoding = ob.CACHE_NATIVE
    rotary = ob.RotarySpec(tokens, query_heads, kv_heads, head_size, cos_sin_cache.shape[1],
                           cos_sin_cache.shape[0], ORACLE_DTYPE[dtype], bool(is_neox))
    spec = ob.RopeKvSpec(rotary, value_head_size, num_blocks, block_size, encoding)
    q, k, v = bits(query), bits(key), bits(value)
    kc, vc = bits(key_cache), bits(value_cache)
    slots = np.full(tokens, -1, dtype=np.int64)
    slots[: slot_mapping.numel()] = slot_mapping.detach().cpu().numpy()
    if fp8:
        ob.rope_paged_kv_write_fp8(ORACLE_DTYPE[dtype], q, k, v, bits(positions), bits(cos_sin_cache), kc, vc,
                                   slots, key_scales.detach().cpu().numpy(),
                                   value_scales.detach().cpu().numpy(), spec)
        kc_t = torch.from_numpy(kc).reshape(key_cache.shape)
        vc_t = torch.from_numpy(vc).reshape(value_cache.shape)
    else:
        ob.rope_paged_kv_write(ORACLE_DTYPE[dtype], q, k, v, bits(positions), bits(cos_sin_cache), kc, vc,
                               slots, spec)
        kc_t = from_bits(kc, dtype, key_cache.shape)
        vc_t = from_bits(vc, dtype, value_cache.shape)
    return from_bits(q, dtype, query.shape), from_bits(k, dtype, key.shape), kc_t, vc_t


def same_bits(left: torch.Tensor, right: torch.Tensor) -> bool:
    """Bitwise equality (so that -0.0 != 0.0 and NaN payloads count)."""
    left, right = left.detach().cpu().contiguous(), right.detach().cpu().contiguous()
    if left.dtype != right.dtype or left.shape != right.shape:
        return False
    if left.dtype == torch.float32:
        return bool(torch.equal(left.view(torch.int32), right.view(torch.int32)))
    if left.dtype in (torch.float16, torch.bfloat16):
        return bool(torch.equal(left.view(torch.int16), right.view(torch.int16)))
    return bool(torch.equal(left, right))


def assert_close(actual: torch.Tensor, expected: torch.Tensor, dtype: torch.dtype, what: str = ""):
    tolerance = TOLERANCE[dtype]
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert a.shape == e.shape, (a.shape, e.shape)
    error = (a - e).abs()
    bound = tolerance + tolerance * e.abs()
    worst = (error - bound).max().item()
    assert torch.isfinite(a).all(), f"{what}: non-finite output"
    assert worst <= 0, f"{what}: max abs error {error.max().item():.3e} exceeds rtol=atol={tolerance}"
