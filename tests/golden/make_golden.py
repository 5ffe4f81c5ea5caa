"""Generates ``tests/golden/paged_decode_small.npz``: seeded inputs of the hot
path and the outputs the CPU oracle gives for them.

The reference cannot be built or imported here (its CPU oracle is Rust), so
the fixture is produced by the C++ restatement under ``oracle/``, which is
pinned to the reference's own known-answer tests
(``tests/test_oracle_known_answers.py``). The fixture freezes those outputs:
``tests/test_golden_fixtures.py`` checks that the oracle still reproduces them
bit for bit (CPU) and that the CUDA path matches them (GPU).

Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import torch_glue as glue  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "paged_decode_small.npz")


def rope_table(max_position, rotary_dim, theta, dtype):
    inverse = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim))
    angles = torch.arange(max_position, dtype=torch.float64)[:, None] * inverse[None, :]
    return torch.cat([angles.cos(), angles.sin()], dim=1).to(dtype)


def build(seed=20240607):
    gen = torch.Generator().manual_seed(seed)
    dtype = torch.bfloat16
    lengths = [5, 33, 40, 16]
    batch, query_heads, kv_heads, dim, block = len(lengths), 8, 2, 64, 16
    blocks_per_seq = 3
    num_blocks = batch * blocks_per_seq + 1
    tables = torch.randperm(num_blocks, generator=gen)[: batch * blocks_per_seq].reshape(batch, blocks_per_seq).to(torch.int32)
    key_cache = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(dtype)
    value_cache = torch.randn((num_blocks, block, kv_heads, dim), generator=gen).to(dtype)
    # one new token per sequence, packed QKV row
    qkv = torch.randn((batch, query_heads + 2 * kv_heads, dim), generator=gen).to(dtype)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int64)
    slots = torch.tensor([int(tables[b, (n - 1) // block]) * block + (n - 1) % block for b, n in enumerate(lengths)],
                         dtype=torch.int64)
    table = rope_table(128, dim, 1.0e6, dtype)
    scale = dim ** -0.5
    out = {
        "lengths": np.array(lengths, dtype=np.int32), "block_tables": tables.numpy(), "positions": positions.numpy(),
        "slot_mapping": slots.numpy(), "scale": np.float32(scale),
        "qkv": glue.bits(qkv), "key_cache": glue.bits(key_cache), "value_cache": glue.bits(value_cache),
        "cos_sin_cache": glue.bits(table),
        "shape": np.array([batch, query_heads, kv_heads, dim, block, num_blocks], dtype=np.int64),
    }
    lens = torch.tensor(lengths, dtype=torch.int32)
    for style, is_neox in (("neox", True), ("interleaved", False)):
        q = qkv[:, :query_heads].clone()
        k = qkv[:, query_heads:query_heads + kv_heads].clone()
        v = qkv[:, query_heads + kv_heads:].clone()
        # native cache
        rq, rk, kc, vc = glue.oracle_rope_write(q, k, v, positions, table, key_cache, value_cache, slots, is_neox=is_neox)
        attention = glue.oracle_decode(rq, kc, vc, tables, lens, scale=scale, max_sequence_length=max(lengths))
        out[f"{style}_query"] = glue.bits(rq)
        out[f"{style}_key"] = glue.bits(rk)
        # the write touches one page per sequence: the rest of the cache must stay as it was
        written_blocks, written_pages = slots // block, slots % block
        out[f"{style}_written_keys"] = glue.bits(kc[written_blocks, written_pages])
        out[f"{style}_written_values"] = glue.bits(vc[written_blocks, written_pages])
        assert glue.same_bits(kc.index_put((written_blocks, written_pages), key_cache[written_blocks, written_pages]), key_cache)
        out[f"{style}_attention"] = glue.bits(attention)
        # FP8 E4M3 cache with one scale per KV head
        key_scales = torch.tensor([0.011, 0.017], dtype=torch.float32)
        value_scales = torch.tensor([0.013, 0.009], dtype=torch.float32)
        fp8_k = torch.zeros(key_cache.shape, dtype=torch.uint8)
        fp8_v = torch.zeros(value_cache.shape, dtype=torch.uint8)
        # fill the FP8 caches by writing every cached token through the reference encoder
        from oracle import binding as ob

        for h in range(kv_heads):
            fp8_k[:, :, h] = torch.from_numpy(
                ob.fp8_from_f32((key_cache[:, :, h].float() / key_scales[h]).numpy().ravel())).reshape(num_blocks, block, dim)
            fp8_v[:, :, h] = torch.from_numpy(
                ob.fp8_from_f32((value_cache[:, :, h].float() / value_scales[h]).numpy().ravel())).reshape(num_blocks, block, dim)
        rq8, rk8, kc8, vc8 = glue.oracle_rope_write(q, k, v, positions, table, fp8_k, fp8_v, slots, is_neox=is_neox,
                                                    key_scales=key_scales, value_scales=value_scales)
        attention8 = glue.oracle_decode(rq8, kc8, vc8, tables, lens, scale=scale, max_sequence_length=max(lengths),
                                        key_scales=key_scales, value_scales=value_scales)
        out["fp8_key_scales"] = key_scales.numpy()
        out["fp8_value_scales"] = value_scales.numpy()
        out["fp8_initial_key_cache"] = fp8_k.numpy()
        out["fp8_initial_value_cache"] = fp8_v.numpy()
        out[f"{style}_fp8_written_keys"] = kc8[written_blocks, written_pages].numpy()
        out[f"{style}_fp8_written_values"] = vc8[written_blocks, written_pages].numpy()
        out[f"{style}_fp8_attention"] = glue.bits(attention8)
    return out


if __name__ == "__main__":
    data = build()
    np.savez_compressed(OUT, **data)
    print(OUT, os.path.getsize(OUT), "bytes")
