"""Seeded synthetic workloads shaped like the benchmark configurations.

No dataset or model weight is involved: each configuration is an attention
geometry (heads, head size, block size, batch, context-length distribution)
filled with seeded random data, as the reference's own benchmarks do
(benchmarks/vllm_paged_decode_attention.py, python/tests/
test_paged_decode_attention.py:95-99 for the block-table construction). The
same seed gives the same bytes on any device, because every tensor is drawn on
the CPU generator unless ``fast_device_fill`` is set (bench-only, for caches of
several GB).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field, replace

import numpy as np
import torch

TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


@dataclass(frozen=True)
class DecodeConfig:
    name: str
    batch: int
    query_heads: int
    kv_heads: int
    head_size: int = 128
    block_size: int = 16
    dtype: str = "bf16"
    cache: str = "native"        # "native" or "fp8"
    fp8_granularity: str = "head"  # "tensor" or "head"
    layout: str = "NHD"          # physical order inside a block: NHD or HND
    lengths: tuple = ("uniform", 1, 512)
    partition_tokens: int = 0    # 0 = library default
    rope_style: str = "neox"
    rope_theta: float = 1.0e6
    description: str = ""

    @property
    def torch_dtype(self) -> torch.dtype:
        return TORCH_DTYPES[self.dtype]

    @property
    def cache_element_bytes(self) -> int:
        return 1 if self.cache == "fp8" else {"f32": 4, "f16": 2, "bf16": 2}[self.dtype]

    @property
    def kv_bytes_per_token(self) -> int:
        """Algorithmic K+V bytes one cached token of one sequence costs a decode step."""
        return 2 * self.kv_heads * self.head_size * self.cache_element_bytes


CONFIGS = {
    "cfg1": DecodeConfig("cfg1", 4, 8, 2, dtype="f32", lengths=("uniform", 1, 512),
                         description="CPU-runnable F32 oracle case"),
    "cfg2": DecodeConfig("cfg2", 64, 12, 2, dtype="bf16", lengths=("uniform", 512, 4096),
                         rope_theta=1.0e6,
                         description="Qwen2.5-1.5B-shaped BF16 decode, batch 64"),
    # cfg2's geometry inside the envelope of the reference's own CUDA kernels (contexts up to 1024
    # tokens), for timing both on the same inputs
    "cfg2-1024": DecodeConfig("cfg2-1024", 64, 12, 2, dtype="bf16", lengths=("uniform", 256, 1024),
                              rope_theta=1.0e6,
                              description="Qwen2.5-1.5B-shaped BF16 decode, batch 64, contexts up to 1024"),
    # the reference's largest published case (61.55 us on an H20, its split-K kernels; FA3 30.58 us)
    "ref-b8-ctx1024": DecodeConfig("ref-b8-ctx1024", 8, 32, 8, dtype="bf16", lengths=("fixed", [1024] * 8),
                                   description="the reference's largest published decode case: batch 8, context 1024"),
    "cfg3": DecodeConfig("cfg3", 256, 32, 8, dtype="bf16", layout="HND",
                         lengths=("loguniform", 1024, 8192), partition_tokens=512,
                         description="Llama-3-8B-shaped BF16 decode, batch 256, split-K 512"),
    "cfg4": DecodeConfig("cfg4", 128, 64, 8, dtype="bf16", cache="fp8", fp8_granularity="head",
                         lengths=("uniform", 2048, 16384), rope_style="interleaved", rope_theta=5.0e5,
                         description="Llama-3-70B-shaped decode over an FP8 E4M3 cache, batch 128"),
    "cfg5": DecodeConfig("cfg5", 8, 32, 8, dtype="bf16",
                         lengths=("long_tail", 131072, 256, 32768),
                         description="long-context skewed batch: one 131072 + 7 log-uniform"),
}


def sample_lengths(config: DecodeConfig, rng: np.random.Generator) -> np.ndarray:
    kind = config.lengths[0]
    if kind == "uniform":
        _, low, high = config.lengths
        return rng.integers(low, high + 1, size=config.batch).astype(np.int64)
    if kind == "loguniform":
        _, low, high = config.lengths
        draws = np.exp(rng.uniform(math.log(low), math.log(high), size=config.batch))
        return np.clip(np.rint(draws), low, high).astype(np.int64)
    if kind == "long_tail":
        _, longest, low, high = config.lengths
        draws = np.exp(rng.uniform(math.log(low), math.log(high), size=config.batch - 1))
        rest = np.clip(np.rint(draws), low, high).astype(np.int64)
        return np.concatenate([[longest], rest]).astype(np.int64)
    if kind == "fixed":
        return np.asarray(config.lengths[1], dtype=np.int64)
    raise ValueError(kind)


def rope_table(max_position: int, rotary_dim: int, theta: float, dtype: torch.dtype) -> torch.Tensor:
    """[max_position, rotary_dim]: cosines then sines, computed in float64."""
    half = rotary_dim // 2
    inverse = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / rotary_dim)
    angles = np.arange(max_position, dtype=np.float64)[:, None] * inverse[None, :]
    table = np.concatenate([np.cos(angles), np.sin(angles)], axis=1)
    return torch.from_numpy(table).to(torch.float32).to(dtype)


@dataclass
class DecodeCase:
    config: DecodeConfig
    lengths: np.ndarray                 # int64 [B], context INCLUDING the new token
    max_sequence_length: int
    num_blocks: int
    qkv: torch.Tensor                   # packed [B, (Hq + 2 Hkv) * D] of the new token
    positions: torch.Tensor             # int64 [B] = length - 1
    slot_mapping: torch.Tensor          # int64 [B]
    cos_sin_cache: torch.Tensor         # [max_position, D]
    kv_cache: torch.Tensor              # packed allocation, see `cache_views`
    block_tables: torch.Tensor          # int32 [B, max_blocks]
    sequence_lengths: torch.Tensor      # int32 [B]
    key_scales: torch.Tensor            # float32 [1] or [Hkv]
    value_scales: torch.Tensor
    scale: float
    extras: dict = field(default_factory=dict)

    @property
    def query(self) -> torch.Tensor:
        c = self.config
        return self.qkv.view(c.batch, c.query_heads + 2 * c.kv_heads, c.head_size)[:, : c.query_heads]

    @property
    def key(self) -> torch.Tensor:
        c = self.config
        return self.qkv.view(c.batch, c.query_heads + 2 * c.kv_heads, c.head_size)[
            :, c.query_heads : c.query_heads + c.kv_heads
        ]

    @property
    def value(self) -> torch.Tensor:
        c = self.config
        return self.qkv.view(c.batch, c.query_heads + 2 * c.kv_heads, c.head_size)[:, c.query_heads + c.kv_heads :]

    def cache_views(self) -> tuple[torch.Tensor, torch.Tensor]:
        """Logical [blocks, block_size, kv_heads, D] views of K and V."""
        return logical_cache_views(self.kv_cache, self.config.layout)

    def rope_cache_argument(self) -> torch.Tensor:
        """The [blocks, 2, block_size, kv_heads, D] view the RoPE operator takes."""
        if self.config.layout == "NHD":
            return self.kv_cache
        return self.kv_cache.permute(0, 1, 3, 2, 4)

    @property
    def kv_bytes(self) -> int:
        """Algorithmic bytes one decode step must read from the cache."""
        return int(self.lengths.sum()) * self.config.kv_bytes_per_token


def logical_cache_views(kv_cache: torch.Tensor, layout: str) -> tuple[torch.Tensor, torch.Tensor]:
    if layout == "NHD":  # [blocks, 2, block, heads, D]
        return kv_cache[:, 0], kv_cache[:, 1]
    # HND: [blocks, 2, heads, block, D] -> logical [blocks, block, heads, D]
    return kv_cache[:, 0].permute(0, 2, 1, 3), kv_cache[:, 1].permute(0, 2, 1, 3)


def _fill_normal(shape, dtype, generator, device, fast_device_fill):
    """N(0,1) in `dtype` (F32 for a byte cache); CPU generator unless told otherwise."""
    if fast_device_fill and device.type == "cuda":
        out = torch.randn(shape, device=device, dtype=torch.float32 if dtype == torch.uint8 else dtype,
                          generator=generator)
    else:
        out = torch.randn(shape, dtype=torch.float32, generator=generator)
        if dtype != torch.uint8:
            out = out.to(dtype)
    return out


def build_case(config: DecodeConfig, device="cpu", seed: int = 0, spare_blocks: int = 7,
               fast_device_fill: bool = False, lengths=None) -> DecodeCase:
    """Draws one decode step's inputs. The cache holds every token but the
    newest of each sequence; the RoPE + paged-KV write of `qkv` fills that one."""
    device = torch.device(device)
    rng = np.random.default_rng(seed)
    lengths = sample_lengths(config, rng) if lengths is None else np.asarray(lengths, dtype=np.int64)
    assert len(lengths) == config.batch
    c = config
    dtype = c.torch_dtype
    blocks_per_seq = (lengths + c.block_size - 1) // c.block_size
    max_blocks = int(blocks_per_seq.max())
    max_sequence_length = int(lengths.max())
    num_blocks = int(blocks_per_seq.sum()) + spare_blocks

    permutation = rng.permutation(num_blocks)
    tables = np.zeros((c.batch, max_blocks), dtype=np.int32)
    cursor = 0
    for s in range(c.batch):
        count = int(blocks_per_seq[s])
        tables[s, :count] = permutation[cursor : cursor + count]
        cursor += count

    fill_on_device = fast_device_fill and device.type == "cuda"
    generator = torch.Generator(device=device if fill_on_device else "cpu")
    generator.manual_seed(seed + 1)

    fp8 = c.cache == "fp8"
    inner = (c.block_size, c.kv_heads, c.head_size) if c.layout == "NHD" else (c.kv_heads, c.block_size, c.head_size)
    cache_shape = (num_blocks, 2, *inner)
    head_axis = 3 if c.layout == "NHD" else 2
    if fp8:
        # Per-head standard deviation in [0.5, 4]; the static scale is amax / 448
        # with amax taken as six standard deviations (per head, or of the widest
        # head when one scale serves the whole tensor).
        head_std = torch.from_numpy(rng.uniform(0.5, 4.0, size=(2, c.kv_heads)).astype(np.float32))
        if c.fp8_granularity == "head":
            scales = head_std * 6.0 / 448.0
        else:
            scales = head_std.max(dim=1, keepdim=True).values * 6.0 / 448.0
        key_scales, value_scales = scales[0].contiguous(), scales[1].contiguous()
        ratio_shape = [1, 2, 1, 1, 1]
        ratio_shape[head_axis] = c.kv_heads
        ratio = (head_std / scales).reshape(ratio_shape)  # [K|V, head] broadcast over the cache
        kv_cache = torch.empty(cache_shape, dtype=torch.uint8, device=device)
        step = max(1, (256 << 20) // (int(np.prod(cache_shape[1:])) * 4))
        for start in range(0, num_blocks, step):
            stop = min(num_blocks, start + step)
            chunk = _fill_normal((stop - start, *cache_shape[1:]), torch.uint8, generator, device,
                                 fast_device_fill)
            chunk = (chunk * ratio.to(chunk.device)).clamp_(-448.0, 448.0)
            kv_cache[start:stop] = chunk.to(torch.float8_e4m3fn).view(torch.uint8).to(device)
        source_std = head_std
    else:
        key_scales = torch.ones(1, dtype=torch.float32)
        value_scales = torch.ones(1, dtype=torch.float32)
        if fill_on_device:
            kv_cache = torch.randn(cache_shape, device=device, dtype=dtype, generator=generator)
        else:
            kv_cache = torch.randn(cache_shape, dtype=torch.float32, generator=generator).to(dtype).to(device)
        source_std = None

    width = (c.query_heads + 2 * c.kv_heads) * c.head_size
    qkv = torch.randn((c.batch, width), dtype=torch.float32, generator=torch.Generator().manual_seed(seed + 2))
    if source_std is not None:
        view = qkv.view(c.batch, c.query_heads + 2 * c.kv_heads, c.head_size)
        view[:, c.query_heads : c.query_heads + c.kv_heads] *= source_std[0][None, :, None]
        view[:, c.query_heads + c.kv_heads :] *= source_std[1][None, :, None]
    qkv = qkv.to(dtype).to(device)

    positions = torch.from_numpy(lengths - 1)
    last_block = tables[np.arange(c.batch), (lengths - 1) // c.block_size].astype(np.int64)
    slot_mapping = torch.from_numpy(last_block * c.block_size + (lengths - 1) % c.block_size)
    cos_sin = rope_table(max_sequence_length, c.head_size, c.rope_theta, dtype)

    return DecodeCase(
        config=c,
        lengths=lengths,
        max_sequence_length=max_sequence_length,
        num_blocks=num_blocks,
        qkv=qkv,
        positions=positions.to(device),
        slot_mapping=slot_mapping.to(device),
        cos_sin_cache=cos_sin.to(device),
        kv_cache=kv_cache,
        block_tables=torch.from_numpy(tables).to(device),
        sequence_lengths=torch.from_numpy(lengths.astype(np.int32)).to(device),
        key_scales=key_scales.to(device),
        value_scales=value_scales.to(device),
        scale=1.0 / math.sqrt(c.head_size),
    )


def scaled(config: DecodeConfig, **changes) -> DecodeConfig:
    """A copy of a configuration with some fields replaced (smaller test cases)."""
    return replace(config, **changes)
