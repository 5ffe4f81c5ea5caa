"""Seeded random shapes through the default decode entry point, against the CPU oracle.

Every case draws its geometry (query / KV heads, head size, layout, cache encoding, block size,
dtype) and ragged context lengths from a seeded generator, runs the fused RoPE + paged-KV write and
then the decode through whichever kernel the library picks, and compares both with the oracle: cache
bytes bit for bit, attention rows within the tolerance of the dtype. The fixed cases elsewhere pin
the routes; this file only asks that no combination of the supported axes falls between them.
"""

import numpy as np
import pytest
import torch

from attnarc_b200 import workloads
from tests import helpers

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


def draw_config(seed: int) -> workloads.DecodeConfig:
    rng = np.random.default_rng(seed)
    kv_heads = int(rng.choice([1, 2, 3, 4, 8, 16]))
    group = int(rng.choice([1, 2, 4, 6, 8, 16]))
    cache = str(rng.choice(["native", "fp8"]))
    dtype = str(rng.choice(["bf16", "f16"] if cache == "fp8" else ["bf16", "f16", "f32"]))
    batch = int(rng.integers(1, 9))
    longest = int(rng.choice([40, 300, 2100, 5000]))
    lengths = [int(x) for x in rng.integers(1, longest + 1, size=batch)]
    return workloads.DecodeConfig(
        f"random-{seed}", batch, kv_heads * group, kv_heads, head_size=int(rng.choice([64, 128])),
        block_size=int(rng.choice([16, 32])), dtype=dtype, cache=cache,
        fp8_granularity=str(rng.choice(["tensor", "head"])), layout=str(rng.choice(["NHD", "HND"])),
        lengths=("fixed", lengths), rope_style=str(rng.choice(["neox", "interleaved"])))


@pytest.mark.parametrize("seed", range(40))
def test_random_geometry_matches_the_oracle(seed):
    from attnarc_b200 import ops

    config = draw_config(seed)
    case = workloads.build_case(config, DEVICE, seed=seed)
    key_view, value_view = case.cache_views()
    is_neox = config.rope_style == "neox"
    expected_q, expected_k, expected_kc, expected_vc = helpers.oracle_rope_write(
        case.query, case.key, case.value, case.positions, case.cos_sin_cache, key_view, value_view,
        case.slot_mapping, is_neox=is_neox, key_scales=case.key_scales, value_scales=case.value_scales)
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if config.cache == "fp8" else {}
    expected = helpers.oracle_decode(expected_q, expected_kc, expected_vc, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)

    ops.rope_paged_kv_write_(case.query, case.key, case.value, case.positions, case.cos_sin_cache,
                             case.rope_cache_argument(), case.key_scales, case.value_scales, case.slot_mapping,
                             is_neox=is_neox)
    torch.cuda.synchronize()
    what = f"{config}"
    assert helpers.same_bits(case.query, expected_q), what
    assert helpers.same_bits(key_view, expected_kc) and helpers.same_bits(value_view, expected_vc), what
    for split in (False, True):
        actual = ops.paged_decode_attention_ex(case.query, key_view, value_view, case.block_tables,
                                               case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                               scale=case.scale, split=split, **scales)
        helpers.assert_close(actual, expected, config.torch_dtype, f"{what} split={split} route={ops.last_decode_route()}")
    assert ops.decode_timeout_flag() == 0
