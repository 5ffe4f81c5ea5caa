"""Multi-token queries: causal attention of Tq new tokens per sequence.

The reference has no such operator yet (it names it as a later contract field),
so the expectation is its single-token oracle applied token by token: token t of
a sequence of context `length` sees the first `length - (Tq - 1 - t)` tokens.
"""

import numpy as np
import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

DEVICE = torch.device("cuda:0")


def expanded_metadata(block_tables, lengths, query_tokens):
    """The oracle-side restatement of the expansion (numpy)."""
    tables = np.repeat(block_tables, query_tokens, axis=0)
    steps = np.arange(query_tokens)[None, :]
    visible = np.maximum(lengths[:, None] - (query_tokens - 1 - steps), 0).reshape(-1)
    return tables.astype(np.int32), visible.astype(np.int32)


def test_expansion_kernel_matches_numpy():
    from attnarc_b200 import _native

    rng = np.random.default_rng(0)
    tables = rng.integers(-1, 900, size=(7, 33)).astype(np.int32)
    lengths = np.array([1, 2, 3, 4, 100, 517, 0], dtype=np.int32)
    for query_tokens in (1, 3, 4):
        want_tables, want_lengths = expanded_metadata(tables, lengths, query_tokens)
        out_tables = torch.full((7 * query_tokens, 33), -7, dtype=torch.int32, device=DEVICE)
        out_lengths = torch.full((7 * query_tokens,), -7, dtype=torch.int32, device=DEVICE)
        device_tables, device_lengths = torch.from_numpy(tables).to(DEVICE), torch.from_numpy(lengths).to(DEVICE)
        status = _native.library().loom_cuda_expand_query_tokens(
            device_tables.data_ptr(), device_lengths.data_ptr(), out_tables.data_ptr(), out_lengths.data_ptr(),
            7, query_tokens, 33, None)
        torch.cuda.synchronize()
        assert status == 0
        assert np.array_equal(out_tables.cpu().numpy(), want_tables)
        assert np.array_equal(out_lengths.cpu().numpy(), want_lengths)


@pytest.mark.parametrize("one_pass", [True, False])
@pytest.mark.parametrize("name,query_tokens", [("cfg2", 3), ("cfg3", 4), ("cfg4", 2), ("cfg1", 5)])
def test_multi_token_attention_matches_the_oracle_token_by_token(name, query_tokens, one_pass):
    from attnarc_b200 import ops, workloads

    config = workloads.scaled(workloads.CONFIGS[name], batch=5,
                              lengths=("fixed", [2, 17, 300, 1025, 2300]))  # 2 < Tq for Tq = 3, 4
    case = workloads.build_case(config, DEVICE, seed=13)
    key_cache, value_cache = case.cache_views()
    fp8 = config.cache == "fp8"
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if fp8 else {}
    generator = torch.Generator(device="cpu").manual_seed(17)
    query = torch.randn((5, query_tokens, config.query_heads, config.head_size), generator=generator)
    query = query.to(config.torch_dtype).to(DEVICE)

    got = ops.paged_multi_token_decode_attention(query, key_cache, value_cache, case.block_tables,
                                                 case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                                 scale=case.scale, one_pass=one_pass, **scales)
    assert tuple(got.shape) == (5, query_tokens, config.query_heads, config.head_size)

    tables, visible = expanded_metadata(case.block_tables.cpu().numpy(), case.sequence_lengths.cpu().numpy(),
                                        query_tokens)
    rows = query.reshape(5 * query_tokens, config.query_heads, config.head_size)
    live = np.flatnonzero(visible > 0)
    want = helpers.oracle_decode(rows[live].cpu(), key_cache.cpu(), value_cache.cpu(),
                                 torch.from_numpy(tables[live]), torch.from_numpy(visible[live]), scale=case.scale,
                                 max_sequence_length=case.max_sequence_length,
                                 **{k: v.cpu() for k, v in scales.items()})
    flat = got.reshape(5 * query_tokens, config.query_heads, config.head_size)
    helpers.assert_close(flat[torch.from_numpy(live).to(DEVICE)], want, config.torch_dtype,
                         f"{name} Tq={query_tokens}")
    hidden = np.flatnonzero(visible == 0)
    assert len(hidden) == max(query_tokens - 2, 0)
    assert not flat[torch.from_numpy(hidden).to(DEVICE)].any()  # a token with nothing to see yields a zero row

    # the last token of every sequence is the ordinary single-token decode
    single = ops.paged_decode_attention_ex(query[:, -1], key_cache, value_cache, case.block_tables,
                                           case.sequence_lengths, max_sequence_length=case.max_sequence_length,
                                           scale=case.scale, **scales)
    helpers.assert_close(got[:, -1], single, config.torch_dtype, f"{name} last token")


def test_multi_token_rejects_malformed_arguments():
    from attnarc_b200 import ops, workloads

    config = workloads.scaled(workloads.CONFIGS["cfg2"], batch=2)
    case = workloads.build_case(config, DEVICE, seed=1)
    key_cache, value_cache = case.cache_views()
    query = torch.zeros((2, 2, config.query_heads, config.head_size), dtype=config.torch_dtype, device=DEVICE)
    with pytest.raises(RuntimeError, match=r"\[B, Tq, Hq, D\]"):
        ops.paged_multi_token_decode_attention(query[:, 0], key_cache, value_cache, case.block_tables,
                                               case.sequence_lengths, max_sequence_length=case.max_sequence_length)
    with pytest.raises(RuntimeError, match="scratch"):
        ops.paged_multi_token_decode_attention(
            query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
            max_sequence_length=case.max_sequence_length, one_pass=False,
            scratch=(torch.zeros((3, 1), dtype=torch.int32, device=DEVICE),
                     torch.zeros((4,), dtype=torch.int32, device=DEVICE)))
