"""The sharding plans of ``attnarc_b200.multi_gpu`` driven through the CUDA
operators on one device: every rank's part is decoded in turn, the partial
states are stacked as an all-gather would deliver them, and the merged result
is compared with the oracle's decode of the unsplit batch.
"""

import pytest
import torch

from attnarc_b200 import multi_gpu
from tests.helpers import assert_close, oracle_decode
from tests.test_multi_gpu_host import build_case

pytestmark = pytest.mark.gpu


def expected_output(query, keys, values, tables, lengths, scale):
    live = [i for i, n in enumerate(lengths) if n > 0]
    expected = torch.zeros((len(lengths), query.shape[1], values.shape[3]), dtype=query.dtype)
    expected[live] = oracle_decode(query[live], keys, values, tables[live],
                                   torch.tensor([lengths[i] for i in live], dtype=torch.int32),
                                   scale=scale, max_sequence_length=max(lengths))
    return expected


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_long_context_plan_merges_to_the_unsplit_result(ranks):
    from attnarc_b200 import ops

    query, keys, values, tables, lengths, block, scale = build_case(23)
    device = torch.device("cuda:0")
    q, k, v, t = (x.to(device) for x in (query, keys, values, tables))
    batch, heads, dim = q.shape
    stacked = torch.zeros((ranks, batch, heads, dim + 2), dtype=torch.float32, device=device)
    stacked[:, :, :, dim] = float("-inf")
    plans = multi_gpu.plan_long_context(lengths, ranks, block, split_threshold_tokens=256)
    assert sum(p.tokens for p in plans) == sum(lengths)
    for plan in plans:
        if not plan.rows:
            continue
        local_q, local_t, local_n = multi_gpu.local_decode_inputs(plan, q, t)
        states = ops.paged_decode_attention_ex(local_q, k, v, local_t, local_n,
                                               max_sequence_length=max(plan.lengths + [1]), scale=scale,
                                               emit_state=True)
        stacked[plan.rank].index_copy_(0, torch.tensor(plan.rows, device=device), states)
    merged = ops.merge_decode_states(stacked.reshape(ranks, batch * heads, dim + 2).contiguous(), torch.bfloat16)
    assert_close(merged.reshape(batch, heads, dim).cpu(), expected_output(query, keys, values, tables, lengths, scale),
                 torch.bfloat16, f"{ranks} ranks")


def test_by_sequence_plan_covers_the_batch():
    query, keys, values, tables, lengths, block, scale = build_case(29)
    device = torch.device("cuda:0")
    q, k, v, t = (x.to(device) for x in (query, keys, values, tables))
    result = torch.zeros((len(lengths), q.shape[1], v.shape[3]), dtype=torch.bfloat16)
    for rank in range(3):
        rows, output = multi_gpu.decode_by_sequence(q, k, v, t, lengths, scale=scale, rank=rank, ranks=3)
        if rows:
            result[rows] = output.cpu()
    assert_close(result, expected_output(query, keys, values, tables, lengths, scale), torch.bfloat16, "by sequence")
