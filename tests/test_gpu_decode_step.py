"""The captured serving step (`attnarc_b200.decode_step`): one CUDA graph per step.

The graph replays the host-to-device copy, RoPE + KV write, decode and the copy
back; its cache bytes and attention rows must equal those of the same operators
called one by one, also after the caller has refilled the host views.
"""

import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu


def eager_step(case, config, kv_cache, qkv, positions, slots, tables, lengths):
    from attnarc_b200 import ops

    rows = qkv.clone().view(config.batch, config.query_heads + 2 * config.kv_heads, config.head_size)
    q = rows[:, :config.query_heads]
    k = rows[:, config.query_heads:config.query_heads + config.kv_heads]
    v = rows[:, config.query_heads + config.kv_heads:]
    fp8 = kv_cache.dtype == torch.uint8
    ops.rope_paged_kv_write_(q, k, v, positions, case.cos_sin_cache, kv_cache, case.key_scales, case.value_scales,
                             slots, is_neox=config.rope_style == "neox")
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if fp8 else {}
    return ops.paged_decode_attention_ex(q, kv_cache[:, 0], kv_cache[:, 1], tables, lengths,
                                         max_sequence_length=case.max_sequence_length, scale=case.scale, **scales)


@pytest.mark.parametrize("name,batch", [("cfg2", 8), ("cfg3", 6), ("cfg4", 4)])
def test_captured_step_equals_the_operators_called_one_by_one(name, batch):
    from attnarc_b200 import workloads
    from attnarc_b200.decode_step import CapturedDecodeStep

    device = torch.device("cuda:0")
    config = workloads.scaled(workloads.CONFIGS[name], batch=batch)
    case = workloads.build_case(config, device, seed=5)
    block = config.block_size

    def cache_argument(allocation):
        return allocation if config.layout == "NHD" else allocation.permute(0, 1, 3, 2, 4)

    graph_cache, eager_cache = case.kv_cache.clone(), case.kv_cache.clone()
    fp8 = config.cache == "fp8"
    step = CapturedDecodeStep(
        cache_argument(graph_cache), case.cos_sin_cache, sequences=batch, query_heads=config.query_heads,
        max_blocks_per_sequence=case.block_tables.shape[1], max_sequence_length=case.max_sequence_length,
        dtype=config.torch_dtype, scale=case.scale, is_neox=config.rope_style == "neox",
        key_scales=case.key_scales if fp8 else None, value_scales=case.value_scales if fp8 else None)

    def fill(qkv, positions, slots, tables, lengths):
        step.host_qkv.copy_(qkv.view(step.host_qkv.shape).cpu())
        step.host_positions.copy_(positions.cpu())
        step.host_slot_mapping.copy_(slots.cpu())
        step.host_block_tables.copy_(tables.cpu())
        step.host_sequence_lengths.copy_(lengths.cpu())

    # ---- the step the case describes ----------------------------------------------------
    fill(case.qkv, case.positions, case.slot_mapping, case.block_tables, case.sequence_lengths)
    step.capture()
    got = step.run().clone()
    want = eager_step(case, config, cache_argument(eager_cache), case.qkv, case.positions, case.slot_mapping,
                      case.block_tables, case.sequence_lengths)
    torch.cuda.synchronize()
    assert helpers.same_bits(got, want.cpu())
    assert helpers.same_bits(graph_cache.cpu(), eager_cache.cpu())

    # ---- another step through the same graph: shorter contexts, other rows ------------------
    lengths = torch.clamp(case.sequence_lengths - 5, min=1)
    positions = (lengths - 1).to(torch.int64)
    logical = (positions // block).to(torch.int64)
    physical = case.block_tables.gather(1, logical[:, None])[:, 0].to(torch.int64)
    slots = physical * block + positions % block
    generator = torch.Generator(device="cpu").manual_seed(11)
    qkv = torch.randn(case.qkv.shape, generator=generator).to(config.torch_dtype).to(device)
    fill(qkv, positions, slots, case.block_tables, lengths)
    got = step.run().clone()
    want = eager_step(case, config, cache_argument(eager_cache), qkv, positions, slots, case.block_tables, lengths)
    torch.cuda.synchronize()
    assert helpers.same_bits(got, want.cpu())
    assert helpers.same_bits(graph_cache.cpu(), eager_cache.cpu())
    assert step.kernel_launches in (2, 3) and step.h2d_bytes > 0 and step.d2h_bytes == got.numel() * got.element_size()


def test_run_before_capture_is_an_error():
    from attnarc_b200 import workloads
    from attnarc_b200.decode_step import CapturedDecodeStep

    device = torch.device("cuda:0")
    config = workloads.scaled(workloads.CONFIGS["cfg2"], batch=2)
    case = workloads.build_case(config, device, seed=1)
    step = CapturedDecodeStep(case.kv_cache, case.cos_sin_cache, sequences=2, query_heads=config.query_heads,
                              max_blocks_per_sequence=case.block_tables.shape[1],
                              max_sequence_length=case.max_sequence_length, dtype=config.torch_dtype)
    with pytest.raises(RuntimeError, match="capture"):
        step.run()
