"""The bounded waits of the copy-fed kernels, made to run out without any fault.

``ops.set_wait_policy(attempts, unmatched_bytes)`` arms every copy barrier for
more bytes than its copy delivers and lowers the poll limit: the first wait of
every ring expires although the data arrived. The kernels must then set their
timeout flag, start no further copy, return (the device stays usable), and
work normally again once the policy is back to service values.
"""

import pytest
import torch

from attnarc_b200 import workloads
from tests import helpers

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


@pytest.fixture()
def ops():
    from attnarc_b200 import ops as module

    module.set_wait_policy()
    yield module
    module.set_wait_policy()
    module.set_decode_copy_engine("tma")
    module.decode_timeout_flag(reset=True)
    module.kv_block_move_timeout_flag(reset=True)


@pytest.mark.parametrize("name,engine", [("cfg2", "tma"), ("cfg4", "tma"), ("cfg4", "tma-head"), ("cfg4", "tma-mma")])
def test_an_expired_wait_of_the_decode_kernel_sets_the_flag_and_returns(ops, name, engine):
    # cfg4 / tma: the FP8 kernel that copies a block of eight KV heads per tile; tma-head: one KV head per
    # tile, copies issued by a warp of their own; tma-mma: every warp feeds itself
    ops.set_decode_copy_engine(engine)
    config = workloads.scaled(workloads.CONFIGS[name], batch=3, lengths=("fixed", [700, 64, 300]))
    case = workloads.build_case(config, DEVICE, seed=9)
    key_cache, value_cache = case.cache_views()
    query = case.query.contiguous()
    scales = dict(key_scales=case.key_scales, value_scales=case.value_scales) if config.cache == "fp8" else {}

    def decode():
        out = ops.paged_decode_attention_ex(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                            max_sequence_length=case.max_sequence_length, scale=case.scale,
                                            split=True, **scales)
        torch.cuda.synchronize()  # the kernel returned: no hang, no fault
        return out

    expected = helpers.oracle_decode(query, key_cache, value_cache, case.block_tables, case.sequence_lengths,
                                     scale=case.scale, max_sequence_length=case.max_sequence_length, **scales)
    helpers.assert_close(decode(), expected, config.torch_dtype, "before")
    route = ops.last_decode_route()
    assert "balanced" in route and route.endswith("-tma")
    assert ("producer" in route) == (name == "cfg4" and engine == "tma-head")
    assert ("block" in route) == (name == "cfg4" and engine == "tma")
    assert ops.decode_timeout_flag() == 0

    ops.set_wait_policy(attempts=400, unmatched_bytes=16)
    decode()
    flag = ops.decode_timeout_flag()
    assert flag & 1, "the expiry must be visible to the host"
    assert (flag >> 20) == 1, "the first expiry was a wait on a K/V tile of the streaming kernel"
    assert ops.decode_timeout_flag(reset=True) == flag and ops.decode_timeout_flag() == 0

    ops.set_wait_policy()
    helpers.assert_close(decode(), expected, config.torch_dtype, "after")
    assert ops.decode_timeout_flag() == 0


@pytest.mark.parametrize("swap", [False, True])
def test_an_expired_wait_of_the_block_movement_kernels_sets_the_flag_and_returns(ops, swap):
    generator = torch.Generator(device=DEVICE).manual_seed(3)
    cache = torch.randint(0, 255, (24, 2, 16, 2, 128), dtype=torch.uint8, device=DEVICE, generator=generator)
    pairs = torch.tensor([[0, 12], [1, 13], [2, 14], [3, 15]], dtype=torch.int64, device=DEVICE)
    before = cache.clone()

    def operate(target):
        if swap:
            ops.kv_block_swap_(target, pairs)
        else:
            ops.kv_block_move_(target, target, pairs)
        torch.cuda.synchronize()

    ops.set_wait_policy(attempts=400, unmatched_bytes=16)
    scratch = cache.clone()
    operate(scratch)
    assert ops.kv_block_move_timeout_flag() != 0
    assert ops.kv_block_move_timeout_flag(reset=True) != 0 and ops.kv_block_move_timeout_flag() == 0
    # blocks no pair names are untouched whatever happened to the others
    assert torch.equal(scratch[16:], before[16:]) and torch.equal(scratch[4:12], before[4:12])

    ops.set_wait_policy()
    operate(cache)
    assert ops.kv_block_move_timeout_flag() == 0
    assert torch.equal(cache[12:16], before[0:4])
    assert torch.equal(cache[0:4], before[12:16] if swap else before[0:4])


def test_wait_policy_rejects_odd_byte_counts(ops):
    with pytest.raises(ValueError):
        ops.set_wait_policy(100, 7)


def test_no_launch_needed_a_plain_retry_and_failures_name_their_site(ops):
    assert ops.plain_launch_retries() == 0
    assert ops.last_launch_failure() == "none" or " at " in ops.last_launch_failure()
