"""The long-context exchange on two GPUs: one process per GPU, the partial states
exchanged by NCCL (all-gather + merge operator) and by this library's own push
and merge kernels over peer memory. Skipped where fewer than two devices are
visible.
"""

import os
import socket

import pytest
import torch

from attnarc_b200 import multi_gpu
from tests.helpers import assert_close, oracle_decode
from tests.test_multi_gpu_host import build_case

pytestmark = pytest.mark.gpu


def _rank(rank, world, port, results):
    import faulthandler

    import torch.distributed as dist

    faulthandler.dump_traceback_later(120, exit=True)  # a rank that stops making progress says where, and ends

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        query, keys, values, tables, lengths, block, scale = build_case(41)
        device = torch.device("cuda", rank)
        merged = multi_gpu.decode_long_context(
            query.to(device), keys.to(device), values.to(device), tables.to(device), lengths,
            scale=scale, block_size=block, split_threshold_tokens=256)
        torch.cuda.synchronize()
        results[rank] = merged.cpu()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_long_context_exchange_over_nccl():
    import torch.multiprocessing as mp

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, port, results), nprocs=2, join=True)
    query, keys, values, tables, lengths, block, scale = build_case(41)
    live = [i for i, n in enumerate(lengths) if n > 0]
    expected = torch.zeros((len(lengths), query.shape[1], values.shape[3]), dtype=torch.bfloat16)
    expected[live] = oracle_decode(query[live], keys, values, tables[live],
                                   torch.tensor([lengths[i] for i in live], dtype=torch.int32),
                                   scale=scale, max_sequence_length=max(lengths))
    for rank in (0, 1):
        assert_close(results[rank], expected, torch.bfloat16, f"rank {rank}")


def _peer_rank(rank, world, port, results):
    import faulthandler

    import torch.distributed as dist

    faulthandler.dump_traceback_later(120, exit=True)  # a rank that stops making progress says where, and ends

    from attnarc_b200 import sharded_step, workloads

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        config = workloads.scaled(workloads.CONFIGS["cfg5"], batch=4, lengths=("fixed", [9000, 40, 700, 16]))
        case = workloads.build_case(config, torch.device("cuda", rank), seed=37)
        shard = sharded_step.shard_long_context(case, rank, world)
        rows = {}
        for exchange in ("peer", "nccl"):
            step = sharded_step.ShardedDecodeStep(shard, case.cos_sin_cache, dtype=config.torch_dtype,
                                                  scale=case.scale, is_neox=True, exchange=exchange)
            eager = step.run_eager().clone()
            step.capture()
            for _ in range(3):  # the captured step, several times: step counters, both buffer generations
                replayed = step.run().clone()
            assert torch.equal(eager.view(torch.int16), replayed.view(torch.int16))
            if step.peer_exchange is not None:
                assert step.peer_exchange.status() == (5, 0)  # eager + the capture's own run + three replays
            rows[exchange] = replayed
            # a CUDA graph that holds a captured NCCL collective must be gone before the group is
            # destroyed, and peers must have stopped pushing before a rank frees its exchange buffer
            torch.cuda.synchronize()
            dist.barrier()
            step.close()
            del step
        dist.barrier()
        results[rank] = rows
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_exchange_step_equals_the_nccl_step_and_the_oracle():
    import torch.multiprocessing as mp

    from attnarc_b200 import workloads
    from tests.test_gpu_sharded_decode import _oracle_rows

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_peer_rank, args=(2, port, results), nprocs=2, join=True)
    config = workloads.scaled(workloads.CONFIGS["cfg5"], batch=4, lengths=("fixed", [9000, 40, 700, 16]))
    expected = _oracle_rows(workloads.build_case(config, torch.device("cuda", 0), seed=37))
    for rank in (0, 1):
        assert_close(results[rank]["peer"], expected, torch.bfloat16, f"rank {rank}, peer exchange")
        assert_close(results[rank]["nccl"], expected, torch.bfloat16, f"rank {rank}, NCCL exchange")
