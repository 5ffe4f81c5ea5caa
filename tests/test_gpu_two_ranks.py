"""The long-context exchange on two GPUs: one process per GPU, NCCL all-gather of
the partial states, merge on every rank. Skipped where fewer than two devices
are visible.
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
    import torch.distributed as dist

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
