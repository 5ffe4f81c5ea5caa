"""Sharding the paged-decode path over the GPUs of one node.

The reference runs on one device (its operator catalogue lists distributed
split-KV as planned, docs/operator-catalog.md:109), so nothing here replaces a
reference interface; the names follow its vocabulary (sequences, KV heads,
blocks, partial states).

One process per GPU. A decode step is a set of independent (sequence, KV head)
units, so two of the three modes need no exchange on the data path:

* by sequence: every rank decodes whole sequences of the batch, chosen so that
  the ranks read about the same number of cached tokens;
* by KV head: every rank owns a contiguous range of KV heads (and the query
  heads of their groups) of every sequence: the layout tensor parallelism gives;
* long context: a sequence longer than a rank's fair share is cut into one
  block range per rank. Each rank turns its range into partial (O, max, sum)
  states; one all-gather moves the states (``Dv + 2`` floats per query head and
  rank) and every rank merges them. This is the only collective of the path.

The assignment itself is computed by the C partitioner of the library
(``include/loom_partition.h``): it is deterministic, so every rank computes the
same plan from the same lengths without talking to the others.

The decode and merge kernels are passed in as callables by the few functions
that launch work (default: the CUDA operators of ``attnarc_b200.ops``).
Host-side tests substitute their own checker for them; nothing in this module
computes attention on the CPU.
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Callable, Sequence

import torch

from . import _native


class _Shard(ctypes.Structure):
    _fields_ = [
        ("sequence", ctypes.c_uint32),
        ("rank", ctypes.c_uint32),
        ("first_block", ctypes.c_uint32),
        ("block_count", ctypes.c_uint32),
        ("first_token", ctypes.c_uint64),
        ("token_count", ctypes.c_uint64),
        ("split", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32),
    ]


@dataclasses.dataclass(frozen=True)
class SequenceShard:
    """A whole sequence, or one block range of a split sequence, owned by a rank."""

    sequence: int
    rank: int
    first_block: int
    block_count: int
    first_token: int
    token_count: int
    split: bool


def _lengths_array(lengths: Sequence[int]):
    values = [int(v) for v in lengths]
    return (ctypes.c_int64 * max(len(values), 1))(*values), len(values)


def _check(status: int, what: str) -> None:
    if status != 0:
        raise ValueError(f"{what}: invalid argument")


def partition_by_sequence(lengths: Sequence[int], ranks: int) -> tuple[list[int], list[int]]:
    """Owner rank of every sequence and the cached tokens each rank reads.

    Longest sequence first, each to the rank with the fewest tokens so far;
    ties go to the lower rank.
    """
    array, count = _lengths_array(lengths)
    owners = (ctypes.c_uint32 * max(count, 1))()
    tokens = (ctypes.c_uint64 * max(ranks, 1))()
    _check(_native.library().loom_partition_by_sequence(array, count, ranks, owners, tokens),
           "partition by sequence")
    return list(owners[:count]), list(tokens[:ranks])


def partition_by_kv_head(kv_heads: int, ranks: int) -> list[tuple[int, int]]:
    """(first KV head, KV head count) of every rank; counts differ by at most one."""
    first = (ctypes.c_uint32 * max(ranks, 1))()
    count = (ctypes.c_uint32 * max(ranks, 1))()
    _check(_native.library().loom_partition_by_kv_head(kv_heads, ranks, first, count), "partition by KV head")
    return [(int(first[r]), int(count[r])) for r in range(ranks)]


def partition_long_context(lengths: Sequence[int], ranks: int, block_size: int,
                           split_threshold_tokens: int = 0) -> tuple[list[SequenceShard], list[int]]:
    """Shards of a batch in which long sequences are cut into one block range per rank.

    Returns the shards (ordered by sequence, then rank) and the tokens per rank.
    ``split_threshold_tokens`` of 0 means a rank's fair share of the batch.
    """
    array, count = _lengths_array(lengths)
    capacity = count * (ranks + 1) + 1
    shards = (_Shard * capacity)()
    produced = ctypes.c_uint32(0)
    tokens = (ctypes.c_uint64 * max(ranks, 1))()
    _check(
        _native.library().loom_partition_long_context(
            array, count, ranks, block_size, split_threshold_tokens,
            ctypes.cast(shards, ctypes.c_void_p), capacity, ctypes.byref(produced), tokens),
        "long-context partition",
    )
    out = [
        SequenceShard(int(s.sequence), int(s.rank), int(s.first_block), int(s.block_count),
                      int(s.first_token), int(s.token_count), bool(s.split))
        for s in shards[: produced.value]
    ]
    return out, list(tokens[:ranks])


# ------------------------------------------------------------ plans per rank

@dataclasses.dataclass(frozen=True)
class RankBatch:
    """What one rank decodes in a step.

    ``rows`` are indices into the global batch, in the order of the rank's local
    batch. ``first_blocks``/``lengths`` give, per local row, the first logical
    block of its range and the number of tokens inside the range (the whole
    sequence when it is not split). ``split_rows`` marks rows whose result is a
    partial state that must be merged with other ranks' states.
    """

    rank: int
    rows: list[int]
    first_blocks: list[int]
    lengths: list[int]
    split_rows: list[bool]

    @property
    def tokens(self) -> int:
        return sum(self.lengths)


def plan_by_sequence(lengths: Sequence[int], ranks: int) -> list[RankBatch]:
    owners, _ = partition_by_sequence(lengths, ranks)
    plans = []
    for rank in range(ranks):
        rows = [i for i, owner in enumerate(owners) if owner == rank]
        plans.append(RankBatch(rank, rows, [0] * len(rows), [int(lengths[i]) for i in rows], [False] * len(rows)))
    return plans


def plan_long_context(lengths: Sequence[int], ranks: int, block_size: int,
                      split_threshold_tokens: int = 0) -> list[RankBatch]:
    shards, _ = partition_long_context(lengths, ranks, block_size, split_threshold_tokens)
    plans = []
    for rank in range(ranks):
        mine = [s for s in shards if s.rank == rank]
        plans.append(RankBatch(rank, [s.sequence for s in mine], [s.first_block for s in mine],
                               [s.token_count for s in mine], [s.split for s in mine]))
    return plans


def local_decode_inputs(plan: RankBatch, query: torch.Tensor, block_tables: torch.Tensor
                        ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Slices a rank's rows out of the global query and block table.

    The block table of a split row is shifted so that its range starts at
    logical block 0: the kernels then see an ordinary, shorter sequence.
    Returns (query rows, block tables, lengths) on the device of ``query``.
    """
    device = query.device
    rows = torch.tensor(plan.rows, dtype=torch.int64, device=device)
    local_query = query.index_select(0, rows)
    width = block_tables.shape[1]
    tables = block_tables.index_select(0, rows.to(block_tables.device))
    firsts = torch.tensor(plan.first_blocks, dtype=torch.int64, device=tables.device)
    columns = (torch.arange(width, device=tables.device).unsqueeze(0) + firsts.unsqueeze(1)).clamp_(max=width - 1)
    tables = torch.gather(tables, 1, columns).contiguous()
    lengths = torch.tensor(plan.lengths, dtype=torch.int32, device=device)
    return local_query.contiguous(), tables, lengths


DecodeStates = Callable[..., torch.Tensor]
MergeStates = Callable[[torch.Tensor, torch.dtype], torch.Tensor]


def _default_decode_states(query, key_cache, value_cache, block_tables, lengths, **kwargs):
    from . import ops

    return ops.paged_decode_attention_ex(query, key_cache, value_cache, block_tables, lengths,
                                         emit_state=True, **kwargs)


def _default_merge(states, dtype):
    from . import ops

    return ops.merge_decode_states(states, dtype)


def decode_long_context(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    lengths: Sequence[int],
    *,
    scale: float,
    block_size: int,
    group=None,
    split_threshold_tokens: int = 0,
    decode_states: DecodeStates = _default_decode_states,
    merge_states: MergeStates = _default_merge,
    **decode_kwargs,
) -> torch.Tensor:
    """One decode step of a batch whose long sequences are spread over the ranks.

    Every rank holds the whole (replicated or peer-visible) block table and the
    blocks of its own ranges in its cache. Each rank computes partial states
    for its rows, the states are all-gathered (``Dv + 2`` floats per query head
    per rank), and every rank merges them: all ranks return the full
    ``[B, Hq, Dv]`` output. Rows that a rank does not own contribute an empty
    state (max = -inf, sum = 0), which the merge ignores.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    plan = plan_long_context(lengths, world, block_size, split_threshold_tokens)[rank]
    batch, query_heads, _ = query.shape
    value_dim = value_cache.shape[3]
    states = torch.zeros((batch, query_heads, value_dim + 2), dtype=torch.float32, device=query.device)
    states[:, :, value_dim] = float("-inf")
    if plan.rows:
        local_query, tables, local_lengths = local_decode_inputs(plan, query, block_tables)
        local_states = decode_states(local_query, key_cache, value_cache, tables, local_lengths,
                                     max_sequence_length=int(max(plan.lengths + [1])), scale=scale,
                                     **decode_kwargs)
        # a split sequence appears at most once per rank, so the rows are distinct
        states.index_copy_(0, torch.tensor(plan.rows, dtype=torch.int64, device=query.device),
                           local_states.to(torch.float32))
    gathered = torch.empty(world * states.numel(), dtype=torch.float32, device=query.device)
    dist.all_gather_into_tensor(gathered, states.reshape(-1), group=group)
    merged = merge_states(gathered.reshape(world, batch * query_heads, value_dim + 2).contiguous(), query.dtype)
    return merged.reshape(batch, query_heads, value_dim)


def decode_by_sequence(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    lengths: Sequence[int],
    *,
    scale: float,
    rank: int,
    ranks: int,
    decode: Callable[..., torch.Tensor] | None = None,
    **decode_kwargs,
) -> tuple[list[int], torch.Tensor]:
    """Decodes the sequences this rank owns; no communication.

    Returns the global row indices and the ``[rows, Hq, Dv]`` outputs. A serving
    engine with data-parallel replicas keeps the rows where they are.
    """
    if decode is None:
        from . import ops

        decode = ops.paged_decode_attention_ex
    plan = plan_by_sequence(lengths, ranks)[rank]
    if not plan.rows:
        empty = query.new_empty((0, query.shape[1], value_cache.shape[3]))
        return [], empty
    local_query, tables, local_lengths = local_decode_inputs(plan, query, block_tables)
    output = decode(local_query, key_cache, value_cache, tables, local_lengths,
                    max_sequence_length=int(max(plan.lengths + [1])), scale=scale, **decode_kwargs)
    return plan.rows, output
