"""One decode step of ONE global batch spread over the GPUs of a node.

The reference runs on one device and lists distributed split-KV as planned
(docs/operator-catalog.md:109), so nothing here replaces a reference
interface. One process per GPU; every rank computes the same plan from the
batch's lengths (``attnarc_b200.multi_gpu``, the C partitioner) and holds only
the pages its share of the step reads:

* ``shard_by_sequence``: whole sequences per rank; the rank's blocks are packed
  into a local cache and its block tables renumbered. No exchange.
* ``shard_by_kv_head``: a contiguous range of KV heads (and the query heads of
  their groups) of every sequence per rank; the local cache is the head slice
  of every block. No exchange.
* ``shard_long_context``: a sequence longer than a rank's fair share is cut
  into one block range per rank; the other sequences are placed whole. Every
  rank decodes its ranges into partial (O, max, sum) states, one all-gather
  moves the states and every rank merges them.

``ShardedDecodeStep`` turns a shard into the rank's serving step: host buffers
in, RoPE + paged-KV write, decode (plus all-gather and merge in the
long-context mode), rows out; eagerly or as one CUDA graph per step.
"""

from __future__ import annotations

import dataclasses
from typing import Sequence

import torch

from . import multi_gpu, ops


@dataclasses.dataclass
class RankShard:
    """What one rank holds and computes of a global decode step.

    The local batch has ``len(rows)`` sequences; local row ``i`` is global row
    ``rows[i]``. ``query_heads`` is the (first, count) range of global query
    heads the rank computes, ``kv_heads`` likewise. ``kv_cache`` is the packed
    local allocation ``[local_blocks, 2, ...]`` in the layout of the global one;
    ``rope_cache`` is its ``[blocks, 2, block_size, kv_heads, dim]`` view.
    ``qkv`` holds the local packed rows of the step's new tokens. In the
    long-context mode every rank lists every sequence; a sequence it holds no
    range of has length 0 there, and ``slot_mapping`` is -1 (rotate, do not
    write) unless the rank holds the block of the new token.
    """

    mode: str
    rank: int
    ranks: int
    rows: list[int]
    query_heads: tuple[int, int]
    kv_heads: tuple[int, int]
    kv_cache: torch.Tensor
    rope_cache: torch.Tensor
    block_tables: torch.Tensor
    sequence_lengths: torch.Tensor
    qkv: torch.Tensor
    positions: torch.Tensor
    slot_mapping: torch.Tensor
    key_scales: torch.Tensor
    value_scales: torch.Tensor
    max_sequence_length: int
    kv_bytes: int
    exchange: bool = False

    @property
    def sequences(self) -> int:
        return len(self.rows)


def _rope_view(kv_cache: torch.Tensor, layout: str) -> torch.Tensor:
    return kv_cache if layout == "NHD" else kv_cache.permute(0, 1, 3, 2, 4)


def _pack_blocks(case, wanted_blocks: torch.Tensor, spare_blocks: int = 1):
    """Copies the named global blocks into a fresh local cache, in order.

    Returns (local cache, int32 map global block id -> local id, -1 elsewhere).
    The copy is the library's own block-move operator: a block's K bytes and V
    bytes are each one dense span in NHD and HND alike.
    """
    device = case.kv_cache.device
    count = int(wanted_blocks.numel())
    local = torch.zeros((count + spare_blocks, *case.kv_cache.shape[1:]), dtype=case.kv_cache.dtype, device=device)
    renumber = torch.full((case.num_blocks,), -1, dtype=torch.int32, device=device)
    if count:
        local_ids = torch.arange(count, dtype=torch.int64, device=device)
        renumber[wanted_blocks] = local_ids.to(torch.int32)
        pairs = torch.stack([wanted_blocks.to(torch.int64), local_ids], dim=1).contiguous()
        ops.kv_block_move_(local, case.kv_cache, pairs)
    return local, renumber


def _local_slots(case, renumber, rows: torch.Tensor) -> torch.Tensor:
    """Slots of the new tokens of global ``rows`` in local numbering (-1 if the block is elsewhere)."""
    block_size = case.config.block_size
    global_slots = case.slot_mapping[rows]
    local_block = renumber[(global_slots // block_size)].to(torch.int64)
    slots = local_block * block_size + global_slots % block_size
    return torch.where(local_block < 0, torch.full_like(slots, -1), slots)


def whole_case(case) -> RankShard:
    """The whole batch as the shard of a single rank: the case's own cache, nothing copied."""
    config = case.config
    return RankShard(
        mode="single GPU", rank=0, ranks=1, rows=list(range(config.batch)),
        query_heads=(0, config.query_heads), kv_heads=(0, config.kv_heads),
        kv_cache=case.kv_cache, rope_cache=_rope_view(case.kv_cache, config.layout),
        block_tables=case.block_tables, sequence_lengths=case.sequence_lengths, qkv=case.qkv,
        positions=case.positions, slot_mapping=case.slot_mapping, key_scales=case.key_scales,
        value_scales=case.value_scales, max_sequence_length=case.max_sequence_length, kv_bytes=case.kv_bytes)


def shard_by_sequence(case, rank: int, ranks: int) -> RankShard:
    """The sequences of ``case`` this rank owns, with their blocks packed into a local cache."""
    plan = multi_gpu.plan_by_sequence(case.lengths.tolist(), ranks)[rank]
    return shard_rows(case, plan.rows, rank, ranks)


def shard_rows(case, owned_rows: Sequence[int], rank: int = 0, ranks: int = 1) -> RankShard:
    """The named sequences of ``case`` with their blocks packed into a local cache."""
    config = case.config

    owned = list(owned_rows)
    owned_lengths = [int(case.lengths[r]) for r in owned]
    device = case.kv_cache.device
    rows = torch.tensor(owned, dtype=torch.int64, device=device)
    block_size = config.block_size
    tables = case.block_tables[rows] if owned else case.block_tables[:0]
    lengths = case.sequence_lengths[rows] if owned else case.sequence_lengths[:0]
    blocks_per_row = (lengths + block_size - 1) // block_size
    width = int(blocks_per_row.max()) if owned else 1
    tables = tables[:, :width]
    live = torch.arange(width, device=device)[None, :] < blocks_per_row[:, None]
    wanted = tables[live].to(torch.int64)
    local_cache, renumber = _pack_blocks(case, wanted)
    local_tables = torch.where(live, renumber[tables.to(torch.int64)], torch.zeros_like(tables)).contiguous()
    return RankShard(
        mode="by sequence", rank=rank, ranks=ranks, rows=list(owned),
        query_heads=(0, config.query_heads), kv_heads=(0, config.kv_heads),
        kv_cache=local_cache, rope_cache=_rope_view(local_cache, config.layout),
        block_tables=local_tables.to(torch.int32), sequence_lengths=lengths.contiguous(),
        qkv=case.qkv[rows].contiguous(), positions=case.positions[rows].contiguous(),
        slot_mapping=_local_slots(case, renumber, rows).contiguous(),
        key_scales=case.key_scales, value_scales=case.value_scales,
        max_sequence_length=max(owned_lengths + [1]), kv_bytes=sum(owned_lengths) * config.kv_bytes_per_token)


def shard_by_kv_head(case, rank: int, ranks: int) -> RankShard:
    """KV heads ``first .. first + count`` of every sequence, and the query heads of their groups."""
    config = case.config
    first, count = multi_gpu.partition_by_kv_head(config.kv_heads, ranks)[rank]
    if count == 0:
        raise ValueError(f"rank {rank} of {ranks} owns no KV head of {config.kv_heads}")
    group = config.query_heads // config.kv_heads
    head_axis = 3 if config.layout == "NHD" else 2
    local_cache = case.kv_cache.narrow(head_axis, first, count).contiguous()
    rows = case.qkv.view(config.batch, config.query_heads + 2 * config.kv_heads, config.head_size)
    key0 = config.query_heads
    value0 = config.query_heads + config.kv_heads
    qkv = torch.cat([rows[:, first * group:(first + count) * group], rows[:, key0 + first:key0 + first + count],
                     rows[:, value0 + first:value0 + first + count]], dim=1).reshape(config.batch, -1).contiguous()
    per_head = case.key_scales.numel() > 1
    return RankShard(
        mode="by KV head", rank=rank, ranks=ranks, rows=list(range(config.batch)),
        query_heads=(first * group, count * group), kv_heads=(first, count),
        kv_cache=local_cache, rope_cache=_rope_view(local_cache, config.layout),
        block_tables=case.block_tables, sequence_lengths=case.sequence_lengths,
        qkv=qkv, positions=case.positions, slot_mapping=case.slot_mapping,
        key_scales=case.key_scales[first:first + count].contiguous() if per_head else case.key_scales,
        value_scales=case.value_scales[first:first + count].contiguous() if per_head else case.value_scales,
        max_sequence_length=case.max_sequence_length,
        kv_bytes=int(case.lengths.sum()) * 2 * count * config.head_size * config.cache_element_bytes)


def shard_long_context(case, rank: int, ranks: int, split_threshold_tokens: int = 0) -> RankShard:
    """Block ranges of the long sequences and whole short sequences, as one local batch of every row."""
    config = case.config
    block_size = config.block_size
    plan = multi_gpu.plan_long_context(case.lengths.tolist(), ranks, block_size, split_threshold_tokens)[rank]
    device = case.kv_cache.device
    batch = config.batch
    first_blocks = [0] * batch
    lengths = [0] * batch
    for row, first, tokens in zip(plan.rows, plan.first_blocks, plan.lengths):
        first_blocks[row], lengths[row] = first, tokens
    counts = [(n + block_size - 1) // block_size for n in lengths]
    width = max(counts + [1])
    firsts = torch.tensor(first_blocks, dtype=torch.int64, device=device)
    blocks_per_row = torch.tensor(counts, dtype=torch.int64, device=device)
    columns = torch.arange(width, device=device)[None, :]
    live = columns < blocks_per_row[:, None]
    source = (columns + firsts[:, None]).clamp_(max=case.block_tables.shape[1] - 1)
    tables = torch.gather(case.block_tables.to(torch.int64), 1, source)
    local_cache, renumber = _pack_blocks(case, tables[live])
    local_tables = torch.where(live, renumber[tables].to(torch.int64), torch.zeros_like(tables)).to(torch.int32)
    everyone = torch.arange(batch, dtype=torch.int64, device=device)
    return RankShard(
        mode="long context", rank=rank, ranks=ranks, rows=list(range(batch)),
        query_heads=(0, config.query_heads), kv_heads=(0, config.kv_heads),
        kv_cache=local_cache, rope_cache=_rope_view(local_cache, config.layout),
        block_tables=local_tables.contiguous(),
        sequence_lengths=torch.tensor(lengths, dtype=torch.int32, device=device),
        qkv=case.qkv, positions=case.positions, slot_mapping=_local_slots(case, renumber, everyone).contiguous(),
        key_scales=case.key_scales, value_scales=case.value_scales,
        max_sequence_length=max(lengths + [1]), kv_bytes=plan.tokens * config.kv_bytes_per_token,
        exchange=ranks > 1)


SHARDERS = {"by sequence": shard_by_sequence, "by KV head": shard_by_kv_head, "long context": shard_long_context}


class ShardedDecodeStep:
    """A rank's serving step on its shard: RoPE + paged-KV write, decode, optional exchange.

    ``kv_cache`` is a ``[blocks, 2, block_size, kv_heads, dim]`` view of a local
    cache (several steps may rotate over copies of it). The step's inputs sit in
    one pinned host buffer (``host_*`` views, filled from the shard at
    construction and refillable in place), its rows come back in ``host_output``
    (``[sequences, query_heads, dim]``; in the long-context mode the merged rows
    of the whole batch on every rank).

    Long-context mode: the decode emits F32 (O, max, sum) states of every row
    (an absent row gives the empty state); with ``exchange="peer"`` (default)
    this library's push kernel stores them into every peer's exchange buffer
    over NVLink and its merge kernel waits for all parts and merges
    (``multi_gpu.PeerExchange``), with ``exchange="nccl"``
    ``all_gather_into_tensor`` moves them and ``loom_cuda_merge_decode_states``
    merges. The exchange buffers are set up once; nothing is planned or
    allocated per step, and every rank must run every step. ``group`` is the
    process group of the exchange; ``health`` (``multi_gpu.RankHealth``) makes
    ``run`` return a status instead of launching when a peer has left.
    ``early_metadata`` is the ``stable_metadata`` promise of
    ``ops.paged_decode_attention_ex``, which the step can make for the caller.
    """

    def __init__(self, shard: RankShard, cos_sin_cache: torch.Tensor, *, rope_cache: torch.Tensor | None = None,
                 dtype: torch.dtype, scale: float, is_neox: bool, partition_tokens: int = 0, group=None,
                 health: "multi_gpu.RankHealth | None" = None, early_metadata: bool = True,
                 exchange: str = "peer", rows_to_host: bool = False):
        kv_cache = shard.rope_cache if rope_cache is None else rope_cache
        self.shard = shard
        self.device = kv_cache.device
        self.kv_cache = kv_cache
        self.cos_sin_cache = cos_sin_cache
        self.fp8 = kv_cache.dtype == torch.uint8
        self.sequences = shard.sequences
        self.query_heads = shard.query_heads[1]
        self.kv_heads, self.head_size = int(kv_cache.shape[3]), int(kv_cache.shape[4])
        self.max_sequence_length = int(shard.max_sequence_length)
        self.scale, self.is_neox = float(scale), bool(is_neox)
        self.key_scales, self.value_scales = shard.key_scales, shard.value_scales
        self._decode_scales = (dict(key_scales=shard.key_scales, value_scales=shard.value_scales)
                               if self.fp8 else {})
        self.group, self.health = group, health
        # what the step promises the decode (ops.paged_decode_attention_ex): lengths and tables arrive
        # with the upload, before the RoPE launch
        self.early_metadata = bool(early_metadata)
        self.exchange = bool(shard.exchange)
        self.ranks = shard.ranks

        heads = self.query_heads + 2 * self.kv_heads
        pieces = [("qkv", dtype, (self.sequences, heads, self.head_size)),
                  ("positions", torch.int64, (self.sequences,)),
                  ("slot_mapping", torch.int64, (self.sequences,)),
                  ("block_tables", torch.int32, tuple(shard.block_tables.shape)),
                  ("sequence_lengths", torch.int32, (self.sequences,))]
        offsets, total = [], 0
        for _, piece_dtype, shape in pieces:
            offsets.append(total)
            count = 1
            for extent in shape:
                count *= extent
            total += (count * torch.empty((), dtype=piece_dtype).element_size() + 15) // 16 * 16
        self._host = torch.zeros(max(total, 16), dtype=torch.uint8).pin_memory()
        self._device = torch.zeros(max(total, 16), dtype=torch.uint8, device=self.device)

        def views(buffer):
            out = {}
            for (name, piece_dtype, shape), offset in zip(pieces, offsets):
                count = 1
                for extent in shape:
                    count *= extent
                width = torch.empty((), dtype=piece_dtype).element_size()
                out[name] = buffer[offset:offset + count * width].view(piece_dtype).reshape(shape)
            return out

        self.host = views(self._host)
        self._pieces = views(self._device)
        self.host["qkv"].copy_(shard.qkv.view(self.sequences, heads, self.head_size))
        self.host["positions"].copy_(shard.positions)
        self.host["slot_mapping"].copy_(shard.slot_mapping)
        self.host["block_tables"].copy_(shard.block_tables)
        self.host["sequence_lengths"].copy_(shard.sequence_lengths)
        self.h2d_bytes = total

        needed, partition = ops.decode_workspace_elements_ex(
            max(self.sequences, 1), self.query_heads, self.kv_heads, self.head_size, self.max_sequence_length,
            partition_tokens)
        self._partition = partition
        self._split = self.max_sequence_length > partition
        self._workspace = (torch.empty(needed, device=self.device, dtype=torch.float32)
                           if self._split and needed else None)
        rows = (self.sequences, self.query_heads, self.head_size)
        self.host_output = torch.zeros(rows, dtype=dtype).pin_memory()
        # rows_to_host: the step's last kernel stores the rows into the pinned buffer itself (posted
        # writes over PCIe while it runs) and the device-to-host copy that would follow it is dropped
        self.rows_to_host = bool(rows_to_host)
        self.output = self.host_output if self.rows_to_host else torch.zeros(rows, device=self.device, dtype=dtype)
        self.d2h_bytes = self.host_output.numel() * self.host_output.element_size()
        self.peer_exchange = None
        if self.exchange:
            self._states = torch.zeros((self.sequences, self.query_heads, self.head_size + 2), device=self.device,
                                       dtype=torch.float32)
            if exchange == "peer":
                # this library's own push + merge kernels over NVLink peer memory (set up once, here);
                # where some rank cannot share its buffer every rank learns of it and all use NCCL
                try:
                    self.peer_exchange = multi_gpu.PeerExchange(self.sequences * self.query_heads, self.head_size,
                                                                group=group)
                except multi_gpu.PeerExchangeUnavailable as problem:
                    import warnings

                    warnings.warn(f"peer exchange unavailable, using the NCCL all-gather instead: {problem}")
                    exchange = "nccl"
            if self.peer_exchange is not None:
                pass
            elif exchange == "nccl":
                self._gathered = torch.zeros((self.ranks, self.sequences * self.query_heads, self.head_size + 2),
                                             device=self.device, dtype=torch.float32)
            else:
                raise ValueError("exchange is 'peer' or 'nccl'")
        # RoPE, decode, its merge; the exchange adds push + merge of this library (or the library merge after NCCL)
        self.kernel_launches = (2 + (1 if self._split else 0)
                                + ((2 if self.peer_exchange is not None else 1) if self.exchange else 0))
        self._graph: torch.cuda.CUDAGraph | None = None

    # ---- the step as stream operations ---------------------------------------------------------
    def enqueue_kernels(self, kv_cache: torch.Tensor | None = None, rope: bool = True,
                        exchange: bool = True) -> None:
        """RoPE + KV write, decode and (long-context mode) exchange + merge on the current stream,
        reading the step's inputs from the device mirror of the host buffer. ``rope=False`` and
        ``exchange=False`` leave those parts out (for timing the decode operator alone)."""
        import torch.distributed as dist

        kv_cache = self.kv_cache if kv_cache is None else kv_cache
        if self.sequences == 0:
            return
        qkv = self._pieces["qkv"]
        query = qkv[:, :self.query_heads]
        key = qkv[:, self.query_heads:self.query_heads + self.kv_heads]
        value = qkv[:, self.query_heads + self.kv_heads:]
        if rope:
            ops.rope_paged_kv_write_(query, key, value, self._pieces["positions"], self.cos_sin_cache, kv_cache,
                                     self.key_scales, self.value_scales, self._pieces["slot_mapping"],
                                     is_neox=self.is_neox)
        ops.paged_decode_attention_ex(
            query, kv_cache[:, 0], kv_cache[:, 1], self._pieces["block_tables"], self._pieces["sequence_lengths"],
            max_sequence_length=self.max_sequence_length, scale=self.scale, workspace=self._workspace,
            partition_tokens=self._partition, split=self._split, emit_state=self.exchange,
            output=self._states if self.exchange else self.output, stable_metadata=self.early_metadata,
            **self._decode_scales)
        if self.exchange and exchange:
            rows = self.output.view(self.sequences * self.query_heads, self.head_size)
            if self.peer_exchange is not None:
                self.peer_exchange.push(self._states)
                self.peer_exchange.merge(rows)
            else:
                dist.all_gather_into_tensor(self._gathered.view(-1), self._states.view(-1), group=self.group)
                ops.merge_decode_states(self._gathered, self.output.dtype, output=rows)

    def upload(self) -> None:
        self._device.copy_(self._host, non_blocking=True)

    def _enqueue(self) -> None:
        self.upload()
        self.enqueue_kernels()
        if not self.rows_to_host:
            self.host_output.copy_(self.output, non_blocking=True)

    def run_eager(self) -> torch.Tensor:
        with torch.cuda.device(self.device):
            self._enqueue()
            torch.cuda.current_stream().synchronize()
        return self.host_output

    def capture(self) -> "ShardedDecodeStep":
        """Records the step as one CUDA graph (it is run once eagerly first)."""
        self.run_eager()
        with torch.cuda.device(self.device):
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                self._enqueue()
            torch.cuda.current_stream().wait_stream(stream)
        self._graph = graph
        return self

    def run(self) -> torch.Tensor | int:
        """Replays the recorded step and waits for its rows. With a ``health`` monitor, a peer that
        has left makes this return ``multi_gpu.STATUS_UNAVAILABLE`` before anything is launched."""
        if self._graph is None:
            raise RuntimeError("ShardedDecodeStep.capture() has not been called")
        if self.health is not None and self.exchange:
            status = self.health.before_launch()
            if status != multi_gpu.STATUS_SUCCESS:
                return status
        self._graph.replay()
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_output


    def close(self) -> None:
        """Drops the recorded graph and the exchange buffers. In the long-context mode call it on every
        rank after a barrier (peers store into a rank's buffer until their last step has completed)
        and before the process group is destroyed (a graph holding a captured collective must not
        outlive its communicator)."""
        self._graph = None
        if self.peer_exchange is not None:
            self.peer_exchange.close()
            self.peer_exchange = None


def gather_rows(shard: RankShard, local_rows: torch.Tensor, global_shape: Sequence[int]) -> torch.Tensor:
    """Places a rank's rows into a zero tensor of the global output shape (for checks and tests)."""
    out = torch.zeros(tuple(global_shape), dtype=local_rows.dtype, device=local_rows.device)
    first, count = shard.query_heads
    if shard.rows:
        index = torch.tensor(shard.rows, dtype=torch.int64, device=local_rows.device)
        out[index, first:first + count] = local_rows
    return out
