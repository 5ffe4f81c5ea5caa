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


# ------------------------------------------------------------ failure detection
#
# The exchange of the long-context mode is the one place where a rank waits for
# others. Failures are detected on the host, never on the device: a peer that
# left says so in a key-value store before it goes (or stops updating its
# heartbeat), and a collective that does not complete within the timeout is
# reported as a status. The codes are LoomCudaStatus values
# (include/loom_launch.h): a caller sees the same vocabulary as from a launch.

STATUS_SUCCESS = 0
STATUS_LAUNCH_ERROR = 3
STATUS_UNAVAILABLE = 4


class RankHealth:
    """Who is still taking part, kept in a ``torch.distributed`` store.

    Every rank calls ``beat(step)`` between steps (one store write) and
    ``leave()`` before it stops taking part. ``before_launch()`` is the check a
    rank makes before it enqueues a step that contains a collective: it returns
    ``STATUS_UNAVAILABLE`` (and says why in ``last_error``) if a peer has left
    or has not beaten for ``stale_after`` seconds, so that the caller never
    launches a collective nobody will join.
    """

    def __init__(self, store, rank: int, ranks: int, stale_after: float = 30.0, clock=None):
        import time

        self.store, self.rank, self.ranks = store, int(rank), int(ranks)
        self.stale_after = float(stale_after)
        self.clock = clock or time.monotonic
        self.last_error = ""
        self._seen: dict[int, tuple[bytes, float]] = {}
        self.store.set(f"loom/alive/{self.rank}", "0")

    def beat(self, step: int) -> None:
        self.store.set(f"loom/alive/{self.rank}", str(int(step)))

    def leave(self) -> None:
        self.store.set(f"loom/alive/{self.rank}", "gone")

    def before_launch(self) -> int:
        now = self.clock()
        for peer in range(self.ranks):
            if peer == self.rank:
                continue
            key = f"loom/alive/{peer}"
            try:
                present = self.store.check([key])
                value = self.store.get(key) if present else b""
            except Exception as error:  # the store itself is gone: nobody can be reached
                self.last_error = f"rank store unreachable: {error}"
                return STATUS_UNAVAILABLE
            if value == b"gone":
                self.last_error = f"rank {peer} has left the group"
                return STATUS_UNAVAILABLE
            previous = self._seen.get(peer)
            if previous is None or previous[0] != value:
                self._seen[peer] = (value, now)
            elif now - previous[1] > self.stale_after:
                self.last_error = f"rank {peer} has not reported for {now - previous[1]:.1f} s"
                return STATUS_UNAVAILABLE
        self.last_error = ""
        return STATUS_SUCCESS


def guarded_all_gather(gathered: torch.Tensor, local: torch.Tensor, group=None,
                       timeout_seconds: float | None = None) -> tuple[int, str]:
    """``all_gather_into_tensor`` that reports instead of hanging.

    Without ``timeout_seconds`` the collective is enqueued and the call returns
    at once (the steady-state path: errors surface through the process group's
    own timeout). With it, the host waits for completion at most that long.
    Returns ``(status, message)``: ``STATUS_UNAVAILABLE`` when a peer did not
    arrive in time or the group is gone, ``STATUS_LAUNCH_ERROR`` for any other
    failure of the collective. The buffers hold no result after a failure.
    """
    import datetime

    import torch.distributed as dist

    try:
        work = dist.all_gather_into_tensor(gathered, local, group=group, async_op=True)
        if timeout_seconds is None:
            work.wait()  # on a CUDA group this orders the current stream after the collective, no host wait
            return STATUS_SUCCESS, ""
        work.wait(datetime.timedelta(seconds=float(timeout_seconds)))
        return STATUS_SUCCESS, ""
    except Exception as error:  # torch raises RuntimeError / DistBackendError subclasses
        text = str(error)
        lowered = text.lower()
        gone = any(word in lowered for word in ("timeout", "timed out", "connection", "closed", "reset by peer"))
        return (STATUS_UNAVAILABLE if gone else STATUS_LAUNCH_ERROR), text


class PeerExchangeUnavailable(RuntimeError):
    """The peer exchange could not be set up on some rank; raised on EVERY rank of the group, so that
    all of them can fall back to the library all-gather together."""


class PeerExchange:
    """The long-context exchange over peer memory instead of a library all-gather.

    Every rank owns an exchange buffer in its GPU's memory (created and shared
    with CUDA IPC by the library, ``include/loom_launch.h``: the peer exchange
    section). ``push`` stores this rank's F32 ``[rows, Dv + 2]`` states straight
    into every peer's buffer over NVLink and ``merge`` waits (bounded) for all
    parts of the step in its own buffer and writes the merged ``[rows, Dv]`` rows:
    two kernels of this library per step, no communication-library call, nothing
    allocated after construction. The handles are exchanged once, here, with
    ``all_gather_object`` on ``group`` (any backend). Every rank must run every
    step; ``status()`` (synchronous) tells how many steps completed and whether a
    wait ever ran out, after which every rank calls ``reset()`` and the ranks
    meet at a host barrier before the next step.

    ``buffers`` lets a test hand over buffers that already live in one process
    (several ranks emulated on one GPU); nothing is opened or exchanged then.
    """

    def __init__(self, rows: int, value_head_size: int, *, group=None, rank: int | None = None,
                 world: int | None = None, buffers: Sequence[int] | None = None):
        import torch.distributed as dist

        self._lib = _native.library()
        self.rows, self.value_head_size = int(rows), int(value_head_size)
        self.world = int(world) if world is not None else dist.get_world_size(group)
        self.rank = int(rank) if rank is not None else dist.get_rank(group)
        self.bytes = int(self._lib.loom_cuda_peer_exchange_bytes(self.world, self.rows, self.value_head_size))
        if self.bytes == 0:
            raise ValueError("peer exchange: unsupported shape (at most 16 ranks; rows * (Dv + 2) a multiple of 4)")
        self._opened: list[int] = []
        self._own = None
        if buffers is not None:
            pointers = [int(b) for b in buffers]
        else:
            # Every rank takes part in both collectives below whatever happens to it, and all ranks reach
            # the same conclusion: a rank that raised on its own would leave the others waiting for it.
            own = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            status = self._lib.loom_cuda_peer_exchange_create(self.bytes, ctypes.byref(own), handle, 64)
            problem = None
            if status != 0:
                problem = (f"rank {self.rank}: exchange buffer not created (status {status}, "
                           + self._lib.loom_cuda_last_launch_failure().decode() + ")")
            else:
                self._own = own.value
            handles: list = [None] * self.world
            dist.all_gather_object(handles, None if problem else handle.raw, group=group)
            pointers = []
            for peer, raw in enumerate(handles):
                if peer == self.rank or problem is not None or raw is None:
                    pointers.append(self._own or 0)
                    continue
                mapped = ctypes.c_void_p()
                status = self._lib.loom_cuda_peer_exchange_open(raw, len(raw), ctypes.byref(mapped))
                if status != 0:
                    problem = (f"rank {self.rank}: rank {peer}'s exchange buffer not mapped (status {status}, "
                               + self._lib.loom_cuda_last_launch_failure().decode() + ")")
                    pointers.append(0)
                    continue
                self._opened.append(mapped.value)
                pointers.append(mapped.value)
            problems: list = [None] * self.world
            dist.all_gather_object(problems, problem, group=group)
            if any(problems):
                self.close()
                raise PeerExchangeUnavailable("; ".join(text for text in problems if text))
        self.buffer = pointers[self.rank]
        self._pointers = (ctypes.c_void_p * self.world)(*pointers)

    def push(self, states: torch.Tensor) -> None:
        """Enqueues the stores of this rank's states into every rank's buffer on the current stream."""
        if (states.dtype != torch.float32 or not states.is_contiguous()
                or states.numel() != self.rows * (self.value_head_size + 2)):
            raise RuntimeError("peer exchange expects contiguous float32 [rows, Dv + 2] states")
        from . import ops

        status = self._lib.loom_cuda_peer_exchange_push(states.data_ptr(), self._pointers, self.rank, self.world,
                                                        self.rows, self.value_head_size, ops._stream(states.device))
        if status != 0:
            raise RuntimeError(f"peer exchange push failed (status {status})")

    def merge(self, output: torch.Tensor) -> torch.Tensor:
        """Enqueues the wait for all ranks' parts and their merge into ``output`` ``[rows, Dv]``."""
        from . import ops

        if (output.dtype not in ops._DTYPE_CODES or not output.is_contiguous()
                or output.numel() != self.rows * self.value_head_size):
            raise RuntimeError("peer exchange merges into a contiguous [rows, Dv] tensor of a supported type")
        stream = ops._stream(output.device if output.device.type == "cuda" else torch.device("cuda", torch.cuda.current_device()))
        status = self._lib.loom_cuda_peer_exchange_merge(self.buffer, self.world, self.rows, self.value_head_size,
                                                         ops._DTYPE_CODES[output.dtype], output.data_ptr(), stream)
        if status != 0:
            raise RuntimeError(f"peer exchange merge failed (status {status})")
        return output

    def status(self) -> tuple[int, int]:
        """(steps completed, error word) of this rank's buffer; waits for the device."""
        steps, error = _native.u64(0), _native.u32(0)
        if self._lib.loom_cuda_peer_exchange_status(self.buffer, ctypes.byref(steps), ctypes.byref(error)) != 0:
            raise RuntimeError("peer exchange status could not be read")
        return int(steps.value), int(error.value)

    def reset(self, stream: int = 0) -> None:
        if self._lib.loom_cuda_peer_exchange_reset(self.buffer, self.bytes, stream) != 0:
            raise RuntimeError("peer exchange buffer could not be reset")

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's own (call after a barrier: peers may still push)."""
        for pointer in self._opened:
            self._lib.loom_cuda_peer_exchange_close(pointer)
        self._opened = []
        if self._own is not None:
            self._lib.loom_cuda_peer_exchange_destroy(self._own)
            self._own = None


class LongContextDecoder:
    """The long-context mode for one batch shape: plan, index tensors and buffers made once.

    Every rank holds the whole (replicated or peer-visible) block table and, in
    its cache, the blocks of its own ranges. ``decode`` computes partial states
    of every row (rows the rank holds nothing of give the empty state: max =
    -inf, sum = 0, which the merge ignores), all-gathers them (``Dv + 2`` floats
    per query head per rank) and merges: every rank gets the full ``[B, Hq, Dv]``
    output. A step enqueues three operations (decode, all-gather, merge) and
    builds nothing on the host. ``timeout_seconds`` bounds the host's wait for
    the all-gather; ``health`` is consulted before anything is launched.
    """

    def __init__(self, lengths: Sequence[int], block_tables: torch.Tensor, *, query_heads: int,
                 value_head_size: int, block_size: int, dtype: torch.dtype, group=None,
                 split_threshold_tokens: int = 0, decode_states: DecodeStates = _default_decode_states,
                 merge_states: MergeStates = _default_merge, timeout_seconds: float | None = None,
                 health: RankHealth | None = None):
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.plan = plan_long_context(lengths, self.world, block_size, split_threshold_tokens)[self.rank]
        self.dtype = dtype
        self.decode_states, self.merge_states = decode_states, merge_states
        self.timeout_seconds, self.health = timeout_seconds, health
        self.last_error = ""
        device = block_tables.device
        batch = len(lengths)
        self.batch, self.query_heads, self.value_head_size = batch, int(query_heads), int(value_head_size)
        first_blocks, local_lengths = [0] * batch, [0] * batch
        for row, first, tokens in zip(self.plan.rows, self.plan.first_blocks, self.plan.lengths):
            first_blocks[row], local_lengths[row] = first, tokens
        width = block_tables.shape[1]
        firsts = torch.tensor(first_blocks, dtype=torch.int64, device=device)
        columns = (torch.arange(width, device=device).unsqueeze(0) + firsts.unsqueeze(1)).clamp_(max=width - 1)
        self.block_tables = torch.gather(block_tables, 1, columns).contiguous()
        self.lengths = torch.tensor(local_lengths, dtype=torch.int32, device=device)
        self.max_sequence_length = int(max(local_lengths + [1]))
        self.gathered = torch.empty(self.world * batch * self.query_heads * (self.value_head_size + 2),
                                    dtype=torch.float32, device=device)

    def decode(self, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, *, scale: float,
               **decode_kwargs):
        """Returns the merged ``[B, Hq, Dv]`` rows, or a status code (int) if the step could not run."""
        if self.health is not None:
            status = self.health.before_launch()
            if status != STATUS_SUCCESS:
                self.last_error = self.health.last_error
                return status
        states = self.decode_states(query, key_cache, value_cache, self.block_tables, self.lengths,
                                    max_sequence_length=self.max_sequence_length, scale=scale, **decode_kwargs)
        status, message = guarded_all_gather(self.gathered, states.to(torch.float32).reshape(-1), self.group,
                                             self.timeout_seconds)
        if status != STATUS_SUCCESS:
            self.last_error = message
            return status
        merged = self.merge_states(
            self.gathered.view(self.world, self.batch * self.query_heads, self.value_head_size + 2), self.dtype)
        return merged.reshape(self.batch, self.query_heads, self.value_head_size)


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

    Convenience form of ``LongContextDecoder`` for a single step (it builds the
    plan and its tensors, which a serving loop does once per batch shape by
    keeping the decoder). Raises ``RuntimeError`` if the exchange fails.
    """
    decoder = LongContextDecoder(lengths, block_tables, query_heads=query.shape[1],
                                 value_head_size=value_cache.shape[3], block_size=block_size, dtype=query.dtype,
                                 group=group, split_threshold_tokens=split_threshold_tokens,
                                 decode_states=decode_states, merge_states=merge_states)
    result = decoder.decode(query, key_cache, value_cache, scale=scale, **decode_kwargs)
    if isinstance(result, int):
        raise RuntimeError(f"long-context exchange failed (status {result}): {decoder.last_error}")
    return result


def decode_by_kv_head(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    scale: float,
    max_sequence_length: int,
    rank: int,
    ranks: int,
    key_scales: torch.Tensor | None = None,
    value_scales: torch.Tensor | None = None,
    decode: Callable[..., torch.Tensor] | None = None,
    **decode_kwargs,
) -> tuple[tuple[int, int], torch.Tensor]:
    """Decodes this rank's KV heads of every sequence; no communication.

    ``key_cache``/``value_cache`` are logical ``[blocks, block_size, Hkv, D]``
    views of the full head range (a rank that holds only its own heads passes
    ``ranks=1``-style arguments instead). The rank's share is the head slice
    ``[first, first + count)`` given by the partitioner and the query heads of
    those groups. Returns ((first query head, query head count), ``[B, count *
    group, Dv]`` rows): disjoint column slices of the full output, the layout
    tensor parallelism leaves them in.
    """
    if decode is None:
        from . import ops

        decode = ops.paged_decode_attention_ex
    kv_heads = key_cache.shape[2]
    group = query.shape[1] // kv_heads
    first, count = partition_by_kv_head(kv_heads, ranks)[rank]
    if count == 0:
        return (first * group, 0), query.new_empty((query.shape[0], 0, value_cache.shape[3]))
    local_query = query[:, first * group:(first + count) * group]
    scales = {}
    if key_scales is not None:
        per_head = key_scales.numel() > 1
        scales = dict(key_scales=key_scales[first:first + count].contiguous() if per_head else key_scales,
                      value_scales=value_scales[first:first + count].contiguous() if per_head else value_scales)
    output = decode(local_query, key_cache[:, :, first:first + count], value_cache[:, :, first:first + count],
                    block_tables, sequence_lengths, max_sequence_length=max_sequence_length, scale=scale,
                    **scales, **decode_kwargs)
    return (first * group, count * group), output


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
