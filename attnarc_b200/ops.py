"""PyTorch-facing operators of the paged-decode path.

Same names, arguments and error behaviour as the reference's Python API
(python/src/loom_kernels/ops/attention.py, ops/rope_kv.py, ops/telemetry.py),
so its tests read the same against this package. The differences are
additions: contexts are not capped at 1024 tokens, the decode accepts any cache
stride order and FP8 E4M3 caches (``paged_decode_attention_ex``), and partial
states can be produced and merged. torch is used for device memory and streams
only; all work happens in ``libloom_cuda_bridge.so``.
"""

from __future__ import annotations

import ctypes
import enum
import functools
import math

import torch

from . import _native
from ._native import BridgeError, check, library

_DTYPE_CODES = {torch.float32: _native.F32, torch.float16: _native.F16, torch.bfloat16: _native.BF16}
_DTYPE_NAMES = _DTYPE_CODES  # membership test used by the predicates


class Operator(enum.IntEnum):
    """Launch-counter ids (loom_cuda_bridge.h:28-40)."""

    RMS_NORM = 0
    ADD_RMS_NORM = 1
    RMS_NORM_DYNAMIC_FP8 = 2
    SILU_AND_MUL = 3
    SILU_AND_MUL_DYNAMIC_FP8 = 4
    ROPE_PAGED_KV_WRITE = 5
    GREEDY_SAMPLE_LOGPROBS = 6
    SELECTED_TOKEN_LOGPROBS = 7
    MIN_P_FILTER = 8
    PAGED_DECODE_ATTENTION = 9
    GREEDY_SPECULATIVE_VERIFY = 10


def launch_count(operator: Operator) -> int:
    """Successful launches of one operator since the last reset."""
    count = _native.u64(0)
    check(library().loom_cuda_bridge_launch_count(int(operator), count), "launch count")
    return int(count.value)


def reset_launch_count(operator: Operator) -> None:
    check(library().loom_cuda_bridge_reset_launch_count(int(operator)), "launch count reset")


def last_decode_route() -> str:
    """Kernel family chosen by the last decode launch on this thread."""
    return library().loom_cuda_last_decode_route().decode()


def set_programmatic_launch(mode: int) -> None:
    """0: plain launches; 1 (default): programmatic dependent launch of the library's kernels."""
    if library().loom_cuda_set_programmatic_launch(int(mode)) != 0:
        raise ValueError(f"unknown programmatic launch mode {mode!r}")


def set_decode_copy_engine(engine: str) -> None:
    """How the balanced kernel is fed: ``"tma"`` (default; over an FP8 cache the
    copies are issued by a warp of their own, a whole block of eight KV heads at
    a time where the KV heads come in eights), ``"cp_async"`` (per-lane copies),
    ``"tma-mma"`` (TMA with every computing warp feeding its own ring),
    ``"tma-umma"`` (TMA, and the tcgen05 kernel where it applies: FP8 cache,
    head size 128, up to 8 query heads per KV head) or ``"tma-head"`` (as
    ``"tma"``, but always one KV head per tile)."""
    code = {"tma": 0, "cp_async": 1, "tma-mma": 2, "tma-umma": 3, "tma-head": 4}[engine]
    if library().loom_cuda_set_decode_copy_engine(code) != 0:
        raise RuntimeError("could not select the decode copy engine")


def decode_timeout_flag(device=None, reset: bool = False) -> int:
    """Non-zero if a bounded wait inside the TMA-fed kernel ever expired on the device."""
    value = _native.u32(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        status = library().loom_cuda_decode_timeout_flag(value, 1 if reset else 0)
    if status != 0:
        raise RuntimeError("could not read the decode timeout flag")
    return int(value.value)


def set_wait_policy(attempts: int = 0, unmatched_bytes: int = 0) -> None:
    """Limit of the kernels' waits on copy barriers (0 = default, about a second).

    ``unmatched_bytes`` > 0 is the self-test of the expiry path: barriers are armed
    for more bytes than arrive, every ring's first wait runs out after ``attempts``
    polls, the kernels set their timeout flag and return. Results of launches made
    under it are invalid; call ``set_wait_policy()`` to return to service."""
    if library().loom_cuda_set_wait_policy(int(attempts), int(unmatched_bytes)) != 0:
        raise ValueError("unmatched_bytes must be a multiple of 16 of at most 1 MiB")


def plain_launch_retries() -> int:
    """Launches refused with the programmatic-launch attribute and issued plain instead."""
    return int(library().loom_cuda_plain_launch_retries())


def last_launch_failure() -> str:
    """CUDA error and call site behind this thread's last launch error (``"none"`` if none)."""
    return library().loom_cuda_last_launch_failure().decode()


def _require_inference_tensors(*tensors: torch.Tensor) -> None:
    for tensor in tensors:
        if tensor.requires_grad:
            raise ValueError("Loom operators are inference-only; detach tensors that require grad")


def _stream(device: torch.device) -> int:
    """Raw handle of torch's current stream on the device."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(index)


@functools.lru_cache(maxsize=4096)
def _span_of(shape: tuple, stride: tuple) -> int:
    if 0 in shape:
        return 0
    return 1 + sum((size - 1) * step for size, step in zip(shape, stride))


def _span(tensor: torch.Tensor) -> int:
    """Elements from the first to one past the last addressed element."""
    return _span_of(tuple(tensor.shape), tuple(tensor.stride()))


class _on_device:
    """``torch.cuda.device`` that does nothing when the device is already current."""

    __slots__ = ("guard",)

    def __init__(self, device: torch.device):
        index = device.index
        self.guard = None if index is None or index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            return self.guard.__exit__(*exc)
        return False


@functools.lru_cache(maxsize=1024)
def _cached_workspace_query(device, sequences, query_heads, kv_heads, value_head_size, max_sequence_length,
                            partition_tokens):
    # `device` only keys the cache: the answer depends on the SM count of the current device
    elements, tokens = _native.u64(0), _native.u32(0)
    check(
        library().loom_cuda_bridge_paged_decode_workspace_elements_ex(
            sequences, query_heads, kv_heads, value_head_size, max_sequence_length, partition_tokens,
            elements, tokens,
        ),
        "paged decode workspace query",
    )
    return int(elements.value), int(tokens.value)


def _has_dense_nhd_inner_strides(tensor: torch.Tensor) -> bool:
    if tensor.dim() != 4:
        return False
    _, block_size, heads, width = tensor.shape
    return bool(
        tensor.stride(3) == 1
        and tensor.stride(2) == width
        and tensor.stride(1) == heads * width
        and tensor.stride(0) >= block_size * heads * width
    )


# ------------------------------------------------------------------ decode

def supports_paged_decode_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    max_sequence_length: int,
) -> bool:
    """Whether the tensors fit the reference-shaped decode entry point."""
    if (
        query.dim() != 3 or key_cache.dim() != 4 or value_cache.dim() != 4
        or block_tables.dim() != 2 or sequence_lengths.dim() != 1
        or query.numel() == 0 or key_cache.numel() == 0 or value_cache.numel() == 0
        or isinstance(max_sequence_length, bool) or not isinstance(max_sequence_length, int)
    ):
        return False
    sequences, query_heads, head_size = query.shape
    num_blocks, block_size, kv_heads, key_head_size = key_cache.shape
    if not (
        query.device.type == "cuda"
        and all(t.device == query.device for t in (key_cache, value_cache, block_tables, sequence_lengths))
        and query.dtype in _DTYPE_NAMES
        and key_cache.dtype == query.dtype and value_cache.dtype == query.dtype
        and block_tables.dtype == torch.int32 and sequence_lengths.dtype == torch.int32
        and query.is_contiguous()
        and _has_dense_nhd_inner_strides(key_cache) and _has_dense_nhd_inner_strides(value_cache)
        and block_tables.is_contiguous() and sequence_lengths.is_contiguous()
        and not query.requires_grad and not key_cache.requires_grad and not value_cache.requires_grad
        and head_size == key_head_size
        and tuple(value_cache.shape[:3]) == (num_blocks, block_size, kv_heads)
        and value_cache.shape[3] > 0
        and kv_heads > 0 and query_heads % kv_heads == 0
        and block_tables.shape[0] == sequences and block_tables.shape[1] > 0
        and sequence_lengths.shape[0] == sequences
        and 0 < max_sequence_length <= block_tables.shape[1] * block_size
    ):
        return False
    return bool(
        library().loom_cuda_bridge_supports_paged_decode(
            _DTYPE_CODES[query.dtype], _native.KV_CACHE_NATIVE, sequences, query_heads, kv_heads,
            head_size, value_cache.shape[3], num_blocks, block_size, block_tables.shape[1],
            max_sequence_length, 1.0,
        )
    )


def _check_decode_tensors(query, key_cache, value_cache, block_tables, sequence_lengths, output,
                          strided_query=False):
    if query.dim() != 3 or key_cache.dim() != 4 or value_cache.dim() != 4:
        raise RuntimeError("Loom paged decode expects query [B,Hq,D] and caches [blocks,block,Hkv,D]")
    if block_tables.dim() != 2 or sequence_lengths.dim() != 1:
        raise RuntimeError("Loom paged decode expects block_tables [B,max_blocks] and lengths [B]")
    # the output may also be pinned host memory: the last kernel then stores the rows straight over
    # PCIe and no device-to-host copy follows (pinned allocations are addressable by the device)
    output_ok = output.device == query.device or (output.device.type == "cpu" and output.is_pinned())
    if query.device.type != "cuda" or not output_ok or any(
        t.device != query.device for t in (key_cache, value_cache, block_tables, sequence_lengths)
    ):
        raise RuntimeError("Loom paged decode tensors must share one CUDA device "
                           "(the output may instead be pinned host memory)")
    if query.dtype not in _DTYPE_CODES:
        raise RuntimeError("Loom paged decode supports float32, float16 and bfloat16 queries")
    if block_tables.dtype != torch.int32 or sequence_lengths.dtype != torch.int32:
        raise RuntimeError("Loom paged decode metadata must be int32")
    query_ok = query.stride(2) == 1 if strided_query else query.is_contiguous()
    if not (query_ok and output.is_contiguous() and block_tables.is_contiguous()
            and sequence_lengths.is_contiguous()):
        raise RuntimeError("Loom paged decode query, output and metadata must be contiguous")


def decode_workspace_elements(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                              block_tables: torch.Tensor, *, max_sequence_length: int,
                              scale: float = 1.0) -> int:
    """F32 workspace elements the reference-shaped decode call expects (0 = none)."""
    elements = _native.u64(0)
    check(
        library().loom_cuda_bridge_paged_decode_workspace_elements(
            _DTYPE_CODES[query.dtype], query.shape[0], query.shape[1], key_cache.shape[2], query.shape[2],
            value_cache.shape[3], key_cache.shape[0], key_cache.shape[1], block_tables.shape[1],
            int(max_sequence_length), float(scale), elements,
        ),
        "paged decode workspace query",
    )
    return int(elements.value)


def paged_decode_attention_out(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    output: torch.Tensor,
    *,
    max_sequence_length: int,
    scale: float | None = None,
    workspace: torch.Tensor | None = None,
) -> torch.Tensor:
    """Paged MQA/GQA decode into caller-owned output (dense-inner NHD caches)."""
    _require_inference_tensors(query, key_cache, value_cache, output)
    _check_decode_tensors(query, key_cache, value_cache, block_tables, sequence_lengths, output)
    if not (_has_dense_nhd_inner_strides(key_cache) and _has_dense_nhd_inner_strides(value_cache)):
        raise RuntimeError("Loom paged decode caches must be dense-inner NHD; use paged_decode_attention_ex")
    if scale is None:
        scale = query.shape[-1] ** -0.5
    with _on_device(query.device):
        needed = decode_workspace_elements(query, key_cache, value_cache, block_tables,
                                           max_sequence_length=max_sequence_length, scale=scale)
        if needed and (workspace is None or workspace.numel() != needed):
            workspace = torch.empty(needed, device=query.device, dtype=torch.float32)
        status = library().loom_cuda_bridge_paged_decode_attention(
            _DTYPE_CODES[query.dtype], query.data_ptr(), query.numel(), key_cache.data_ptr(),
            _span(key_cache), value_cache.data_ptr(), _span(value_cache), block_tables.data_ptr(),
            block_tables.numel(), sequence_lengths.data_ptr(), sequence_lengths.numel(),
            output.data_ptr(), output.numel(), workspace.data_ptr() if needed else None, needed,
            query.shape[0], query.shape[1], key_cache.shape[2], query.shape[2], value_cache.shape[3],
            key_cache.shape[0], key_cache.shape[1], key_cache.stride(0), value_cache.stride(0),
            block_tables.shape[1], int(max_sequence_length), float(scale), _stream(query.device),
        )
    check(status, "paged decode attention")
    return output


def paged_decode_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    max_sequence_length: int,
    scale: float | None = None,
) -> torch.Tensor:
    """Paged MQA/GQA decode for one query token per sequence."""
    if query.dim() != 3 or value_cache.dim() != 4:
        raise ValueError("paged decode query/value cache must have ranks 3 and 4")
    output = torch.empty((query.shape[0], query.shape[1], value_cache.shape[3]),
                         device=query.device, dtype=query.dtype)
    return paged_decode_attention_out(query, key_cache, value_cache, block_tables, sequence_lengths,
                                      output, max_sequence_length=max_sequence_length, scale=scale)


def decode_workspace_elements_ex(sequences: int, query_heads: int, kv_heads: int, value_head_size: int,
                                 max_sequence_length: int, partition_tokens: int = 0) -> tuple[int, int]:
    """(workspace elements, partition tokens) of a partitioned decode on the current device."""
    device = torch.cuda.current_device() if torch.cuda.is_available() else -1
    return _cached_workspace_query(device, int(sequences), int(query_heads), int(kv_heads), int(value_head_size),
                                   int(max_sequence_length), int(partition_tokens))


def paged_decode_attention_ex(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    max_sequence_length: int,
    scale: float | None = None,
    key_scales: torch.Tensor | None = None,
    value_scales: torch.Tensor | None = None,
    workspace: torch.Tensor | None = None,
    partition_tokens: int = 0,
    split: bool | None = None,
    emit_state: bool = False,
    output: torch.Tensor | None = None,
    sliding_window: int = 0,
    logits_soft_cap: float = 0.0,
    stable_metadata: bool = False,
) -> torch.Tensor:
    """Decode over caches of any stride order, native or FP8 E4M3.

    ``key_cache``/``value_cache`` are logical ``[blocks, block_size, kv_heads,
    dim]`` views (permute an HND allocation to get one); only the last stride
    must be 1. ``uint8`` caches are FP8 E4M3 and need ``key_scales`` and
    ``value_scales`` (one element, or one per KV head). ``split`` chooses the
    partitioned path (default: when the context spans several partitions);
    ``emit_state`` returns F32 ``[B, Hq, Dv + 2]`` partial states. ``query``
    may be a strided view (unit innermost stride), e.g. the rotated Q inside a
    packed QKV row. ``sliding_window`` W > 0 lets a query see only the last W
    tokens of its sequence; ``logits_soft_cap`` c > 0 turns every scaled score
    s into ``c * tanh(s / c)`` before the softmax (both are options the
    reference names as later contract fields; 0 = off).

    ``stable_metadata`` is a promise that lets a serving loop shed latency:
    ``block_tables`` and ``sequence_lengths`` were written before the operation
    preceding this call in the stream began (e.g. before the step's RoPE + KV
    write); the kernel then plans its work while that operation still runs.
    """
    _require_inference_tensors(query, key_cache, value_cache)
    sequences, query_heads, head_size = query.shape
    num_blocks, block_size, kv_heads, _ = key_cache.shape
    value_head_size = value_cache.shape[3]
    fp8 = key_cache.dtype == torch.uint8
    if scale is None:
        scale = head_size ** -0.5
    if key_cache.stride(3) != 1 or value_cache.stride(3) != 1:
        raise RuntimeError("Loom paged decode caches need a unit innermost stride")
    if output is None:
        shape = (sequences, query_heads, value_head_size + 2) if emit_state else (sequences, query_heads, value_head_size)
        output = torch.empty(shape, device=query.device, dtype=torch.float32 if emit_state else query.dtype)
    _check_decode_tensors(query, key_cache, value_cache, block_tables, sequence_lengths, output,
                          strided_query=True)
    with _on_device(query.device):
        needed, tokens = decode_workspace_elements_ex(sequences, query_heads, kv_heads, value_head_size,
                                                      int(max_sequence_length), partition_tokens)
        if split is None:
            split = max_sequence_length > (tokens if tokens else 256)
        if split:
            if workspace is None or workspace.numel() < needed:
                workspace = torch.empty(needed, device=query.device, dtype=torch.float32)
        else:
            workspace = None
        scales = (key_scales, value_scales) if fp8 else (None, None)
        status = library().loom_cuda_bridge_paged_decode_attention_with_options(
            _DTYPE_CODES[query.dtype], _native.KV_CACHE_FP8_E4M3 if fp8 else _native.KV_CACHE_NATIVE,
            query.data_ptr(), _span(query), key_cache.data_ptr(), _span(key_cache),
            value_cache.data_ptr(), _span(value_cache),
            scales[0].data_ptr() if scales[0] is not None else None,
            scales[0].numel() if scales[0] is not None else 0,
            scales[1].data_ptr() if scales[1] is not None else None,
            scales[1].numel() if scales[1] is not None else 0,
            block_tables.data_ptr(), block_tables.numel(), sequence_lengths.data_ptr(),
            sequence_lengths.numel(), output.data_ptr(), output.numel(),
            workspace.data_ptr() if workspace is not None else None,
            workspace.numel() if workspace is not None else 0,
            sequences, query_heads, kv_heads, head_size, value_head_size, num_blocks, block_size,
            key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
            value_cache.stride(0), value_cache.stride(1), value_cache.stride(2),
            block_tables.shape[1], int(max_sequence_length), partition_tokens if split else 0, float(scale),
            1 if emit_state else 0,
            0 if query.is_contiguous() else query.stride(0), 0 if query.is_contiguous() else query.stride(1),
            int(sliding_window), float(logits_soft_cap),
            _native.DECODE_STABLE_METADATA if stable_metadata else 0,
            _stream(query.device),
        )
    check(status, "paged decode attention")
    return output


def merge_decode_states(states: torch.Tensor, out_dtype: torch.dtype,
                        output: torch.Tensor | None = None) -> torch.Tensor:
    """Merges ``[parts, rows, Dv + 2]`` F32 states into ``[rows, Dv]`` outputs (into ``output`` if given)."""
    if states.dim() != 3 or states.dtype != torch.float32 or not states.is_contiguous():
        raise RuntimeError("decode states must be a contiguous float32 [parts, rows, Dv + 2] tensor")
    parts, rows, width = states.shape
    if output is None:
        output = torch.empty((rows, width - 2), device=states.device, dtype=out_dtype)
    elif (output.dtype != out_dtype or tuple(output.shape) != (rows, width - 2) or not output.is_contiguous()
          or not (output.device == states.device or (output.device.type == "cpu" and output.is_pinned()))):
        raise RuntimeError("merge output must be a contiguous [rows, Dv] tensor of the requested dtype")
    with _on_device(states.device):
        status = library().loom_cuda_bridge_merge_decode_states(
            states.data_ptr(), states.numel(), parts, rows, width - 2, _DTYPE_CODES[out_dtype],
            output.data_ptr(), output.numel(), _stream(states.device),
        )
    check(status, "decode state merge")
    return output


# -------------------------------------------------------------------- RoPE

def supports_rope_paged_kv_write(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    positions: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    kv_cache: torch.Tensor,
    key_scales: torch.Tensor,
    value_scales: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> bool:
    """Whether the tensors fit the fused RoPE + paged-KV write."""
    if query.dim() != 3 or key.dim() != 3 or value.dim() != 3 or cos_sin_cache.dim() != 2:
        return False
    if query.numel() == 0 or key.numel() == 0 or value.numel() == 0 or kv_cache.dim() != 5:
        return False
    rotary_dim = cos_sin_cache.shape[1]
    others = (key, value, positions, cos_sin_cache, kv_cache, key_scales, value_scales, slot_mapping)
    span = (kv_cache.shape[2] - 1) * kv_cache.stride(2) + (kv_cache.shape[3] - 1) * kv_cache.stride(3) + kv_cache.shape[4]
    return bool(
        query.device.type == "cuda"
        and all(t.device == query.device for t in others)
        and query.dtype in _DTYPE_NAMES
        and key.dtype == query.dtype and value.dtype == query.dtype and cos_sin_cache.dtype == query.dtype
        and kv_cache.dtype in (query.dtype, torch.uint8)
        and key_scales.dtype == torch.float32 and value_scales.dtype == torch.float32
        and key_scales.numel() == value_scales.numel() and key_scales.numel() in (1, key.shape[1])
        and key_scales.is_contiguous() and value_scales.is_contiguous()
        and positions.dtype == torch.int64 and slot_mapping.dtype == torch.int64
        and query.shape[0] == key.shape[0] == value.shape[0]
        and query.shape[2] == key.shape[2]
        and key.shape[1] == value.shape[1] and key.shape[2] == value.shape[2]
        and positions.dim() == 1 and positions.numel() == query.shape[0]
        and slot_mapping.dim() == 1 and 0 < slot_mapping.numel() <= query.shape[0]
        and cos_sin_cache.shape[0] > 0 and rotary_dim > 0 and rotary_dim % 2 == 0
        and rotary_dim <= query.shape[2]
        and kv_cache.shape[0] > 0 and kv_cache.shape[1] == 2 and kv_cache.shape[2] > 0
        and tuple(kv_cache.shape[3:]) == tuple(key.shape[1:])
        and query.stride(2) == 1 and key.stride(2) == 1 and value.stride(2) == 1
        and all(s > 0 for s in query.stride()[:2]) and all(s > 0 for s in key.stride()[:2])
        and all(s > 0 for s in value.stride()[:2])
        and positions.is_contiguous() and cos_sin_cache.is_contiguous() and slot_mapping.is_contiguous()
        and kv_cache.stride(4) == 1 and all(s > 0 for s in kv_cache.stride()[:4])
        and kv_cache.stride(1) >= span and kv_cache.stride(0) >= kv_cache.stride(1) + span
        and not any(t.requires_grad for t in (query, key, value, cos_sin_cache))
    )


def rope_paged_kv_write_(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    positions: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    kv_cache: torch.Tensor,
    key_scales: torch.Tensor,
    value_scales: torch.Tensor,
    slot_mapping: torch.Tensor,
    is_neox: bool = True,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Rotates Q/K in place and writes K/V into a packed paged cache.

    ``kv_cache`` is ``[blocks, 2, block_size, kv_heads, head_size]`` with any
    positive strides (vLLM's NHD and HND layouts both qualify); ``uint8``
    storage selects the static FP8 E4M3 encoding with the given scales.
    """
    _require_inference_tensors(query, key, value, cos_sin_cache, kv_cache, key_scales, value_scales)
    if query.dim() != 3 or key.dim() != 3 or value.dim() != 3 or kv_cache.dim() != 5 or kv_cache.shape[1] != 2:
        raise RuntimeError(
            "Loom RoPE+paged-KV expects [tokens, heads, dim] sources and a "
            "[blocks, 2, block_size, kv_heads, head_size] cache"
        )
    if query.dtype not in _DTYPE_CODES:
        raise RuntimeError("Loom RoPE+paged-KV supports float32, float16 and bfloat16 sources")
    if query.stride(2) != 1 or key.stride(2) != 1 or value.stride(2) != 1 or kv_cache.stride(4) != 1:
        raise RuntimeError("Loom RoPE+paged-KV needs unit innermost strides")
    fp8 = kv_cache.dtype == torch.uint8
    view_span = (
        (kv_cache.shape[0] - 1) * kv_cache.stride(0) + (kv_cache.shape[2] - 1) * kv_cache.stride(2)
        + (kv_cache.shape[3] - 1) * kv_cache.stride(3) + kv_cache.shape[4]
    )
    key_cache_pointer = kv_cache.data_ptr()
    value_cache_pointer = key_cache_pointer + kv_cache.stride(1) * kv_cache.element_size()
    with _on_device(query.device):
        status = library().loom_cuda_bridge_rope_paged_kv_write(
            _DTYPE_CODES[query.dtype], _native.KV_CACHE_FP8_E4M3 if fp8 else _native.KV_CACHE_NATIVE,
            query.data_ptr(), _span(query), key.data_ptr(), _span(key), value.data_ptr(), _span(value),
            positions.data_ptr(), positions.numel(), cos_sin_cache.data_ptr(), cos_sin_cache.numel(),
            key_cache_pointer, view_span, value_cache_pointer, view_span,
            key_scales.data_ptr(), key_scales.numel(), value_scales.data_ptr(), value_scales.numel(),
            slot_mapping.data_ptr(), slot_mapping.numel(),
            query.shape[0], slot_mapping.numel(), query.shape[1], key.shape[1], query.shape[2],
            value.shape[2], cos_sin_cache.shape[1], cos_sin_cache.shape[0], kv_cache.shape[0],
            kv_cache.shape[2],
            query.stride(0), query.stride(1), key.stride(0), key.stride(1), value.stride(0), value.stride(1),
            kv_cache.stride(0), kv_cache.stride(2), kv_cache.stride(3),
            kv_cache.stride(0), kv_cache.stride(2), kv_cache.stride(3),
            1 if is_neox else 0, _stream(query.device),
        )
    check(status, "RoPE+paged-KV")
    return query, key, kv_cache


# ---- multi-token queries -------------------------------------------------------------------

def _multi_token_one_pass(query, key_cache, value_cache, block_tables, sequence_lengths, max_sequence_length,
                          scale, key_scales, value_scales):
    sequences, query_tokens, query_heads, head_size = query.shape
    kv_heads, value_head_size = key_cache.shape[2], value_cache.shape[3]
    fp8 = key_cache.dtype == torch.uint8
    device = query.device
    wide_heads = query_tokens * query_heads  # the rows of a (sequence, KV head) pair form one group of Tq x group
    packed = torch.empty((sequences, wide_heads, head_size), dtype=query.dtype, device=device)
    prefix_lengths = torch.empty((sequences,), dtype=torch.int32, device=device)
    states = torch.empty((sequences, wide_heads, value_head_size + 2), dtype=torch.float32, device=device)
    output = torch.empty((sequences, query_tokens, query_heads, value_head_size), dtype=query.dtype, device=device)
    lib = library()
    with _on_device(device):
        needed, tokens = decode_workspace_elements_ex(sequences, wide_heads, kv_heads, value_head_size,
                                                      max_sequence_length, 0)
        split = needed > 0 and max_sequence_length > (tokens if tokens else 256)
        workspace = torch.empty(needed, dtype=torch.float32, device=device) if split else None
        args = _native.LoomDecodeArgs()
        args.struct_size = ctypes.sizeof(_native.LoomDecodeArgs)
        args.dtype = _DTYPE_CODES[query.dtype]
        args.cache_encoding = _native.KV_CACHE_FP8_E4M3 if fp8 else _native.KV_CACHE_NATIVE
        args.scale_stride = 0 if not fp8 or key_scales.numel() == 1 else 1
        args.query, args.key_cache, args.value_cache = query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr()
        args.key_scales = key_scales.data_ptr() if fp8 else None
        args.value_scales = value_scales.data_ptr() if fp8 else None
        args.block_tables, args.sequence_lengths = block_tables.data_ptr(), sequence_lengths.data_ptr()
        args.output = output.data_ptr()
        args.workspace = workspace.data_ptr() if split else None
        args.workspace_elements = needed if split else 0
        args.sequences, args.query_heads, args.kv_heads = sequences, query_heads, kv_heads
        args.head_size, args.value_head_size = head_size, value_head_size
        args.num_blocks, args.block_size = key_cache.shape[0], key_cache.shape[1]
        args.max_blocks_per_sequence, args.max_sequence_length = block_tables.shape[1], max_sequence_length
        args.key_block_stride, args.key_page_stride, args.key_head_stride = key_cache.stride()[:3]
        args.value_block_stride, args.value_page_stride, args.value_head_stride = value_cache.stride()[:3]
        args.scale = scale
        args.stream = _stream(device)
        status = lib.loom_cuda_paged_multi_token_decode(ctypes.byref(args), query_tokens, packed.data_ptr(),
                                                        prefix_lengths.data_ptr(), states.data_ptr())
        if status != 0:
            raise RuntimeError("Loom multi-token decode failed: " + lib.loom_cuda_status_string(status).decode())
    return output


def paged_multi_token_decode_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    max_sequence_length: int,
    scale: float | None = None,
    key_scales: torch.Tensor | None = None,
    value_scales: torch.Tensor | None = None,
    scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
    one_pass: bool | None = None,
) -> torch.Tensor:
    """Causal attention of ``Tq`` new tokens per sequence over a paged cache.

    ``query`` is ``[B, Tq, Hq, D]`` (contiguous); ``sequence_lengths`` counts
    each context INCLUDING its ``Tq`` new tokens, whose K/V are already in the
    cache. Token ``t`` attends to the first ``length - (Tq - 1 - t)`` tokens.
    Returns ``[B, Tq, Hq, Dv]``. Caches, scales and tables as in
    ``paged_decode_attention_ex``. ``scratch`` may carry reusable int32 tensors
    ``([B * Tq, max_blocks], [B * Tq])`` for the expanded metadata.

    ``one_pass`` (default: whenever head sizes are at most 256) streams the KV
    once: the ``Tq x group`` rows of a (sequence, KV head) pair run as one GQA
    group over the common prefix ``length - (Tq - 1)`` and a finishing kernel
    adds each row's up to ``Tq - 1`` tail tokens. Otherwise the single-token
    decode runs on ``B * Tq`` rows with expanded metadata (any shape, but a
    sequence's pages are streamed once per query token).
    """
    if query.dim() != 4 or not query.is_contiguous():
        raise RuntimeError("Loom multi-token decode expects a contiguous query [B, Tq, Hq, D]")
    if block_tables.dtype != torch.int32 or sequence_lengths.dtype != torch.int32:
        raise RuntimeError("Loom paged decode metadata must be int32")
    if (block_tables.dim() != 2 or sequence_lengths.dim() != 1 or not block_tables.is_contiguous()
            or not sequence_lengths.is_contiguous() or block_tables.shape[0] != query.shape[0]
            or sequence_lengths.shape[0] != query.shape[0]):
        raise RuntimeError("Loom multi-token decode expects block_tables [B, max_blocks] and lengths [B]")
    if query.device.type != "cuda" or block_tables.device != query.device or sequence_lengths.device != query.device:
        raise RuntimeError("Loom paged decode tensors must share one CUDA device")
    sequences, query_tokens, query_heads, head_size = query.shape
    rows, max_blocks = sequences * query_tokens, block_tables.shape[1]
    fp8 = key_cache.dtype == torch.uint8
    if one_pass is None:
        one_pass = (query_tokens > 1 and head_size <= 256 and value_cache.shape[3] <= 256
                    and not (fp8 and query.dtype == torch.float32))
    if one_pass:
        return _multi_token_one_pass(query, key_cache, value_cache, block_tables, sequence_lengths,
                                     int(max_sequence_length), head_size ** -0.5 if scale is None else float(scale),
                                     key_scales if fp8 else None, value_scales if fp8 else None)
    if scratch is None:
        scratch = (torch.empty((rows, max_blocks), dtype=torch.int32, device=query.device),
                   torch.empty((rows,), dtype=torch.int32, device=query.device))
    tables, lengths = scratch
    if (tuple(tables.shape) != (rows, max_blocks) or tuple(lengths.shape) != (rows,) or tables.dtype != torch.int32
            or lengths.dtype != torch.int32 or not tables.is_contiguous() or not lengths.is_contiguous()
            or tables.device != query.device or lengths.device != query.device):
        raise RuntimeError("Loom multi-token decode scratch must be int32 [B*Tq, max_blocks] and [B*Tq] on the device")
    with _on_device(query.device):
        status = library().loom_cuda_expand_query_tokens(
            block_tables.data_ptr(), sequence_lengths.data_ptr(), tables.data_ptr(), lengths.data_ptr(),
            sequences, query_tokens, max_blocks, _stream(query.device))
    if status != 0:
        raise RuntimeError("Loom multi-token metadata expansion failed: "
                           + library().loom_cuda_status_string(status).decode())
    scales = dict(key_scales=key_scales, value_scales=value_scales) if key_cache.dtype == torch.uint8 else {}
    output = paged_decode_attention_ex(query.view(rows, query_heads, head_size), key_cache, value_cache, tables,
                                       lengths, max_sequence_length=max_sequence_length, scale=scale, **scales)
    return output.view(sequences, query_tokens, query_heads, output.shape[-1])


# ---- KV block movement ---------------------------------------------------------------------

def kv_block_movement_launches() -> int:
    """Successful move, swap and table-remap launches since the library was loaded."""
    count = _native.u64(0)
    check(library().loom_cuda_bridge_kv_block_movement_launches(count), "KV block movement launch count")
    return int(count.value)


_BLOCK_MOVE_ENGINES = {"bulk": 0, "vector": 1}


def set_kv_block_move_engine(engine: str) -> None:
    """``"bulk"`` (default): cp.async.bulk through shared memory; ``"vector"``: 16-byte loads and stores."""
    if library().loom_cuda_set_kv_block_move_engine(_BLOCK_MOVE_ENGINES[engine]) != 0:
        raise RuntimeError(f"unknown KV block move engine {engine!r}")


def kv_block_move_timeout_flag(device=None, reset: bool = False) -> int:
    """Non-zero after a bounded wait of the bulk-copy move kernel expired on this device."""
    value = _native.u32(0)
    with _on_device(torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)):
        status = library().loom_cuda_kv_block_move_timeout_flag(value, 1 if reset else 0)
    if status != 0:
        raise RuntimeError("reading the KV block move timeout flag failed")
    return int(value.value)


def _block_spans(kv_cache: torch.Tensor, name: str, host_allowed: bool = False):
    """(K pointer, V pointer, span bytes, block bytes, block stride bytes) of a packed cache.

    The cache is ``[blocks, 2, ...]`` with each block's K part and V part dense
    in memory (any order of the inner axes: NHD, HND).
    """
    if kv_cache.dim() < 3 or kv_cache.shape[1] != 2:
        raise RuntimeError(f"Loom KV block movement expects a [blocks, 2, ...] cache; {name} is not")
    if kv_cache.device.type != "cuda" and not (host_allowed and kv_cache.device.type == "cpu"
                                               and kv_cache.is_pinned()):
        raise RuntimeError("Loom KV block movement tensors must live on a CUDA device"
                           + (" or in pinned host memory" if host_allowed else ""))
    inner = kv_cache[0, 0]
    block_elements = inner.numel()
    if _span(inner) != block_elements:
        raise RuntimeError(f"the K and V parts of a block must be dense in memory; {name} has gaps inside a block")
    size = kv_cache.element_size()
    block_stride = kv_cache.stride(0) * size
    span = ((kv_cache.shape[0] - 1) * kv_cache.stride(0) + block_elements) * size
    key_pointer = kv_cache.data_ptr()
    value_pointer = key_pointer + kv_cache.stride(1) * size
    return key_pointer, value_pointer, span, block_elements * size, block_stride


def _pairs_argument(block_pairs: torch.Tensor, device: torch.device) -> torch.Tensor:
    if block_pairs.dtype != torch.int64 or block_pairs.dim() != 2 or block_pairs.shape[1] != 2:
        raise RuntimeError("Loom KV block pairs must be an int64 [pairs, 2] tensor")
    if block_pairs.device != device or not block_pairs.is_contiguous():
        raise RuntimeError("Loom KV block pairs must be contiguous and live on the cache's device")
    return block_pairs


def kv_block_move_(destination: torch.Tensor, source: torch.Tensor, block_pairs: torch.Tensor) -> torch.Tensor:
    """Copies whole KV blocks: ``destination[pairs[i, 1]] = source[pairs[i, 0]]``, K and V.

    Both caches are packed ``[blocks, 2, ...]`` allocations with the same block
    shape and dtype; they may be the same tensor (copy-on-write of a shared
    block, compaction) or different ones (gather into a staging buffer,
    scatter back). Either may also be a pinned host tensor: blocks swapped out
    to host memory on preemption and back in on resume travel over PCIe, read or
    written by the kernel directly. ``block_pairs`` is int64 ``[pairs, 2]`` on
    the device, whose current stream carries the launch. No block may be both
    read and written, nor written twice, in one call.
    """
    _require_inference_tensors(destination, source)
    if destination.dtype != source.dtype:
        raise RuntimeError("Loom KV block move needs caches of one dtype")
    device = block_pairs.device
    if device.type != "cuda" or any(t.device.type == "cuda" and t.device != device for t in (source, destination)):
        raise RuntimeError("Loom KV block pairs and the device caches must live on one CUDA device")
    pairs = _pairs_argument(block_pairs, device)
    source_key, source_value, source_span, block_bytes, source_stride = _block_spans(source, "source", True)
    to_key, to_value, to_span, to_block_bytes, to_stride = _block_spans(destination, "destination", True)
    if block_bytes != to_block_bytes:
        raise RuntimeError("Loom KV block move needs source and destination blocks of one size")
    with _on_device(device):
        status = library().loom_cuda_bridge_kv_block_move(
            source_key, source_span, source_value, source_span, to_key, to_span, to_value, to_span,
            pairs.data_ptr(), pairs.numel(), source.shape[0], destination.shape[0], block_bytes,
            source_stride, source_stride, to_stride, to_stride, _stream(device),
        )
    check(status, "KV block move")
    return destination


def kv_block_swap_(kv_cache: torch.Tensor, block_pairs: torch.Tensor) -> torch.Tensor:
    """Exchanges the contents of blocks ``pairs[i, 0]`` and ``pairs[i, 1]``, K and V, in place.

    A block may occur in one pair only.
    """
    _require_inference_tensors(kv_cache)
    pairs = _pairs_argument(block_pairs, kv_cache.device)
    key, value, span, block_bytes, stride = _block_spans(kv_cache, "kv_cache")
    with _on_device(kv_cache.device):
        status = library().loom_cuda_bridge_kv_block_swap(
            key, span, value, span, pairs.data_ptr(), pairs.numel(), kv_cache.shape[0], block_bytes, stride,
            stride, _stream(kv_cache.device),
        )
    check(status, "KV block swap")
    return kv_cache


def block_table_remap_(block_tables: torch.Tensor, new_block_ids: torch.Tensor) -> torch.Tensor:
    """``block_tables[i] = new_block_ids[block_tables[i]]`` in place, for ids inside the cache.

    Entries outside ``[0, len(new_block_ids))`` (negative sentinels) stay.
    """
    if block_tables.dtype != torch.int32 or new_block_ids.dtype != torch.int32:
        raise RuntimeError("Loom block tables and new block ids must be int32")
    if (block_tables.device.type != "cuda" or new_block_ids.device != block_tables.device
            or not block_tables.is_contiguous() or not new_block_ids.is_contiguous() or new_block_ids.dim() != 1):
        raise RuntimeError("Loom block table remap needs contiguous tensors on one CUDA device")
    with _on_device(block_tables.device):
        status = library().loom_cuda_bridge_block_table_remap(
            block_tables.data_ptr(), block_tables.numel(), new_block_ids.data_ptr(), new_block_ids.numel(),
            _stream(block_tables.device),
        )
    check(status, "block table remap")
    return block_tables


def default_scale(head_size: int) -> float:
    return 1.0 / math.sqrt(head_size)


__all__ = [
    "BridgeError",
    "Operator",
    "decode_workspace_elements",
    "decode_workspace_elements_ex",
    "last_decode_route",
    "launch_count",
    "merge_decode_states",
    "paged_decode_attention",
    "paged_decode_attention_ex",
    "paged_decode_attention_out",
    "reset_launch_count",
    "rope_paged_kv_write_",
    "supports_paged_decode_attention",
    "supports_rope_paged_kv_write",
]
