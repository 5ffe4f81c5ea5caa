"""One serving step, host buffers in and host buffer out, as a CUDA graph.

A decode step of a serving engine is: copy the step's packed QKV rows and its
metadata (positions, slots, block tables, context lengths) to the device,
rotate Q/K and write K/V into the paged cache, attend over the cache, and read
the attention rows back. Issued call by call that is two copies in, three
kernel launches and one copy out, and the host's own work between the calls
(argument checks, ctypes marshalling) is longer than the kernels of a small
batch. ``CapturedDecodeStep`` records the whole sequence once and replays it
with one launch per step, the way serving engines run their decode loop.

The inputs live in one pinned host buffer (one copy per step); the caller
refills its views in place before each ``run``. Shapes, the cache and the
buffers are fixed at capture time; the kernels read lengths and tables from
the device, so every step may carry different contexts up to
``max_sequence_length``.
"""

from __future__ import annotations

import torch

from . import ops


class CapturedDecodeStep:
    """RoPE + paged-KV write and paged decode attention of one step, captured.

    ``kv_cache`` is the packed cache ``[blocks, 2, block_size, kv_heads, dim]``
    (any positive strides: NHD, or an HND allocation permuted to this order);
    ``uint8`` storage selects the FP8 E4M3 cache and needs both scale tensors.

    Pinned host views to fill before every ``run``:

    - ``host_qkv``            ``[sequences, query_heads + 2 * kv_heads, dim]``
    - ``host_positions``      ``[sequences]`` int64
    - ``host_slot_mapping``   ``[sequences]`` int64
    - ``host_block_tables``   ``[sequences, max_blocks_per_sequence]`` int32
    - ``host_sequence_lengths`` ``[sequences]`` int32

    ``run`` returns ``host_output`` ``[sequences, query_heads, dim]`` (pinned),
    valid until the next ``run``.
    """

    def __init__(
        self,
        kv_cache: torch.Tensor,
        cos_sin_cache: torch.Tensor,
        *,
        sequences: int,
        query_heads: int,
        max_blocks_per_sequence: int,
        max_sequence_length: int,
        dtype: torch.dtype,
        scale: float | None = None,
        is_neox: bool = True,
        key_scales: torch.Tensor | None = None,
        value_scales: torch.Tensor | None = None,
        partition_tokens: int = 0,
    ):
        if kv_cache.device.type != "cuda":
            raise RuntimeError("CapturedDecodeStep needs a CUDA device; there is no CPU path")
        if kv_cache.dim() != 5 or kv_cache.shape[1] != 2:
            raise RuntimeError("CapturedDecodeStep expects a [blocks, 2, block_size, kv_heads, dim] cache")
        fp8 = kv_cache.dtype == torch.uint8
        if fp8 and (key_scales is None or value_scales is None):
            raise RuntimeError("an FP8 E4M3 cache needs key_scales and value_scales")
        if not fp8 and kv_cache.dtype != dtype:
            raise RuntimeError("a native cache has the dtype of the queries")
        self.device = kv_cache.device
        self.kv_cache = kv_cache
        self.cos_sin_cache = cos_sin_cache
        self.sequences, self.query_heads = int(sequences), int(query_heads)
        self.kv_heads, self.head_size = int(kv_cache.shape[3]), int(kv_cache.shape[4])
        self.max_sequence_length = int(max_sequence_length)
        self.scale = float(scale) if scale is not None else self.head_size ** -0.5
        self.is_neox = bool(is_neox)
        one = None if fp8 else torch.ones(1, dtype=torch.float32, device=self.device)
        self.key_scales = key_scales if fp8 else one
        self.value_scales = value_scales if fp8 else one
        self._decode_scales = dict(key_scales=key_scales, value_scales=value_scales) if fp8 else {}

        # ---- one pinned host buffer and its device mirror ----------------------------------
        rows = self.query_heads + 2 * self.kv_heads
        element = torch.empty((), dtype=dtype).element_size()
        layout = [  # (name, dtype, shape); 8-byte pieces before 4-byte ones keeps every offset aligned
            ("qkv", dtype, (self.sequences, rows, self.head_size)),
            ("positions", torch.int64, (self.sequences,)),
            ("slot_mapping", torch.int64, (self.sequences,)),
            ("block_tables", torch.int32, (self.sequences, int(max_blocks_per_sequence))),
            ("sequence_lengths", torch.int32, (self.sequences,)),
        ]
        sizes = []
        for _, piece_dtype, shape in layout:
            count = 1
            for extent in shape:
                count *= extent
            sizes.append(count * torch.empty((), dtype=piece_dtype).element_size())
        sizes[0] = (self.sequences * rows * self.head_size * element + 15) // 16 * 16
        offsets = [sum(sizes[:i]) for i in range(len(sizes))]
        self._host = torch.empty(sum(sizes), dtype=torch.uint8).pin_memory()
        self._host.zero_()
        self._device = torch.zeros(sum(sizes), dtype=torch.uint8, device=self.device)

        def views(buffer):
            out = {}
            for (name, piece_dtype, shape), offset in zip(layout, offsets):
                count = 1
                for extent in shape:
                    count *= extent
                width = torch.empty((), dtype=piece_dtype).element_size()
                out[name] = buffer[offset:offset + count * width].view(piece_dtype).reshape(shape)
            return out

        host, device = views(self._host), views(self._device)
        self.host_qkv = host["qkv"]
        self.host_positions = host["positions"]
        self.host_slot_mapping = host["slot_mapping"]
        self.host_block_tables = host["block_tables"]
        self.host_sequence_lengths = host["sequence_lengths"]
        self._pieces = device
        self.h2d_bytes = self._host.numel()

        needed, partition = ops.decode_workspace_elements_ex(
            self.sequences, self.query_heads, self.kv_heads, self.head_size, self.max_sequence_length,
            partition_tokens)
        self._partition = partition
        self._split = self.max_sequence_length > partition
        self._workspace = (torch.empty(needed, device=self.device, dtype=torch.float32)
                           if self._split and needed else None)
        self.output = torch.empty((self.sequences, self.query_heads, self.head_size), device=self.device,
                                  dtype=dtype)
        self.host_output = torch.empty(self.output.shape, dtype=dtype).pin_memory()
        self.d2h_bytes = self.host_output.numel() * self.host_output.element_size()
        self.kernel_launches = 2 + (1 if self._split else 0)
        self._graph: torch.cuda.CUDAGraph | None = None

    # The step as a sequence of stream operations (eager, or under capture).
    def _enqueue(self) -> None:
        self._device.copy_(self._host, non_blocking=True)
        qkv = self._pieces["qkv"]
        query = qkv[:, :self.query_heads]
        key = qkv[:, self.query_heads:self.query_heads + self.kv_heads]
        value = qkv[:, self.query_heads + self.kv_heads:]
        ops.rope_paged_kv_write_(query, key, value, self._pieces["positions"], self.cos_sin_cache, self.kv_cache,
                                 self.key_scales, self.value_scales, self._pieces["slot_mapping"],
                                 is_neox=self.is_neox)
        ops.paged_decode_attention_ex(
            query, self.kv_cache[:, 0], self.kv_cache[:, 1], self._pieces["block_tables"],
            self._pieces["sequence_lengths"], max_sequence_length=self.max_sequence_length, scale=self.scale,
            workspace=self._workspace, partition_tokens=self._partition, split=self._split, output=self.output,
            stable_metadata=True,  # lengths and tables arrive with the copy above, before the RoPE launch
            **self._decode_scales)
        self.host_output.copy_(self.output, non_blocking=True)

    def run_eager(self) -> torch.Tensor:
        """The same step issued call by call on the current stream (no graph)."""
        with torch.cuda.device(self.device):
            self._enqueue()
            torch.cuda.current_stream().synchronize()
        return self.host_output

    def capture(self) -> "CapturedDecodeStep":
        """Records the step. The host views must hold a valid step: it is run once first."""
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

    def launch(self) -> None:
        """Replays the recorded step on the current stream without waiting for it."""
        if self._graph is None:
            raise RuntimeError("CapturedDecodeStep.capture() has not been called")
        self._graph.replay()

    def run(self) -> torch.Tensor:
        """Replays the recorded step and waits for its result in ``host_output``."""
        self.launch()
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_output
