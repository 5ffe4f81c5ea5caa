"""ctypes binding of ``libloom_cuda_bridge.so`` (the checked bridge ABI).

The library is the product: if it has not been built, importing the operators
fails with instructions instead of falling back to anything else.
"""

from __future__ import annotations

import ctypes
import os

_PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_PACKAGE_DIR, "libloom_cuda_bridge.so")

SUCCESS, INVALID_ARGUMENT, LAUNCH_ERROR, UNAVAILABLE = 0, 1, 2, 3
F32, F16, BF16 = 0, 1, 2
KV_CACHE_NATIVE, KV_CACHE_FP8_E4M3 = 0, 1
DECODE_STABLE_METADATA = 2
BRIDGE_ABI_VERSION = 2

u32, u64, f32 = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_float
ptr = ctypes.c_void_p


class LoomDecodeArgs(ctypes.Structure):
    """ctypes mirror of ``LoomDecodeArgs`` (include/loom_launch.h)."""

    _fields_ = (
        [(name, u32) for name in ("struct_size", "dtype", "cache_encoding", "scale_stride")]
        + [(name, ptr) for name in ("query", "key_cache", "value_cache", "key_scales", "value_scales",
                                    "block_tables", "sequence_lengths", "output", "workspace")]
        + [("workspace_elements", u64)]
        + [(name, u32) for name in ("sequences", "query_heads", "kv_heads", "head_size", "value_head_size",
                                    "num_blocks", "block_size", "max_blocks_per_sequence", "max_sequence_length",
                                    "partition_tokens")]
        + [(name, u64) for name in ("key_block_stride", "key_page_stride", "key_head_stride", "value_block_stride",
                                    "value_page_stride", "value_head_stride", "query_token_stride",
                                    "query_head_stride")]
        + [("scale", f32), ("emit_state", u32), ("stream", ptr)]
        + [("sliding_window", u32), ("logits_soft_cap", f32), ("flags", u32), ("reserved", u32)]
    )


class NativeLibraryMissing(ImportError):
    pass


class BridgeError(RuntimeError):
    """A bridge call returned a non-zero status."""

    def __init__(self, operation: str, status: int, message: str):
        super().__init__(f"Loom {operation} bridge failed: {message} (status {status})")
        self.operation = operation
        self.status = status
        self.bridge_message = message


_lib = None


def _declare(lib):
    lib.loom_cuda_bridge_abi_version.restype = u32
    lib.loom_cuda_bridge_abi_version.argtypes = []
    lib.loom_cuda_bridge_last_error_message.restype = ctypes.c_char_p
    lib.loom_cuda_bridge_last_error_message.argtypes = []
    lib.loom_cuda_bridge_launch_count.argtypes = [u32, ctypes.POINTER(u64)]
    lib.loom_cuda_bridge_reset_launch_count.argtypes = [u32]
    lib.loom_cuda_bridge_paged_decode_workspace_elements.argtypes = [u32] * 10 + [f32, ctypes.POINTER(u64)]
    lib.loom_cuda_bridge_paged_decode_attention.argtypes = (
        [u32, ptr, u64, ptr, u64, ptr, u64, ptr, u64, ptr, u64, ptr, u64, ptr, u64]
        + [u32] * 7 + [u64, u64, u32, u32, f32, ptr]
    )
    lib.loom_cuda_bridge_paged_decode_workspace_elements_ex.argtypes = (
        [u32] * 6 + [ctypes.POINTER(u64), ctypes.POINTER(u32)]
    )
    lib.loom_cuda_bridge_paged_decode_attention_ex.argtypes = (
        [u32, u32] + [ptr, u64] * 9 + [u32] * 7 + [u64] * 6 + [u32, u32, u32, f32, u32, u64, u64, ptr]
    )
    lib.loom_cuda_bridge_paged_decode_attention_with_options.argtypes = (
        [u32, u32] + [ptr, u64] * 9 + [u32] * 7 + [u64] * 6 + [u32, u32, u32, f32, u32, u64, u64, u32, f32, u32, ptr]
    )
    lib.loom_cuda_bridge_merge_decode_states.argtypes = [ptr, u64, u32, u32, u32, u32, ptr, u64, ptr]
    lib.loom_cuda_bridge_supports_paged_decode.argtypes = [u32] * 11 + [f32]
    lib.loom_cuda_bridge_supports_rope_paged_kv_write.argtypes = [u32] * 11
    lib.loom_cuda_bridge_rope_paged_kv_write.argtypes = (
        [u32, u32] + [ptr, u64] * 10 + [u32] * 10 + [u64] * 12 + [u32, ptr]
    )
    lib.loom_cuda_last_decode_route.restype = ctypes.c_char_p
    lib.loom_cuda_last_decode_route.argtypes = []
    lib.loom_cuda_last_launch_failure.restype = ctypes.c_char_p
    lib.loom_cuda_last_launch_failure.argtypes = []
    lib.loom_cuda_plain_launch_retries.restype = u64
    lib.loom_cuda_plain_launch_retries.argtypes = []
    lib.loom_cuda_set_wait_policy.argtypes = [u32, u32]
    lib.loom_cuda_set_decode_copy_engine.argtypes = [u32]
    lib.loom_cuda_set_programmatic_launch.argtypes = [u32]
    lib.loom_cuda_decode_timeout_flag.argtypes = [ctypes.POINTER(u32), u32]
    lib.loom_cuda_status_string.restype = ctypes.c_char_p
    lib.loom_cuda_status_string.argtypes = [ctypes.c_int]
    lib.loom_cuda_paged_decode_default_partition_tokens.restype = u32
    lib.loom_cuda_paged_decode_default_partition_tokens.argtypes = [u32, u32, u32]
    for name in ("f32", "f16", "bf16"):
        getattr(lib, f"loom_cuda_paged_decode_attention_{name}").argtypes = (
            [ptr] * 6 + [u32] * 7 + [u64, u64, u32, u32, f32, ptr]
        )
        getattr(lib, f"loom_cuda_paged_decode_attention_split_k_{name}").argtypes = (
            [ptr] * 7 + [u64] + [u32] * 7 + [u64, u64, u32, u32, f32, ptr]
        )
        getattr(lib, f"loom_cuda_rope_paged_kv_write_{name}").argtypes = (
            [ptr] * 10 + [u32] * 12 + [u64] * 12 + [u32, ptr]
        )
    lib.loom_cuda_paged_decode_attention_split_k_workspace_elements.restype = u64
    lib.loom_cuda_paged_decode_attention_split_k_workspace_elements.argtypes = [u32] * 6
    lib.loom_cuda_paged_decode_workspace_elements.restype = u64
    lib.loom_cuda_paged_decode_workspace_elements.argtypes = [u32] * 6
    lib.loom_cuda_merge_decode_states.argtypes = [ptr, u32, u32, u32, u32, ptr, ptr]
    lib.loom_cuda_expand_query_tokens.argtypes = [ptr, ptr, ptr, ptr, u32, u32, u32, ptr]
    lib.loom_cuda_multi_token_prepare.argtypes = [ptr, ptr, ptr, ptr] + [u32] * 6 + [ptr]
    lib.loom_cuda_multi_token_finish.argtypes = [ctypes.POINTER(LoomDecodeArgs), u32, ptr]
    lib.loom_cuda_paged_multi_token_decode.argtypes = [ctypes.POINTER(LoomDecodeArgs), u32, ptr, ptr, ptr]
    # KV block movement
    lib.loom_cuda_bridge_kv_block_move.argtypes = [ptr, u64] * 5 + [u32, u32] + [u64] * 5 + [ptr]
    lib.loom_cuda_bridge_kv_block_swap.argtypes = [ptr, u64] * 3 + [u32] + [u64] * 3 + [ptr]
    lib.loom_cuda_bridge_block_table_remap.argtypes = [ptr, u64, ptr, u64, ptr]
    lib.loom_cuda_bridge_kv_block_movement_launches.argtypes = [ctypes.POINTER(u64)]
    lib.loom_cuda_kv_block_move.argtypes = [ptr] * 5 + [u32] * 3 + [u64] * 5 + [ptr]
    lib.loom_cuda_kv_block_swap.argtypes = [ptr] * 3 + [u32, u32] + [u64] * 3 + [ptr]
    lib.loom_cuda_block_table_remap.argtypes = [ptr, u64, ptr, u32, ptr]
    lib.loom_cuda_set_kv_block_move_engine.argtypes = [u32]
    lib.loom_cuda_kv_block_move_timeout_flag.argtypes = [ctypes.POINTER(u32), u32]
    # peer exchange of partial states
    lib.loom_cuda_peer_exchange_bytes.restype = u64
    lib.loom_cuda_peer_exchange_bytes.argtypes = [u32, u32, u32]
    lib.loom_cuda_peer_exchange_create.argtypes = [u64, ctypes.POINTER(ptr), ctypes.c_char_p, u64]
    lib.loom_cuda_peer_exchange_open.argtypes = [ctypes.c_char_p, u64, ctypes.POINTER(ptr)]
    lib.loom_cuda_peer_exchange_close.argtypes = [ptr]
    lib.loom_cuda_peer_exchange_destroy.argtypes = [ptr]
    lib.loom_cuda_peer_exchange_reset.argtypes = [ptr, u64, ptr]
    lib.loom_cuda_peer_exchange_status.argtypes = [ptr, ctypes.POINTER(u64), ctypes.POINTER(u32)]
    lib.loom_cuda_peer_exchange_push.argtypes = [ptr, ctypes.POINTER(ptr), u32, u32, u32, u32, ptr]
    lib.loom_cuda_peer_exchange_merge.argtypes = [ptr, u32, u32, u32, u32, ptr, ptr]
    # partitioner
    i64p, u32p, u64p = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(u32), ctypes.POINTER(u64)
    lib.loom_partition_by_sequence.argtypes = [i64p, u32, u32, u32p, u64p]
    lib.loom_partition_by_kv_head.argtypes = [u32, u32, u32p, u32p]
    lib.loom_partition_long_context.argtypes = [i64p, u32, u32, u32, u64, ptr, u32, u32p, u64p]


def library() -> ctypes.CDLL:
    """Loads the built library once; raises if it is absent or of another ABI."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise NativeLibraryMissing(
                f"{LIBRARY_PATH} has not been built. Run `python -m attnarc_b200.build` "
                "(needs nvcc with sm_100a support). There is no fallback implementation."
            )
        lib = ctypes.CDLL(LIBRARY_PATH)
        _declare(lib)
        version = lib.loom_cuda_bridge_abi_version()
        if version != BRIDGE_ABI_VERSION:
            raise NativeLibraryMissing(
                f"{LIBRARY_PATH} has bridge ABI {version}, expected {BRIDGE_ABI_VERSION}"
            )
        _lib = lib
    return _lib


def last_error() -> str:
    return library().loom_cuda_bridge_last_error_message().decode("utf-8", "replace")


def check(status: int, operation: str) -> None:
    if status != SUCCESS:
        raise BridgeError(operation, status, last_error())
