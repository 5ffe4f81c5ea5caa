"""ctypes binding of the CPU oracle (``libloom_oracle.so``).

TEST INFRASTRUCTURE ONLY. Tests, the smoke check and the CPU-baseline leg of
the benchmark import this module to check or to time the oracle. The shipped
package never does.

Arrays are numpy. F32 data is ``float32``; F16 and BF16 data are ``uint16``
bit patterns; FP8 data is ``uint8``. Integer metadata is ``int64`` as in the
reference's CPU functions.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np

F32, F16, BF16, FP8 = 0, 1, 2, 3
CACHE_NATIVE, CACHE_FP8_PER_TENSOR, CACHE_FP8_PER_HEAD = 0, 1, 2

ERROR_NAMES = {
    0: "Ok",
    1: "ZeroDimension",
    2: "ElementCountOverflow",
    3: "InvalidRotaryDimension",
    4: "PositionOutOfBounds",
    5: "SlotOutOfBounds",
    6: "DuplicateSlot",
    7: "InvalidScale",
    8: "HeadCountNotDivisible",
    9: "SequenceLengthOutOfBounds",
    10: "MaxSequenceLengthOutOfBounds",
    11: "BlockIdOutOfBounds",
    12: "LengthMismatch",
    13: "UnsupportedDType",
}

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libloom_oracle.so")


class _Error(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int32),
        ("a", ctypes.c_int64),
        ("b", ctypes.c_int64),
        ("c", ctypes.c_int64),
        ("d", ctypes.c_int64),
        ("value", ctypes.c_float),
        ("buffer", ctypes.c_char * 32),
    ]


class _DecodeSpec(ctypes.Structure):
    _fields_ = [
        ("sequences", ctypes.c_uint64),
        ("query_heads", ctypes.c_uint64),
        ("kv_heads", ctypes.c_uint64),
        ("head_size", ctypes.c_uint64),
        ("value_head_size", ctypes.c_uint64),
        ("num_blocks", ctypes.c_uint64),
        ("block_size", ctypes.c_uint64),
        ("max_blocks_per_sequence", ctypes.c_uint64),
        ("max_sequence_length", ctypes.c_uint64),
        ("scale", ctypes.c_float),
        ("dtype", ctypes.c_int32),
    ]


class _RotarySpec(ctypes.Structure):
    _fields_ = [
        ("tokens", ctypes.c_uint64),
        ("query_heads", ctypes.c_uint64),
        ("key_heads", ctypes.c_uint64),
        ("head_size", ctypes.c_uint64),
        ("rotary_dim", ctypes.c_uint64),
        ("max_position", ctypes.c_uint64),
        ("dtype", ctypes.c_int32),
        ("is_neox", ctypes.c_int32),
    ]


class _RopeKvSpec(ctypes.Structure):
    _fields_ = [
        ("rotary", _RotarySpec),
        ("value_head_size", ctypes.c_uint64),
        ("num_blocks", ctypes.c_uint64),
        ("block_size", ctypes.c_uint64),
        ("cache_encoding", ctypes.c_int32),
    ]


class OracleError(Exception):
    """A contract error raised by the oracle, with the reference's fields."""

    def __init__(self, kind: int, fields: dict, message: str):
        super().__init__(message)
        self.kind = ERROR_NAMES.get(kind, str(kind))
        self.fields = fields
        self.message = message


@dataclass(frozen=True)
class DecodeSpec:
    sequences: int
    query_heads: int
    kv_heads: int
    head_size: int
    value_head_size: int
    num_blocks: int
    block_size: int
    max_blocks_per_sequence: int
    max_sequence_length: int
    scale: float
    dtype: int

    def c(self) -> _DecodeSpec:
        return _DecodeSpec(
            self.sequences, self.query_heads, self.kv_heads, self.head_size,
            self.value_head_size, self.num_blocks, self.block_size,
            self.max_blocks_per_sequence, self.max_sequence_length, self.scale,
            self.dtype,
        )


@dataclass(frozen=True)
class RotarySpec:
    tokens: int
    query_heads: int
    key_heads: int
    head_size: int
    rotary_dim: int
    max_position: int
    dtype: int
    is_neox: bool

    def c(self) -> _RotarySpec:
        return _RotarySpec(
            self.tokens, self.query_heads, self.key_heads, self.head_size,
            self.rotary_dim, self.max_position, self.dtype, int(self.is_neox),
        )


@dataclass(frozen=True)
class RopeKvSpec:
    rotary: RotarySpec
    value_head_size: int
    num_blocks: int
    block_size: int
    cache_encoding: int

    def c(self) -> _RopeKvSpec:
        return _RopeKvSpec(
            self.rotary.c(), self.value_head_size, self.num_blocks,
            self.block_size, self.cache_encoding,
        )

    def scale_elements(self) -> int:
        if self.cache_encoding == CACHE_FP8_PER_TENSOR:
            return 1
        if self.cache_encoding == CACHE_FP8_PER_HEAD:
            return self.rotary.key_heads
        return 0


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the library is missing."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_fp8_e4m3fn_to_f32.restype = ctypes.c_float
        _lib.oracle_fp8_e4m3fn_to_f32.argtypes = [ctypes.c_uint8]
        _lib.oracle_fp8_e4m3fn_from_f32.restype = ctypes.c_uint8
        _lib.oracle_fp8_e4m3fn_from_f32.argtypes = [ctypes.c_float]
        _lib.oracle_fp8_e4m3fn_from_f32_direct.restype = ctypes.c_uint8
        _lib.oracle_fp8_e4m3fn_from_f32_direct.argtypes = [ctypes.c_float]
        for name in ("oracle_f32_to_bf16", "oracle_f32_to_f16"):
            getattr(_lib, name).restype = ctypes.c_uint16
            getattr(_lib, name).argtypes = [ctypes.c_float]
        for name in ("oracle_bf16_to_f32", "oracle_f16_to_f32"):
            getattr(_lib, name).restype = ctypes.c_float
            getattr(_lib, name).argtypes = [ctypes.c_uint16]
    return _lib


def _ptr(array):
    if array is None:
        return None
    assert array.flags["C_CONTIGUOUS"], "oracle buffers are contiguous"
    return array.ctypes.data_as(ctypes.c_void_p)


def _len(array) -> ctypes.c_uint64:
    return ctypes.c_uint64(0 if array is None else array.size)


def _raise(error: _Error):
    text = ctypes.create_string_buffer(512)
    lib().oracle_error_message(ctypes.byref(error), text, 512)
    fields = {
        "a": error.a, "b": error.b, "c": error.c, "d": error.d,
        "value": error.value, "buffer": error.buffer.decode(),
    }
    raise OracleError(error.kind, fields, text.value.decode())


def _check(status: int, error: _Error):
    if status != 0:
        _raise(error)


# ------------------------------------------------------------ conversions

def _convert(name: str, source: np.ndarray, out_dtype) -> np.ndarray:
    source = np.ascontiguousarray(source)
    out = np.empty(source.shape, dtype=out_dtype)
    getattr(lib(), name)(_ptr(source), _ptr(out), ctypes.c_uint64(source.size))
    return out


def f32_to_bf16(values) -> np.ndarray:
    return _convert("oracle_f32_to_bf16_n", np.asarray(values, np.float32), np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    return _convert("oracle_bf16_to_f32_n", np.asarray(bits, np.uint16), np.float32)


def f32_to_f16(values) -> np.ndarray:
    return _convert("oracle_f32_to_f16_n", np.asarray(values, np.float32), np.uint16)


def f16_to_f32(bits) -> np.ndarray:
    return _convert("oracle_f16_to_f32_n", np.asarray(bits, np.uint16), np.float32)


def fp8_from_f32(values) -> np.ndarray:
    return _convert("oracle_fp8_e4m3fn_from_f32_n", np.asarray(values, np.float32), np.uint8)


def fp8_to_f32(bits) -> np.ndarray:
    return _convert("oracle_fp8_e4m3fn_to_f32_n", np.asarray(bits, np.uint8), np.float32)


def to_storage(values, dtype: int) -> np.ndarray:
    """Rounds F32 values to the storage type (bit patterns for 16-bit types)."""
    values = np.asarray(values, np.float32)
    if dtype == F32:
        return np.ascontiguousarray(values)
    return f32_to_f16(values) if dtype == F16 else f32_to_bf16(values)


def from_storage(bits, dtype: int) -> np.ndarray:
    if dtype == F32:
        return np.asarray(bits, np.float32)
    return f16_to_f32(bits) if dtype == F16 else bf16_to_f32(bits)


# ------------------------------------------------------------------ specs

def check_decode_spec(spec: DecodeSpec):
    error = _Error()
    c_spec = spec.c()
    _check(lib().oracle_decode_spec_check(ctypes.byref(c_spec), ctypes.byref(error)), error)


def check_rotary_spec(spec: RotarySpec):
    error = _Error()
    c_spec = spec.c()
    _check(lib().oracle_rotary_spec_check(ctypes.byref(c_spec), ctypes.byref(error)), error)


def check_rope_kv_spec(spec: RopeKvSpec):
    error = _Error()
    c_spec = spec.c()
    _check(lib().oracle_rope_kv_spec_check(ctypes.byref(c_spec), ctypes.byref(error)), error)


# -------------------------------------------------------------- operators

import contextlib


@contextlib.contextmanager
def decode_options(sliding_window: int = 0, logits_soft_cap: float = 0.0):
    """Decode calls inside the block use a sliding window and/or a logits soft cap (extensions,
    parity unpinned); the reference's arithmetic is restored on exit."""
    library = lib()
    library.oracle_set_decode_options.argtypes = [ctypes.c_uint64, ctypes.c_double]
    if library.oracle_set_decode_options(int(sliding_window), float(logits_soft_cap)) != 0:
        raise ValueError("logits_soft_cap must be finite and not negative")
    try:
        yield
    finally:
        library.oracle_set_decode_options(0, 0.0)


def paged_decode_attention(call_dtype, query, key_cache, value_cache, block_tables,
                           sequence_lengths, output, spec: DecodeSpec, threads: int = 1):
    """Runs the reference decode in place on ``output``; raises OracleError."""
    error = _Error()
    c_spec = spec.c()
    block_tables = np.ascontiguousarray(block_tables, np.int64)
    sequence_lengths = np.ascontiguousarray(sequence_lengths, np.int64)
    status = lib().oracle_paged_decode_attention(
        ctypes.c_int32(call_dtype), _ptr(query), _len(query), _ptr(key_cache),
        _len(key_cache), _ptr(value_cache), _len(value_cache), _ptr(block_tables),
        _len(block_tables), _ptr(sequence_lengths), _len(sequence_lengths),
        _ptr(output), _len(output), ctypes.byref(c_spec), ctypes.c_int32(threads),
        ctypes.byref(error),
    )
    _check(status, error)
    return output


def paged_decode_attention_fp8(call_dtype, query, key_cache, value_cache, key_scales,
                               value_scales, scale_stride, block_tables,
                               sequence_lengths, output, spec: DecodeSpec,
                               threads: int = 1):
    error = _Error()
    c_spec = spec.c()
    block_tables = np.ascontiguousarray(block_tables, np.int64)
    sequence_lengths = np.ascontiguousarray(sequence_lengths, np.int64)
    key_scales = np.ascontiguousarray(key_scales, np.float32)
    value_scales = np.ascontiguousarray(value_scales, np.float32)
    status = lib().oracle_paged_decode_attention_fp8(
        ctypes.c_int32(call_dtype), _ptr(query), _len(query), _ptr(key_cache),
        _len(key_cache), _ptr(value_cache), _len(value_cache), _ptr(key_scales),
        _ptr(value_scales), ctypes.c_uint32(scale_stride), _ptr(block_tables),
        _len(block_tables), _ptr(sequence_lengths), _len(sequence_lengths),
        _ptr(output), _len(output), ctypes.byref(c_spec), ctypes.c_int32(threads),
        ctypes.byref(error),
    )
    _check(status, error)
    return output


def rotary_embedding(call_dtype, query, key, positions, cos_sin_cache, spec: RotarySpec):
    error = _Error()
    c_spec = spec.c()
    positions = np.ascontiguousarray(positions, np.int64)
    status = lib().oracle_rotary_embedding(
        ctypes.c_int32(call_dtype), _ptr(query), _len(query), _ptr(key), _len(key),
        _ptr(positions), _len(positions), _ptr(cos_sin_cache), _len(cos_sin_cache),
        ctypes.byref(c_spec), ctypes.byref(error),
    )
    _check(status, error)


def rope_paged_kv_write(call_dtype, query, key, value, positions, cos_sin_cache,
                        key_cache, value_cache, slot_mapping, spec: RopeKvSpec):
    error = _Error()
    c_spec = spec.c()
    positions = np.ascontiguousarray(positions, np.int64)
    slot_mapping = np.ascontiguousarray(slot_mapping, np.int64)
    status = lib().oracle_rope_paged_kv_write(
        ctypes.c_int32(call_dtype), _ptr(query), _len(query), _ptr(key), _len(key),
        _ptr(value), _len(value), _ptr(positions), _len(positions),
        _ptr(cos_sin_cache), _len(cos_sin_cache), _ptr(key_cache), _len(key_cache),
        _ptr(value_cache), _len(value_cache), _ptr(slot_mapping), _len(slot_mapping),
        ctypes.byref(c_spec), ctypes.byref(error),
    )
    _check(status, error)


def rope_paged_kv_write_fp8(call_dtype, query, key, value, positions, cos_sin_cache,
                            key_cache, value_cache, slot_mapping, key_scales,
                            value_scales, spec: RopeKvSpec):
    error = _Error()
    c_spec = spec.c()
    positions = np.ascontiguousarray(positions, np.int64)
    slot_mapping = np.ascontiguousarray(slot_mapping, np.int64)
    key_scales = np.ascontiguousarray(key_scales, np.float32)
    value_scales = np.ascontiguousarray(value_scales, np.float32)
    status = lib().oracle_rope_paged_kv_write_fp8(
        ctypes.c_int32(call_dtype), _ptr(query), _len(query), _ptr(key), _len(key),
        _ptr(value), _len(value), _ptr(positions), _len(positions),
        _ptr(cos_sin_cache), _len(cos_sin_cache), _ptr(key_cache), _len(key_cache),
        _ptr(value_cache), _len(value_cache), _ptr(slot_mapping), _len(slot_mapping),
        _ptr(key_scales), _len(key_scales), _ptr(value_scales), _len(value_scales),
        ctypes.byref(c_spec), ctypes.byref(error),
    )
    _check(status, error)


def max_threads() -> int:
    return int(lib().oracle_max_threads())
