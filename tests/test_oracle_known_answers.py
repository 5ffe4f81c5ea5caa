"""Pins the CPU oracle to the reference's own known-answer tests.

Each test replays one test of the reference's contract crate against the C++
restatement: crates/loom-kernels/src/tests/attention_tests.rs and
crates/loom-kernels/src/tests/rope_kv_tests.rs. Inputs and expected values are
the ones those tests state; nothing here needs a GPU.
"""

import math

import numpy as np
import pytest

from oracle import binding as ob


def f32(values):
    return np.array(values, dtype=np.float32)


# ------------------------------------------------ attention_tests.rs:5-30
def test_decode_follows_block_indirection_and_gqa_mapping():
    spec = ob.DecodeSpec(1, 2, 1, 1, 1, 2, 2, 2, 4, 1.0, ob.F32)
    query = f32([1.0, 1.0])
    # Physical block 0 is the second logical block; its second slot lies
    # beyond the active length and must not influence the result.
    key_cache = f32([2.0, 99.0, 0.0, 1.0])
    value_cache = f32([20.0, 99.0, 1.0, 10.0])
    output = f32([-1.0, -1.0])
    ob.paged_decode_attention(ob.F32, query, key_cache, value_cache, [1, 0], [3], output, spec)
    e1, e2 = np.float32(np.exp(np.float32(1.0))), np.float32(np.exp(np.float32(2.0)))
    expected = (1.0 + 10.0 * e1 + 20.0 * e2) / (1.0 + e1 + e2)
    assert abs(output[0] - expected) < 1.0e-6
    assert abs(output[1] - expected) < 1.0e-6


# ----------------------------------------------- attention_tests.rs:32-56
def test_decode_supports_low_precision_and_distinct_value_width():
    spec = ob.DecodeSpec(1, 1, 1, 2, 3, 1, 1, 1, 1, 0.5, ob.BF16)
    query = ob.f32_to_bf16([2.0, -1.0])
    key_cache = ob.f32_to_bf16([4.0, 3.0])
    value_cache = ob.f32_to_bf16([1.25, -2.5, 7.0])
    output = np.zeros(3, dtype=np.uint16)
    ob.paged_decode_attention(ob.BF16, query, key_cache, value_cache, [0], [1], output, spec)
    assert np.array_equal(output, value_cache)


# ---------------------------------------------- attention_tests.rs:58-118
def test_decode_validates_metadata_before_mutating_output():
    with pytest.raises(ob.OracleError) as info:
        ob.check_decode_spec(ob.DecodeSpec(1, 3, 2, 4, 4, 1, 16, 1, 16, 0.5, ob.F16))
    assert info.value.kind == "HeadCountNotDivisible"
    assert (info.value.fields["a"], info.value.fields["b"]) == (3, 2)

    with pytest.raises(ob.OracleError) as info:
        ob.check_decode_spec(ob.DecodeSpec(1, 2, 1, 4, 4, 1, 16, 1, 16, 0.0, ob.F16))
    assert info.value.kind == "InvalidScale"
    assert info.value.fields["value"] == 0.0

    spec = ob.DecodeSpec(2, 1, 1, 1, 1, 2, 2, 2, 4, 1.0, ob.F32)
    query = f32([1.0, 1.0])
    key_cache = f32([1.0] * 4)
    value_cache = f32([2.0] * 4)
    output = f32([-7.0, -7.0])

    with pytest.raises(ob.OracleError) as info:
        ob.paged_decode_attention(
            ob.F32, query, key_cache, value_cache, [0, 1, 1, -1], [3, 5], output, spec
        )
    assert info.value.kind == "SequenceLengthOutOfBounds"
    fields = info.value.fields
    assert (fields["a"], fields["b"], fields["c"]) == (1, 5, 4)
    assert np.array_equal(output, f32([-7.0, -7.0]))

    with pytest.raises(ob.OracleError) as info:
        ob.paged_decode_attention(
            ob.F32, query, key_cache, value_cache, [0, 2, 1, -1], [3, 1], output, spec
        )
    assert info.value.kind == "BlockIdOutOfBounds"
    fields = info.value.fields
    assert (fields["a"], fields["b"], fields["c"], fields["d"]) == (0, 1, 2, 2)
    assert np.array_equal(output, f32([-7.0, -7.0]))


# -------------------------------------------------- rope_kv_tests.rs:3-19
def test_rotary_contract_rejects_invalid_partial_dimensions():
    for rotary_dim in (3, 10):
        with pytest.raises(ob.OracleError) as info:
            ob.check_rotary_spec(ob.RotarySpec(1, 2, 1, 8, rotary_dim, 16, ob.F16, True))
        assert info.value.kind == "InvalidRotaryDimension"
        assert (info.value.fields["a"], info.value.fields["b"]) == (rotary_dim, 8)


# ------------------------------------------------- rope_kv_tests.rs:21-54
def test_rotary_supports_both_pairing_styles_and_partial_rope():
    cos_sin = f32([1.0, 1.0, 0.0, 0.0, 0.0, 0.0, 1.0, 1.0])
    positions = [1]

    neox = ob.RotarySpec(1, 1, 1, 6, 4, 2, ob.F32, True)
    query = f32([1.0, 2.0, 3.0, 4.0, 5.0, 6.0])
    key = f32([7.0, 8.0, 9.0, 10.0, 11.0, 12.0])
    ob.rotary_embedding(ob.F32, query, key, positions, cos_sin, neox)
    assert query.tolist() == [-3.0, -4.0, 1.0, 2.0, 5.0, 6.0]
    assert key.tolist() == [-9.0, -10.0, 7.0, 8.0, 11.0, 12.0]

    interleaved = ob.RotarySpec(1, 1, 1, 6, 4, 2, ob.F32, False)
    query = f32([1.0, 2.0, 3.0, 4.0, 5.0, 6.0])
    key = f32([7.0, 8.0, 9.0, 10.0, 11.0, 12.0])
    ob.rotary_embedding(ob.F32, query, key, positions, cos_sin, interleaved)
    assert query.tolist() == [-2.0, 1.0, -4.0, 3.0, 5.0, 6.0]
    assert key.tolist() == [-8.0, 7.0, -10.0, 9.0, 11.0, 12.0]


# ------------------------------------------------- rope_kv_tests.rs:56-90
def test_fused_write_rotates_padding_but_skips_its_cache_slot():
    rotary = ob.RotarySpec(2, 1, 1, 4, 4, 2, ob.F32, True)
    spec = ob.RopeKvSpec(rotary, 2, 2, 2, ob.CACHE_NATIVE)
    assert spec.scale_elements() == 0
    query = f32([1, 2, 3, 4, 5, 6, 7, 8])
    key = f32([9, 10, 11, 12, 13, 14, 15, 16])
    value = f32([17, 18, 19, 20])
    cos_sin = f32([1.0, 1.0, 0.0, 0.0, 0.0, 0.0, 1.0, 1.0])
    key_cache = np.full(16, -99.0, dtype=np.float32)
    value_cache = np.full(8, -99.0, dtype=np.float32)

    ob.rope_paged_kv_write(
        ob.F32, query, key, value, [0, 1], cos_sin, key_cache, value_cache, [3, -1], spec
    )

    assert query[:4].tolist() == [1.0, 2.0, 3.0, 4.0]
    assert query[4:].tolist() == [-7.0, -8.0, 5.0, 6.0]
    assert key[4:].tolist() == [-15.0, -16.0, 13.0, 14.0]
    assert np.all(key_cache[:12] == -99.0)
    assert key_cache[12:].tolist() == [9.0, 10.0, 11.0, 12.0]
    assert np.all(value_cache[:6] == -99.0)
    assert value_cache[6:].tolist() == [17.0, 18.0]


# ------------------------------------------------ rope_kv_tests.rs:92-139
def test_fused_write_rejects_bad_metadata_before_mutation():
    rotary = ob.RotarySpec(2, 1, 1, 4, 4, 2, ob.F32, True)
    spec = ob.RopeKvSpec(rotary, 4, 1, 2, ob.CACHE_NATIVE)
    original = f32([1.0] * 8)
    query, key = original.copy(), original.copy()
    value = f32([2.0] * 8)
    cache = f32([1.0, 1.0, 0.0, 0.0, 1.0, 1.0, 0.0, 0.0])
    key_cache = np.zeros(8, dtype=np.float32)
    value_cache = np.zeros(8, dtype=np.float32)

    with pytest.raises(ob.OracleError) as info:
        ob.rope_paged_kv_write(
            ob.F32, query, key, value, [0, 1], cache, key_cache, value_cache, [1, 1], spec
        )
    assert info.value.kind == "DuplicateSlot"
    fields = info.value.fields
    assert (fields["a"], fields["b"], fields["c"]) == (0, 1, 1)
    assert np.array_equal(query, original) and np.array_equal(key, original)

    with pytest.raises(ob.OracleError) as info:
        ob.rotary_embedding(ob.F32, query, key, [0, 2], cache, rotary)
    assert info.value.kind == "PositionOutOfBounds"
    fields = info.value.fields
    assert (fields["a"], fields["b"], fields["c"]) == (1, 2, 2)
    assert np.array_equal(query, original) and np.array_equal(key, original)


# ----------------------------------------------- rope_kv_tests.rs:141-188
def test_fused_write_quantizes_fp8_with_per_head_scales():
    rotary = ob.RotarySpec(1, 1, 2, 4, 4, 1, ob.F32, True)
    spec = ob.RopeKvSpec(rotary, 2, 1, 2, ob.CACHE_FP8_PER_HEAD)
    assert spec.scale_elements() == 2
    query = f32([1, 2, 3, 4])
    key = f32([1, 2, 3, 4, 10, 20, 30, 40])
    value = f32([2, 4, 8, 12])
    cos_sin = f32([1.0, 1.0, 0.0, 0.0])
    key_cache = np.full(16, 0xAA, dtype=np.uint8)
    value_cache = np.full(8, 0xAA, dtype=np.uint8)

    ob.rope_paged_kv_write_fp8(
        ob.F32, query, key, value, [0], cos_sin, key_cache, value_cache, [1],
        [1.0, 10.0], [2.0, 4.0], spec,
    )

    assert np.all(key_cache[:8] == 0xAA)
    assert np.array_equal(key_cache[8:], ob.fp8_from_f32([1, 2, 3, 4, 1, 2, 3, 4]))
    assert np.all(value_cache[:4] == 0xAA)
    assert np.array_equal(value_cache[4:], ob.fp8_from_f32([1, 2, 2, 3]))


# ----------------------------------------------- rope_kv_tests.rs:190-226
def test_fp8_write_rejects_invalid_scales_before_mutation():
    rotary = ob.RotarySpec(1, 1, 1, 4, 4, 1, ob.F32, True)
    spec = ob.RopeKvSpec(rotary, 4, 1, 1, ob.CACHE_FP8_PER_TENSOR)
    original = f32([1, 2, 3, 4])
    query, key, value = original.copy(), original.copy(), original.copy()
    key_cache = np.zeros(4, dtype=np.uint8)
    value_cache = np.zeros(4, dtype=np.uint8)
    with pytest.raises(ob.OracleError) as info:
        ob.rope_paged_kv_write_fp8(
            ob.F32, query, key, value, [0], f32([0.0, 0.0, 1.0, 1.0]), key_cache,
            value_cache, [0], [0.0], [1.0], spec,
        )
    assert info.value.kind == "InvalidScale"
    assert info.value.fields["value"] == 0.0
    assert np.array_equal(query, original) and np.array_equal(key, original)


# ---- the deterministic fixtures the reference runs against its GPU wrappers:
# crates/loom-cuda/src/attention_dispatch.rs:487-606 and
# crates/loom-cuda/src/rope_kv_dispatch.rs:596-741. Here they check the oracle
# against a float64 numpy evaluation written independently of it.
def _numpy_decode(query, key_cache, value_cache, tables, lengths, spec):
    q = query.reshape(spec.sequences, spec.query_heads, spec.head_size).astype(np.float64)
    k = key_cache.reshape(spec.num_blocks, spec.block_size, spec.kv_heads, spec.head_size)
    v = value_cache.reshape(spec.num_blocks, spec.block_size, spec.kv_heads, spec.value_head_size)
    tables = np.asarray(tables).reshape(spec.sequences, spec.max_blocks_per_sequence)
    out = np.zeros((spec.sequences, spec.query_heads, spec.value_head_size))
    group = spec.query_heads // spec.kv_heads
    for s in range(spec.sequences):
        tokens = np.arange(lengths[s])
        blocks = tables[s, tokens // spec.block_size]
        for h in range(spec.query_heads):
            keys = k[blocks, tokens % spec.block_size, h // group].astype(np.float64)
            values = v[blocks, tokens % spec.block_size, h // group].astype(np.float64)
            scores = keys @ q[s, h] * np.float64(np.float32(spec.scale))
            weights = np.exp(scores - scores.max())
            out[s, h] = weights @ values / weights.sum()
    return out.astype(np.float32).reshape(-1)


def test_decode_matches_independent_float64_on_the_wrapper_fixture():
    spec = ob.DecodeSpec(2, 4, 2, 4, 3, 4, 2, 2, 4, 0.5, ob.F32)
    query = f32([(i - 9.0) * 0.07 for i in range(2 * 4 * 4)])
    key_cache = f32([(np.float32(i) % np.float32(13.0) - 6.0) * 0.11 for i in range(4 * 2 * 2 * 4)])
    value_cache = f32([(np.float32(i) % np.float32(17.0) - 8.0) * 0.09 for i in range(4 * 2 * 2 * 3)])
    tables, lengths = [2, 0, 1, 3], [3, 2]
    output = np.zeros(2 * 4 * 3, dtype=np.float32)
    ob.paged_decode_attention(ob.F32, query, key_cache, value_cache, tables, lengths, output, spec)
    expected = _numpy_decode(query, key_cache, value_cache, tables, lengths, spec)
    assert np.allclose(output, expected, rtol=0, atol=1e-6)


def test_decode_matches_independent_float64_on_the_split_k_fixture():
    spec = ob.DecodeSpec(1, 4, 1, 128, 128, 8, 16, 8, 128, 0.125, ob.F32)
    query = f32([(i % 29 - 14.0) * 0.013 for i in range(4 * 128)])
    key_cache = f32([(i % 37 - 18.0) * 0.011 for i in range(8 * 16 * 128)])
    value_cache = f32([(i % 41 - 20.0) * 0.009 for i in range(8 * 16 * 128)])
    tables, lengths = list(range(8)), [128]
    output = np.zeros(4 * 128, dtype=np.float32)
    ob.paged_decode_attention(ob.F32, query, key_cache, value_cache, tables, lengths, output, spec)
    expected = _numpy_decode(query, key_cache, value_cache, tables, lengths, spec)
    assert np.allclose(output, expected, rtol=0, atol=1e-6)


def test_threaded_oracle_equals_the_single_threaded_loop():
    rng = np.random.default_rng(5)
    spec = ob.DecodeSpec(3, 8, 2, 32, 24, 16, 4, 5, 19, 0.2, ob.BF16)
    query = ob.f32_to_bf16(rng.standard_normal(3 * 8 * 32))
    key_cache = ob.f32_to_bf16(rng.standard_normal(16 * 4 * 2 * 32))
    value_cache = ob.f32_to_bf16(rng.standard_normal(16 * 4 * 2 * 24))
    tables = rng.permutation(16)[:15].reshape(3, 5)
    lengths = [19, 1, 7]
    single = np.zeros(3 * 8 * 24, dtype=np.uint16)
    threaded = np.zeros_like(single)
    ob.paged_decode_attention(ob.BF16, query, key_cache, value_cache, tables, lengths, single, spec, 1)
    ob.paged_decode_attention(ob.BF16, query, key_cache, value_cache, tables, lengths, threaded, spec, 4)
    assert np.array_equal(single, threaded)


def test_error_messages_follow_the_reference_wording():
    # contract.rs:163-303.
    with pytest.raises(ob.OracleError) as info:
        ob.check_decode_spec(ob.DecodeSpec(1, 3, 2, 4, 4, 1, 16, 1, 16, 0.5, ob.F16))
    assert info.value.message == "query head count 3 must be divisible by KV head count 2"
    with pytest.raises(ob.OracleError) as info:
        ob.check_decode_spec(ob.DecodeSpec(1, 2, 1, 4, 4, 1, 16, 1, 16, 0.0, ob.F16))
    assert info.value.message == "attention scale must be finite and positive, got 0"
    with pytest.raises(ob.OracleError) as info:
        ob.check_decode_spec(ob.DecodeSpec(1, 2, 1, 4, 4, 1, 16, 1, 17, 0.5, ob.F16))
    assert info.value.message == "maximum sequence length 17 exceeds block-table capacity 16"
    with pytest.raises(ob.OracleError) as info:
        ob.check_rotary_spec(ob.RotarySpec(1, 2, 1, 8, 3, 16, ob.F16, True))
    assert info.value.message == (
        "rotary dimension must be non-zero, even, and no larger than head size; "
        "got rotary_dim=3, head_size=8"
    )
    spec = ob.DecodeSpec(1, 1, 1, 1, 1, 1, 1, 1, 1, 1.0, ob.F32)
    with pytest.raises(ob.OracleError) as info:
        ob.paged_decode_attention(ob.F32, f32([1, 2]), f32([1]), f32([1]), [0], [1], f32([0]), spec)
    assert info.value.message == "query length mismatch: expected 1, got 2"
    with pytest.raises(ob.OracleError) as info:
        ob.paged_decode_attention(ob.F16, f32([1]), f32([1]), f32([1]), [0], [1], f32([0]), spec)
    assert info.value.message == "CPU reference does not support dtype F32"


def test_softmax_weights_use_the_f32_scale_widened_to_f64():
    # attention.rs:404-411 multiplies the F64 dot product by f64::from(scale).
    spec = ob.DecodeSpec(1, 1, 1, 1, 1, 1, 2, 1, 2, 1 / math.sqrt(128), ob.F32)
    output = np.zeros(1, dtype=np.float32)
    ob.paged_decode_attention(ob.F32, f32([3.0]), f32([1.0, -2.0]), f32([1.0, 5.0]), [0], [2], output, spec)
    scale = np.float64(np.float32(1 / math.sqrt(128)))
    weights = np.exp(np.array([3.0, -6.0]) * scale - 3.0 * scale)
    expected = np.float32((weights @ np.array([1.0, 5.0])) / weights.sum())
    assert output[0] == expected
