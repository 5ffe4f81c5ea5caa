// CPU oracle for the paged-decode hot path.
//
// TEST INFRASTRUCTURE ONLY: see loom_oracle.h. Each function names the place
// in the reference (path within the Loom Kernels project) that it restates.
// Build with -O2 -ffp-contract=off: the reference never fuses a multiply with
// an add, and the rotated K values must come out bit-identical.

#include "loom_oracle.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <unordered_map>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

using usize = uint64_t;

// ---------------------------------------------------------------- errors

int fail(oracle_error* error, int kind, int64_t a = 0, int64_t b = 0,
         int64_t c = 0, int64_t d = 0, float value = 0.0f,
         const char* buffer = "") {
  if (error != nullptr) {
    error->kind = kind;
    error->a = a;
    error->b = b;
    error->c = c;
    error->d = d;
    error->value = value;
    std::snprintf(error->buffer, sizeof(error->buffer), "%s", buffer);
  }
  return kind;
}

int ok(oracle_error* error) { return fail(error, ORACLE_OK); }

// contract.rs:321-335 (require_len).
int require_len(oracle_error* error, const char* buffer, usize actual,
                usize expected) {
  if (actual == expected) return ORACLE_OK;
  return fail(error, ORACLE_LENGTH_MISMATCH, (int64_t)expected, (int64_t)actual,
              0, 0, 0.0f, buffer);
}

bool checked_mul(usize left, usize right, usize* out) {
  return !__builtin_mul_overflow(left, right, out);
}

// attention.rs:428-435 (checked_product).
bool checked_product(std::initializer_list<usize> dimensions) {
  usize product = 1;
  for (usize dimension : dimensions) {
    if (!checked_mul(product, dimension, &product)) return false;
  }
  return true;
}

const char* dtype_name(int64_t dtype) {
  switch (dtype) {
    case ORACLE_F32: return "F32";
    case ORACLE_F16: return "F16";
    case ORACLE_BF16: return "Bf16";
    case ORACLE_FP8_E4M3FN: return "Fp8E4M3Fn";
    default: return "?";
  }
}

// Rust prints an f32 with `{}` as the shortest string that round-trips, and
// whole numbers without a trailing ".0". "%g" with nine digits is too long,
// so try increasing precision until the value round-trips.
void format_f32(float value, char* out, int capacity) {
  if (std::isnan(value)) {
    std::snprintf(out, capacity, "NaN");
    return;
  }
  if (std::isinf(value)) {
    std::snprintf(out, capacity, value < 0 ? "-inf" : "inf");
    return;
  }
  for (int precision = 1; precision <= 9; ++precision) {
    char text[64];
    std::snprintf(text, sizeof(text), "%.*g", precision, (double)value);
    float back = std::strtof(text, nullptr);
    if (back == value) {
      // Expand an exponent form only when Rust would not use one; the values
      // that reach this path in tests are small decimals and integers.
      if (std::strchr(text, 'e') == nullptr) {
        std::snprintf(out, capacity, "%s", text);
        return;
      }
      break;
    }
  }
  std::snprintf(out, capacity, "%.9g", (double)value);
}

// ------------------------------------------------- element conversions

uint32_t f32_bits(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  return bits;
}

float bits_f32(uint32_t bits) {
  float value;
  std::memcpy(&value, &bits, 4);
  return value;
}

// half::bf16::from_f32: quiet any NaN, otherwise round to nearest even.
uint16_t f32_to_bf16(float value) {
  const uint32_t bits = f32_bits(value);
  if ((bits & 0x7fffffffu) > 0x7f800000u) {
    return (uint16_t)((bits >> 16) | 0x0040u);
  }
  const uint32_t round_bit = 0x00008000u;
  if ((bits & round_bit) != 0 && (bits & (3u * round_bit - 1u)) != 0) {
    return (uint16_t)((bits >> 16) + 1u);
  }
  return (uint16_t)(bits >> 16);
}

float bf16_to_f32(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

// half::f16::from_f32: IEEE binary16, round to nearest even, gradual
// underflow, overflow to infinity.
uint16_t f32_to_f16(float value) {
  const uint32_t bits = f32_bits(value);
  const uint32_t sign = (bits >> 16) & 0x8000u;
  const uint32_t magnitude = bits & 0x7fffffffu;
  if (magnitude > 0x7f800000u) {  // NaN: keep the top mantissa bits, force quiet
    return (uint16_t)(sign | 0x7e00u | ((magnitude >> 13) & 0x03ffu));
  }
  if (magnitude == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
  const int32_t exponent = (int32_t)(magnitude >> 23) - 127;
  uint32_t mantissa = magnitude & 0x007fffffu;
  if (exponent > 15) return (uint16_t)(sign | 0x7c00u);
  if (exponent >= -14) {
    uint32_t half_bits = ((uint32_t)(exponent + 15) << 10) | (mantissa >> 13);
    const uint32_t remainder = mantissa & 0x1fffu;
    if (remainder > 0x1000u || (remainder == 0x1000u && (half_bits & 1u))) {
      ++half_bits;  // a carry into the exponent (and on to infinity) is correct
    }
    return (uint16_t)(sign | half_bits);
  }
  if (exponent < -25) return (uint16_t)sign;  // below half the smallest subnormal
  mantissa |= 0x00800000u;
  const int shift = -exponent - 14 + 13;  // 14..24
  uint32_t half_bits = mantissa >> shift;
  const uint32_t remainder = mantissa & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (remainder > halfway || (remainder == halfway && (half_bits & 1u))) {
    ++half_bits;
  }
  return (uint16_t)(sign | half_bits);
}

float f16_to_f32(uint16_t bits) {
  const uint32_t sign = ((uint32_t)bits & 0x8000u) << 16;
  const uint32_t exponent = (bits >> 10) & 0x1fu;
  const uint32_t mantissa = bits & 0x03ffu;
  if (exponent == 0x1fu) {
    return bits_f32(sign | 0x7f800000u | (mantissa << 13));
  }
  if (exponent == 0) {
    const float magnitude = std::ldexp((float)mantissa, -24);
    return (sign != 0) ? -magnitude : magnitude;
  }
  return bits_f32(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

struct F32 {
  using Storage = float;
  static constexpr int kDType = ORACLE_F32;
  static float to_f32(Storage value) { return value; }
  static Storage from_f32(float value) { return value; }
};

struct F16 {
  using Storage = uint16_t;
  static constexpr int kDType = ORACLE_F16;
  static float to_f32(Storage value) { return f16_to_f32(value); }
  static Storage from_f32(float value) { return f32_to_f16(value); }
};

struct Bf16 {
  using Storage = uint16_t;
  static constexpr int kDType = ORACLE_BF16;
  static float to_f32(Storage value) { return bf16_to_f32(value); }
  static Storage from_f32(float value) { return f32_to_bf16(value); }
};

// ------------------------------------------------------------------ FP8

// quantization.rs:13-28.
float fp8_to_f32(uint8_t bits) {
  const uint8_t magnitude = bits & 0x7f;
  const float sign = (bits & 0x80) == 0 ? 1.0f : -1.0f;
  if (magnitude == 0x7f) {
    return std::copysign(std::numeric_limits<float>::quiet_NaN(), sign);
  }
  const int exponent = magnitude >> 3;
  const int mantissa = magnitude & 0x07;
  float value;
  if (exponent == 0) {
    value = (float)mantissa * std::ldexp(1.0f, -9);
  } else {
    value = (1.0f + (float)mantissa / 8.0f) * std::ldexp(1.0f, exponent - 7);
  }
  return sign * value;
}

// quantization.rs:32-56: scan all finite codes for the nearest, ties to the
// even code, saturate at 448.
uint8_t fp8_from_f32_scan(float value) {
  const uint8_t sign = std::signbit(value) ? 0x80 : 0x00;
  if (std::isnan(value)) return sign | 0x7f;
  const float magnitude = std::fabs(value);
  if (magnitude >= 448.0f) return sign | 0x7e;
  uint8_t best_bits = 0;
  float best_distance = std::numeric_limits<float>::infinity();
  for (int candidate = 0; candidate <= 0x7e; ++candidate) {
    const float decoded = fp8_to_f32((uint8_t)candidate);
    const float distance = std::fabs(decoded - magnitude);
    if (distance < best_distance ||
        (distance == best_distance && (candidate & 1) == 0 &&
         (best_bits & 1) != 0)) {
      best_bits = (uint8_t)candidate;
      best_distance = distance;
    }
  }
  return sign | best_bits;
}

// The same mapping computed from the bit pattern: round the 23-bit mantissa to
// 3 bits (nearest even) in the normal range, to a multiple of 2^-9 below it.
uint8_t fp8_from_f32_direct(float value) {
  const uint32_t bits = f32_bits(value);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
  const uint32_t magnitude = bits & 0x7fffffffu;
  if (magnitude > 0x7f800000u) return sign | 0x7f;
  if (magnitude >= 0x43e00000u) return sign | 0x7e;  // >= 448
  const int32_t exponent = (int32_t)(magnitude >> 23) - 127;
  if (exponent >= -6) {
    uint32_t code = ((uint32_t)(exponent + 7) << 3) | ((magnitude >> 20) & 0x7u);
    const uint32_t remainder = magnitude & 0x000fffffu;
    if (remainder > 0x00080000u || (remainder == 0x00080000u && (code & 1u))) {
      ++code;
    }
    // 448 is the largest input that reaches here unrounded; anything that
    // rounds past 0x7e was >= 464 and has already been saturated above, but a
    // value in (448-16, 448) can round up to exactly 0x7e, which is finite.
    return sign | (uint8_t)(code > 0x7eu ? 0x7eu : code);
  }
  if (exponent < -10) {
    // Below 2^-10 the nearest code is 0 (2^-10 itself is the tie, to even 0).
    return sign;
  }
  // Subnormal target: units of 2^-9, value = m * 2^e with m in [1,2).
  const uint32_t mantissa = (magnitude & 0x007fffffu) | 0x00800000u;
  const int shift = 23 + (-9 - exponent);  // exponent -7 -> 21, ..., -10 -> 24
  uint32_t code = mantissa >> shift;
  const uint32_t remainder = mantissa & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (remainder > halfway || (remainder == halfway && (code & 1u))) ++code;
  return sign | (uint8_t)code;
}

// --------------------------------------------------------------- specs

// attention.rs:34-97.
int check_decode_spec(const oracle_decode_spec& s, oracle_error* error) {
  if (s.sequences == 0 || s.query_heads == 0 || s.kv_heads == 0 ||
      s.head_size == 0 || s.value_head_size == 0 || s.num_blocks == 0 ||
      s.block_size == 0 || s.max_blocks_per_sequence == 0 ||
      s.max_sequence_length == 0) {
    return fail(error, ORACLE_ZERO_DIMENSION);
  }
  if (s.query_heads % s.kv_heads != 0) {
    return fail(error, ORACLE_HEAD_COUNT_NOT_DIVISIBLE, (int64_t)s.query_heads,
                (int64_t)s.kv_heads);
  }
  if (!std::isfinite(s.scale) || s.scale <= 0.0f) {
    return fail(error, ORACLE_INVALID_SCALE, 0, 0, 0, 0, s.scale);
  }
  if (!checked_product({s.sequences, s.query_heads, s.head_size}) ||
      !checked_product({s.sequences, s.query_heads, s.value_head_size}) ||
      !checked_product({s.num_blocks, s.block_size, s.kv_heads, s.head_size}) ||
      !checked_product(
          {s.num_blocks, s.block_size, s.kv_heads, s.value_head_size}) ||
      !checked_product({s.sequences, s.max_blocks_per_sequence})) {
    return fail(error, ORACLE_ELEMENT_COUNT_OVERFLOW);
  }
  usize table_capacity = 0;
  if (!checked_mul(s.max_blocks_per_sequence, s.block_size, &table_capacity)) {
    return fail(error, ORACLE_ELEMENT_COUNT_OVERFLOW);
  }
  if (s.max_sequence_length > table_capacity) {
    return fail(error, ORACLE_MAX_SEQUENCE_LENGTH_OUT_OF_BOUNDS,
                (int64_t)s.max_sequence_length, (int64_t)table_capacity);
  }
  return ok(error);
}

// rope_kv.rs:69-112.
int check_rotary_spec(const oracle_rotary_spec& s, oracle_error* error) {
  if (s.tokens == 0 || s.query_heads == 0 || s.key_heads == 0 ||
      s.head_size == 0 || s.max_position == 0) {
    return fail(error, ORACLE_ZERO_DIMENSION);
  }
  if (s.rotary_dim == 0 || s.rotary_dim % 2 != 0 || s.rotary_dim > s.head_size) {
    return fail(error, ORACLE_INVALID_ROTARY_DIMENSION, (int64_t)s.rotary_dim,
                (int64_t)s.head_size);
  }
  if (!checked_product({s.tokens, s.query_heads, s.head_size}) ||
      !checked_product({s.tokens, s.key_heads, s.head_size}) ||
      !checked_product({s.max_position, s.rotary_dim})) {
    return fail(error, ORACLE_ELEMENT_COUNT_OVERFLOW);
  }
  return ok(error);
}

// rope_kv.rs:177-210.
int check_rope_kv_spec(const oracle_rope_kv_spec& s, oracle_error* error) {
  if (int status = check_rotary_spec(s.rotary, error)) return status;
  if (s.value_head_size == 0 || s.num_blocks == 0 || s.block_size == 0) {
    return fail(error, ORACLE_ZERO_DIMENSION);
  }
  if (!checked_product({s.rotary.tokens, s.rotary.key_heads, s.value_head_size}) ||
      !checked_product({s.num_blocks, s.block_size, s.rotary.key_heads,
                        s.rotary.head_size}) ||
      !checked_product({s.num_blocks, s.block_size, s.rotary.key_heads,
                        s.value_head_size})) {
    return fail(error, ORACLE_ELEMENT_COUNT_OVERFLOW);
  }
  return ok(error);
}

// rope_kv.rs:39-45.
usize scale_elements(int32_t encoding, usize kv_heads) {
  switch (encoding) {
    case ORACLE_CACHE_FP8_PER_TENSOR: return 1;
    case ORACLE_CACHE_FP8_PER_HEAD: return kv_heads;
    default: return 0;
  }
}

// ------------------------------------------------------------ attention

// attention.rs:359-402: every check that can fail runs before the output is
// touched.
int validate_decode_buffers(const oracle_decode_spec& s, int32_t call_dtype,
                            usize query_len, usize key_cache_len,
                            usize value_cache_len, const int64_t* block_tables,
                            usize block_tables_len,
                            const int64_t* sequence_lengths,
                            usize sequence_lengths_len, usize output_len,
                            oracle_error* error) {
  if (s.dtype != call_dtype) {
    return fail(error, ORACLE_UNSUPPORTED_DTYPE, s.dtype);
  }
  const usize query_numel = s.sequences * s.query_heads * s.head_size;
  const usize output_numel = s.sequences * s.query_heads * s.value_head_size;
  const usize key_numel = s.num_blocks * s.block_size * s.kv_heads * s.head_size;
  const usize value_numel =
      s.num_blocks * s.block_size * s.kv_heads * s.value_head_size;
  const usize table_numel = s.sequences * s.max_blocks_per_sequence;
  if (require_len(error, "query", query_len, query_numel) ||
      require_len(error, "key_cache", key_cache_len, key_numel) ||
      require_len(error, "value_cache", value_cache_len, value_numel) ||
      require_len(error, "block_tables", block_tables_len, table_numel) ||
      require_len(error, "sequence_lengths", sequence_lengths_len, s.sequences) ||
      require_len(error, "output", output_len, output_numel)) {
    return error != nullptr ? error->kind : ORACLE_LENGTH_MISMATCH;
  }
  for (usize sequence = 0; sequence < s.sequences; ++sequence) {
    const int64_t length = sequence_lengths[sequence];
    if (length <= 0 || (usize)length > s.max_sequence_length) {
      return fail(error, ORACLE_SEQUENCE_LENGTH_OUT_OF_BOUNDS, (int64_t)sequence,
                  length, (int64_t)s.max_sequence_length);
    }
    const usize active_blocks = ((usize)length + s.block_size - 1) / s.block_size;
    const usize table_offset = sequence * s.max_blocks_per_sequence;
    for (usize logical = 0; logical < active_blocks; ++logical) {
      const int64_t block_id = block_tables[table_offset + logical];
      if (block_id < 0 || (usize)block_id >= s.num_blocks) {
        return fail(error, ORACLE_BLOCK_ID_OUT_OF_BOUNDS, (int64_t)sequence,
                    (int64_t)logical, block_id, (int64_t)s.num_blocks);
      }
    }
  }
  return ok(error);
}

// attention.rs:413-426.
inline usize cache_offset(const oracle_decode_spec& s, usize sequence,
                          usize position, usize kv_head, usize head_size,
                          const int64_t* block_tables) {
  const usize logical_block = position / s.block_size;
  const usize block_offset = position % s.block_size;
  const usize table_offset = sequence * s.max_blocks_per_sequence;
  const usize physical_block = (usize)block_tables[table_offset + logical_block];
  return ((physical_block * s.block_size + block_offset) * s.kv_heads + kv_head) *
         head_size;
}

// Options beyond the reference's contract (its design note lists sliding windows
// and logits soft caps as later contract fields,
// docs/design/paged-decode-attention.md:42-52; parity unpinned). Process-wide,
// set by oracle_set_decode_options: with a window of W > 0 tokens a query only
// sees the last W positions of its sequence; with a cap c > 0 every scaled score
// s becomes c * tanh(s / c) before the softmax. Zero (the default) is the
// reference's arithmetic, untouched.
static uint64_t g_sliding_window = 0;
static double g_logits_soft_cap = 0.0;

// One (sequence, query head): attention.rs:294-353. `KeyAt`/`ValueAt` return
// the F32 value of a cache element given its NHD offset and KV head; for the
// native cache that is a plain widening.
template <typename Q, typename KeyAt, typename ValueAt>
void attend_one(const oracle_decode_spec& s, const typename Q::Storage* query,
                const int64_t* block_tables, usize sequence,
                usize sequence_length, usize query_head,
                typename Q::Storage* output, KeyAt key_at, ValueAt value_at) {
  const usize queries_per_kv = s.query_heads / s.kv_heads;
  const usize kv_head = query_head / queries_per_kv;
  const typename Q::Storage* q =
      query + (sequence * s.query_heads + query_head) * s.head_size;

  // attention.rs:404-411: F64 products summed left to right, scaled after.
  auto score = [&](usize key_offset) {
    double sum = 0.0;
    for (usize d = 0; d < s.head_size; ++d) {
      sum += (double)Q::to_f32(q[d]) * (double)key_at(key_offset + d, kv_head);
    }
    const double scaled = sum * (double)s.scale;
    return g_logits_soft_cap > 0.0 ? g_logits_soft_cap * std::tanh(scaled / g_logits_soft_cap) : scaled;
  };
  const usize first_position =
      (g_sliding_window > 0 && sequence_length > g_sliding_window) ? sequence_length - (usize)g_sliding_window : 0;

  double maximum = -std::numeric_limits<double>::infinity();
  for (usize position = first_position; position < sequence_length; ++position) {
    const usize key_offset =
        cache_offset(s, sequence, position, kv_head, s.head_size, block_tables);
    // f64::max ignores a NaN operand, as fmax does.
    maximum = std::fmax(maximum, score(key_offset));
  }

  double denominator = 0.0;
  std::vector<double> accumulator(s.value_head_size, 0.0);
  for (usize position = first_position; position < sequence_length; ++position) {
    const usize key_offset =
        cache_offset(s, sequence, position, kv_head, s.head_size, block_tables);
    const double weight = std::exp(score(key_offset) - maximum);
    denominator += weight;
    const usize value_offset = cache_offset(s, sequence, position, kv_head,
                                            s.value_head_size, block_tables);
    for (usize d = 0; d < s.value_head_size; ++d) {
      accumulator[d] += weight * (double)value_at(value_offset + d, kv_head);
    }
  }

  typename Q::Storage* out =
      output + (sequence * s.query_heads + query_head) * s.value_head_size;
  for (usize d = 0; d < s.value_head_size; ++d) {
    out[d] = Q::from_f32((float)(accumulator[d] / denominator));
  }
}

template <typename Q, typename KeyAt, typename ValueAt>
void attend_all(const oracle_decode_spec& s, const typename Q::Storage* query,
                const int64_t* block_tables, const int64_t* sequence_lengths,
                typename Q::Storage* output, int32_t threads, KeyAt key_at,
                ValueAt value_at) {
  const int64_t items = (int64_t)(s.sequences * s.query_heads);
  if (threads <= 1) {
    // attention.rs:292-294: sequences outermost, heads inside.
    for (int64_t item = 0; item < items; ++item) {
      const usize sequence = (usize)item / s.query_heads;
      const usize head = (usize)item % s.query_heads;
      attend_one<Q>(s, query, block_tables, sequence,
                    (usize)sequence_lengths[sequence], head, output, key_at,
                    value_at);
    }
    return;
  }
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
  for (int64_t item = 0; item < items; ++item) {
    const usize sequence = (usize)item / s.query_heads;
    const usize head = (usize)item % s.query_heads;
    attend_one<Q>(s, query, block_tables, sequence,
                  (usize)sequence_lengths[sequence], head, output, key_at,
                  value_at);
  }
}

template <typename Q>
int decode_native(const void* query, const void* key_cache,
                  const void* value_cache, const int64_t* block_tables,
                  const int64_t* sequence_lengths, void* output,
                  const oracle_decode_spec& s, int32_t threads) {
  using Storage = typename Q::Storage;
  const Storage* keys = static_cast<const Storage*>(key_cache);
  const Storage* values = static_cast<const Storage*>(value_cache);
  attend_all<Q>(
      s, static_cast<const Storage*>(query), block_tables, sequence_lengths,
      static_cast<Storage*>(output), threads,
      [keys](usize offset, usize) { return Q::to_f32(keys[offset]); },
      [values](usize offset, usize) { return Q::to_f32(values[offset]); });
  return ORACLE_OK;
}

template <typename Q>
int decode_fp8(const void* query, const uint8_t* key_cache,
               const uint8_t* value_cache, const float* key_scales,
               const float* value_scales, uint32_t scale_stride,
               const int64_t* block_tables, const int64_t* sequence_lengths,
               void* output, const oracle_decode_spec& s, int32_t threads) {
  using Storage = typename Q::Storage;
  attend_all<Q>(
      s, static_cast<const Storage*>(query), block_tables, sequence_lengths,
      static_cast<Storage*>(output), threads,
      [=](usize offset, usize head) {
        return fp8_to_f32(key_cache[offset]) * key_scales[head * scale_stride];
      },
      [=](usize offset, usize head) {
        return fp8_to_f32(value_cache[offset]) *
               value_scales[head * scale_stride];
      });
  return ORACLE_OK;
}

// ----------------------------------------------------------------- RoPE

// rope_kv.rs:669-698.
int validate_rotary_buffers(const oracle_rotary_spec& s, int32_t call_dtype,
                            usize query_len, usize key_len,
                            const int64_t* positions, usize positions_len,
                            usize cos_sin_len, oracle_error* error) {
  if (s.dtype != call_dtype) {
    return fail(error, ORACLE_UNSUPPORTED_DTYPE, s.dtype);
  }
  if (require_len(error, "query", query_len,
                  s.tokens * s.query_heads * s.head_size) ||
      require_len(error, "key", key_len, s.tokens * s.key_heads * s.head_size) ||
      require_len(error, "positions", positions_len, s.tokens) ||
      require_len(error, "cos_sin_cache", cos_sin_len,
                  s.max_position * s.rotary_dim)) {
    return error != nullptr ? error->kind : ORACLE_LENGTH_MISMATCH;
  }
  for (usize token = 0; token < s.tokens; ++token) {
    const int64_t position = positions[token];
    if (position < 0 || (usize)position >= s.max_position) {
      return fail(error, ORACLE_POSITION_OUT_OF_BOUNDS, (int64_t)token, position,
                  (int64_t)s.max_position);
    }
  }
  return ok(error);
}

// rope_kv.rs:700-724.
int validate_slot_mapping(const int64_t* slot_mapping, usize count,
                          usize slot_capacity, oracle_error* error) {
  std::unordered_map<usize, usize> owners;
  owners.reserve(count);
  for (usize token = 0; token < count; ++token) {
    const int64_t slot = slot_mapping[token];
    if (slot < 0) continue;
    if ((usize)slot >= slot_capacity) {
      return fail(error, ORACLE_SLOT_OUT_OF_BOUNDS, (int64_t)token, slot,
                  (int64_t)slot_capacity);
    }
    auto found = owners.find((usize)slot);
    if (found != owners.end()) {
      return fail(error, ORACLE_DUPLICATE_SLOT, (int64_t)found->second,
                  (int64_t)token, slot);
    }
    owners.emplace((usize)slot, token);
  }
  return ok(error);
}

// rope_kv.rs:633-652.
int validate_rope_kv_buffers(const oracle_rope_kv_spec& s, int32_t call_dtype,
                             usize query_len, usize key_len, usize value_len,
                             const int64_t* positions, usize positions_len,
                             usize cos_sin_len, usize key_cache_len,
                             usize value_cache_len, const int64_t* slot_mapping,
                             usize slot_mapping_len, oracle_error* error) {
  const oracle_rotary_spec& r = s.rotary;
  if (int status = validate_rotary_buffers(r, call_dtype, query_len, key_len,
                                           positions, positions_len, cos_sin_len,
                                           error)) {
    return status;
  }
  const usize slot_capacity = s.num_blocks * s.block_size;
  if (require_len(error, "value", value_len,
                  r.tokens * r.key_heads * s.value_head_size) ||
      require_len(error, "key_cache", key_cache_len,
                  slot_capacity * r.key_heads * r.head_size) ||
      require_len(error, "value_cache", value_cache_len,
                  slot_capacity * r.key_heads * s.value_head_size) ||
      require_len(error, "slot_mapping", slot_mapping_len, r.tokens)) {
    return error != nullptr ? error->kind : ORACLE_LENGTH_MISMATCH;
  }
  return validate_slot_mapping(slot_mapping, slot_mapping_len, slot_capacity,
                               error);
}

// rope_kv.rs:759-777. Four separate F32 roundings per output: two products,
// then a difference or a sum. -ffp-contract=off keeps them apart.
template <typename T>
void rotate_head(typename T::Storage* head, const typename T::Storage* cos_sin,
                 const oracle_rotary_spec& s) {
  const usize half = s.rotary_dim / 2;
  for (usize pair = 0; pair < half; ++pair) {
    const usize first_index = s.is_neox ? pair : pair * 2;
    const usize second_index = s.is_neox ? pair + half : pair * 2 + 1;
    const float first = T::to_f32(head[first_index]);
    const float second = T::to_f32(head[second_index]);
    const float cosine = T::to_f32(cos_sin[pair]);
    const float sine = T::to_f32(cos_sin[half + pair]);
    const float first_cos = first * cosine;
    const float second_sin = second * sine;
    const float second_cos = second * cosine;
    const float first_sin = first * sine;
    head[first_index] = T::from_f32(first_cos - second_sin);
    head[second_index] = T::from_f32(second_cos + first_sin);
  }
}

// rope_kv.rs:726-757.
template <typename T>
void apply_rotary(typename T::Storage* query, typename T::Storage* key,
                  const int64_t* positions, const typename T::Storage* cos_sin,
                  const oracle_rotary_spec& s) {
  for (usize token = 0; token < s.tokens; ++token) {
    const typename T::Storage* row = cos_sin + (usize)positions[token] * s.rotary_dim;
    for (usize head = 0; head < s.query_heads; ++head) {
      rotate_head<T>(query + (token * s.query_heads + head) * s.head_size, row, s);
    }
    for (usize head = 0; head < s.key_heads; ++head) {
      rotate_head<T>(key + (token * s.key_heads + head) * s.head_size, row, s);
    }
  }
}

// rope_kv.rs:513-562.
template <typename T>
void write_native(typename T::Storage* key, const typename T::Storage* value,
                  typename T::Storage* key_cache,
                  typename T::Storage* value_cache, const int64_t* slot_mapping,
                  const oracle_rope_kv_spec& s) {
  const oracle_rotary_spec& r = s.rotary;
  for (usize token = 0; token < r.tokens; ++token) {
    const int64_t slot = slot_mapping[token];
    if (slot < 0) continue;
    for (usize head = 0; head < r.key_heads; ++head) {
      std::memcpy(key_cache + ((usize)slot * r.key_heads + head) * r.head_size,
                  key + (token * r.key_heads + head) * r.head_size,
                  r.head_size * sizeof(typename T::Storage));
      std::memcpy(
          value_cache + ((usize)slot * r.key_heads + head) * s.value_head_size,
          value + (token * r.key_heads + head) * s.value_head_size,
          s.value_head_size * sizeof(typename T::Storage));
    }
  }
}

// rope_kv.rs:602-628: quantise the already-rounded K and the source V.
template <typename T>
void write_fp8(const typename T::Storage* key, const typename T::Storage* value,
               uint8_t* key_cache, uint8_t* value_cache,
               const int64_t* slot_mapping, const float* key_scales,
               const float* value_scales, const oracle_rope_kv_spec& s) {
  const oracle_rotary_spec& r = s.rotary;
  for (usize token = 0; token < r.tokens; ++token) {
    const int64_t slot = slot_mapping[token];
    if (slot < 0) continue;
    for (usize head = 0; head < r.key_heads; ++head) {
      const usize scale_index =
          s.cache_encoding == ORACLE_CACHE_FP8_PER_HEAD ? head : 0;
      const float key_scale = key_scales[scale_index];
      const float value_scale = value_scales[scale_index];
      const usize source_key = (token * r.key_heads + head) * r.head_size;
      const usize target_key = ((usize)slot * r.key_heads + head) * r.head_size;
      for (usize d = 0; d < r.head_size; ++d) {
        key_cache[target_key + d] =
            fp8_from_f32_scan(T::to_f32(key[source_key + d]) / key_scale);
      }
      const usize source_value = (token * r.key_heads + head) * s.value_head_size;
      const usize target_value =
          ((usize)slot * r.key_heads + head) * s.value_head_size;
      for (usize d = 0; d < s.value_head_size; ++d) {
        value_cache[target_value + d] =
            fp8_from_f32_scan(T::to_f32(value[source_value + d]) / value_scale);
      }
    }
  }
}

template <typename F>
int by_dtype(int32_t dtype, oracle_error* error, F&& body) {
  switch (dtype) {
    case ORACLE_F32: return body(F32{});
    case ORACLE_F16: return body(F16{});
    case ORACLE_BF16: return body(Bf16{});
    default: return fail(error, ORACLE_UNSUPPORTED_DTYPE, dtype);
  }
}

}  // namespace

// ================================================================ C ABI

extern "C" {

int oracle_error_message(const oracle_error* e, char* out, int capacity) {
  if (e == nullptr || out == nullptr || capacity <= 0) return 0;
  char number[64];
  switch (e->kind) {
    case ORACLE_OK:
      return std::snprintf(out, capacity, "ok");
    case ORACLE_ZERO_DIMENSION:
      return std::snprintf(out, capacity, "tensor dimensions must be non-zero");
    case ORACLE_ELEMENT_COUNT_OVERFLOW:
      return std::snprintf(out, capacity, "tensor element count overflowed");
    case ORACLE_INVALID_ROTARY_DIMENSION:
      return std::snprintf(
          out, capacity,
          "rotary dimension must be non-zero, even, and no larger than head "
          "size; got rotary_dim=%lld, head_size=%lld",
          (long long)e->a, (long long)e->b);
    case ORACLE_POSITION_OUT_OF_BOUNDS:
      return std::snprintf(out, capacity,
                           "position %lld for token %lld is outside [0, %lld)",
                           (long long)e->b, (long long)e->a, (long long)e->c);
    case ORACLE_SLOT_OUT_OF_BOUNDS:
      return std::snprintf(out, capacity,
                           "cache slot %lld for token %lld is outside [0, %lld)",
                           (long long)e->b, (long long)e->a, (long long)e->c);
    case ORACLE_DUPLICATE_SLOT:
      return std::snprintf(
          out, capacity,
          "cache slot %lld is assigned to both token %lld and token %lld",
          (long long)e->c, (long long)e->a, (long long)e->b);
    case ORACLE_INVALID_SCALE:
      format_f32(e->value, number, sizeof(number));
      return std::snprintf(
          out, capacity, "attention scale must be finite and positive, got %s",
          number);
    case ORACLE_HEAD_COUNT_NOT_DIVISIBLE:
      return std::snprintf(
          out, capacity,
          "query head count %lld must be divisible by KV head count %lld",
          (long long)e->a, (long long)e->b);
    case ORACLE_SEQUENCE_LENGTH_OUT_OF_BOUNDS:
      return std::snprintf(
          out, capacity,
          "sequence length %lld for sequence %lld is outside [1, %lld]",
          (long long)e->b, (long long)e->a, (long long)e->c);
    case ORACLE_MAX_SEQUENCE_LENGTH_OUT_OF_BOUNDS:
      return std::snprintf(
          out, capacity,
          "maximum sequence length %lld exceeds block-table capacity %lld",
          (long long)e->a, (long long)e->b);
    case ORACLE_BLOCK_ID_OUT_OF_BOUNDS:
      return std::snprintf(out, capacity,
                           "physical block ID %lld for sequence %lld, logical "
                           "block %lld is outside [0, %lld)",
                           (long long)e->c, (long long)e->a, (long long)e->b,
                           (long long)e->d);
    case ORACLE_LENGTH_MISMATCH:
      return std::snprintf(out, capacity,
                           "%s length mismatch: expected %lld, got %lld",
                           e->buffer, (long long)e->a, (long long)e->b);
    case ORACLE_UNSUPPORTED_DTYPE:
      return std::snprintf(out, capacity,
                           "CPU reference does not support dtype %s",
                           dtype_name(e->a));
    default:
      return std::snprintf(out, capacity, "unknown oracle error %d", e->kind);
  }
}

uint16_t oracle_f32_to_bf16(float value) { return f32_to_bf16(value); }
float oracle_bf16_to_f32(uint16_t bits) { return bf16_to_f32(bits); }
uint16_t oracle_f32_to_f16(float value) { return f32_to_f16(value); }
float oracle_f16_to_f32(uint16_t bits) { return f16_to_f32(bits); }

void oracle_f32_to_bf16_n(const float* in, uint16_t* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
void oracle_bf16_to_f32_n(const uint16_t* in, float* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}
void oracle_f32_to_f16_n(const float* in, uint16_t* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = f32_to_f16(in[i]);
}
void oracle_f16_to_f32_n(const uint16_t* in, float* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = f16_to_f32(in[i]);
}

float oracle_fp8_e4m3fn_to_f32(uint8_t bits) { return fp8_to_f32(bits); }
uint8_t oracle_fp8_e4m3fn_from_f32(float value) { return fp8_from_f32_scan(value); }
uint8_t oracle_fp8_e4m3fn_from_f32_direct(float value) {
  return fp8_from_f32_direct(value);
}
void oracle_fp8_e4m3fn_from_f32_n(const float* in, uint8_t* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = fp8_from_f32_scan(in[i]);
}
void oracle_fp8_e4m3fn_to_f32_n(const uint8_t* in, float* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = fp8_to_f32(in[i]);
}

int oracle_decode_spec_check(const oracle_decode_spec* spec, oracle_error* error) {
  return check_decode_spec(*spec, error);
}
int oracle_rotary_spec_check(const oracle_rotary_spec* spec, oracle_error* error) {
  return check_rotary_spec(*spec, error);
}
int oracle_rope_kv_spec_check(const oracle_rope_kv_spec* spec,
                              oracle_error* error) {
  return check_rope_kv_spec(*spec, error);
}

int oracle_set_decode_options(uint64_t sliding_window, double logits_soft_cap) {
  if (!(logits_soft_cap >= 0.0) || !std::isfinite(logits_soft_cap)) return 1;
  g_sliding_window = sliding_window;
  g_logits_soft_cap = logits_soft_cap;
  return 0;
}

int oracle_paged_decode_attention(
    int32_t call_dtype, const void* query, uint64_t query_len,
    const void* key_cache, uint64_t key_cache_len, const void* value_cache,
    uint64_t value_cache_len, const int64_t* block_tables,
    uint64_t block_tables_len, const int64_t* sequence_lengths,
    uint64_t sequence_lengths_len, void* output, uint64_t output_len,
    const oracle_decode_spec* spec, int32_t threads, oracle_error* error) {
  if (int status = check_decode_spec(*spec, error)) return status;
  if (int status = validate_decode_buffers(
          *spec, call_dtype, query_len, key_cache_len, value_cache_len,
          block_tables, block_tables_len, sequence_lengths, sequence_lengths_len,
          output_len, error)) {
    return status;
  }
  return by_dtype(call_dtype, error, [&](auto tag) {
    using Q = decltype(tag);
    return decode_native<Q>(query, key_cache, value_cache, block_tables,
                            sequence_lengths, output, *spec, threads);
  });
}

int oracle_paged_decode_attention_fp8(
    int32_t call_dtype, const void* query, uint64_t query_len,
    const uint8_t* key_cache, uint64_t key_cache_len,
    const uint8_t* value_cache, uint64_t value_cache_len,
    const float* key_scales, const float* value_scales, uint32_t scale_stride,
    const int64_t* block_tables, uint64_t block_tables_len,
    const int64_t* sequence_lengths, uint64_t sequence_lengths_len,
    void* output, uint64_t output_len, const oracle_decode_spec* spec,
    int32_t threads, oracle_error* error) {
  if (int status = check_decode_spec(*spec, error)) return status;
  if (int status = validate_decode_buffers(
          *spec, call_dtype, query_len, key_cache_len, value_cache_len,
          block_tables, block_tables_len, sequence_lengths, sequence_lengths_len,
          output_len, error)) {
    return status;
  }
  const uint64_t scales = scale_stride == 0 ? 1 : spec->kv_heads;
  for (uint64_t i = 0; i < scales; ++i) {
    for (float scale : {key_scales[i], value_scales[i]}) {
      if (!std::isfinite(scale) || scale <= 0.0f) {
        return fail(error, ORACLE_INVALID_SCALE, 0, 0, 0, 0, scale);
      }
    }
  }
  return by_dtype(call_dtype, error, [&](auto tag) {
    using Q = decltype(tag);
    return decode_fp8<Q>(query, key_cache, value_cache, key_scales, value_scales,
                         scale_stride, block_tables, sequence_lengths, output,
                         *spec, threads);
  });
}

int oracle_rotary_embedding(int32_t call_dtype, void* query, uint64_t query_len,
                            void* key, uint64_t key_len,
                            const int64_t* positions, uint64_t positions_len,
                            const void* cos_sin_cache, uint64_t cos_sin_len,
                            const oracle_rotary_spec* spec, oracle_error* error) {
  if (int status = check_rotary_spec(*spec, error)) return status;
  if (int status =
          validate_rotary_buffers(*spec, call_dtype, query_len, key_len,
                                  positions, positions_len, cos_sin_len, error)) {
    return status;
  }
  return by_dtype(call_dtype, error, [&](auto tag) {
    using T = decltype(tag);
    using Storage = typename T::Storage;
    apply_rotary<T>(static_cast<Storage*>(query), static_cast<Storage*>(key),
                    positions, static_cast<const Storage*>(cos_sin_cache), *spec);
    return (int)ORACLE_OK;
  });
}

int oracle_rope_paged_kv_write(
    int32_t call_dtype, void* query, uint64_t query_len, void* key,
    uint64_t key_len, const void* value, uint64_t value_len,
    const int64_t* positions, uint64_t positions_len,
    const void* cos_sin_cache, uint64_t cos_sin_len, void* key_cache,
    uint64_t key_cache_len, void* value_cache, uint64_t value_cache_len,
    const int64_t* slot_mapping, uint64_t slot_mapping_len,
    const oracle_rope_kv_spec* spec, oracle_error* error) {
  if (int status = check_rope_kv_spec(*spec, error)) return status;
  // rope_kv.rs:525-527.
  if (spec->cache_encoding != ORACLE_CACHE_NATIVE) {
    return fail(error, ORACLE_UNSUPPORTED_DTYPE, ORACLE_FP8_E4M3FN);
  }
  if (int status = validate_rope_kv_buffers(
          *spec, call_dtype, query_len, key_len, value_len, positions,
          positions_len, cos_sin_len, key_cache_len, value_cache_len,
          slot_mapping, slot_mapping_len, error)) {
    return status;
  }
  return by_dtype(call_dtype, error, [&](auto tag) {
    using T = decltype(tag);
    using Storage = typename T::Storage;
    apply_rotary<T>(static_cast<Storage*>(query), static_cast<Storage*>(key),
                    positions, static_cast<const Storage*>(cos_sin_cache),
                    spec->rotary);
    write_native<T>(static_cast<Storage*>(key),
                    static_cast<const Storage*>(value),
                    static_cast<Storage*>(key_cache),
                    static_cast<Storage*>(value_cache), slot_mapping, *spec);
    return (int)ORACLE_OK;
  });
}

int oracle_rope_paged_kv_write_fp8(
    int32_t call_dtype, void* query, uint64_t query_len, void* key,
    uint64_t key_len, const void* value, uint64_t value_len,
    const int64_t* positions, uint64_t positions_len,
    const void* cos_sin_cache, uint64_t cos_sin_len, uint8_t* key_cache,
    uint64_t key_cache_len, uint8_t* value_cache, uint64_t value_cache_len,
    const int64_t* slot_mapping, uint64_t slot_mapping_len,
    const float* key_scales, uint64_t key_scales_len,
    const float* value_scales, uint64_t value_scales_len,
    const oracle_rope_kv_spec* spec, oracle_error* error) {
  if (int status = check_rope_kv_spec(*spec, error)) return status;
  // rope_kv.rs:579-584.
  if (spec->cache_encoding == ORACLE_CACHE_NATIVE) {
    return fail(error, ORACLE_UNSUPPORTED_DTYPE, spec->rotary.dtype);
  }
  if (int status = validate_rope_kv_buffers(
          *spec, call_dtype, query_len, key_len, value_len, positions,
          positions_len, cos_sin_len, key_cache_len, value_cache_len,
          slot_mapping, slot_mapping_len, error)) {
    return status;
  }
  // rope_kv.rs:654-667.
  const uint64_t expected_scales =
      scale_elements(spec->cache_encoding, spec->rotary.key_heads);
  if (require_len(error, "key_scales", key_scales_len, expected_scales) ||
      require_len(error, "value_scales", value_scales_len, expected_scales)) {
    return error != nullptr ? error->kind : ORACLE_LENGTH_MISMATCH;
  }
  for (uint64_t i = 0; i < key_scales_len; ++i) {
    if (!std::isfinite(key_scales[i]) || key_scales[i] <= 0.0f) {
      return fail(error, ORACLE_INVALID_SCALE, 0, 0, 0, 0, key_scales[i]);
    }
  }
  for (uint64_t i = 0; i < value_scales_len; ++i) {
    if (!std::isfinite(value_scales[i]) || value_scales[i] <= 0.0f) {
      return fail(error, ORACLE_INVALID_SCALE, 0, 0, 0, 0, value_scales[i]);
    }
  }
  return by_dtype(call_dtype, error, [&](auto tag) {
    using T = decltype(tag);
    using Storage = typename T::Storage;
    apply_rotary<T>(static_cast<Storage*>(query), static_cast<Storage*>(key),
                    positions, static_cast<const Storage*>(cos_sin_cache),
                    spec->rotary);
    write_fp8<T>(static_cast<const Storage*>(key),
                 static_cast<const Storage*>(value), key_cache, value_cache,
                 slot_mapping, key_scales, value_scales, *spec);
    return (int)ORACLE_OK;
  });
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
