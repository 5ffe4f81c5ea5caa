// Operator contracts of the paged-decode path, host side, header only.
//
// These are the B200 library's equivalents of the reference's contract types:
//   PagedDecodeAttentionSpec   crates/loom-kernels/src/attention.rs:16-166
//   RotaryEmbeddingSpec        crates/loom-kernels/src/rope_kv.rs:55-157
//   RopePagedKvWriteSpec       crates/loom-kernels/src/rope_kv.rs:168-251
//   KvCacheEncoding            crates/loom-kernels/src/rope_kv.rs:30-46
//   ContractError (+ wording)  crates/loom-kernels/src/contract.rs:79-303
// Construction validates in the same order and fails with the same wording,
// so a message that reaches a caller through the bridge reads the same.
#pragma once

#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <string>

namespace loom {

enum class DType : uint32_t { F32 = 0, F16 = 1, Bf16 = 2, Fp8E4M3Fn = 3 };

inline size_t size_in_bytes(DType dtype) {
  switch (dtype) {
    case DType::F32: return 4;
    case DType::F16:
    case DType::Bf16: return 2;
    default: return 1;
  }
}

inline const char* debug_name(DType dtype) {
  switch (dtype) {
    case DType::F32: return "F32";
    case DType::F16: return "F16";
    case DType::Bf16: return "Bf16";
    default: return "Fp8E4M3Fn";
  }
}

enum class RotaryStyle : uint32_t { Interleaved = 0, NeoX = 1 };

enum class KvCacheEncoding : uint32_t {
  Native = 0,
  Fp8E4M3FnPerTensor = 1,
  Fp8E4M3FnPerHead = 2,
};

inline bool is_fp8(KvCacheEncoding encoding) {
  return encoding != KvCacheEncoding::Native;
}

// Number of scale values one K or V cache needs (rope_kv.rs:39-45).
inline size_t scale_elements(KvCacheEncoding encoding, size_t kv_heads) {
  switch (encoding) {
    case KvCacheEncoding::Fp8E4M3FnPerTensor: return 1;
    case KvCacheEncoding::Fp8E4M3FnPerHead: return kv_heads;
    default: return 0;
  }
}

// A failed construction or validation. `message` is final user-facing text.
struct ContractError {
  bool failed = false;
  std::string message;

  static ContractError none() { return {}; }
  static ContractError make(std::string text) {
    ContractError error;
    error.failed = true;
    error.message = std::move(text);
    return error;
  }
  explicit operator bool() const { return failed; }
};

namespace detail {

inline std::string format(const char* pattern, ...) __attribute__((format(printf, 1, 2)));
inline std::string format(const char* pattern, ...) {
  char text[512];
  va_list arguments;
  va_start(arguments, pattern);
  std::vsnprintf(text, sizeof(text), pattern, arguments);
  va_end(arguments);
  return std::string(text);
}

// Shortest decimal text that reads back as the same float, without a trailing
// ".0": how the reference prints a scale inside its messages.
inline std::string shortest_float(float value) {
  if (std::isnan(value)) return "NaN";
  if (std::isinf(value)) return value < 0 ? "-inf" : "inf";
  char text[64];
  for (int precision = 1; precision <= 9; ++precision) {
    std::snprintf(text, sizeof(text), "%.*g", precision, (double)value);
    if (std::strtof(text, nullptr) == value) break;
  }
  return std::string(text);
}

inline bool mul_overflows(size_t left, size_t right, size_t* out) {
  return __builtin_mul_overflow(left, right, out);
}

inline bool product_fits(std::initializer_list<size_t> dimensions) {
  size_t product = 1;
  for (size_t dimension : dimensions) {
    if (mul_overflows(product, dimension, &product)) return false;
  }
  return true;
}

}  // namespace detail

namespace messages {
inline std::string zero_dimension() { return "tensor dimensions must be non-zero"; }
inline std::string overflow() { return "tensor element count overflowed"; }
inline std::string invalid_scale(float value) {
  return "attention scale must be finite and positive, got " +
         detail::shortest_float(value);
}
}  // namespace messages

// One decode query token per sequence over a block-paged K/V cache.
struct PagedDecodeAttentionSpec {
  size_t sequences = 0, query_heads = 0, kv_heads = 0;
  size_t head_size = 0, value_head_size = 0;
  size_t num_blocks = 0, block_size = 0;
  size_t max_blocks_per_sequence = 0, max_sequence_length = 0;
  float scale = 0.0f;
  DType dtype = DType::F32;

  static ContractError create(size_t sequences, size_t query_heads,
                              size_t kv_heads, size_t head_size,
                              size_t value_head_size, size_t num_blocks,
                              size_t block_size, size_t max_blocks_per_sequence,
                              size_t max_sequence_length, float scale,
                              DType dtype, PagedDecodeAttentionSpec* out) {
    if (sequences == 0 || query_heads == 0 || kv_heads == 0 || head_size == 0 ||
        value_head_size == 0 || num_blocks == 0 || block_size == 0 ||
        max_blocks_per_sequence == 0 || max_sequence_length == 0) {
      return ContractError::make(messages::zero_dimension());
    }
    if (query_heads % kv_heads != 0) {
      return ContractError::make(detail::format(
          "query head count %zu must be divisible by KV head count %zu",
          query_heads, kv_heads));
    }
    if (!std::isfinite(scale) || scale <= 0.0f) {
      return ContractError::make(messages::invalid_scale(scale));
    }
    if (!detail::product_fits({sequences, query_heads, head_size}) ||
        !detail::product_fits({sequences, query_heads, value_head_size}) ||
        !detail::product_fits({num_blocks, block_size, kv_heads, head_size}) ||
        !detail::product_fits({num_blocks, block_size, kv_heads, value_head_size}) ||
        !detail::product_fits({sequences, max_blocks_per_sequence})) {
      return ContractError::make(messages::overflow());
    }
    size_t table_capacity = 0;
    if (detail::mul_overflows(max_blocks_per_sequence, block_size, &table_capacity)) {
      return ContractError::make(messages::overflow());
    }
    if (max_sequence_length > table_capacity) {
      return ContractError::make(detail::format(
          "maximum sequence length %zu exceeds block-table capacity %zu",
          max_sequence_length, table_capacity));
    }
    out->sequences = sequences;
    out->query_heads = query_heads;
    out->kv_heads = kv_heads;
    out->head_size = head_size;
    out->value_head_size = value_head_size;
    out->num_blocks = num_blocks;
    out->block_size = block_size;
    out->max_blocks_per_sequence = max_blocks_per_sequence;
    out->max_sequence_length = max_sequence_length;
    out->scale = scale;
    out->dtype = dtype;
    return ContractError::none();
  }

  size_t queries_per_kv() const { return query_heads / kv_heads; }
  size_t query_numel() const { return sequences * query_heads * head_size; }
  size_t output_numel() const { return sequences * query_heads * value_head_size; }
  size_t key_cache_numel() const { return num_blocks * block_size * kv_heads * head_size; }
  size_t value_cache_numel() const { return num_blocks * block_size * kv_heads * value_head_size; }
  size_t block_table_numel() const { return sequences * max_blocks_per_sequence; }
};

// In-place rotary embedding of Q and K; cos_sin_cache is [max_position,
// rotary_dim] with the cosines in its first half.
struct RotaryEmbeddingSpec {
  size_t tokens = 0, query_heads = 0, key_heads = 0, head_size = 0;
  size_t rotary_dim = 0, max_position = 0;
  DType dtype = DType::F32;
  RotaryStyle style = RotaryStyle::NeoX;

  static ContractError create(size_t tokens, size_t query_heads, size_t key_heads,
                              size_t head_size, size_t rotary_dim,
                              size_t max_position, DType dtype, RotaryStyle style,
                              RotaryEmbeddingSpec* out) {
    if (tokens == 0 || query_heads == 0 || key_heads == 0 || head_size == 0 ||
        max_position == 0) {
      return ContractError::make(messages::zero_dimension());
    }
    if (rotary_dim == 0 || rotary_dim % 2 != 0 || rotary_dim > head_size) {
      return ContractError::make(detail::format(
          "rotary dimension must be non-zero, even, and no larger than head "
          "size; got rotary_dim=%zu, head_size=%zu",
          rotary_dim, head_size));
    }
    if (!detail::product_fits({tokens, query_heads, head_size}) ||
        !detail::product_fits({tokens, key_heads, head_size}) ||
        !detail::product_fits({max_position, rotary_dim})) {
      return ContractError::make(messages::overflow());
    }
    out->tokens = tokens;
    out->query_heads = query_heads;
    out->key_heads = key_heads;
    out->head_size = head_size;
    out->rotary_dim = rotary_dim;
    out->max_position = max_position;
    out->dtype = dtype;
    out->style = style;
    return ContractError::none();
  }

  size_t query_numel() const { return tokens * query_heads * head_size; }
  size_t key_numel() const { return tokens * key_heads * head_size; }
  size_t cos_sin_cache_numel() const { return max_position * rotary_dim; }
};

// Fused RoPE plus the paged write of the rotated K and of V.
struct RopePagedKvWriteSpec {
  RotaryEmbeddingSpec rotary;
  size_t value_head_size = 0, num_blocks = 0, block_size = 0;
  KvCacheEncoding cache_encoding = KvCacheEncoding::Native;

  static ContractError create(const RotaryEmbeddingSpec& rotary,
                              size_t value_head_size, size_t num_blocks,
                              size_t block_size, KvCacheEncoding cache_encoding,
                              RopePagedKvWriteSpec* out) {
    if (value_head_size == 0 || num_blocks == 0 || block_size == 0) {
      return ContractError::make(messages::zero_dimension());
    }
    if (!detail::product_fits({rotary.tokens, rotary.key_heads, value_head_size}) ||
        !detail::product_fits({num_blocks, block_size, rotary.key_heads, rotary.head_size}) ||
        !detail::product_fits({num_blocks, block_size, rotary.key_heads, value_head_size})) {
      return ContractError::make(messages::overflow());
    }
    out->rotary = rotary;
    out->value_head_size = value_head_size;
    out->num_blocks = num_blocks;
    out->block_size = block_size;
    out->cache_encoding = cache_encoding;
    return ContractError::none();
  }

  size_t scale_elements() const {
    return loom::scale_elements(cache_encoding, rotary.key_heads);
  }
  size_t slot_capacity() const { return num_blocks * block_size; }
  size_t value_numel() const { return rotary.tokens * rotary.key_heads * value_head_size; }
};

}  // namespace loom
