// Physical layouts and the error type of the safe dispatch layer.
//
// Equivalents of crates/loom-cuda/src/layout.rs (PagedDecodeLayout :107-198,
// RopePagedKvLayout :200-491, strided_span :23-41,
// validate_non_overlapping_layout :43-69) and of CudaExecutorError
// (crates/loom-cuda/src/lib.rs:41-48). A failed check throws ExecutorFailure;
// the bridge turns it into a status code and a last-error message, which is
// what the reference's `?` propagation plus bridge_call do.
#pragma once

#include <algorithm>
#include <cstdarg>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "contract.hpp"

namespace loom {

struct ExecutorFailure : std::exception {
  enum class Kind { InvalidContract, BackendUnavailable, KernelSubmission };
  Kind kind;
  int status = 0;
  std::string text;  // already formatted like the reference's Display impl

  ExecutorFailure(Kind kind_, int status_, std::string text_)
      : kind(kind_), status(status_), text(std::move(text_)) {}
  const char* what() const noexcept override { return text.c_str(); }
};

inline ExecutorFailure invalid(const std::string& message) {
  return ExecutorFailure(ExecutorFailure::Kind::InvalidContract, 0,
                         "invalid operator contract: " + message);
}

inline ExecutorFailure invalid(const ContractError& error) {
  return invalid(error.message);
}

inline ExecutorFailure submission(int status, const char* status_text) {
  return ExecutorFailure(
      ExecutorFailure::Kind::KernelSubmission, status,
      detail::format("CUDA kernel submission failed with status %d: %s", status,
                     status_text != nullptr ? status_text
                                            : "unknown Loom CUDA status"));
}

namespace layout_detail {

inline size_t add(size_t left, size_t right, const char* name) {
  size_t out;
  if (__builtin_add_overflow(left, right, &out)) {
    throw invalid(std::string(name) + " storage span overflows usize");
  }
  return out;
}

inline size_t mul(size_t left, size_t right, const char* name) {
  size_t out;
  if (__builtin_mul_overflow(left, right, &out)) {
    throw invalid(std::string(name) + " storage span overflows usize");
  }
  return out;
}

using Dimension = std::pair<size_t, size_t>;  // (size, element stride)

// Elements from the first to one past the last addressed element.
inline size_t strided_span(const std::vector<Dimension>& dimensions,
                           size_t contiguous_width, const char* name) {
  if (contiguous_width == 0) {
    throw invalid(std::string(name) + " contiguous width must be positive");
  }
  size_t span = contiguous_width;
  for (const Dimension& dimension : dimensions) {
    if (dimension.first == 0 || dimension.second == 0) {
      throw invalid(std::string(name) + " dimensions and strides must be positive");
    }
    span = add(span, mul(dimension.first - 1, dimension.second, name), name);
  }
  return span;
}

// Sorted by stride, every dimension must step over everything nested in it.
inline void require_non_overlapping(std::vector<Dimension> dimensions,
                                    size_t contiguous_width, const char* name) {
  dimensions.insert(dimensions.begin(), Dimension(contiguous_width, 1));
  std::stable_sort(dimensions.begin(), dimensions.end(),
                   [](const Dimension& a, const Dimension& b) {
                     return a.second < b.second;
                   });
  size_t occupied = 1;
  for (const Dimension& dimension : dimensions) {
    if (dimension.first == 0 || dimension.second == 0) {
      throw invalid(std::string(name) + " dimensions and strides must be positive");
    }
    if (dimension.first == 1) continue;
    if (dimension.second < occupied) {
      throw invalid(std::string(name) + " layout overlaps itself");
    }
    occupied = add(occupied, mul(dimension.first - 1, dimension.second, name), name);
  }
}

}  // namespace layout_detail

// Dense-inner NHD cache views with a free stride between blocks: the only
// freedom the reference's decode ABI has (layout.rs:107-198).
struct PagedDecodeLayout {
  size_t key_block_stride = 0, value_block_stride = 0;

  static PagedDecodeLayout create(const PagedDecodeAttentionSpec& spec,
                                  size_t key_block_stride,
                                  size_t value_block_stride) {
    size_t key_block = 0, value_block = 0;
    if (!block_elements(spec, spec.head_size, &key_block)) {
      throw invalid("paged key block size overflows usize");
    }
    if (!block_elements(spec, spec.value_head_size, &value_block)) {
      throw invalid("paged value block size overflows usize");
    }
    if (key_block_stride < key_block) {
      throw invalid("paged key block stride is smaller than one dense NHD block");
    }
    if (value_block_stride < value_block) {
      throw invalid("paged value block stride is smaller than one dense NHD block");
    }
    PagedDecodeLayout layout;
    layout.key_block_stride = key_block_stride;
    layout.value_block_stride = value_block_stride;
    return layout;
  }

  static PagedDecodeLayout contiguous(const PagedDecodeAttentionSpec& spec) {
    size_t key_block = 0, value_block = 0;
    if (!block_elements(spec, spec.head_size, &key_block)) {
      throw invalid("paged key block size overflows usize");
    }
    if (!block_elements(spec, spec.value_head_size, &value_block)) {
      throw invalid("paged value block size overflows usize");
    }
    return create(spec, key_block, value_block);
  }

  size_t key_storage_elements(const PagedDecodeAttentionSpec& spec) const {
    return layout_detail::add(
        layout_detail::mul(spec.num_blocks - 1, key_block_stride, "paged key cache"),
        spec.block_size * spec.kv_heads * spec.head_size, "paged key cache");
  }
  size_t value_storage_elements(const PagedDecodeAttentionSpec& spec) const {
    return layout_detail::add(
        layout_detail::mul(spec.num_blocks - 1, value_block_stride, "paged value cache"),
        spec.block_size * spec.kv_heads * spec.value_head_size, "paged value cache");
  }

 private:
  static bool block_elements(const PagedDecodeAttentionSpec& spec, size_t width,
                             size_t* out) {
    size_t partial = 0;
    return !__builtin_mul_overflow(spec.block_size, spec.kv_heads, &partial) &&
           !__builtin_mul_overflow(partial, width, out);
  }
};

// Addition: block, page and head strides all explicit, so HND caches and K/V
// views of one interleaved allocation can be read by the decode kernels. The
// checks are the ones RopePagedKvLayout applies to the same cache views.
struct StridedDecodeLayout {
  size_t key_block_stride = 0, key_page_stride = 0, key_head_stride = 0;
  size_t value_block_stride = 0, value_page_stride = 0, value_head_stride = 0;

  static StridedDecodeLayout create(const PagedDecodeAttentionSpec& spec,
                                    size_t key_block_stride, size_t key_page_stride,
                                    size_t key_head_stride, size_t value_block_stride,
                                    size_t value_page_stride, size_t value_head_stride) {
    layout_detail::require_non_overlapping(
        {{spec.num_blocks, key_block_stride},
         {spec.block_size, key_page_stride},
         {spec.kv_heads, key_head_stride}},
        spec.head_size, "paged key cache");
    layout_detail::require_non_overlapping(
        {{spec.num_blocks, value_block_stride},
         {spec.block_size, value_page_stride},
         {spec.kv_heads, value_head_stride}},
        spec.value_head_size, "paged value cache");
    StridedDecodeLayout layout;
    layout.key_block_stride = key_block_stride;
    layout.key_page_stride = key_page_stride;
    layout.key_head_stride = key_head_stride;
    layout.value_block_stride = value_block_stride;
    layout.value_page_stride = value_page_stride;
    layout.value_head_stride = value_head_stride;
    return layout;
  }

  static StridedDecodeLayout from_nhd(const PagedDecodeAttentionSpec& spec,
                                      const PagedDecodeLayout& dense) {
    StridedDecodeLayout layout;
    layout.key_block_stride = dense.key_block_stride;
    layout.key_page_stride = spec.kv_heads * spec.head_size;
    layout.key_head_stride = spec.head_size;
    layout.value_block_stride = dense.value_block_stride;
    layout.value_page_stride = spec.kv_heads * spec.value_head_size;
    layout.value_head_stride = spec.value_head_size;
    return layout;
  }

  size_t key_storage_elements(const PagedDecodeAttentionSpec& spec) const {
    return layout_detail::strided_span({{spec.num_blocks, key_block_stride},
                                        {spec.block_size, key_page_stride},
                                        {spec.kv_heads, key_head_stride}},
                                       spec.head_size, "paged key cache");
  }
  size_t value_storage_elements(const PagedDecodeAttentionSpec& spec) const {
    return layout_detail::strided_span({{spec.num_blocks, value_block_stride},
                                        {spec.block_size, value_page_stride},
                                        {spec.kv_heads, value_head_stride}},
                                       spec.value_head_size, "paged value cache");
  }
};

// Strides of the Q/K/V sources and of both cache views for the fused RoPE +
// paged-KV write (layout.rs:200-491).
struct RopePagedKvLayout {
  size_t cache_tokens = 0;
  size_t query_token_stride = 0, query_head_stride = 0;
  size_t key_token_stride = 0, source_key_head_stride = 0;
  size_t value_token_stride = 0, source_value_head_stride = 0;
  size_t key_block_stride = 0, key_page_stride = 0, key_head_stride = 0;
  size_t value_block_stride = 0, value_page_stride = 0, value_head_stride = 0;

  static RopePagedKvLayout create(
      const RopePagedKvWriteSpec& spec, size_t cache_tokens,
      size_t query_token_stride, size_t query_head_stride,
      size_t key_token_stride, size_t source_key_head_stride,
      size_t value_token_stride, size_t source_value_head_stride,
      size_t key_block_stride, size_t key_page_stride, size_t key_head_stride,
      size_t value_block_stride, size_t value_page_stride,
      size_t value_head_stride) {
    const RotaryEmbeddingSpec& rotary = spec.rotary;
    if (cache_tokens == 0 || cache_tokens > rotary.tokens) {
      throw invalid("RoPE+paged-KV cache token count must be in [1, tokens]");
    }
    using layout_detail::require_non_overlapping;
    require_non_overlapping({{rotary.tokens, query_token_stride},
                             {rotary.query_heads, query_head_stride}},
                            rotary.head_size, "RoPE query");
    require_non_overlapping({{rotary.tokens, key_token_stride},
                             {rotary.key_heads, source_key_head_stride}},
                            rotary.head_size, "RoPE key");
    require_non_overlapping({{rotary.tokens, value_token_stride},
                             {rotary.key_heads, source_value_head_stride}},
                            spec.value_head_size, "RoPE value");
    require_non_overlapping({{spec.num_blocks, key_block_stride},
                             {spec.block_size, key_page_stride},
                             {rotary.key_heads, key_head_stride}},
                            rotary.head_size, "paged key cache");
    require_non_overlapping({{spec.num_blocks, value_block_stride},
                             {spec.block_size, value_page_stride},
                             {rotary.key_heads, value_head_stride}},
                            spec.value_head_size, "paged value cache");
    RopePagedKvLayout layout;
    layout.cache_tokens = cache_tokens;
    layout.query_token_stride = query_token_stride;
    layout.query_head_stride = query_head_stride;
    layout.key_token_stride = key_token_stride;
    layout.source_key_head_stride = source_key_head_stride;
    layout.value_token_stride = value_token_stride;
    layout.source_value_head_stride = source_value_head_stride;
    layout.key_block_stride = key_block_stride;
    layout.key_page_stride = key_page_stride;
    layout.key_head_stride = key_head_stride;
    layout.value_block_stride = value_block_stride;
    layout.value_page_stride = value_page_stride;
    layout.value_head_stride = value_head_stride;
    return layout;
  }

  static RopePagedKvLayout contiguous(const RopePagedKvWriteSpec& spec) {
    const RotaryEmbeddingSpec& r = spec.rotary;
    return create(spec, r.tokens, r.query_heads * r.head_size, r.head_size,
                  r.key_heads * r.head_size, r.head_size,
                  r.key_heads * spec.value_head_size, spec.value_head_size,
                  spec.block_size * r.key_heads * r.head_size,
                  r.key_heads * r.head_size, r.head_size,
                  spec.block_size * r.key_heads * spec.value_head_size,
                  r.key_heads * spec.value_head_size, spec.value_head_size);
  }

  size_t key_block_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::strided_span({{spec.block_size, key_page_stride},
                                        {spec.rotary.key_heads, key_head_stride}},
                                       spec.rotary.head_size, "paged key cache block");
  }
  size_t value_block_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::strided_span({{spec.block_size, value_page_stride},
                                        {spec.rotary.key_heads, value_head_stride}},
                                       spec.value_head_size, "paged value cache block");
  }
  size_t query_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::strided_span({{spec.rotary.tokens, query_token_stride},
                                        {spec.rotary.query_heads, query_head_stride}},
                                       spec.rotary.head_size, "RoPE query");
  }
  size_t key_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::strided_span({{spec.rotary.tokens, key_token_stride},
                                        {spec.rotary.key_heads, source_key_head_stride}},
                                       spec.rotary.head_size, "RoPE key");
  }
  size_t value_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::strided_span({{spec.rotary.tokens, value_token_stride},
                                        {spec.rotary.key_heads, source_value_head_stride}},
                                       spec.value_head_size, "RoPE value");
  }
  size_t key_cache_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::add(
        layout_detail::mul(spec.num_blocks - 1, key_block_stride, "paged key cache"),
        key_block_storage_elements(spec), "paged key cache");
  }
  size_t value_cache_storage_elements(const RopePagedKvWriteSpec& spec) const {
    return layout_detail::add(
        layout_detail::mul(spec.num_blocks - 1, value_block_stride, "paged value cache"),
        value_block_storage_elements(spec), "paged value cache");
  }
};

}  // namespace loom
