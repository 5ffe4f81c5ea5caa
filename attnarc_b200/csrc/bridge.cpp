// Checked bridge: the C ABI that framework dispatchers call.
//
// The library's equivalent of the reference's bridge crate for this path:
//   crates/loom-cuda-bridge/src/cuda/mod.rs           (ranges, overlap rules,
//                                                      last error, counters,
//                                                      panic containment)
//   crates/loom-cuda-bridge/src/cuda/attention_bridge.rs
//   crates/loom-cuda-bridge/src/cuda/rope_kv_bridge.rs
// It validates every pointer/length pair and the aliasing rules, builds the
// contract and layout, and only then calls the safe dispatch layer. Checks run
// in the reference's order and fail with its wording.

#include "../../include/loom_bridge.h"
#include "../../include/loom_launch.h"

#include <atomic>
#include <cstdint>
#include <exception>
#include <functional>
#include <optional>
#include <string>
#include <vector>

#include "dispatch.hpp"

namespace {

using loom::DType;
using loom::ExecutorFailure;
using loom::invalid;
using loom::Region;
using loom::detail::format;

constexpr int kOperatorCount = 11;
std::atomic<uint64_t> g_launch_counts[kOperatorCount];
std::atomic<uint64_t> g_block_movement_launches{0};  // outside the reference's operator ids

thread_local std::string g_last_error = "no bridge error has been recorded";

void set_last_error(const std::string& message) {
  g_last_error.clear();
  for (char c : message) {
    if (c == '\0') g_last_error += "\\0";
    else g_last_error += c;
  }
}

void record_launch(int operation) { g_launch_counts[operation].fetch_add(1, std::memory_order_relaxed); }

int error_status(const ExecutorFailure& failure) {
  switch (failure.kind) {
    case ExecutorFailure::Kind::InvalidContract: return LOOM_CUDA_BRIDGE_INVALID_ARGUMENT;
    case ExecutorFailure::Kind::BackendUnavailable: return LOOM_CUDA_BRIDGE_UNAVAILABLE;
    default: return LOOM_CUDA_BRIDGE_LAUNCH_ERROR;
  }
}

// Nothing thrown below may cross the C boundary (mod.rs:696-708).
template <typename Body>
int bridge_call(Body&& body) noexcept {
  try {
    body();
    return LOOM_CUDA_BRIDGE_SUCCESS;
  } catch (const ExecutorFailure& failure) {
    set_last_error(failure.text);
    return error_status(failure);
  } catch (const std::exception& error) {
    set_last_error(std::string("C++ exception was contained at the Loom CUDA bridge: ") + error.what());
    return LOOM_CUDA_BRIDGE_LAUNCH_ERROR;
  } catch (...) {
    set_last_error("C++ exception was contained at the Loom CUDA bridge");
    return LOOM_CUDA_BRIDGE_LAUNCH_ERROR;
  }
}

struct ByteRange {
  uintptr_t start = 0, end = 0;
};

bool ranges_overlap(ByteRange left, ByteRange right) { return left.start < right.end && right.start < left.end; }

// mod.rs:88-117.
ByteRange checked_byte_range(const void* pointer, uint64_t elements, size_t element_size, const char* name) {
  if (pointer == nullptr) throw invalid(format("%s pointer is null", name));
  if (elements == 0) throw invalid(format("%s region is empty", name));
  const uintptr_t start = reinterpret_cast<uintptr_t>(pointer);
  if (start % element_size != 0) {
    throw invalid(format("%s pointer is not aligned to %zu bytes", name, element_size));
  }
  size_t bytes = 0;
  if (__builtin_mul_overflow((size_t)elements, element_size, &bytes)) {
    throw invalid(format("%s byte size overflows usize", name));
  }
  uintptr_t end = 0;
  if (__builtin_add_overflow(start, (uintptr_t)bytes, &end)) {
    throw invalid(format("%s address range overflows usize", name));
  }
  return ByteRange{start, end};
}

struct Checked {
  Region region;
  ByteRange range;
};

Checked borrow(const void* pointer, uint64_t elements, size_t element_size, const char* name) {
  Checked out;
  out.range = checked_byte_range(pointer, elements, element_size, name);
  out.region.pointer = pointer;
  out.region.elements = (size_t)elements;
  return out;
}

using Named = std::pair<const char*, ByteRange>;

// mod.rs:139-153.
void require_disjoint_from(const char* target_name, ByteRange target, const std::vector<Named>& others,
                           const char* operation) {
  for (const Named& other : others) {
    if (ranges_overlap(target, other.second)) {
      throw invalid(format("%s regions %s and %s must not overlap", operation, target_name, other.first));
    }
  }
}

// mod.rs:156-233: two views of one packed allocation may overlap in their
// bounding spans if their rows are dense, share the outer stride, and sit side
// by side inside every row.
void require_disjoint_or_dense_packed_axis(size_t element_size, const char* left_name, ByteRange left,
                                           size_t left_outer_stride, std::optional<size_t> left_inner,
                                           const char* right_name, ByteRange right,
                                           size_t right_outer_stride, std::optional<size_t> right_inner,
                                           const char* operation) {
  if (!ranges_overlap(left, right)) return;
  if (!left_inner || !right_inner) {
    throw invalid(format("%s regions %s and %s overlap without a dense packed layout", operation,
                         left_name, right_name));
  }
  if (left_outer_stride != right_outer_stride) {
    throw invalid(format("%s packed regions %s and %s must share an outer stride", operation, left_name,
                         right_name));
  }
  size_t outer_bytes = 0, left_bytes = 0, right_bytes = 0;
  if (__builtin_mul_overflow(left_outer_stride, element_size, &outer_bytes)) {
    throw invalid(format("%s packed outer stride overflows usize", operation));
  }
  if (__builtin_mul_overflow(*left_inner, element_size, &left_bytes)) {
    throw invalid(format("%s %s packed inner span overflows usize", operation, left_name));
  }
  if (__builtin_mul_overflow(*right_inner, element_size, &right_bytes)) {
    throw invalid(format("%s %s packed inner span overflows usize", operation, right_name));
  }
  const bool left_first = left.start <= right.start;
  const char* earlier_name = left_first ? left_name : right_name;
  const char* later_name = left_first ? right_name : left_name;
  const ByteRange earlier = left_first ? left : right;
  const ByteRange later = left_first ? right : left;
  const size_t earlier_bytes = left_first ? left_bytes : right_bytes;
  const size_t later_bytes = left_first ? right_bytes : left_bytes;
  const size_t offset = later.start - earlier.start;
  size_t later_end = 0;
  if (__builtin_add_overflow(offset, later_bytes, &later_end)) {
    throw invalid(format("%s packed inner span overflows usize", operation));
  }
  if (offset >= outer_bytes || earlier_bytes > offset || later_end > outer_bytes) {
    throw invalid(format("%s logical elements in packed regions %s and %s overlap", operation,
                         earlier_name, later_name));
  }
}

DType scalar_kind(uint32_t dtype) {
  switch (dtype) {
    case LOOM_CUDA_BRIDGE_F32: return DType::F32;
    case LOOM_CUDA_BRIDGE_F16: return DType::F16;
    case LOOM_CUDA_BRIDGE_BF16: return DType::Bf16;
    default: throw invalid(format("unknown bridge dtype code %u", dtype));
  }
}

loom::PagedDecodeAttentionSpec decode_spec(DType dtype, uint32_t sequences, uint32_t query_heads,
                                           uint32_t kv_heads, uint32_t head_size, uint32_t value_head_size,
                                           uint32_t num_blocks, uint32_t block_size,
                                           uint32_t max_blocks_per_sequence, uint32_t max_sequence_length,
                                           float scale) {
  loom::PagedDecodeAttentionSpec spec;
  if (auto error = loom::PagedDecodeAttentionSpec::create(sequences, query_heads, kv_heads, head_size,
                                                          value_head_size, num_blocks, block_size,
                                                          max_blocks_per_sequence, max_sequence_length,
                                                          scale, dtype, &spec)) {
    throw invalid(error);
  }
  return spec;
}

int unavailable(const char* operation) {
  set_last_error(std::string("invalid operator contract: ") + operation +
                 " is outside the paged-decode library; link the operator's own provider");
  return LOOM_CUDA_BRIDGE_UNAVAILABLE;
}

int checked_operation(uint32_t operation) {
  if (operation >= (uint32_t)kOperatorCount) throw invalid(format("unknown bridge operator code %u", operation));
  return (int)operation;
}

}  // namespace

extern "C" {

uint32_t loom_cuda_bridge_abi_version(void) { return 2; }

const char* loom_cuda_bridge_last_error_message(void) { return g_last_error.c_str(); }

int loom_cuda_bridge_launch_count(uint32_t operation, uint64_t* count) {
  return bridge_call([&] {
    const int index = checked_operation(operation);
    if (count == nullptr || reinterpret_cast<uintptr_t>(count) % alignof(uint64_t) != 0) {
      throw invalid("launch-count output pointer is null or misaligned");
    }
    *count = g_launch_counts[index].load(std::memory_order_relaxed);
  });
}

int loom_cuda_bridge_reset_launch_count(uint32_t operation) {
  return bridge_call([&] { g_launch_counts[checked_operation(operation)].store(0, std::memory_order_relaxed); });
}

// ------------------------------------------------------------------ decode

int loom_cuda_bridge_paged_decode_workspace_elements(
    uint32_t dtype, uint32_t sequences, uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size, uint32_t max_blocks_per_sequence,
    uint32_t max_sequence_length, float scale, uint64_t* workspace_elements) {
  return bridge_call([&] {
    if (workspace_elements == nullptr ||
        reinterpret_cast<uintptr_t>(workspace_elements) % alignof(uint64_t) != 0) {
      throw invalid("workspace-size output pointer is null or misaligned");
    }
    const auto spec = decode_spec(scalar_kind(dtype), sequences, query_heads, kv_heads, head_size,
                                  value_head_size, num_blocks, block_size, max_blocks_per_sequence,
                                  max_sequence_length, scale);
    *workspace_elements = loom::paged_decode_attention_split_k_workspace_elements(spec).value_or(0);
  });
}

int loom_cuda_bridge_paged_decode_attention(
    uint32_t dtype, const void* query, uint64_t query_elements, const void* key_cache,
    uint64_t key_cache_elements, const void* value_cache, uint64_t value_cache_elements,
    const int32_t* block_tables, uint64_t block_table_elements, const int32_t* sequence_lengths,
    uint64_t sequence_length_elements, void* output, uint64_t output_elements, float* workspace,
    uint64_t workspace_elements, uint32_t sequences, uint32_t query_heads, uint32_t kv_heads,
    uint32_t head_size, uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size,
    uint64_t key_block_stride, uint64_t value_block_stride, uint32_t max_blocks_per_sequence,
    uint32_t max_sequence_length, float scale, void* stream) {
  return bridge_call([&] {
    const DType kind = scalar_kind(dtype);
    const size_t width = loom::size_in_bytes(kind);
    // attention_bridge.rs:100-133.
    const auto spec = decode_spec(kind, sequences, query_heads, kv_heads, head_size, value_head_size,
                                  num_blocks, block_size, max_blocks_per_sequence, max_sequence_length,
                                  scale);
    const auto layout = loom::PagedDecodeLayout::create(spec, key_block_stride, value_block_stride);
    const size_t expected = loom::paged_decode_attention_split_k_workspace_elements(spec).value_or(0);
    if (workspace_elements != expected) {
      throw invalid(format("paged decode workspace has %llu F32 elements, expected %zu",
                           (unsigned long long)workspace_elements, expected));
    }
    if (expected == 0 && workspace != nullptr) {
      throw invalid("base paged decode requires a null workspace pointer");
    }
    if (expected != 0 && workspace == nullptr) {
      throw invalid("split-K paged decode requires a workspace pointer");
    }
    // attention_bridge.rs:135-168.
    const Checked q = borrow(query, query_elements, width, "paged decode query");
    const Checked k = borrow(key_cache, key_cache_elements, width, "paged decode key cache");
    const Checked v = borrow(value_cache, value_cache_elements, width, "paged decode value cache");
    const Checked tables = borrow(block_tables, block_table_elements, 4, "paged decode block tables");
    const Checked lengths = borrow(sequence_lengths, sequence_length_elements, 4, "paged decode sequence lengths");
    const Checked out = borrow(output, output_elements, width, "paged decode output");
    const std::vector<Named> inputs = {{"query", q.range},
                                       {"key cache", k.range},
                                       {"value cache", v.range},
                                       {"block tables", tables.range},
                                       {"sequence lengths", lengths.range}};
    require_disjoint_from("output", out.range, inputs, "paged decode");
    if (expected == 0) {
      loom::paged_decode_attention(kind, q.region, k.region, v.region, tables.region, lengths.region,
                                   out.region, spec, layout, stream);
    } else {
      const Checked ws = borrow(workspace, workspace_elements, 4, "paged decode split-K workspace");
      std::vector<Named> all = inputs;
      all.push_back({"output", out.range});
      require_disjoint_from("workspace", ws.range, all, "paged decode");
      loom::paged_decode_attention_split_k(kind, q.region, k.region, v.region, tables.region,
                                           lengths.region, out.region, ws.region, spec, layout, stream);
    }
    record_launch(LOOM_CUDA_BRIDGE_PAGED_DECODE_ATTENTION);
  });
}

int loom_cuda_bridge_paged_decode_workspace_elements_ex(uint32_t sequences, uint32_t query_heads,
                                                        uint32_t kv_heads, uint32_t value_head_size,
                                                        uint32_t max_sequence_length,
                                                        uint32_t partition_tokens,
                                                        uint64_t* workspace_elements,
                                                        uint32_t* chosen_partition_tokens) {
  return bridge_call([&] {
    if (workspace_elements == nullptr ||
        reinterpret_cast<uintptr_t>(workspace_elements) % alignof(uint64_t) != 0) {
      throw invalid("workspace-size output pointer is null or misaligned");
    }
    if (sequences == 0 || query_heads == 0 || kv_heads == 0 || value_head_size == 0 ||
        max_sequence_length == 0) {
      throw invalid(loom::messages::zero_dimension());
    }
    if (partition_tokens % 16 != 0) {
      throw invalid("paged decode partition length must be a multiple of 16 tokens");
    }
    const uint32_t tokens = partition_tokens;  // 0 = the library chooses at launch
    const uint64_t elements = loom_cuda_paged_decode_workspace_elements(
        sequences, query_heads, kv_heads, value_head_size, max_sequence_length, tokens);
    if (elements == 0) throw invalid("paged decode workspace size overflows the CUDA ABI");
    *workspace_elements = elements;
    if (chosen_partition_tokens != nullptr) *chosen_partition_tokens = tokens;
  });
}

int loom_cuda_bridge_paged_decode_attention_with_options(
    uint32_t dtype, uint32_t cache_encoding, const void* query, uint64_t query_elements,
    const void* key_cache, uint64_t key_cache_elements, const void* value_cache,
    uint64_t value_cache_elements, const float* key_scales, uint64_t key_scale_elements,
    const float* value_scales, uint64_t value_scale_elements, const int32_t* block_tables,
    uint64_t block_table_elements, const int32_t* sequence_lengths, uint64_t sequence_length_elements,
    void* output, uint64_t output_elements, float* workspace, uint64_t workspace_elements,
    uint32_t sequences, uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size, uint64_t key_block_stride,
    uint64_t key_page_stride, uint64_t key_head_stride, uint64_t value_block_stride,
    uint64_t value_page_stride, uint64_t value_head_stride, uint32_t max_blocks_per_sequence,
    uint32_t max_sequence_length, uint32_t partition_tokens, float scale, uint32_t emit_state,
    uint64_t query_token_stride, uint64_t query_head_stride, uint32_t sliding_window, float logits_soft_cap,
    uint32_t flags, void* stream) {
  return bridge_call([&] {
    const DType kind = scalar_kind(dtype);
    const size_t width = loom::size_in_bytes(kind);
    const auto spec = decode_spec(kind, sequences, query_heads, kv_heads, head_size, value_head_size,
                                  num_blocks, block_size, max_blocks_per_sequence, max_sequence_length,
                                  scale);
    const auto layout = loom::StridedDecodeLayout::create(spec, key_block_stride, key_page_stride,
                                                          key_head_stride, value_block_stride,
                                                          value_page_stride, value_head_stride);
    loom::DecodeOptions options;
    options.sliding_window = sliding_window;
    options.logits_soft_cap = logits_soft_cap;
    options.flags = flags;
    options.partition_tokens = partition_tokens;
    options.emit_state = emit_state != 0;
    options.query_token_stride = (size_t)query_token_stride;
    options.query_head_stride = (size_t)query_head_stride;
    size_t cache_width = width;
    std::vector<Named> inputs;
    if (cache_encoding == LOOM_CUDA_BRIDGE_KV_CACHE_FP8_E4M3) {
      if (key_scale_elements != value_scale_elements) {
        throw invalid("paged K/V cache scale tensors must have the same length");
      }
      if (key_scale_elements != 1 && key_scale_elements != kv_heads) {
        throw invalid("paged K/V cache scales must contain one value or one value per KV head");
      }
      options.encoding = key_scale_elements == 1 ? loom::KvCacheEncoding::Fp8E4M3FnPerTensor
                                                 : loom::KvCacheEncoding::Fp8E4M3FnPerHead;
      // A single KV head makes the two granularities coincide; keep per tensor.
      const Checked ks = borrow(key_scales, key_scale_elements, 4, "paged key cache scales");
      const Checked vs = borrow(value_scales, value_scale_elements, 4, "paged value cache scales");
      options.key_scales = ks.region;
      options.value_scales = vs.region;
      inputs.push_back({"key scales", ks.range});
      inputs.push_back({"value scales", vs.range});
      cache_width = 1;
    } else if (cache_encoding != LOOM_CUDA_BRIDGE_KV_CACHE_NATIVE) {
      throw invalid("unsupported paged K/V cache encoding");
    }
    if (emit_state > 1) throw invalid("paged decode state flag must be 0 or 1");
    const Checked q = borrow(query, query_elements, width, "paged decode query");
    const Checked k = borrow(key_cache, key_cache_elements, cache_width, "paged decode key cache");
    const Checked v = borrow(value_cache, value_cache_elements, cache_width, "paged decode value cache");
    const Checked tables = borrow(block_tables, block_table_elements, 4, "paged decode block tables");
    const Checked lengths = borrow(sequence_lengths, sequence_length_elements, 4, "paged decode sequence lengths");
    const Checked out = borrow(output, output_elements, options.emit_state ? 4 : width, "paged decode output");
    inputs.push_back({"query", q.range});
    inputs.push_back({"key cache", k.range});
    inputs.push_back({"value cache", v.range});
    inputs.push_back({"block tables", tables.range});
    inputs.push_back({"sequence lengths", lengths.range});
    require_disjoint_from("output", out.range, inputs, "paged decode");
    if (workspace != nullptr || workspace_elements != 0) {
      const Checked ws = borrow(workspace, workspace_elements, 4, "paged decode split-K workspace");
      inputs.push_back({"output", out.range});
      require_disjoint_from("workspace", ws.range, inputs, "paged decode");
      options.workspace = ws.region;
    }
    loom::paged_decode_attention_strided(kind, q.region, k.region, v.region, tables.region,
                                         lengths.region, out.region, spec, layout, options, stream);
    record_launch(LOOM_CUDA_BRIDGE_PAGED_DECODE_ATTENTION);
  });
}

int loom_cuda_bridge_paged_decode_attention_ex(
    uint32_t dtype, uint32_t cache_encoding, const void* query, uint64_t query_elements,
    const void* key_cache, uint64_t key_cache_elements, const void* value_cache,
    uint64_t value_cache_elements, const float* key_scales, uint64_t key_scale_elements,
    const float* value_scales, uint64_t value_scale_elements, const int32_t* block_tables,
    uint64_t block_table_elements, const int32_t* sequence_lengths, uint64_t sequence_length_elements,
    void* output, uint64_t output_elements, float* workspace, uint64_t workspace_elements,
    uint32_t sequences, uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size, uint64_t key_block_stride,
    uint64_t key_page_stride, uint64_t key_head_stride, uint64_t value_block_stride,
    uint64_t value_page_stride, uint64_t value_head_stride, uint32_t max_blocks_per_sequence,
    uint32_t max_sequence_length, uint32_t partition_tokens, float scale, uint32_t emit_state,
    uint64_t query_token_stride, uint64_t query_head_stride, void* stream) {
  return loom_cuda_bridge_paged_decode_attention_with_options(
      dtype, cache_encoding, query, query_elements, key_cache, key_cache_elements, value_cache,
      value_cache_elements, key_scales, key_scale_elements, value_scales, value_scale_elements, block_tables,
      block_table_elements, sequence_lengths, sequence_length_elements, output, output_elements, workspace,
      workspace_elements, sequences, query_heads, kv_heads, head_size, value_head_size, num_blocks, block_size,
      key_block_stride, key_page_stride, key_head_stride, value_block_stride, value_page_stride,
      value_head_stride, max_blocks_per_sequence, max_sequence_length, partition_tokens, scale, emit_state,
      query_token_stride, query_head_stride, 0u, 0.0f, 0u, stream);
}

int loom_cuda_bridge_merge_decode_states(const float* states, uint64_t state_elements, uint32_t parts,
                                         uint32_t rows, uint32_t value_head_size, uint32_t out_dtype,
                                         void* output, uint64_t output_elements, void* stream) {
  return bridge_call([&] {
    const DType kind = scalar_kind(out_dtype);
    const Checked in = borrow(states, state_elements, 4, "decode partial states");
    const Checked out = borrow(output, output_elements, loom::size_in_bytes(kind), "decode merge output");
    require_disjoint_from("output", out.range, {{"states", in.range}}, "decode merge");
    loom::merge_decode_states(in.region, parts, rows, value_head_size, kind, out.region, stream);
    record_launch(LOOM_CUDA_BRIDGE_PAGED_DECODE_ATTENTION);
  });
}

// ---- KV block movement (no counterpart in the reference yet; checks in the bridge's style) ----

namespace {

// The span of a cache that `blocks` blocks of `block_bytes` at `stride` cover.
void require_block_span(const char* name, uint64_t span_bytes, uint32_t blocks, uint64_t block_bytes,
                        uint64_t stride) {
  if (blocks == 0) throw invalid(format("%s holds no blocks", name));
  if (block_bytes == 0) throw invalid("KV block size is zero bytes");
  if (stride < block_bytes) throw invalid(format("%s block stride %llu is smaller than a block (%llu bytes)", name,
                                                 (unsigned long long)stride, (unsigned long long)block_bytes));
  uint64_t needed = 0;
  if (__builtin_mul_overflow((uint64_t)(blocks - 1), stride, &needed) ||
      __builtin_add_overflow(needed, block_bytes, &needed)) {
    throw invalid(format("%s byte span overflows", name));
  }
  if (span_bytes < needed) {
    throw invalid(format("%s span of %llu bytes is shorter than its %u blocks need (%llu bytes)", name,
                         (unsigned long long)span_bytes, blocks, (unsigned long long)needed));
  }
  if (block_bytes % 16 != 0 || stride % 16 != 0) {
    throw invalid(format("%s blocks and strides must be multiples of 16 bytes", name));
  }
}

void raise_launch_status(int status, const char* operation) {
  if (status == LOOM_CUDA_SUCCESS) return;
  if (status == LOOM_CUDA_INVALID_ARGUMENT || status == LOOM_CUDA_UNSUPPORTED) {
    throw invalid(format("%s rejected its arguments: %s", operation, loom_cuda_status_string(status)));
  }
  if (status == LOOM_CUDA_UNAVAILABLE) {
    throw ExecutorFailure(ExecutorFailure::Kind::BackendUnavailable, status,
                          format("%s: CUDA backend unavailable", operation));
  }
  throw loom::submission(status, loom_cuda_status_string(status));
}

// A cache pointer with its byte span: non-null, 16-byte aligned, no address overflow.
ByteRange cache_range(const void* pointer, uint64_t bytes, const char* name) {
  if (pointer == nullptr) throw invalid(format("%s pointer is null", name));
  const uintptr_t start = reinterpret_cast<uintptr_t>(pointer);
  if (start % 16 != 0) throw invalid(format("%s pointer is not aligned to 16 bytes", name));
  uintptr_t end = 0;
  if (__builtin_add_overflow(start, (uintptr_t)bytes, &end)) {
    throw invalid(format("%s address range overflows usize", name));
  }
  return ByteRange{start, end};
}

}  // namespace

int loom_cuda_bridge_kv_block_move(const void* source_key_cache, uint64_t source_key_bytes,
                                   const void* source_value_cache, uint64_t source_value_bytes,
                                   void* destination_key_cache, uint64_t destination_key_bytes,
                                   void* destination_value_cache, uint64_t destination_value_bytes,
                                   const int64_t* block_pairs, uint64_t pair_elements, uint32_t source_blocks,
                                   uint32_t destination_blocks, uint64_t block_bytes,
                                   uint64_t source_key_block_stride, uint64_t source_value_block_stride,
                                   uint64_t destination_key_block_stride, uint64_t destination_value_block_stride,
                                   void* stream) {
  return bridge_call([&] {
    if (pair_elements % 2 != 0) throw invalid("KV block pairs must hold two ids per pair");
    if (pair_elements / 2 > 0xffffffffull) throw invalid("too many KV block pairs for one call");
    cache_range(source_key_cache, source_key_bytes, "source key cache");
    cache_range(source_value_cache, source_value_bytes, "source value cache");
    const ByteRange written_key = cache_range(destination_key_cache, destination_key_bytes, "destination key cache");
    const ByteRange written_value =
        cache_range(destination_value_cache, destination_value_bytes, "destination value cache");
    require_block_span("source key cache", source_key_bytes, source_blocks, block_bytes, source_key_block_stride);
    require_block_span("source value cache", source_value_bytes, source_blocks, block_bytes,
                       source_value_block_stride);
    require_block_span("destination key cache", destination_key_bytes, destination_blocks, block_bytes,
                       destination_key_block_stride);
    require_block_span("destination value cache", destination_value_bytes, destination_blocks, block_bytes,
                       destination_value_block_stride);
    if (pair_elements == 0) return;  // nothing to move
    const Checked pairs = borrow(block_pairs, pair_elements, 8, "KV block pairs");
    require_disjoint_from("block pairs", pairs.range,
                          {{"destination key cache", written_key}, {"destination value cache", written_value}},
                          "KV block move");
    raise_launch_status(
        loom_cuda_kv_block_move(source_key_cache, source_value_cache, destination_key_cache,
                                destination_value_cache, block_pairs, (uint32_t)(pair_elements / 2), source_blocks,
                                destination_blocks, block_bytes, source_key_block_stride,
                                source_value_block_stride, destination_key_block_stride,
                                destination_value_block_stride, stream),
        "KV block move");
    g_block_movement_launches.fetch_add(1, std::memory_order_relaxed);
  });
}

int loom_cuda_bridge_kv_block_swap(void* key_cache, uint64_t key_bytes, void* value_cache, uint64_t value_bytes,
                                   const int64_t* block_pairs, uint64_t pair_elements, uint32_t num_blocks,
                                   uint64_t block_bytes, uint64_t key_block_stride, uint64_t value_block_stride,
                                   void* stream) {
  return bridge_call([&] {
    if (pair_elements % 2 != 0) throw invalid("KV block pairs must hold two ids per pair");
    if (pair_elements / 2 > 0xffffffffull) throw invalid("too many KV block pairs for one call");
    const ByteRange keys = cache_range(key_cache, key_bytes, "key cache");
    const ByteRange values = cache_range(value_cache, value_bytes, "value cache");
    require_block_span("key cache", key_bytes, num_blocks, block_bytes, key_block_stride);
    require_block_span("value cache", value_bytes, num_blocks, block_bytes, value_block_stride);
    if (pair_elements == 0) return;
    const Checked pairs = borrow(block_pairs, pair_elements, 8, "KV block pairs");
    require_disjoint_from("block pairs", pairs.range, {{"key cache", keys}, {"value cache", values}},
                          "KV block swap");
    raise_launch_status(loom_cuda_kv_block_swap(key_cache, value_cache, block_pairs, (uint32_t)(pair_elements / 2),
                                                num_blocks, block_bytes, key_block_stride, value_block_stride,
                                                stream),
                        "KV block swap");
    g_block_movement_launches.fetch_add(1, std::memory_order_relaxed);
  });
}

int loom_cuda_bridge_block_table_remap(int32_t* block_tables, uint64_t table_elements,
                                       const int32_t* new_block_ids, uint64_t id_elements, void* stream) {
  return bridge_call([&] {
    if (id_elements == 0 || id_elements > 0xffffffffull) throw invalid("new block ids must name 1..2^32-1 blocks");
    const Checked ids = borrow(new_block_ids, id_elements, 4, "new block ids");
    if (table_elements == 0) return;
    const Checked tables = borrow(block_tables, table_elements, 4, "block tables");
    require_disjoint_from("block tables", tables.range, {{"new block ids", ids.range}}, "block table remap");
    raise_launch_status(
        loom_cuda_block_table_remap(block_tables, table_elements, new_block_ids, (uint32_t)id_elements, stream),
        "block table remap");
    g_block_movement_launches.fetch_add(1, std::memory_order_relaxed);
  });
}

int loom_cuda_bridge_kv_block_movement_launches(uint64_t* count) {
  return bridge_call([&] {
    if (count == nullptr || reinterpret_cast<uintptr_t>(count) % alignof(uint64_t) != 0) {
      throw invalid("launch-count output pointer is null or misaligned");
    }
    *count = g_block_movement_launches.load(std::memory_order_relaxed);
  });
}

int loom_cuda_bridge_supports_paged_decode(uint32_t dtype, uint32_t cache_encoding, uint32_t sequences,
                                           uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
                                           uint32_t value_head_size, uint32_t num_blocks,
                                           uint32_t block_size, uint32_t max_blocks_per_sequence,
                                           uint32_t max_sequence_length, float scale) {
  bool supported = false;
  bridge_call([&] {
    if (cache_encoding > 1) throw invalid("unsupported paged K/V cache encoding");
    const auto spec = decode_spec(scalar_kind(dtype), sequences, query_heads, kv_heads, head_size,
                                  value_head_size, num_blocks, block_size, max_blocks_per_sequence,
                                  max_sequence_length, scale);
    const loom::Support answer = loom::supports(spec, cache_encoding == 1);
    if (!answer.supported) throw invalid(answer.reason);
    supported = true;
  });
  return supported ? 1 : 0;
}

int loom_cuda_bridge_supports_rope_paged_kv_write(uint32_t dtype, uint32_t cache_encoding, uint32_t tokens,
                                                  uint32_t query_heads, uint32_t kv_heads,
                                                  uint32_t head_size, uint32_t value_head_size,
                                                  uint32_t rotary_dim, uint32_t max_position,
                                                  uint32_t num_blocks, uint32_t block_size) {
  bool supported = false;
  bridge_call([&] {
    if (cache_encoding > 1) throw invalid("unsupported paged K/V cache encoding");
    loom::RotaryEmbeddingSpec rotary;
    if (auto error = loom::RotaryEmbeddingSpec::create(tokens, query_heads, kv_heads, head_size, rotary_dim,
                                                       max_position, scalar_kind(dtype),
                                                       loom::RotaryStyle::NeoX, &rotary)) {
      throw invalid(error);
    }
    loom::RopePagedKvWriteSpec spec;
    if (auto error = loom::RopePagedKvWriteSpec::create(
            rotary, value_head_size, num_blocks, block_size,
            cache_encoding == 1 ? loom::KvCacheEncoding::Fp8E4M3FnPerTensor : loom::KvCacheEncoding::Native,
            &spec)) {
      throw invalid(error);
    }
    const loom::Support answer = loom::supports(spec);
    if (!answer.supported) throw invalid(answer.reason);
    supported = true;
  });
  return supported ? 1 : 0;
}

// -------------------------------------------------------------------- RoPE

int loom_cuda_bridge_rope_paged_kv_write(
    uint32_t dtype, uint32_t cache_encoding, void* query, uint64_t query_elements, void* key,
    uint64_t key_elements, const void* value, uint64_t value_elements, const int64_t* positions,
    uint64_t position_elements, const void* cos_sin_cache, uint64_t cos_sin_cache_elements,
    void* key_cache, uint64_t key_cache_elements, void* value_cache, uint64_t value_cache_elements,
    const float* key_scales, uint64_t key_scale_elements, const float* value_scales,
    uint64_t value_scale_elements, const int64_t* slot_mapping, uint64_t slot_mapping_elements,
    uint32_t tokens, uint32_t cache_tokens, uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t rotary_dim, uint32_t max_position, uint32_t num_blocks,
    uint32_t block_size, uint64_t query_token_stride, uint64_t query_head_stride,
    uint64_t key_token_stride, uint64_t source_key_head_stride, uint64_t value_token_stride,
    uint64_t source_value_head_stride, uint64_t key_block_stride, uint64_t key_page_stride,
    uint64_t key_head_stride, uint64_t value_block_stride, uint64_t value_page_stride,
    uint64_t value_cache_head_stride, uint32_t is_neox, void* stream) {
  return bridge_call([&] {
    const DType kind = scalar_kind(dtype);
    const size_t width = loom::size_in_bytes(kind);
    // rope_kv_bridge.rs:64-141.
    if (is_neox > 1) throw invalid("RoPE style flag must be 0 or 1");
    loom::RotaryEmbeddingSpec rotary;
    if (auto error = loom::RotaryEmbeddingSpec::create(
            tokens, query_heads, kv_heads, head_size, rotary_dim, max_position, kind,
            is_neox == 1 ? loom::RotaryStyle::NeoX : loom::RotaryStyle::Interleaved, &rotary)) {
      throw invalid(error);
    }
    if (key_scale_elements != value_scale_elements) {
      throw invalid("paged K/V cache scale tensors must have the same length");
    }
    if (key_scale_elements != 1 && key_scale_elements != kv_heads) {
      throw invalid("paged K/V cache scales must contain one value or one value per KV head");
    }
    loom::KvCacheEncoding encoding;
    if (cache_encoding == LOOM_CUDA_BRIDGE_KV_CACHE_NATIVE) {
      encoding = loom::KvCacheEncoding::Native;
    } else if (cache_encoding == LOOM_CUDA_BRIDGE_KV_CACHE_FP8_E4M3) {
      encoding = key_scale_elements == 1 ? loom::KvCacheEncoding::Fp8E4M3FnPerTensor
                                         : loom::KvCacheEncoding::Fp8E4M3FnPerHead;
    } else {
      throw invalid("unsupported paged K/V cache encoding");
    }
    loom::RopePagedKvWriteSpec spec;
    if (auto error = loom::RopePagedKvWriteSpec::create(rotary, value_head_size, num_blocks, block_size,
                                                        encoding, &spec)) {
      throw invalid(error);
    }
    const auto layout = loom::RopePagedKvLayout::create(
        spec, cache_tokens, query_token_stride, query_head_stride, key_token_stride,
        source_key_head_stride, value_token_stride, source_value_head_stride, key_block_stride,
        key_page_stride, key_head_stride, value_block_stride, value_page_stride,
        value_cache_head_stride);

    // rope_kv_bridge.rs:143-190.
    const bool fp8 = loom::is_fp8(encoding);
    const size_t cache_width = fp8 ? 1 : width;
    const Checked q = borrow(query, query_elements, width, "RoPE query");
    const Checked k = borrow(key, key_elements, width, "RoPE key");
    const Checked v = borrow(value, value_elements, width, "RoPE value");
    const Checked pos = borrow(positions, position_elements, 8, "RoPE positions");
    const Checked cs = borrow(cos_sin_cache, cos_sin_cache_elements, width, "RoPE cos/sin cache");
    const Checked kc = borrow(key_cache, key_cache_elements, cache_width,
                              fp8 ? "paged FP8 key cache" : "paged key cache");
    const Checked vc = borrow(value_cache, value_cache_elements, cache_width,
                              fp8 ? "paged FP8 value cache" : "paged value cache");
    const Checked ks = borrow(key_scales, key_scale_elements, 4, "paged key cache scales");
    const Checked vs = borrow(value_scales, value_scale_elements, 4, "paged value cache scales");
    const Checked slots = borrow(slot_mapping, slot_mapping_elements, 8, "paged slot mapping");

    // rope_kv_bridge.rs:192-245: packed QKV views.
    std::optional<size_t> dense_query, dense_key, dense_value;
    size_t product = 0;
    if (layout.query_head_stride == rotary.head_size &&
        !__builtin_mul_overflow(rotary.query_heads, rotary.head_size, &product)) {
      dense_query = product;
    }
    if (layout.source_key_head_stride == rotary.head_size &&
        !__builtin_mul_overflow(rotary.key_heads, rotary.head_size, &product)) {
      dense_key = product;
    }
    if (layout.source_value_head_stride == spec.value_head_size &&
        !__builtin_mul_overflow(rotary.key_heads, spec.value_head_size, &product)) {
      dense_value = product;
    }
    require_disjoint_or_dense_packed_axis(width, "query", q.range, layout.query_token_stride, dense_query,
                                          "key", k.range, layout.key_token_stride, dense_key,
                                          "RoPE+paged-KV");
    require_disjoint_or_dense_packed_axis(width, "query", q.range, layout.query_token_stride, dense_query,
                                          "value", v.range, layout.value_token_stride, dense_value,
                                          "RoPE+paged-KV");
    require_disjoint_or_dense_packed_axis(width, "key", k.range, layout.key_token_stride, dense_key,
                                          "value", v.range, layout.value_token_stride, dense_value,
                                          "RoPE+paged-KV");

    // rope_kv_bridge.rs:247-286: K and V views of one interleaved cache.
    size_t key_block_elements = 0, value_block_elements = 0;
    if (__builtin_mul_overflow(spec.block_size, rotary.key_heads, &product) ||
        __builtin_mul_overflow(product, rotary.head_size, &key_block_elements)) {
      throw invalid("paged key cache block size overflows usize");
    }
    if (__builtin_mul_overflow(spec.block_size, rotary.key_heads, &product) ||
        __builtin_mul_overflow(product, spec.value_head_size, &value_block_elements)) {
      throw invalid("paged value cache block size overflows usize");
    }
    std::optional<size_t> dense_key_block, dense_value_block;
    if (layout.key_block_storage_elements(spec) == key_block_elements) dense_key_block = key_block_elements;
    if (layout.value_block_storage_elements(spec) == value_block_elements) {
      dense_value_block = value_block_elements;
    }
    require_disjoint_or_dense_packed_axis(cache_width, "key cache", kc.range, layout.key_block_stride,
                                          dense_key_block, "value cache", vc.range,
                                          layout.value_block_stride, dense_value_block, "RoPE+paged-KV");

    // rope_kv_bridge.rs:288-324.
    const std::vector<Named> metadata_and_caches = {
        {"positions", pos.range},   {"cos/sin cache", cs.range}, {"key cache", kc.range},
        {"value cache", vc.range},  {"key scales", ks.range},    {"value scales", vs.range},
        {"slot mapping", slots.range}};
    require_disjoint_from("query", q.range, metadata_and_caches, "RoPE+paged-KV");
    require_disjoint_from("key", k.range, metadata_and_caches, "RoPE+paged-KV");
    const std::vector<Named> cache_neighbours = {
        {"value", v.range},         {"positions", pos.range},    {"cos/sin cache", cs.range},
        {"key scales", ks.range},   {"value scales", vs.range},  {"slot mapping", slots.range}};
    require_disjoint_from("key cache", kc.range, cache_neighbours, "RoPE+paged-KV");
    require_disjoint_from("value cache", vc.range, cache_neighbours, "RoPE+paged-KV");

    if (fp8) {
      loom::rope_paged_kv_write_fp8_e4m3(kind, q.region, k.region, v.region, pos.region, cs.region,
                                         kc.region, vc.region, slots.region, ks.region, vs.region, spec,
                                         layout, stream);
    } else {
      loom::rope_paged_kv_write(kind, q.region, k.region, v.region, pos.region, cs.region, kc.region,
                                vc.region, slots.region, spec, layout, stream);
    }
    record_launch(LOOM_CUDA_BRIDGE_ROPE_PAGED_KV_WRITE);
  });
}

// ----------------------------------------- operators outside this library

int loom_cuda_bridge_rms_norm(uint32_t, const void*, uint64_t, const void*, uint64_t, void*, uint64_t,
                              uint32_t, uint32_t, float, void*) {
  return unavailable("RMSNorm");
}
int loom_cuda_bridge_add_rms_norm(uint32_t, void*, uint64_t, void*, uint64_t, const void*, uint64_t,
                                  uint32_t, uint32_t, float, void*) {
  return unavailable("Add+RMSNorm");
}
int loom_cuda_bridge_rms_norm_dynamic_fp8(uint32_t, const void*, uint64_t, const void*, uint64_t, uint8_t*,
                                          uint64_t, float*, uint64_t, uint32_t, uint32_t, float, void*) {
  return unavailable("RMSNorm dynamic FP8");
}
int loom_cuda_bridge_silu_and_mul(uint32_t, const void*, uint64_t, void*, uint64_t, uint32_t, uint32_t,
                                  void*) {
  return unavailable("SiLU-and-Mul");
}
int loom_cuda_bridge_silu_and_mul_dynamic_fp8(uint32_t, const void*, uint64_t, uint8_t*, uint64_t, float*,
                                              uint64_t, const float*, uint64_t, uint32_t, uint32_t,
                                              uint32_t, uint32_t, void*) {
  return unavailable("SiLU-and-Mul dynamic FP8");
}
int loom_cuda_bridge_greedy_sample_logprobs(uint32_t, const void*, uint64_t, int32_t*, uint64_t, float*,
                                            uint64_t, int64_t*, uint64_t, uint32_t, uint32_t, uint64_t,
                                            void*) {
  return unavailable("greedy sampling");
}
int loom_cuda_bridge_selected_token_logprobs(uint32_t, const void*, uint64_t, const int64_t*, uint64_t,
                                             float*, uint64_t, int64_t*, uint64_t, uint32_t, uint32_t,
                                             uint64_t, void*) {
  return unavailable("selected-token logprobs");
}
int loom_cuda_bridge_greedy_speculative_verify(const int32_t*, uint64_t, const int64_t*, uint64_t,
                                               const int32_t*, uint64_t, const int32_t*, uint64_t,
                                               int32_t*, uint64_t, int32_t*, uint64_t, int32_t*, uint64_t,
                                               uint32_t, uint32_t, uint32_t, void*) {
  return unavailable("greedy speculative verify");
}
int loom_cuda_bridge_min_p_filter(uint32_t, void*, uint64_t, const float*, uint64_t, uint32_t, uint32_t,
                                  uint64_t, void*) {
  return unavailable("min-p filter");
}

}  // extern "C"
