// Safe dispatch: checks borrowed device regions against a contract and a
// layout, narrows to the launch ABI, launches, and turns a status into an
// error. This is the library's equivalent of the reference's `CudaBackend`
// methods for this path:
//   crates/loom-cuda/src/attention_dispatch.rs:14-478
//   crates/loom-cuda/src/rope_kv_dispatch.rs:18-585
//   crates/loom-cuda/src/cuda_backend.rs:112-145 (capability answers)
// Every function throws loom::ExecutorFailure on a rejected call.
#pragma once

#include <cstdint>
#include <optional>

#include "contract.hpp"
#include "layout.hpp"

namespace loom {

// A borrowed span of device memory with its element count.
struct Region {
  const void* pointer = nullptr;
  size_t elements = 0;

  void require_len(size_t expected, const char* name) const {
    if (elements != expected) {
      throw invalid(detail::format("%s has %zu elements, expected %zu", name, elements, expected));
    }
  }
};

struct Support {
  bool supported = true;
  const char* reason = "supported";
};

// ---- paged decode attention ------------------------------------------------

// Whether the decode contract runs on this library (no launch happens).
Support supports(const PagedDecodeAttentionSpec& spec, bool fp8_cache = false);
Support supports(const RopePagedKvWriteSpec& spec);

// F32 workspace the split-K path needs for this contract, or nothing when one
// partition covers the longest allowed context.
std::optional<size_t> paged_decode_attention_split_k_workspace_elements(
    const PagedDecodeAttentionSpec& spec);

void paged_decode_attention(DType call_dtype, Region query, Region key_cache, Region value_cache,
                            Region block_tables, Region sequence_lengths, Region output,
                            const PagedDecodeAttentionSpec& spec, const PagedDecodeLayout& layout,
                            void* stream);

void paged_decode_attention_split_k(DType call_dtype, Region query, Region key_cache, Region value_cache,
                                    Region block_tables, Region sequence_lengths, Region output,
                                    Region workspace, const PagedDecodeAttentionSpec& spec,
                                    const PagedDecodeLayout& layout, void* stream);

// Addition: explicit strides, optional FP8 cache and workspace, optional state
// output. `encoding` Native ignores the scale regions.
struct DecodeOptions {
  KvCacheEncoding encoding = KvCacheEncoding::Native;
  Region key_scales, value_scales;
  Region workspace;              // empty = single pass
  uint32_t partition_tokens = 0; // 0 = library default
  bool emit_state = false;
  // Element strides of the query between sequences and heads; both 0 = dense.
  size_t query_token_stride = 0, query_head_stride = 0;
  // Options the reference lists as later contract fields (docs/design/paged-decode-attention.md:42-52).
  uint32_t sliding_window = 0;   // > 0: only the last `sliding_window` tokens are attended to
  float logits_soft_cap = 0.0f;  // > 0: score -> cap * tanh(score / cap)
  uint32_t flags = 0;            // LOOM_DECODE_* promises (include/loom_launch.h)
};

uint32_t decode_partition_tokens(const PagedDecodeAttentionSpec& spec, uint32_t requested);
size_t decode_workspace_elements(const PagedDecodeAttentionSpec& spec, uint32_t partition_tokens);

void paged_decode_attention_strided(DType call_dtype, Region query, Region key_cache, Region value_cache,
                                    Region block_tables, Region sequence_lengths, Region output,
                                    const PagedDecodeAttentionSpec& spec, const StridedDecodeLayout& layout,
                                    const DecodeOptions& options, void* stream);

void merge_decode_states(Region states, uint32_t parts, uint32_t rows, uint32_t value_head_size,
                         DType out_dtype, Region output, void* stream);

// ---- fused RoPE + paged-KV write --------------------------------------------

void rope_paged_kv_write(DType call_dtype, Region query, Region key, Region value, Region positions,
                         Region cos_sin_cache, Region key_cache, Region value_cache, Region slot_mapping,
                         const RopePagedKvWriteSpec& spec, const RopePagedKvLayout& layout, void* stream);

void rope_paged_kv_write_fp8_e4m3(DType call_dtype, Region query, Region key, Region value, Region positions,
                                  Region cos_sin_cache, Region key_cache, Region value_cache,
                                  Region slot_mapping, Region key_scales, Region value_scales,
                                  const RopePagedKvWriteSpec& spec, const RopePagedKvLayout& layout,
                                  void* stream);

}  // namespace loom
