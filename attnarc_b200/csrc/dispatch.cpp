// Safe dispatch layer; see dispatch.hpp for what it mirrors.

#include "dispatch.hpp"

#include <cmath>

#include <limits>

#include "../../include/loom_launch.h"

namespace loom {
namespace {

constexpr size_t kU32Max = 0xffffffffull;

void status_result(int status) {
  if (status != LOOM_CUDA_SUCCESS) throw submission(status, loom_cuda_status_string(status));
}

uint32_t narrow_u32(size_t value, const char* name) {
  if (value > kU32Max) throw invalid(std::string(name) + " exceeds the CUDA ABI");
  return (uint32_t)value;
}

bool fits_u32(size_t value) { return value <= kU32Max; }

// attention_dispatch.rs:330-345, minus the reference kernels' 1024-token cap.
bool decode_shape_fits_abi(const PagedDecodeAttentionSpec& spec) {
  size_t grid = 0;
  return fits_u32(spec.sequences) && fits_u32(spec.query_heads) && fits_u32(spec.kv_heads) &&
         fits_u32(spec.head_size) && fits_u32(spec.value_head_size) && fits_u32(spec.num_blocks) &&
         fits_u32(spec.block_size) && fits_u32(spec.max_blocks_per_sequence) &&
         spec.max_sequence_length <= (1u << 30) &&
         !__builtin_mul_overflow(spec.sequences, spec.query_heads, &grid) &&
         grid <= (size_t)std::numeric_limits<int32_t>::max();
}

void require_decode_dtype(const PagedDecodeAttentionSpec& spec, DType expected) {
  if (spec.dtype != expected) {
    throw invalid(detail::format("paged decode attention for %s cannot execute %s", debug_name(expected),
                                 debug_name(spec.dtype)));
  }
}

void require_decode_abi(const PagedDecodeAttentionSpec& spec) {
  if (!decode_shape_fits_abi(spec)) throw invalid("paged decode shape exceeds the CUDA ABI");
}

// attention_dispatch.rs:458-478.
void validate_decode_regions(const Region& query, const Region& key_cache, const Region& value_cache,
                             const Region& block_tables, const Region& sequence_lengths,
                             const Region& output, const PagedDecodeAttentionSpec& spec,
                             size_t key_storage, size_t value_storage, size_t output_elements,
                             size_t query_storage = 0) {
  query.require_len(query_storage != 0 ? query_storage : spec.query_numel(), "paged decode query");
  key_cache.require_len(key_storage, "paged decode key cache");
  value_cache.require_len(value_storage, "paged decode value cache");
  block_tables.require_len(spec.block_table_numel(), "paged decode block tables");
  sequence_lengths.require_len(spec.sequences, "paged decode sequence lengths");
  output.require_len(output_elements, "paged decode output");
  require_decode_abi(spec);
}

LoomDecodeArgs decode_args(DType call_dtype, const Region& query, const Region& key_cache,
                           const Region& value_cache, const Region& block_tables,
                           const Region& sequence_lengths, const Region& output,
                           const PagedDecodeAttentionSpec& spec, const StridedDecodeLayout& layout,
                           void* stream) {
  LoomDecodeArgs a{};
  a.struct_size = sizeof(LoomDecodeArgs);
  a.dtype = (uint32_t)call_dtype;
  a.query = query.pointer;
  a.key_cache = key_cache.pointer;
  a.value_cache = value_cache.pointer;
  a.block_tables = static_cast<const int32_t*>(block_tables.pointer);
  a.sequence_lengths = static_cast<const int32_t*>(sequence_lengths.pointer);
  a.output = const_cast<void*>(output.pointer);
  a.sequences = narrow_u32(spec.sequences, "sequence count");
  a.query_heads = narrow_u32(spec.query_heads, "query head count");
  a.kv_heads = narrow_u32(spec.kv_heads, "KV head count");
  a.head_size = narrow_u32(spec.head_size, "head size");
  a.value_head_size = narrow_u32(spec.value_head_size, "value head size");
  a.num_blocks = narrow_u32(spec.num_blocks, "cache block count");
  a.block_size = narrow_u32(spec.block_size, "cache block size");
  a.max_blocks_per_sequence = narrow_u32(spec.max_blocks_per_sequence, "maximum blocks per sequence");
  a.max_sequence_length = narrow_u32(spec.max_sequence_length, "maximum context");
  a.key_block_stride = layout.key_block_stride;
  a.key_page_stride = layout.key_page_stride;
  a.key_head_stride = layout.key_head_stride;
  a.value_block_stride = layout.value_block_stride;
  a.value_page_stride = layout.value_page_stride;
  a.value_head_stride = layout.value_head_stride;
  a.scale = spec.scale;
  a.stream = stream;
  return a;
}

}  // namespace

Support supports(const PagedDecodeAttentionSpec& spec, bool fp8_cache) {
  Support answer;
  if (spec.dtype != DType::F32 && spec.dtype != DType::F16 && spec.dtype != DType::Bf16) {
    answer.supported = false;
    answer.reason = "B200 paged decode attention supports F32, FP16, and BF16 queries";
    return answer;
  }
  if (!decode_shape_fits_abi(spec)) {
    answer.supported = false;
    answer.reason = "paged decode attention shape exceeds the CUDA ABI";
    return answer;
  }
  const char* reason = nullptr;
  const int ok = loom_cuda_supports_paged_decode(
      (uint32_t)spec.dtype, fp8_cache ? 1u : 0u, (uint32_t)spec.sequences, (uint32_t)spec.query_heads,
      (uint32_t)spec.kv_heads, (uint32_t)spec.head_size, (uint32_t)spec.value_head_size,
      (uint32_t)spec.num_blocks, (uint32_t)spec.block_size, (uint32_t)spec.max_blocks_per_sequence,
      (uint32_t)spec.max_sequence_length, &reason);
  answer.supported = ok == 1;
  answer.reason = reason;
  return answer;
}

// cuda_backend.rs:135-145: the fused RoPE + paged-KV write takes F32, F16 and
// BF16 sources with a native or FP8 cache.
Support supports(const RopePagedKvWriteSpec& spec) {
  Support answer;
  const DType dtype = spec.rotary.dtype;
  if (dtype != DType::F32 && dtype != DType::F16 && dtype != DType::Bf16) {
    answer.supported = false;
    answer.reason = "CUDA RoPE+paged-KV supports F32, FP16, and BF16 sources";
  } else if (!fits_u32(spec.rotary.tokens) || spec.rotary.tokens > 0x7fffffffull ||
             !fits_u32(spec.rotary.query_heads) || !fits_u32(spec.rotary.key_heads) ||
             !fits_u32(spec.rotary.head_size) || !fits_u32(spec.value_head_size) ||
             !fits_u32(spec.rotary.max_position) || !fits_u32(spec.num_blocks) ||
             !fits_u32(spec.block_size)) {
    answer.supported = false;
    answer.reason = "RoPE+paged-KV shape exceeds the CUDA ABI";
  }
  return answer;
}

std::optional<size_t> paged_decode_attention_split_k_workspace_elements(
    const PagedDecodeAttentionSpec& spec) {
  require_decode_abi(spec);
  const uint64_t elements = loom_cuda_paged_decode_attention_split_k_workspace_elements(
      (uint32_t)spec.sequences, (uint32_t)spec.query_heads, (uint32_t)spec.kv_heads,
      (uint32_t)spec.head_size, (uint32_t)spec.value_head_size, (uint32_t)spec.max_sequence_length);
  if (elements == 0) return std::nullopt;
  return (size_t)elements;
}

void paged_decode_attention(DType call_dtype, Region query, Region key_cache, Region value_cache,
                            Region block_tables, Region sequence_lengths, Region output,
                            const PagedDecodeAttentionSpec& spec, const PagedDecodeLayout& layout,
                            void* stream) {
  require_decode_dtype(spec, call_dtype);
  validate_decode_regions(query, key_cache, value_cache, block_tables, sequence_lengths, output, spec,
                          layout.key_storage_elements(spec), layout.value_storage_elements(spec),
                          spec.output_numel());
  LoomDecodeArgs a = decode_args(call_dtype, query, key_cache, value_cache, block_tables,
                                 sequence_lengths, output, spec,
                                 StridedDecodeLayout::from_nhd(spec, layout), stream);
  status_result(loom_cuda_paged_decode_attention_ex(&a));
}

void paged_decode_attention_split_k(DType call_dtype, Region query, Region key_cache, Region value_cache,
                                    Region block_tables, Region sequence_lengths, Region output,
                                    Region workspace, const PagedDecodeAttentionSpec& spec,
                                    const PagedDecodeLayout& layout, void* stream) {
  require_decode_dtype(spec, call_dtype);
  validate_decode_regions(query, key_cache, value_cache, block_tables, sequence_lengths, output, spec,
                          layout.key_storage_elements(spec), layout.value_storage_elements(spec),
                          spec.output_numel());
  // attention_dispatch.rs:433-455.
  const std::optional<size_t> required = paged_decode_attention_split_k_workspace_elements(spec);
  if (!required) throw invalid("paged decode shape does not select the qualified split-K path");
  if (workspace.elements < *required) {
    throw invalid(detail::format(
        "paged decode split-K workspace has %zu F32 elements, requires at least %zu",
        workspace.elements, *required));
  }
  LoomDecodeArgs a = decode_args(call_dtype, query, key_cache, value_cache, block_tables,
                                 sequence_lengths, output, spec,
                                 StridedDecodeLayout::from_nhd(spec, layout), stream);
  a.workspace = static_cast<float*>(const_cast<void*>(workspace.pointer));
  a.workspace_elements = workspace.elements;
  status_result(loom_cuda_paged_decode_attention_ex(&a));
}

uint32_t decode_partition_tokens(const PagedDecodeAttentionSpec& spec, uint32_t requested) {
  require_decode_abi(spec);
  if (requested % 16 != 0) throw invalid("paged decode partition length must be a multiple of 16 tokens");
  return requested;  // 0 = the library chooses at launch
}

size_t decode_workspace_elements(const PagedDecodeAttentionSpec& spec, uint32_t partition_tokens) {
  require_decode_abi(spec);
  const uint64_t elements = loom_cuda_paged_decode_workspace_elements(
      (uint32_t)spec.sequences, (uint32_t)spec.query_heads, (uint32_t)spec.kv_heads,
      (uint32_t)spec.value_head_size, (uint32_t)spec.max_sequence_length, partition_tokens);
  if (elements == 0) throw invalid("paged decode workspace size overflows the CUDA ABI");
  return (size_t)elements;
}

void paged_decode_attention_strided(DType call_dtype, Region query, Region key_cache, Region value_cache,
                                    Region block_tables, Region sequence_lengths, Region output,
                                    const PagedDecodeAttentionSpec& spec, const StridedDecodeLayout& layout,
                                    const DecodeOptions& options, void* stream) {
  require_decode_dtype(spec, call_dtype);
  const size_t state_elements = spec.sequences * spec.query_heads * (spec.value_head_size + 2);
  size_t query_storage = 0;
  if (options.query_token_stride != 0 || options.query_head_stride != 0) {
    layout_detail::require_non_overlapping({{spec.sequences, options.query_token_stride},
                                            {spec.query_heads, options.query_head_stride}},
                                           spec.head_size, "paged decode query");
    query_storage = layout_detail::strided_span({{spec.sequences, options.query_token_stride},
                                                 {spec.query_heads, options.query_head_stride}},
                                                spec.head_size, "paged decode query");
  }
  validate_decode_regions(query, key_cache, value_cache, block_tables, sequence_lengths, output, spec,
                          layout.key_storage_elements(spec), layout.value_storage_elements(spec),
                          options.emit_state ? state_elements : spec.output_numel(), query_storage);
  LoomDecodeArgs a = decode_args(call_dtype, query, key_cache, value_cache, block_tables,
                                 sequence_lengths, output, spec, layout, stream);
  a.query_token_stride = options.query_token_stride;
  a.query_head_stride = options.query_head_stride;
  if (is_fp8(options.encoding)) {
    const size_t scales = scale_elements(options.encoding, spec.kv_heads);
    options.key_scales.require_len(scales, "paged key cache scales");
    options.value_scales.require_len(scales, "paged value cache scales");
    a.cache_encoding = LOOM_CUDA_KV_CACHE_FP8_E4M3;
    a.scale_stride = options.encoding == KvCacheEncoding::Fp8E4M3FnPerHead ? 1 : 0;
    a.key_scales = static_cast<const float*>(options.key_scales.pointer);
    a.value_scales = static_cast<const float*>(options.value_scales.pointer);
  }
  a.emit_state = options.emit_state ? 1 : 0;
  if (!std::isfinite(options.logits_soft_cap) || options.logits_soft_cap < 0.0f) {
    throw invalid("paged decode logits soft cap must be finite and not negative");
  }
  a.sliding_window = options.sliding_window;
  a.logits_soft_cap = options.logits_soft_cap;
  if ((options.flags & ~LOOM_DECODE_STABLE_METADATA) != 0) {
    throw invalid("paged decode flags contain an unknown bit");
  }
  a.flags = options.flags;
  if (options.workspace.pointer != nullptr || options.workspace.elements != 0) {
    const uint32_t tokens = decode_partition_tokens(spec, options.partition_tokens);
    const size_t required = decode_workspace_elements(spec, tokens);
    if (options.workspace.pointer == nullptr || options.workspace.elements < required) {
      throw invalid(detail::format(
          "paged decode split-K workspace has %zu F32 elements, requires at least %zu",
          options.workspace.elements, required));
    }
    a.workspace = static_cast<float*>(const_cast<void*>(options.workspace.pointer));
    a.workspace_elements = options.workspace.elements;
    a.partition_tokens = tokens;
  }
  status_result(loom_cuda_paged_decode_attention_ex(&a));
}

void merge_decode_states(Region states, uint32_t parts, uint32_t rows, uint32_t value_head_size,
                         DType out_dtype, Region output, void* stream) {
  if (parts == 0 || rows == 0 || value_head_size == 0) throw invalid(messages::zero_dimension());
  size_t per_part = 0, total = 0, out_elements = 0;
  if (__builtin_mul_overflow((size_t)rows, (size_t)value_head_size + 2, &per_part) ||
      __builtin_mul_overflow(per_part, (size_t)parts, &total) ||
      __builtin_mul_overflow((size_t)rows, (size_t)value_head_size, &out_elements)) {
    throw invalid(messages::overflow());
  }
  states.require_len(total, "decode partial states");
  output.require_len(out_elements, "decode merge output");
  status_result(loom_cuda_merge_decode_states(static_cast<const float*>(states.pointer), parts, rows,
                                              value_head_size, (uint32_t)out_dtype,
                                              const_cast<void*>(output.pointer), stream));
}

// ------------------------------------------------------------------ RoPE

namespace {

void require_rope_dtype(const RopePagedKvWriteSpec& spec, DType expected) {
  if (spec.rotary.dtype != expected) {
    throw invalid(detail::format("%s RoPE+paged-KV cannot execute %s", debug_name(expected),
                                 debug_name(spec.rotary.dtype)));
  }
}

// rope_kv_dispatch.rs:520-585.
void validate_rope_regions(const Region& query, const Region& key, const Region& value,
                           const Region& positions, const Region& cos_sin_cache,
                           const Region& key_cache, const Region& value_cache,
                           const Region& slot_mapping, const RopePagedKvWriteSpec& spec,
                           const RopePagedKvLayout& layout) {
  query.require_len(layout.query_storage_elements(spec), "RoPE query");
  key.require_len(layout.key_storage_elements(spec), "RoPE key");
  value.require_len(layout.value_storage_elements(spec), "RoPE value");
  positions.require_len(spec.rotary.tokens, "RoPE positions");
  cos_sin_cache.require_len(spec.rotary.cos_sin_cache_numel(), "RoPE cos/sin cache");
  key_cache.require_len(layout.key_cache_storage_elements(spec), "paged key cache");
  value_cache.require_len(layout.value_cache_storage_elements(spec), "paged value cache");
  slot_mapping.require_len(layout.cache_tokens, "paged slot mapping");
}

void launch_rope(DType call_dtype, const Region& query, const Region& key, const Region& value,
                 const Region& positions, const Region& cos_sin_cache, const Region& key_cache,
                 const Region& value_cache, const Region& slot_mapping, const float* key_scales,
                 const float* value_scales, uint32_t cache_encoding, uint32_t scale_stride,
                 const RopePagedKvWriteSpec& spec, const RopePagedKvLayout& layout, void* stream) {
  const RotaryEmbeddingSpec& r = spec.rotary;
#define LOOM_ROPE_CALL(symbol, scalar)                                                              \
  symbol(static_cast<scalar*>(const_cast<void*>(query.pointer)),                                    \
         static_cast<scalar*>(const_cast<void*>(key.pointer)),                                      \
         static_cast<const scalar*>(value.pointer), static_cast<const int64_t*>(positions.pointer), \
         static_cast<const scalar*>(cos_sin_cache.pointer), const_cast<void*>(key_cache.pointer),   \
         const_cast<void*>(value_cache.pointer), key_scales, value_scales,                          \
         static_cast<const int64_t*>(slot_mapping.pointer), narrow_u32(r.tokens, "token count"),    \
         narrow_u32(layout.cache_tokens, "cache token count"),                                      \
         narrow_u32(r.query_heads, "query head count"), narrow_u32(r.key_heads, "KV head count"),   \
         narrow_u32(r.head_size, "head size"), narrow_u32(spec.value_head_size, "value head size"), \
         narrow_u32(r.rotary_dim, "rotary dimension"),                                              \
         narrow_u32(r.max_position, "maximum position"),                                            \
         narrow_u32(spec.num_blocks, "cache block count"),                                          \
         narrow_u32(spec.block_size, "cache block size"), cache_encoding, scale_stride,             \
         layout.query_token_stride, layout.query_head_stride, layout.key_token_stride,              \
         layout.source_key_head_stride, layout.value_token_stride,                                  \
         layout.source_value_head_stride, layout.key_block_stride, layout.key_page_stride,          \
         layout.key_head_stride, layout.value_block_stride, layout.value_page_stride,               \
         layout.value_head_stride, r.style == RotaryStyle::NeoX ? 1u : 0u, stream)
  switch (call_dtype) {
    case DType::F32: status_result(LOOM_ROPE_CALL(loom_cuda_rope_paged_kv_write_f32, float)); break;
    case DType::F16: status_result(LOOM_ROPE_CALL(loom_cuda_rope_paged_kv_write_f16, uint16_t)); break;
    case DType::Bf16: status_result(LOOM_ROPE_CALL(loom_cuda_rope_paged_kv_write_bf16, uint16_t)); break;
    default: throw invalid("RoPE+paged-KV source type must be F32, F16 or BF16");
  }
#undef LOOM_ROPE_CALL
}

}  // namespace

void rope_paged_kv_write(DType call_dtype, Region query, Region key, Region value, Region positions,
                         Region cos_sin_cache, Region key_cache, Region value_cache, Region slot_mapping,
                         const RopePagedKvWriteSpec& spec, const RopePagedKvLayout& layout, void* stream) {
  require_rope_dtype(spec, call_dtype);
  if (spec.cache_encoding != KvCacheEncoding::Native) {
    throw invalid("native RoPE+paged-KV dispatch requires native cache encoding");
  }
  validate_rope_regions(query, key, value, positions, cos_sin_cache, key_cache, value_cache,
                        slot_mapping, spec, layout);
  launch_rope(call_dtype, query, key, value, positions, cos_sin_cache, key_cache, value_cache,
              slot_mapping, nullptr, nullptr, LOOM_CUDA_KV_CACHE_NATIVE, 0, spec, layout, stream);
}

void rope_paged_kv_write_fp8_e4m3(DType call_dtype, Region query, Region key, Region value,
                                  Region positions, Region cos_sin_cache, Region key_cache,
                                  Region value_cache, Region slot_mapping, Region key_scales,
                                  Region value_scales, const RopePagedKvWriteSpec& spec,
                                  const RopePagedKvLayout& layout, void* stream) {
  require_rope_dtype(spec, call_dtype);
  if (!is_fp8(spec.cache_encoding)) {
    throw invalid("FP8 RoPE+paged-KV dispatch requires FP8 E4M3 cache encoding");
  }
  const uint32_t scale_stride = spec.cache_encoding == KvCacheEncoding::Fp8E4M3FnPerHead ? 1 : 0;
  validate_rope_regions(query, key, value, positions, cos_sin_cache, key_cache, value_cache,
                        slot_mapping, spec, layout);
  key_scales.require_len(spec.scale_elements(), "paged key cache scales");
  value_scales.require_len(spec.scale_elements(), "paged value cache scales");
  launch_rope(call_dtype, query, key, value, positions, cos_sin_cache, key_cache, value_cache,
              slot_mapping, static_cast<const float*>(key_scales.pointer),
              static_cast<const float*>(value_scales.pointer), LOOM_CUDA_KV_CACHE_FP8_E4M3,
              scale_stride, spec, layout, stream);
}

}  // namespace loom
