/*
 * Checked bridge ABI (version 2) of the B200 paged-decode library.
 *
 * This is the drop-in boundary: the reference's PyTorch dispatcher
 * (python/csrc/{attention,rope_kv,telemetry}.cpp) is compiled against
 * crates/loom-cuda-bridge/include/loom_cuda_bridge.h and linked to
 * libloom_cuda_bridge.so. The library built from this repository exports the
 * same symbols with the same argument lists and status codes, so that
 * dispatcher, and the Python and vLLM adapters above it, run unchanged.
 *
 * The hot-path symbols (version, last error, launch counters, RoPE + paged-KV
 * write, decode workspace size, decode) are implemented. The remaining symbols
 * of that header belong to operators outside this library's scope; they are
 * exported so the dispatcher still loads, and they return
 * LOOM_CUDA_BRIDGE_UNAVAILABLE with an explanatory last-error message.
 *
 * Every pointer is borrowed device memory on the current device and comes with
 * the element count of the span it may address. The bridge checks null,
 * empty, misaligned and overflowing regions, the overlap rules between
 * regions, and the contract, before anything is launched. A failing call
 * records a message readable through loom_cuda_bridge_last_error_message() on
 * the same host thread. No C++ exception leaves these functions.
 */
#ifndef LOOM_BRIDGE_H_
#define LOOM_BRIDGE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* loom_cuda_bridge.h:10-15 */
enum loom_cuda_bridge_status {
  LOOM_CUDA_BRIDGE_SUCCESS = 0,
  LOOM_CUDA_BRIDGE_INVALID_ARGUMENT = 1,
  LOOM_CUDA_BRIDGE_LAUNCH_ERROR = 2,
  LOOM_CUDA_BRIDGE_UNAVAILABLE = 3,
};

/* loom_cuda_bridge.h:17-21 */
enum loom_cuda_bridge_dtype {
  LOOM_CUDA_BRIDGE_F32 = 0,
  LOOM_CUDA_BRIDGE_F16 = 1,
  LOOM_CUDA_BRIDGE_BF16 = 2,
};

/* loom_cuda_bridge.h:23-26 */
enum loom_cuda_bridge_kv_cache_encoding {
  LOOM_CUDA_BRIDGE_KV_CACHE_NATIVE = 0,
  LOOM_CUDA_BRIDGE_KV_CACHE_FP8_E4M3 = 1,
};

/* loom_cuda_bridge.h:28-40: operator ids of the launch counters. Only 5 and 9
 * are ever incremented by this library. */
enum loom_cuda_bridge_operator {
  LOOM_CUDA_BRIDGE_RMS_NORM = 0,
  LOOM_CUDA_BRIDGE_ADD_RMS_NORM = 1,
  LOOM_CUDA_BRIDGE_RMS_NORM_DYNAMIC_FP8 = 2,
  LOOM_CUDA_BRIDGE_SILU_AND_MUL = 3,
  LOOM_CUDA_BRIDGE_SILU_AND_MUL_DYNAMIC_FP8 = 4,
  LOOM_CUDA_BRIDGE_ROPE_PAGED_KV_WRITE = 5,
  LOOM_CUDA_BRIDGE_GREEDY_SAMPLE_LOGPROBS = 6,
  LOOM_CUDA_BRIDGE_SELECTED_TOKEN_LOGPROBS = 7,
  LOOM_CUDA_BRIDGE_MIN_P_FILTER = 8,
  LOOM_CUDA_BRIDGE_PAGED_DECODE_ATTENTION = 9,
  LOOM_CUDA_BRIDGE_GREEDY_SPECULATIVE_VERIFY = 10,
};

/* loom_cuda_bridge.h:42-45 */
uint32_t loom_cuda_bridge_abi_version(void); /* 2 */
const char* loom_cuda_bridge_last_error_message(void);
int loom_cuda_bridge_launch_count(uint32_t operation, uint64_t* count);
int loom_cuda_bridge_reset_launch_count(uint32_t operation);

/*
 * loom_cuda_bridge.h:103-122. Fused RoPE + paged-KV write. The scale tensors
 * are always passed (one element, or one per KV head); a native cache ignores
 * their values, an FP8 cache takes its granularity from their length.
 * Q, K and V may be views of one packed QKV allocation: overlapping bounding
 * spans are accepted only when the rows are dense, share the token stride and
 * interleave without touching.
 */
int loom_cuda_bridge_rope_paged_kv_write(
    uint32_t dtype, uint32_t cache_encoding, void* query,
    uint64_t query_elements, void* key, uint64_t key_elements,
    const void* value, uint64_t value_elements, const int64_t* positions,
    uint64_t position_elements, const void* cos_sin_cache,
    uint64_t cos_sin_cache_elements, void* key_cache,
    uint64_t key_cache_elements, void* value_cache,
    uint64_t value_cache_elements, const float* key_scales,
    uint64_t key_scale_elements, const float* value_scales,
    uint64_t value_scale_elements, const int64_t* slot_mapping,
    uint64_t slot_mapping_elements, uint32_t tokens, uint32_t cache_tokens,
    uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t rotary_dim, uint32_t max_position,
    uint32_t num_blocks, uint32_t block_size, uint64_t query_token_stride,
    uint64_t query_head_stride, uint64_t key_token_stride,
    uint64_t source_key_head_stride, uint64_t value_token_stride,
    uint64_t source_value_head_stride, uint64_t key_block_stride,
    uint64_t key_page_stride, uint64_t key_head_stride,
    uint64_t value_block_stride, uint64_t value_page_stride,
    uint64_t value_cache_head_stride, uint32_t is_neox, void* stream);

/* loom_cuda_bridge.h:124-129. Exact F32 workspace the decode call expects for
 * this contract (0 = pass a null workspace). */
int loom_cuda_bridge_paged_decode_workspace_elements(
    uint32_t dtype, uint32_t sequences, uint32_t query_heads,
    uint32_t kv_heads, uint32_t head_size, uint32_t value_head_size,
    uint32_t num_blocks, uint32_t block_size,
    uint32_t max_blocks_per_sequence, uint32_t max_sequence_length,
    float scale, uint64_t* workspace_elements);

/* loom_cuda_bridge.h:131-142. Null workspace with zero elements selects the
 * single-pass path; the exact non-zero size selects split-K. */
int loom_cuda_bridge_paged_decode_attention(
    uint32_t dtype, const void* query, uint64_t query_elements,
    const void* key_cache, uint64_t key_cache_elements,
    const void* value_cache, uint64_t value_cache_elements,
    const int32_t* block_tables, uint64_t block_table_elements,
    const int32_t* sequence_lengths, uint64_t sequence_length_elements,
    void* output, uint64_t output_elements, float* workspace,
    uint64_t workspace_elements, uint32_t sequences, uint32_t query_heads,
    uint32_t kv_heads, uint32_t head_size, uint32_t value_head_size,
    uint32_t num_blocks, uint32_t block_size, uint64_t key_block_stride,
    uint64_t value_block_stride, uint32_t max_blocks_per_sequence,
    uint32_t max_sequence_length, float scale, void* stream);

/* --------------------------------------------------------------------- *
 * Additions (no counterpart in the reference)
 * --------------------------------------------------------------------- */

/*
 * Checked decode over explicit cache strides, with an optional FP8 E4M3 cache
 * (dequantised on load) and a caller-chosen partition length. Element counts
 * accompany every pointer as above. cache_encoding 0 ignores the scale
 * arguments (they may be null). partition_tokens 0 lets the library choose.
 * workspace may be null (single pass); otherwise workspace_elements must be at
 * least what loom_cuda_bridge_paged_decode_workspace_elements_ex reports.
 * emit_state 1 writes F32 (O, max, sum) states of [sequences, query_heads,
 * value_head_size + 2] to `output` (output_elements counts floats then).
 * query_token_stride / query_head_stride are the element strides of `query`
 * between sequences and heads (both 0 = contiguous), so the rotated Q inside a
 * packed QKV row can be read without a copy; query_elements is then the span
 * of that view.
 */
int loom_cuda_bridge_paged_decode_attention_ex(
    uint32_t dtype, uint32_t cache_encoding, const void* query,
    uint64_t query_elements, const void* key_cache,
    uint64_t key_cache_elements, const void* value_cache,
    uint64_t value_cache_elements, const float* key_scales,
    uint64_t key_scale_elements, const float* value_scales,
    uint64_t value_scale_elements, const int32_t* block_tables,
    uint64_t block_table_elements, const int32_t* sequence_lengths,
    uint64_t sequence_length_elements, void* output, uint64_t output_elements,
    float* workspace, uint64_t workspace_elements, uint32_t sequences,
    uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size,
    uint64_t key_block_stride, uint64_t key_page_stride,
    uint64_t key_head_stride, uint64_t value_block_stride,
    uint64_t value_page_stride, uint64_t value_head_stride,
    uint32_t max_blocks_per_sequence, uint32_t max_sequence_length,
    uint32_t partition_tokens, float scale, uint32_t emit_state,
    uint64_t query_token_stride, uint64_t query_head_stride, void* stream);

/*
 * The same call with the two attention options the reference names as later
 * contract fields (docs/design/paged-decode-attention.md:42-52), both off at 0:
 * sliding_window W > 0 lets a query see only the last W tokens of its sequence;
 * logits_soft_cap c > 0 (finite) turns every scaled score s into
 * c * tanh(s / c) before the softmax. `flags` carries the caller's
 * LOOM_DECODE_* promises (0 = none; include/loom_launch.h).
 */
int loom_cuda_bridge_paged_decode_attention_with_options(
    uint32_t dtype, uint32_t cache_encoding, const void* query,
    uint64_t query_elements, const void* key_cache,
    uint64_t key_cache_elements, const void* value_cache,
    uint64_t value_cache_elements, const float* key_scales,
    uint64_t key_scale_elements, const float* value_scales,
    uint64_t value_scale_elements, const int32_t* block_tables,
    uint64_t block_table_elements, const int32_t* sequence_lengths,
    uint64_t sequence_length_elements, void* output, uint64_t output_elements,
    float* workspace, uint64_t workspace_elements, uint32_t sequences,
    uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size,
    uint64_t key_block_stride, uint64_t key_page_stride,
    uint64_t key_head_stride, uint64_t value_block_stride,
    uint64_t value_page_stride, uint64_t value_head_stride,
    uint32_t max_blocks_per_sequence, uint32_t max_sequence_length,
    uint32_t partition_tokens, float scale, uint32_t emit_state,
    uint64_t query_token_stride, uint64_t query_head_stride,
    uint32_t sliding_window, float logits_soft_cap, uint32_t flags,
    void* stream);


int loom_cuda_bridge_paged_decode_workspace_elements_ex(
    uint32_t sequences, uint32_t query_heads, uint32_t kv_heads,
    uint32_t value_head_size, uint32_t max_sequence_length,
    uint32_t partition_tokens, uint64_t* workspace_elements,
    uint32_t* chosen_partition_tokens);

/* Checked merge of partial states; see loom_cuda_merge_decode_states. */
int loom_cuda_bridge_merge_decode_states(
    const float* states, uint64_t state_elements, uint32_t parts,
    uint32_t rows, uint32_t value_head_size, uint32_t out_dtype, void* output,
    uint64_t output_elements, void* stream);

/*
 * Checked KV block movement; see loom_cuda_kv_block_move, loom_cuda_kv_block_swap
 * and loom_cuda_block_table_remap in loom_launch.h. Every cache pointer comes
 * with the BYTE length of its addressable span; the bridge checks that the
 * named number of blocks fits the span at the given stride, that blocks,
 * strides and bases are multiples of 16 bytes, and that the id buffers do not
 * overlap what is written. K and V spans of one packed allocation may
 * interleave. The ids themselves are device memory and are not inspected.
 */
int loom_cuda_bridge_kv_block_move(
    const void* source_key_cache, uint64_t source_key_bytes,
    const void* source_value_cache, uint64_t source_value_bytes,
    void* destination_key_cache, uint64_t destination_key_bytes,
    void* destination_value_cache, uint64_t destination_value_bytes,
    const int64_t* block_pairs, uint64_t pair_elements, uint32_t source_blocks,
    uint32_t destination_blocks, uint64_t block_bytes,
    uint64_t source_key_block_stride, uint64_t source_value_block_stride,
    uint64_t destination_key_block_stride,
    uint64_t destination_value_block_stride, void* stream);

int loom_cuda_bridge_kv_block_swap(
    void* key_cache, uint64_t key_bytes, void* value_cache,
    uint64_t value_bytes, const int64_t* block_pairs, uint64_t pair_elements,
    uint32_t num_blocks, uint64_t block_bytes, uint64_t key_block_stride,
    uint64_t value_block_stride, void* stream);

int loom_cuda_bridge_block_table_remap(
    int32_t* block_tables, uint64_t table_elements,
    const int32_t* new_block_ids, uint64_t id_elements, void* stream);

/* Successful launches of the three calls above since the library was loaded
 * (kept apart from the reference's operator ids, whose range stays 0..10). */
int loom_cuda_bridge_kv_block_movement_launches(uint64_t* count);

/*
 * Capability query in the style of the reference's Backend::supports
 * (crates/loom-kernels/src/backend.rs:28-42). Returns 1 and leaves the error
 * message untouched when the contract runs on this library, 0 with the reason
 * recorded as the thread's last error when it does not.
 */
int loom_cuda_bridge_supports_paged_decode(
    uint32_t dtype, uint32_t cache_encoding, uint32_t sequences,
    uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size,
    uint32_t max_blocks_per_sequence, uint32_t max_sequence_length,
    float scale);
int loom_cuda_bridge_supports_rope_paged_kv_write(
    uint32_t dtype, uint32_t cache_encoding, uint32_t tokens,
    uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t rotary_dim, uint32_t max_position,
    uint32_t num_blocks, uint32_t block_size);

/* --------------------------------------------------------------------- *
 * Symbols of loom_cuda_bridge.h:47-101 that are outside this library's
 * scope. Exported for link compatibility; each returns
 * LOOM_CUDA_BRIDGE_UNAVAILABLE.
 * --------------------------------------------------------------------- */
int loom_cuda_bridge_rms_norm(uint32_t, const void*, uint64_t, const void*,
                              uint64_t, void*, uint64_t, uint32_t, uint32_t,
                              float, void*);
int loom_cuda_bridge_add_rms_norm(uint32_t, void*, uint64_t, void*, uint64_t,
                                  const void*, uint64_t, uint32_t, uint32_t,
                                  float, void*);
int loom_cuda_bridge_rms_norm_dynamic_fp8(uint32_t, const void*, uint64_t,
                                          const void*, uint64_t, uint8_t*,
                                          uint64_t, float*, uint64_t, uint32_t,
                                          uint32_t, float, void*);
int loom_cuda_bridge_silu_and_mul(uint32_t, const void*, uint64_t, void*,
                                  uint64_t, uint32_t, uint32_t, void*);
int loom_cuda_bridge_silu_and_mul_dynamic_fp8(uint32_t, const void*, uint64_t,
                                              uint8_t*, uint64_t, float*,
                                              uint64_t, const float*, uint64_t,
                                              uint32_t, uint32_t, uint32_t,
                                              uint32_t, void*);
int loom_cuda_bridge_greedy_sample_logprobs(uint32_t, const void*, uint64_t,
                                            int32_t*, uint64_t, float*,
                                            uint64_t, int64_t*, uint64_t,
                                            uint32_t, uint32_t, uint64_t,
                                            void*);
int loom_cuda_bridge_selected_token_logprobs(uint32_t, const void*, uint64_t,
                                             const int64_t*, uint64_t, float*,
                                             uint64_t, int64_t*, uint64_t,
                                             uint32_t, uint32_t, uint64_t,
                                             void*);
int loom_cuda_bridge_greedy_speculative_verify(
    const int32_t*, uint64_t, const int64_t*, uint64_t, const int32_t*,
    uint64_t, const int32_t*, uint64_t, int32_t*, uint64_t, int32_t*, uint64_t,
    int32_t*, uint64_t, uint32_t, uint32_t, uint32_t, void*);
int loom_cuda_bridge_min_p_filter(uint32_t, void*, uint64_t, const float*,
                                  uint64_t, uint32_t, uint32_t, uint64_t,
                                  void*);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* LOOM_BRIDGE_H_ */
