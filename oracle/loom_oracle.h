/*
 * CPU oracle for the paged-decode hot path: C ABI.
 *
 * TEST INFRASTRUCTURE ONLY. This library restates, in C++, the deterministic
 * CPU reference that the Loom Kernels project keeps in Rust
 * (crates/loom-kernels/src/{attention,rope_kv,quantization,contract}.rs). It
 * exists so that GPU results can be checked and so that a CPU baseline can be
 * timed beside them. Nothing in the shipped library links, loads or calls it.
 *
 * Pinning: every known-answer test the reference holds for this path
 * (crates/loom-kernels/src/tests/attention_tests.rs, rope_kv_tests.rs) is
 * replayed against this restatement by tests/test_oracle_known_answers.py.
 * Two pieces are extensions with no reference counterpart, so their parity is
 * UNPINNED: the FP8-cache decode (dequantise, then the same F64 attention) and
 * anything that depends on a cache layout other than contiguous NHD.
 */
#ifndef LOOM_ORACLE_H_
#define LOOM_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types; values match the bridge ABI's dtype codes. */
enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_BF16 = 2, ORACLE_FP8_E4M3FN = 3 };

/* Cache encodings of the RoPE + paged-KV write contract. */
enum {
  ORACLE_CACHE_NATIVE = 0,
  ORACLE_CACHE_FP8_PER_TENSOR = 1,
  ORACLE_CACHE_FP8_PER_HEAD = 2
};

/* One value per ContractError variant this path can raise
 * (crates/loom-kernels/src/contract.rs:79-161). */
enum {
  ORACLE_OK = 0,
  ORACLE_ZERO_DIMENSION = 1,
  ORACLE_ELEMENT_COUNT_OVERFLOW = 2,
  ORACLE_INVALID_ROTARY_DIMENSION = 3, /* a=rotary_dim b=head_size */
  ORACLE_POSITION_OUT_OF_BOUNDS = 4,   /* a=token b=position c=max_position */
  ORACLE_SLOT_OUT_OF_BOUNDS = 5,       /* a=token b=slot c=slot_capacity */
  ORACLE_DUPLICATE_SLOT = 6,           /* a=first_token b=second_token c=slot */
  ORACLE_INVALID_SCALE = 7,            /* value=scale */
  ORACLE_HEAD_COUNT_NOT_DIVISIBLE = 8, /* a=query_heads b=kv_heads */
  ORACLE_SEQUENCE_LENGTH_OUT_OF_BOUNDS = 9, /* a=sequence b=length c=capacity */
  ORACLE_MAX_SEQUENCE_LENGTH_OUT_OF_BOUNDS = 10, /* a=length b=capacity */
  ORACLE_BLOCK_ID_OUT_OF_BOUNDS = 11, /* a=sequence b=logical_block c=block_id d=num_blocks */
  ORACLE_LENGTH_MISMATCH = 12,        /* buffer, a=expected b=actual */
  ORACLE_UNSUPPORTED_DTYPE = 13       /* a=dtype code */
};

typedef struct oracle_error {
  int32_t kind;
  int64_t a, b, c, d;
  float value;
  char buffer[32];
} oracle_error;

/* Formats the error like the reference's Display impl
 * (crates/loom-kernels/src/contract.rs:163-303). Returns bytes written. */
int oracle_error_message(const oracle_error* error, char* out, int capacity);

/* ---- element conversions (crate half 2.7.1 semantics: RNE, exact widening) */
uint16_t oracle_f32_to_bf16(float value);
float oracle_bf16_to_f32(uint16_t bits);
uint16_t oracle_f32_to_f16(float value);
float oracle_f16_to_f32(uint16_t bits);
void oracle_f32_to_bf16_n(const float* in, uint16_t* out, uint64_t n);
void oracle_bf16_to_f32_n(const uint16_t* in, float* out, uint64_t n);
void oracle_f32_to_f16_n(const float* in, uint16_t* out, uint64_t n);
void oracle_f16_to_f32_n(const uint16_t* in, float* out, uint64_t n);

/* ---- FP8 E4M3FN (crates/loom-kernels/src/quantization.rs:13-56) */
float oracle_fp8_e4m3fn_to_f32(uint8_t bits);
/* The reference's nearest-candidate scan, restated. */
uint8_t oracle_fp8_e4m3fn_from_f32(float value);
/* A direct bit-level encoder; tests prove it equal to the scan. */
uint8_t oracle_fp8_e4m3fn_from_f32_direct(float value);
void oracle_fp8_e4m3fn_from_f32_n(const float* in, uint8_t* out, uint64_t n);
void oracle_fp8_e4m3fn_to_f32_n(const uint8_t* in, float* out, uint64_t n);

/* ---- contracts */
typedef struct oracle_decode_spec {
  uint64_t sequences, query_heads, kv_heads, head_size, value_head_size;
  uint64_t num_blocks, block_size, max_blocks_per_sequence, max_sequence_length;
  float scale;
  int32_t dtype;
} oracle_decode_spec;

typedef struct oracle_rotary_spec {
  uint64_t tokens, query_heads, key_heads, head_size, rotary_dim, max_position;
  int32_t dtype;
  int32_t is_neox; /* 1 = NeoX halves, 0 = interleaved pairs */
} oracle_rotary_spec;

typedef struct oracle_rope_kv_spec {
  oracle_rotary_spec rotary;
  uint64_t value_head_size, num_blocks, block_size;
  int32_t cache_encoding;
} oracle_rope_kv_spec;

/* PagedDecodeAttentionSpec::new (attention.rs:34-97). */
int oracle_decode_spec_check(const oracle_decode_spec* spec, oracle_error* error);
/* RotaryEmbeddingSpec::new (rope_kv.rs:69-112). */
int oracle_rotary_spec_check(const oracle_rotary_spec* spec, oracle_error* error);
/* RopePagedKvWriteSpec::new (rope_kv.rs:177-210); checks the rotary part first. */
int oracle_rope_kv_spec_check(const oracle_rope_kv_spec* spec, oracle_error* error);

/* ---- paged decode attention (attention.rs:169-426).
 * `call_dtype` is the element type of the entry point used (the reference has
 * one function per type and rejects a spec of another type). Buffers are
 * contiguous; *_len are element counts and are validated like slice lengths.
 * threads <= 1 reproduces the reference's single-threaded loop; threads > 1
 * runs the same per-(sequence, head) arithmetic under OpenMP. */
int oracle_paged_decode_attention(
    int32_t call_dtype, const void* query, uint64_t query_len,
    const void* key_cache, uint64_t key_cache_len, const void* value_cache,
    uint64_t value_cache_len, const int64_t* block_tables,
    uint64_t block_tables_len, const int64_t* sequence_lengths,
    uint64_t sequence_lengths_len, void* output, uint64_t output_len,
    const oracle_decode_spec* spec, int32_t threads, oracle_error* error);

/* Extension (parity unpinned; the reference's design note names both as later
 * contract fields, docs/design/paged-decode-attention.md:42-52): options of the
 * two decode functions, process-wide, not thread-safe against running calls.
 * sliding_window W > 0: a query sees only the last W positions of its sequence.
 * logits_soft_cap c > 0: each scaled score s becomes c * tanh(s / c) before the
 * softmax. (0, 0) restores the reference's arithmetic. Returns 0, or 1 for a
 * negative or non-finite cap. */
int oracle_set_decode_options(uint64_t sliding_window, double logits_soft_cap);

/* Extension (parity unpinned): the caches hold FP8 E4M3FN bytes; each element
 * is decoded to F32, multiplied in F32 by its static scale (scale_stride 0 =
 * per tensor, 1 = per KV head), and then fed to the same F64 attention. */
int oracle_paged_decode_attention_fp8(
    int32_t call_dtype, const void* query, uint64_t query_len,
    const uint8_t* key_cache, uint64_t key_cache_len,
    const uint8_t* value_cache, uint64_t value_cache_len,
    const float* key_scales, const float* value_scales, uint32_t scale_stride,
    const int64_t* block_tables, uint64_t block_tables_len,
    const int64_t* sequence_lengths, uint64_t sequence_lengths_len,
    void* output, uint64_t output_len, const oracle_decode_spec* spec,
    int32_t threads, oracle_error* error);

/* ---- rotary embedding and fused RoPE + paged-KV write (rope_kv.rs:254-777) */
int oracle_rotary_embedding(int32_t call_dtype, void* query, uint64_t query_len,
                            void* key, uint64_t key_len,
                            const int64_t* positions, uint64_t positions_len,
                            const void* cos_sin_cache, uint64_t cos_sin_len,
                            const oracle_rotary_spec* spec, oracle_error* error);

int oracle_rope_paged_kv_write(
    int32_t call_dtype, void* query, uint64_t query_len, void* key,
    uint64_t key_len, const void* value, uint64_t value_len,
    const int64_t* positions, uint64_t positions_len,
    const void* cos_sin_cache, uint64_t cos_sin_len, void* key_cache,
    uint64_t key_cache_len, void* value_cache, uint64_t value_cache_len,
    const int64_t* slot_mapping, uint64_t slot_mapping_len,
    const oracle_rope_kv_spec* spec, oracle_error* error);

int oracle_rope_paged_kv_write_fp8(
    int32_t call_dtype, void* query, uint64_t query_len, void* key,
    uint64_t key_len, const void* value, uint64_t value_len,
    const int64_t* positions, uint64_t positions_len,
    const void* cos_sin_cache, uint64_t cos_sin_len, uint8_t* key_cache,
    uint64_t key_cache_len, uint8_t* value_cache, uint64_t value_cache_len,
    const int64_t* slot_mapping, uint64_t slot_mapping_len,
    const float* key_scales, uint64_t key_scales_len,
    const float* value_scales, uint64_t value_scales_len,
    const oracle_rope_kv_spec* spec, oracle_error* error);

/* Threads OpenMP would use (1 when built without it). */
int oracle_max_threads(void);

#ifdef __cplusplus
}
#endif

#endif /* LOOM_ORACLE_H_ */
