/*
 * Launch ABI of the B200 paged-decode library (plain C, no framework types).
 *
 * Part 1 re-declares, symbol for symbol, the hot-path entry points of the
 * reference's internal launch header
 * (crates/loom-cuda-sys/cuda/include/loom_cuda.h): its dispatch layer
 * (crates/loom-cuda/src/{attention_dispatch,rope_kv_dispatch}.rs) binds to
 * exactly these names and argument lists, so it links against this library
 * unchanged. Part 2 adds entry points in the same style for what the reference
 * does not have: any cache stride order (HND as well as NHD), FP8 E4M3 caches
 * read with the dequantisation fused into the load, contexts of any length,
 * partial (O, max, sum) states and their merge.
 *
 * Conventions shared by every function here:
 *  - all pointers are device pointers valid on the current device;
 *  - 16-bit element types travel as uint16_t*; strides count ELEMENTS;
 *  - the call only enqueues work on `stream`; it never allocates, frees or
 *    synchronises;
 *  - the return value is a LoomCudaStatus;
 *  - device metadata (lengths, block ids, positions, slots) is trusted engine
 *    state; the kernels only guard against reading or writing out of bounds.
 */
#ifndef LOOM_LAUNCH_H_
#define LOOM_LAUNCH_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* loom_cuda.h:10-16 */
enum LoomCudaStatus {
  LOOM_CUDA_SUCCESS = 0,
  LOOM_CUDA_INVALID_ARGUMENT = 1,
  LOOM_CUDA_UNSUPPORTED = 2,
  LOOM_CUDA_LAUNCH_ERROR = 3,
  LOOM_CUDA_UNAVAILABLE = 4,
};

/* loom_cuda.h:18-21 */
enum LoomCudaKvCacheEncoding {
  LOOM_CUDA_KV_CACHE_NATIVE = 0,
  LOOM_CUDA_KV_CACHE_FP8_E4M3 = 1,
};

/* loom_cuda.h:23 */
const char* loom_cuda_status_string(int status);

/* ====================================================================== *
 * Part 1: the reference's symbols
 * ====================================================================== */

/*
 * Paged MQA/GQA decode, one query token per sequence (loom_cuda.h:182-210).
 * query/output: contiguous [sequences, query_heads, dim]. Caches: dense-inner
 * NHD [block_size, kv_heads, dim] with a free element stride between blocks.
 * block_tables [sequences, max_blocks_per_sequence] and sequence_lengths
 * [sequences] are int32. Unlike the reference there is no 1024-token cap:
 * max_sequence_length is bounded only by the table capacity.
 */
#define LOOM_DECLARE_DECODE(suffix, scalar)                                     \
  int loom_cuda_paged_decode_attention_##suffix(                                \
      const scalar* query, const scalar* key_cache, const scalar* value_cache,  \
      const int32_t* block_tables, const int32_t* sequence_lengths,             \
      scalar* output, uint32_t sequences, uint32_t query_heads,                 \
      uint32_t kv_heads, uint32_t head_size, uint32_t value_head_size,          \
      uint32_t num_blocks, uint32_t block_size, uint64_t key_block_stride,      \
      uint64_t value_block_stride, uint32_t max_blocks_per_sequence,            \
      uint32_t max_sequence_length, float scale, void* stream);
LOOM_DECLARE_DECODE(f32, float)
LOOM_DECLARE_DECODE(f16, uint16_t)
LOOM_DECLARE_DECODE(bf16, uint16_t)
#undef LOOM_DECLARE_DECODE

/*
 * Split-K sizing (loom_cuda.h:217-220). Returns the F32 element count of the
 * caller-owned workspace that the split-K entry points below need for this
 * shape, or 0 when the shape should use the workspace-free entry points above
 * (a context so short that one partition covers it).
 */
uint64_t loom_cuda_paged_decode_attention_split_k_workspace_elements(
    uint32_t sequences, uint32_t query_heads, uint32_t kv_heads,
    uint32_t head_size, uint32_t value_head_size, uint32_t max_sequence_length);

/*
 * Split-K decode (loom_cuda.h:222-250): a partial kernel over KV partitions
 * followed by a log-sum-exp merge kernel. `workspace` holds at least
 * `workspace_elements` floats as reported by the sizing function.
 */
#define LOOM_DECLARE_DECODE_SPLIT_K(suffix, scalar)                             \
  int loom_cuda_paged_decode_attention_split_k_##suffix(                        \
      const scalar* query, const scalar* key_cache, const scalar* value_cache,  \
      const int32_t* block_tables, const int32_t* sequence_lengths,             \
      scalar* output, float* workspace, uint64_t workspace_elements,            \
      uint32_t sequences, uint32_t query_heads, uint32_t kv_heads,              \
      uint32_t head_size, uint32_t value_head_size, uint32_t num_blocks,        \
      uint32_t block_size, uint64_t key_block_stride,                           \
      uint64_t value_block_stride, uint32_t max_blocks_per_sequence,            \
      uint32_t max_sequence_length, float scale, void* stream);
LOOM_DECLARE_DECODE_SPLIT_K(f32, float)
LOOM_DECLARE_DECODE_SPLIT_K(f16, uint16_t)
LOOM_DECLARE_DECODE_SPLIT_K(bf16, uint16_t)
#undef LOOM_DECLARE_DECODE_SPLIT_K

/*
 * Fused in-place RoPE on Q and K plus the paged write of the rotated K and of
 * V (loom_cuda.h:264-312). Q/K/V are [tokens, heads, dim] views with unit dim
 * stride and explicit token/head strides (packed QKV needs no copy).
 * cos_sin_cache is contiguous [max_position, rotary_dim], cosines then sines.
 * The caches are [blocks, block_size, kv_heads, dim] with explicit strides, so
 * NHD and HND both fit. slot_mapping has cache_tokens <= tokens entries; a
 * negative slot, or a token beyond cache_tokens, is rotated but not written.
 * cache_encoding is a LoomCudaKvCacheEncoding; for FP8 the stored byte is
 * e4m3(round_to_storage(x) / scale), scale_stride 0 = one scale, 1 = per head.
 */
#define LOOM_DECLARE_ROPE_WRITE(suffix, scalar)                                 \
  int loom_cuda_rope_paged_kv_write_##suffix(                                   \
      scalar* query, scalar* key, const scalar* value,                          \
      const int64_t* positions, const scalar* cos_sin_cache, void* key_cache,   \
      void* value_cache, const float* key_scales, const float* value_scales,    \
      const int64_t* slot_mapping, uint32_t tokens, uint32_t cache_tokens,      \
      uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,              \
      uint32_t value_head_size, uint32_t rotary_dim, uint32_t max_position,     \
      uint32_t num_blocks, uint32_t block_size, uint32_t cache_encoding,        \
      uint32_t scale_stride, uint64_t query_token_stride,                       \
      uint64_t query_head_stride, uint64_t key_token_stride,                    \
      uint64_t key_head_stride, uint64_t value_token_stride,                    \
      uint64_t value_head_stride, uint64_t key_cache_block_stride,              \
      uint64_t key_cache_page_stride, uint64_t key_cache_head_stride,           \
      uint64_t value_cache_block_stride, uint64_t value_cache_page_stride,      \
      uint64_t value_cache_head_stride, uint32_t is_neox, void* stream);
LOOM_DECLARE_ROPE_WRITE(f32, float)
LOOM_DECLARE_ROPE_WRITE(f16, uint16_t)
LOOM_DECLARE_ROPE_WRITE(bf16, uint16_t)
#undef LOOM_DECLARE_ROPE_WRITE

/* ====================================================================== *
 * Part 2: additions (no counterpart in the reference; same conventions)
 * ====================================================================== */

/*
 * Everything a decode launch needs, in one plain struct, so that the additive
 * entry points do not multiply into one symbol per combination. Zero-fill it,
 * then set the fields; `struct_size` must be sizeof(LoomDecodeArgs) (or
 * LOOM_DECODE_ARGS_BASE_SIZE, see the end of the struct).
 */
typedef struct LoomDecodeArgs {
  uint32_t struct_size;
  uint32_t dtype;          /* 0 = F32, 1 = F16, 2 = BF16: query/output type */
  uint32_t cache_encoding; /* LoomCudaKvCacheEncoding */
  uint32_t scale_stride;   /* FP8 only: 0 = per tensor, 1 = per KV head */
  const void* query;       /* [sequences, query_heads, head_size]; see strides below */
  const void* key_cache;   /* native: same type as query; FP8: bytes */
  const void* value_cache;
  const float* key_scales; /* FP8 only */
  const float* value_scales;
  const int32_t* block_tables;     /* [sequences, max_blocks_per_sequence] */
  const int32_t* sequence_lengths; /* [sequences] */
  void* output;            /* [sequences, query_heads, value_head_size], or   */
                           /* F32 states when `emit_state` is set            */
  float* workspace;        /* null = single pass over each sequence */
  uint64_t workspace_elements;
  uint32_t sequences, query_heads, kv_heads, head_size, value_head_size;
  uint32_t num_blocks, block_size, max_blocks_per_sequence, max_sequence_length;
  uint32_t partition_tokens; /* 0 = balanced persistent kernel where possible; */
                             /* else fixed partitions of this multiple of 16   */
  uint64_t key_block_stride, key_page_stride, key_head_stride;
  uint64_t value_block_stride, value_page_stride, value_head_stride;
  /* Element strides of `query` between sequences and between heads; 0 and 0
   * mean contiguous. A rotated Q that is still a view of a packed QKV row can
   * be read in place this way. */
  uint64_t query_token_stride, query_head_stride;
  float scale;
  uint32_t emit_state;     /* 1 = write [sequences, query_heads, Dv + 2] F32   */
                           /* states (O unnormalised, max, sum) instead of O  */
  void* stream;
  /* Options the reference names as later contract fields
   * (docs/design/paged-decode-attention.md:42-52). Added at the end: a caller
   * built against the struct without them passes its smaller struct_size
   * (LOOM_DECODE_ARGS_BASE_SIZE) and gets both off. They apply to the
   * single-token decode; the multi-token entry points refuse them. */
  uint32_t sliding_window; /* W > 0: the query sees only the last W tokens of  */
                           /* its sequence (positions length - W .. length - 1) */
  float logits_soft_cap;   /* c > 0: every scaled score s becomes              */
                           /* c * tanh(s / c) before the softmax               */
  uint32_t flags;          /* LOOM_DECODE_* promises of the caller, see below  */
  uint32_t reserved;       /* 0 */
} LoomDecodeArgs;

/*
 * LoomDecodeArgs.flags: promises by the caller that let the launch skip work;
 * without them nothing is assumed.
 *
 * LOOM_DECODE_STABLE_METADATA: block_tables and sequence_lengths were written
 *   before the operation that precedes this launch in the stream began (in a
 *   serving step: before the RoPE + KV-write launch). The balanced kernel then
 *   reads them, and plans its share of the batch, while that preceding kernel
 *   is still running; the query, the caches and the outputs are still only
 *   touched after it has completed.
 */
#define LOOM_DECODE_STABLE_METADATA 2u

/* struct_size of the LoomDecodeArgs layout that ends with `stream`. */
#define LOOM_DECODE_ARGS_BASE_SIZE ((uint32_t)offsetof(LoomDecodeArgs, sliding_window))

/* Copies a caller's LoomDecodeArgs of either known layout into `out` in the
 * current layout (options off for the base layout). Returns 1, or 0 for a null
 * pointer or an unknown struct_size. Host only; every entry point that takes a
 * LoomDecodeArgs reads it through this. */
int loom_cuda_read_decode_args(const LoomDecodeArgs* args, LoomDecodeArgs* out);

/* Partition length (tokens) the fixed-partition kernels default to. */
uint32_t loom_cuda_paged_decode_default_partition_tokens(
    uint32_t sequences, uint32_t kv_heads, uint32_t max_sequence_length);

/*
 * F32 workspace elements of a partitioned decode. partition_tokens 0 sizes for
 * the library's own choice (the balanced persistent kernel when the shape
 * allows it, fixed partitions of the default length otherwise; the size
 * covers both). A non-zero multiple of 16 sizes for fixed partitions of that
 * length: sequences * query_heads * ceil(max_sequence_length / partition) *
 * (value_head_size + 2). Returns 0 if the arguments are invalid or overflow.
 * The balanced kernel's share depends on the SM count of the current device.
 */
uint64_t loom_cuda_paged_decode_workspace_elements(
    uint32_t sequences, uint32_t query_heads, uint32_t kv_heads,
    uint32_t value_head_size, uint32_t max_sequence_length,
    uint32_t partition_tokens);

/* General decode: any stride order, native or FP8 cache, optional workspace. */
int loom_cuda_paged_decode_attention_ex(const LoomDecodeArgs* args);

/*
 * Merge of `parts` partial states per row into normalised output rows.
 * states: [parts, rows, value_head_size + 2] F32, each row holding the
 * unnormalised O (value_head_size floats), then the running maximum of the
 * scaled scores (natural-log units) and the sum of exp(score - max). A part
 * whose sum is 0 is ignored. out_dtype as in LoomDecodeArgs.dtype; output is
 * [rows, value_head_size]. This is the kernel the multi-GPU long-context mode
 * runs after gathering every GPU's states.
 */
int loom_cuda_merge_decode_states(const float* states, uint32_t parts,
                                  uint32_t rows, uint32_t value_head_size,
                                  uint32_t out_dtype, void* output,
                                  void* stream);

/*
 * Capability query (crates/loom-cuda/src/cuda_backend.rs:112-145 answers the
 * same question for the reference). Returns 1 if the decode shape runs here,
 * 0 if not; `reason`, when non-null, receives a short static string.
 */
int loom_cuda_supports_paged_decode(uint32_t dtype, uint32_t cache_encoding,
                                    uint32_t sequences, uint32_t query_heads,
                                    uint32_t kv_heads, uint32_t head_size,
                                    uint32_t value_head_size,
                                    uint32_t num_blocks, uint32_t block_size,
                                    uint32_t max_blocks_per_sequence,
                                    uint32_t max_sequence_length,
                                    const char** reason);

/* Name of the kernel family the last decode launch on this thread selected
 * ("mma16", "scalar", ...); for tests and profiling notes. */
const char* loom_cuda_last_decode_route(void);

/* The CUDA runtime error behind the last LOOM_CUDA_LAUNCH_ERROR that any launch
 * function of this library returned on this thread, and the runtime call it
 * came from ("cudaErrorInvalidValue at shared-memory limit of a decode kernel
 * (cudaFuncSetAttribute)", ...); "none" if there was none. Kernel launches,
 * shared-memory limits and device queries of the decode, RoPE, multi-token and
 * KV block movement paths all report here. With LOOM_DEBUG_LAUNCH set in the
 * environment the same text is printed on stderr when it happens. */
const char* loom_cuda_last_launch_failure(void);

/* Launches that the runtime refused with the programmatic-launch attribute and
 * that this library then issued as plain launches, since the process started.
 * 0 in a healthy process; a non-zero count makes a refused attribute visible
 * instead of silent. */
uint64_t loom_cuda_plain_launch_retries(void);

/*
 * How the balanced decode kernel fills its shared-memory rings: 0 (default)
 * uses the Tensor Memory Accelerator whenever the cache can be described by a
 * tensor map, and over an FP8 cache (up to 8 query heads per KV head, no window
 * or soft cap) the kernel whose copies are issued by a warp of their own; 1
 * always uses per-lane cp.async copies; 2 is 0 without that copy-issuing warp
 * (every computing warp feeds its own ring); 3 is 0 plus the tcgen05 kernel
 * (E4M3 operands read by the tensor cores straight from shared memory,
 * accumulators in tensor memory) for FP8 caches with head size 128 and up to 8
 * query heads per KV head; 4 is 0 without the kernel that, where the KV heads
 * come in multiples of eight (head size 128, FP8 cache, a workspace of the size
 * the workspace query returns), copies one 16-token block of eight KV heads per
 * copy and gives each computing warp one KV head. Process-wide; meant for
 * comparisons and as a switch to fall back on.
 */
int loom_cuda_set_decode_copy_engine(uint32_t engine);

/*
 * Programmatic dependent launch of every kernel of this library (no
 * counterpart in the reference). Process-wide.
 *   0  plain launches.
 *   1  (default) kernels carry the programmatic-serialisation launch attribute:
 *      their CTAs may become resident while the preceding kernel of the stream
 *      drains. Each kernel waits for that kernel to complete before its first
 *      access to global memory, so results never depend on the mode.
 */
int loom_cuda_set_programmatic_launch(uint32_t mode);

/*
 * The TMA-fed kernels bound every wait on a copy; if one ever expires the warp
 * concerned sets a flag on the device instead of hanging, starts no further
 * copy, gives the copies it has in flight one more bounded wait and does
 * nothing more (the rows of its work items are then wrong: the flag is the
 * status). This reads the flag of the current device into *value (0 = never
 * happened; otherwise bit 0 is set and the upper bits say which wait expired
 * first) and optionally clears it. Unlike the launch functions this call
 * synchronises with the device.
 */
int loom_cuda_decode_timeout_flag(uint32_t* value, uint32_t reset);

/*
 * Limit of those waits, for the decode kernels and the KV block movement
 * kernels alike. Process-wide, read at each launch.
 *   attempts         polls of a barrier before a wait gives up; 0 = each
 *                    kernel's default (about a second).
 *   unmatched_bytes  0 in service. A non-zero multiple of 16 is a self-test:
 *                    every copy barrier is armed for that many bytes more than
 *                    its copy delivers, so the first wait of every ring runs out
 *                    although the data arrives. With a small `attempts` the
 *                    expiry path (flag, no further copies, drain, return) is
 *                    exercised in microseconds and without any fault; results
 *                    of such a launch are invalid by construction.
 */
int loom_cuda_set_wait_policy(uint32_t attempts, uint32_t unmatched_bytes);

/*
 * Partitioned decode without a caller workspace. This entry point has no
 * counterpart in the reference.
 *
 * Who it is for: code that must run a split decode but has no means of getting
 * device memory when it does so. Typical cases are a serving engine that
 * claims its whole GPU budget at start-up and forbids allocation afterwards, a
 * latency-critical handler that will not risk the device-wide pause an
 * allocation may cause, and a host application that passes its plug-ins input
 * and output buffers only.
 *
 * What it does: the same as loom_cuda_paged_decode_attention_ex, with the
 * partial (O, max, sum) states kept in a block of device memory that is part of
 * the library itself. args->workspace and args->workspace_elements are
 * ignored; inputs and outputs are still the caller's. Neither this call nor
 * anything it reaches allocates or frees memory.
 *
 * Limits and rules:
 *  - the block holds 4,194,304 F32 elements (16 MiB) and exists once per GPU
 *    that loads the library, for the life of the process. A shape whose
 *    scratch need (loom_cuda_paged_decode_workspace_elements) is larger is
 *    refused with LOOM_CUDA_UNSUPPORTED and a message saying how much it
 *    needs;
 *  - the first call on each device looks up the block's device address (one
 *    runtime query, no allocation). Make that first call outside any stream
 *    capture;
 *  - the address is looked up, and remembered, for the device that is CURRENT
 *    when the call is made: make the device that owns args->stream current
 *    first, as for every other function of this header;
 *  - all calls on a device share the one block, and it keeps whatever the last
 *    call left there. No clearing is needed, because a call writes every word
 *    it later reads. Two such calls that can overlap on the GPU (different
 *    streams without an ordering between them) race on the block: serialise
 *    them.
 * error_text, if non-null, receives a NUL-terminated explanation of a failure
 * (up to error_capacity bytes). Returns a LoomCudaStatus.
 */
int loom_cuda_paged_decode_attention_built_in_scratch(
    const LoomDecodeArgs* args, char* error_text, uint64_t error_capacity);

/*
 * Multi-token queries (speculative verification, short chunked prefill) over
 * the single-token decode: the reference names them as a later contract field
 * (docs/design/paged-decode-attention.md:42-52). Writes the metadata of the
 * expanded problem: row s * query_tokens + t of expanded_block_tables
 * [sequences * query_tokens, max_blocks_per_sequence] is sequence s's table
 * row, and expanded_sequence_lengths[s * query_tokens + t] =
 * max(0, sequence_lengths[s] - (query_tokens - 1 - t)), where sequence_lengths
 * counts the context INCLUDING the query_tokens new tokens (already written to
 * the cache). A decode call on query rows [sequences * query_tokens, heads,
 * dim] with this metadata is causal attention of every new token; a length of
 * 0 yields a zero row.
 */
int loom_cuda_expand_query_tokens(const int32_t* block_tables,
                                  const int32_t* sequence_lengths,
                                  int32_t* expanded_block_tables,
                                  int32_t* expanded_sequence_lengths,
                                  uint32_t sequences, uint32_t query_tokens,
                                  uint32_t max_blocks_per_sequence,
                                  void* stream);

/*
 * Multi-token queries at one pass over the KV, in three launches.
 *  1. loom_cuda_multi_token_prepare: query [sequences, query_tokens,
 *     query_heads, head_size] (contiguous, dtype 0/1/2 = F32/F16/BF16) is
 *     packed as [sequences, kv_heads, query_tokens, group, head_size], and
 *     prefix_lengths[s] = max(0, sequence_lengths[s] - (query_tokens - 1)).
 *  2. An ordinary decode (loom_cuda_paged_decode_attention_ex) of the packed
 *     query as [sequences, query_tokens * query_heads, head_size] with
 *     prefix_lengths and emit_state = 1: the rows of a (sequence, KV head) pair
 *     form one GQA group over the prefix every one of them sees.
 *  3. loom_cuda_multi_token_finish: args as for the decode, but with the
 *     ORIGINAL query, block tables and sequence lengths (counting all new
 *     tokens), query_heads the per-token head count, and output [sequences,
 *     query_tokens, query_heads, value_head_size] of the query's type;
 *     prefix_states is what step 2 wrote. Each row's up to query_tokens - 1
 *     tail tokens are added to its state, the row is normalised and stored.
 *     workspace, partition_tokens, emit_state and the query strides of args
 *     are ignored. Head sizes up to 256; an FP8 cache needs a 16-bit query.
 */
int loom_cuda_multi_token_prepare(const void* query, void* packed_query,
                                  const int32_t* sequence_lengths,
                                  int32_t* prefix_lengths, uint32_t dtype,
                                  uint32_t sequences, uint32_t query_tokens,
                                  uint32_t query_heads, uint32_t kv_heads,
                                  uint32_t head_size, void* stream);
int loom_cuda_multi_token_finish(const LoomDecodeArgs* args,
                                 uint32_t query_tokens,
                                 const float* prefix_states);

/*
 * The three steps above as one call. args as for loom_cuda_multi_token_finish;
 * args->workspace / workspace_elements (may be null / 0 for short contexts)
 * serve the decode of step 2 and are sized with
 * loom_cuda_paged_decode_workspace_elements for query_tokens * query_heads
 * heads. Caller-owned scratch: packed_query (as many elements as the query),
 * prefix_lengths [sequences] and prefix_states [sequences, query_tokens *
 * query_heads, value_head_size + 2] F32.
 */
int loom_cuda_paged_multi_token_decode(const LoomDecodeArgs* args,
                                       uint32_t query_tokens,
                                       void* packed_query,
                                       int32_t* prefix_lengths,
                                       float* prefix_states);

/* ====================================================================== *
 * Exchange of partial decode states between the GPUs of one node
 *
 * No counterpart in the reference (docs/operator-catalog.md:109 lists
 * distributed split-KV as planned). For the long-context mode, in which every
 * GPU holds one block range of a sequence and produces partial (O, max, sum)
 * states (emit_state): instead of an all-gather by a communication library
 * followed by loom_cuda_merge_decode_states, every GPU PUSHES its states into
 * every peer's exchange buffer with plain stores over NVLink, and MERGES what
 * has arrived in its own buffer. One process per GPU; `world` GPUs, at most
 * LOOM_CUDA_PEER_EXCHANGE_MAX_RANKS.
 *
 * Set-up, once: every rank creates its buffer (device memory of the current
 * device, zeroed; this is the only allocating function of the library), sends
 * the returned handle bytes to the other ranks by any means, and opens theirs.
 * rank_buffers[r] is then rank r's buffer as this process sees it (its own
 * pointer for r == rank). Per step, on every rank, in this order on one stream:
 * push, then merge. Every rank must run every step: the kernels count steps in
 * the buffers and a rank that skips one leaves the others waiting (bounded: a
 * wait that runs out sets the buffer's error word, the step's rows are then
 * invalid; loom_cuda_peer_exchange_status reads it, and after an error every
 * rank resets its buffer and the ranks synchronise on the host before the next
 * step). states: [rows, value_head_size + 2] F32 as emit_state writes them,
 * 16-byte aligned, rows * (value_head_size + 2) a multiple of 4.
 * ====================================================================== */
#define LOOM_CUDA_PEER_EXCHANGE_MAX_RANKS 16
#define LOOM_CUDA_PEER_EXCHANGE_HANDLE_BYTES 64

/* Size of a rank's exchange buffer; 0 for an invalid shape. */
uint64_t loom_cuda_peer_exchange_bytes(uint32_t world, uint32_t rows,
                                       uint32_t value_head_size);
int loom_cuda_peer_exchange_create(uint64_t bytes, void** buffer,
                                   unsigned char* handle,
                                   uint64_t handle_capacity);
int loom_cuda_peer_exchange_open(const unsigned char* handle,
                                 uint64_t handle_bytes, void** buffer);
int loom_cuda_peer_exchange_close(void* peer_buffer);
int loom_cuda_peer_exchange_destroy(void* buffer);
/* Zeroes a rank's own buffer (step counters, arrivals, error) on `stream`. */
int loom_cuda_peer_exchange_reset(void* buffer, uint64_t bytes, void* stream);
/* Synchronous read of a rank's own buffer: steps completed, error word. */
int loom_cuda_peer_exchange_status(const void* buffer,
                                   uint64_t* completed_steps, uint32_t* error);
int loom_cuda_peer_exchange_push(const float* states,
                                 void* const* rank_buffers, uint32_t rank,
                                 uint32_t world, uint32_t rows,
                                 uint32_t value_head_size, void* stream);
/* out_dtype as LoomDecodeArgs.dtype; output [rows, value_head_size]. */
int loom_cuda_peer_exchange_merge(void* buffer, uint32_t world, uint32_t rows,
                                  uint32_t value_head_size, uint32_t out_dtype,
                                  void* output, void* stream);

/* ====================================================================== *
 * Part 3: KV block movement
 *
 * The reference names these operators as the next ones around its paged
 * cache (docs/operator-catalog.md:61: "KV block copy, swap, gather, scatter,
 * compact, and remap"; docs/operator-catalog.md:140) and has no symbol for
 * them yet. A block is what a block-table entry names: its K bytes are one
 * contiguous span of `block_bytes` bytes, its V bytes another, in any layout
 * (NHD, HND) and any element type. Sizes and strides of this part count
 * BYTES, because the movement is blind to the element type; spans, strides and
 * base pointers must be multiples of 16 bytes (LOOM_CUDA_UNSUPPORTED
 * otherwise). Block ids are device memory and trusted like block tables: a
 * pair that names a block outside its cache is skipped, nothing else is
 * checked on the device. A count of zero succeeds without a launch.
 * ====================================================================== */

/*
 * For every pair i: block block_pairs[2 i] of the source cache is copied over
 * block block_pairs[2 i + 1] of the destination cache, K and V. Source and
 * destination may be the same cache (copy-on-write of a shared prefix block,
 * compaction) or different allocations (gather into a dense staging buffer,
 * scatter back, migration between caches). Either cache may also lie in
 * pinned host memory (blocks swapped out on preemption, swapped in on resume):
 * the kernel then reads or writes it over PCIe with vector loads and stores;
 * memory the device cannot address is refused with
 * LOOM_CUDA_INVALID_ARGUMENT. No block may be both read and written, and no
 * destination may occur twice, in one call.
 */
int loom_cuda_kv_block_move(
    const void* source_key_cache, const void* source_value_cache,
    void* destination_key_cache, void* destination_value_cache,
    const int64_t* block_pairs, uint32_t pair_count, uint32_t source_blocks,
    uint32_t destination_blocks, uint64_t block_bytes,
    uint64_t source_key_block_stride, uint64_t source_value_block_stride,
    uint64_t destination_key_block_stride,
    uint64_t destination_value_block_stride, void* stream);

/*
 * How loom_cuda_kv_block_move and loom_cuda_kv_block_swap move bytes: 0
 * (default) stages 8 KB chunks through shared memory with the bulk-copy
 * engine (cp.async.bulk in, then out, no register round trip), 1 uses 16-byte
 * vector loads and stores. Process-wide; results are identical.
 */
int loom_cuda_set_kv_block_move_engine(uint32_t engine);

/*
 * The bulk-copy kernel bounds every wait on a copy; if one ever expired, a
 * flag on the current device is set and the affected launch left some
 * destinations unwritten. *value receives the flag; reset != 0 clears it.
 * Synchronous (a small device-to-host copy); never needed on a healthy device.
 */
int loom_cuda_kv_block_move_timeout_flag(uint32_t* value, uint32_t reset);

/*
 * For every pair i: blocks block_pairs[2 i] and block_pairs[2 i + 1] of one
 * cache exchange their contents, K and V. A block may occur in one pair only;
 * a pair of equal ids is left alone.
 */
int loom_cuda_kv_block_swap(void* key_cache, void* value_cache,
                            const int64_t* block_pairs, uint32_t pair_count,
                            uint32_t num_blocks, uint64_t block_bytes,
                            uint64_t key_block_stride,
                            uint64_t value_block_stride, void* stream);

/*
 * After blocks have moved: block_tables[i] = new_block_ids[block_tables[i]]
 * for each of the `entries` table entries whose id lies in [0, num_blocks);
 * other entries (negative sentinels in unused tails) are left alone.
 * new_block_ids has num_blocks elements.
 */
int loom_cuda_block_table_remap(int32_t* block_tables, uint64_t entries,
                                const int32_t* new_block_ids,
                                uint32_t num_blocks, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* LOOM_LAUNCH_H_ */
