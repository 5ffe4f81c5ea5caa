// Multi-token queries (speculative verification, short chunked prefill) on top
// of the single-token decode kernels.
//
// The reference's decode contract is one query token per sequence and names
// "multi-token speculative or chunked-prefill queries" as a later contract
// field (docs/design/paged-decode-attention.md:42-52). Causal attention of
// `query_tokens` new tokens per sequence is the single-token problem
// `query_tokens` times over the same pages: token t of a sequence whose context
// (all new tokens included) is `length` attends to the first
// length - (query_tokens - 1 - t) cached tokens. This file holds the one kernel
// that writes that expanded problem's metadata: row s * query_tokens + t of the
// output gets sequence s's block-table row and the shortened length (0 when the
// sequence is shorter than its query-token count allows, which the decode
// kernels answer with a zero row). The decode kernels then run unchanged on
// sequences * query_tokens rows. That form works for every shape but streams a
// sequence's pages once per query token; the second half of this file holds
// the one-pass form (the tokens' rows beside the GQA group over the common
// prefix, then a short per-token tail).

#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/loom_launch.h"
#include "launch_util.cuh"

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
expand_query_tokens_kernel(const int32_t* __restrict__ block_tables, const int32_t* __restrict__ lengths,
                           int32_t* __restrict__ out_tables, int32_t* __restrict__ out_lengths, uint32_t sequences,
                           uint32_t query_tokens, uint32_t max_blocks) {
  loom_launch::grid_dependency_wait();
  const uint64_t rows = (uint64_t)sequences * query_tokens;
  const uint64_t entries = rows * max_blocks;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < entries; i += (uint64_t)gridDim.x * kThreads) {
    const uint64_t row = i / max_blocks;
    const uint32_t column = (uint32_t)(i - row * max_blocks);
    const uint32_t sequence = (uint32_t)(row / query_tokens);
    out_tables[i] = block_tables[(uint64_t)sequence * max_blocks + column];
    if (column == 0) {
      const uint32_t token = (uint32_t)(row - (uint64_t)sequence * query_tokens);
      const int64_t visible = (int64_t)lengths[sequence] - (int64_t)(query_tokens - 1u - token);
      out_lengths[row] = visible > 0 ? (int32_t)visible : 0;
    }
  }
}

}  // namespace

extern "C" int loom_cuda_expand_query_tokens(const int32_t* block_tables, const int32_t* sequence_lengths,
                                             int32_t* expanded_block_tables, int32_t* expanded_sequence_lengths,
                                             uint32_t sequences, uint32_t query_tokens,
                                             uint32_t max_blocks_per_sequence, void* stream) {
  if (!block_tables || !sequence_lengths || !expanded_block_tables || !expanded_sequence_lengths || sequences == 0 ||
      query_tokens == 0 || max_blocks_per_sequence == 0) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const uint64_t rows = (uint64_t)sequences * query_tokens;
  if (rows > 0x7fffffffull) return LOOM_CUDA_INVALID_ARGUMENT;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return LOOM_CUDA_UNAVAILABLE;
  }
  const uint64_t entries = rows * max_blocks_per_sequence;
  const uint64_t wanted = (entries + kThreads - 1) / kThreads;
  const uint64_t resident = (uint64_t)sms * 8u;
  const cudaError_t status = loom_launch::launch(
      expand_query_tokens_kernel, dim3((uint32_t)(wanted < resident ? wanted : resident)), dim3(kThreads), 0,
      static_cast<cudaStream_t>(stream), block_tables, sequence_lengths, expanded_block_tables,
      expanded_sequence_lengths, sequences, query_tokens, max_blocks_per_sequence);
  return loom_launch::failed(status, "query-token expansion kernel launch");
}

// ---- one pass over the KV for all query tokens ------------------------------------------
//
// The Tq x group rows of a (sequence, KV head) pair all attend to the common
// prefix of length - (Tq - 1) tokens; row (t, g) sees t more tokens after it.
// So: (1) `prepare` packs the queries as [sequences, kv_heads, Tq, group, dim],
// which makes the rows of a pair one GQA group of Tq x group heads, and writes
// the prefix lengths; (2) the ordinary decode runs once over the prefix with
// that widened group and emits F32 (O, max, sum) states; (3) `finish` adds each
// row's at most Tq - 1 tail tokens to its state, normalises and stores the row
// at [sequence, token, head]. The KV is streamed once per 8 or 16 rows of a pair
// (the decode kernels' rows per work item) instead of once per query token.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace {

template <typename T>
__device__ __forceinline__ float to_float(T value);
template <>
__device__ __forceinline__ float to_float<float>(float value) { return value; }
template <>
__device__ __forceinline__ float to_float<__half>(__half value) { return __half2float(value); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 value) { return __bfloat162float(value); }

__device__ __forceinline__ float e4m3_to_float(uint8_t byte) {
  const __half_raw raw = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&raw));
}

template <typename T>
__device__ __forceinline__ T from_float(float value);
template <>
__device__ __forceinline__ float from_float<float>(float value) { return value; }
template <>
__device__ __forceinline__ __half from_float<__half>(float value) { return __float2half_rn(value); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float value) { return __float2bfloat16_rn(value); }

// packed[s][kv][t][g][:] = query[s][t][kv * group + g][:]; prefix_lengths[s] = max(0, length - (Tq - 1)).
template <typename T>
__global__ void __launch_bounds__(kThreads)
multi_token_prepare_kernel(const T* __restrict__ query, T* __restrict__ packed, const int32_t* __restrict__ lengths,
                           int32_t* __restrict__ prefix_lengths, uint32_t sequences, uint32_t query_tokens,
                           uint32_t query_heads, uint32_t kv_heads, uint32_t head_size) {
  loom_launch::grid_dependency_wait();
  const uint32_t group = query_heads / kv_heads;
  const uint64_t elements = (uint64_t)sequences * query_tokens * query_heads * head_size;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < elements; i += (uint64_t)gridDim.x * kThreads) {
    const uint32_t d = (uint32_t)(i % head_size);
    uint64_t rest = i / head_size;
    const uint32_t g = (uint32_t)(rest % group);
    rest /= group;
    const uint32_t t = (uint32_t)(rest % query_tokens);
    rest /= query_tokens;
    const uint32_t kv = (uint32_t)(rest % kv_heads);
    const uint64_t s = rest / kv_heads;
    packed[i] = query[((s * query_tokens + t) * query_heads + (uint64_t)kv * group + g) * head_size + d];
    if (i < sequences) {
      const int64_t prefix = (int64_t)lengths[i] - (int64_t)(query_tokens - 1u);
      prefix_lengths[i] = prefix > 0 ? (int32_t)prefix : 0;
    }
  }
}

struct FinishParams {
  const void* query;          // [sequences, Tq, query_heads, head_size]
  const float* states;        // [sequences, kv_heads * Tq * group, value_head_size + 2]
  const void* key_cache;
  const void* value_cache;
  const float* key_scales;
  const float* value_scales;
  const int32_t* block_tables;
  const int32_t* lengths;
  void* output;               // [sequences, Tq, query_heads, value_head_size]
  uint64_t key_block, key_page, key_head, value_block, value_page, value_head;  // element strides
  uint32_t sequences, query_tokens, query_heads, kv_heads, head_size, value_head_size;
  uint32_t num_blocks, block_size, max_blocks, scale_stride;
  float scale;
};

constexpr int kFinishWarps = 4;
constexpr int kMaxPerLane = 8;  // head sizes up to 256

// One warp per output row (sequence, token, query head).
template <typename T, bool kFp8>
__global__ void __launch_bounds__(kFinishWarps * 32) multi_token_finish_kernel(const FinishParams p) {
  loom_launch::grid_dependency_wait();
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t row = (uint64_t)blockIdx.x * kFinishWarps + (threadIdx.x >> 5);
  const uint64_t rows = (uint64_t)p.sequences * p.query_tokens * p.query_heads;
  if (row >= rows) return;
  const uint32_t head = (uint32_t)(row % p.query_heads);
  const uint32_t token = (uint32_t)((row / p.query_heads) % p.query_tokens);
  const uint32_t sequence = (uint32_t)(row / ((uint64_t)p.query_heads * p.query_tokens));
  const uint32_t group = p.query_heads / p.kv_heads;
  const uint32_t kv = head / group, g = head % group;

  const int64_t length = p.lengths[sequence];
  const int64_t prefix = length - (int64_t)(p.query_tokens - 1u) > 0 ? length - (int64_t)(p.query_tokens - 1u) : 0;
  const int64_t visible = length - (int64_t)(p.query_tokens - 1u - token) > 0
                              ? length - (int64_t)(p.query_tokens - 1u - token) : 0;

  const uint32_t wide = p.value_head_size + 2u;
  const float* state = p.states + ((uint64_t)sequence * p.query_tokens * p.query_heads +
                                   ((uint64_t)kv * p.query_tokens + token) * group + g) * wide;
  float sum = state[p.value_head_size + 1];
  float top = sum > 0.0f ? state[p.value_head_size] : -INFINITY;
  if (!(sum > 0.0f)) sum = 0.0f;
  float acc[kMaxPerLane];
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const uint32_t d = lane + 32u * j;
    acc[j] = (d < p.value_head_size && sum > 0.0f) ? state[d] : 0.0f;
  }
  const T* q = static_cast<const T*>(p.query) + row * p.head_size;
  float qv[kMaxPerLane];
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const uint32_t d = lane + 32u * j;
    qv[j] = d < p.head_size ? to_float<T>(q[d]) : 0.0f;
  }
  float key_scale = 1.0f, value_scale = 1.0f;
  if constexpr (kFp8) {
    key_scale = p.key_scales[(uint64_t)kv * p.scale_stride];
    value_scale = p.value_scales[(uint64_t)kv * p.scale_stride];
  }

  for (int64_t position = prefix; position < visible; ++position) {
    const int64_t logical = position / p.block_size;
    if (logical >= (int64_t)p.max_blocks) break;
    const int32_t block = p.block_tables[(uint64_t)sequence * p.max_blocks + logical];
    if (block < 0 || (uint32_t)block >= p.num_blocks) continue;
    const uint32_t page = (uint32_t)(position - logical * p.block_size);
    const uint64_t key_at = (uint64_t)block * p.key_block + (uint64_t)page * p.key_page + (uint64_t)kv * p.key_head;
    const uint64_t value_at =
        (uint64_t)block * p.value_block + (uint64_t)page * p.value_page + (uint64_t)kv * p.value_head;
    float dot = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const uint32_t d = lane + 32u * j;
      if (d < p.head_size) {
        float k;
        if constexpr (kFp8) k = e4m3_to_float(static_cast<const uint8_t*>(p.key_cache)[key_at + d]);
        else k = to_float<T>(static_cast<const T*>(p.key_cache)[key_at + d]);
        dot = fmaf(qv[j], k, dot);
      }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, offset);
    const float score = dot * p.scale * key_scale;
    const float raised = fmaxf(top, score);
    const float keep = top == -INFINITY ? 0.0f : __expf(top - raised);
    const float weight = __expf(score - raised);
    sum = sum * keep + weight;
    top = raised;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const uint32_t d = lane + 32u * j;
      if (d < p.value_head_size) {
        float v;
        if constexpr (kFp8) v = e4m3_to_float(static_cast<const uint8_t*>(p.value_cache)[value_at + d]) * value_scale;
        else v = to_float<T>(static_cast<const T*>(p.value_cache)[value_at + d]);
        acc[j] = acc[j] * keep + weight * v;
      }
    }
  }
  T* out = static_cast<T*>(p.output) + row * p.value_head_size;
  const float inverse = sum > 0.0f ? 1.0f / sum : 0.0f;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const uint32_t d = lane + 32u * j;
    if (d < p.value_head_size) out[d] = from_float<T>(acc[j] * inverse);
  }
}

int device_sms() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return sms;
}

int launch_status(cudaError_t status) { return loom_launch::failed(status, "multi-token kernel launch"); }

}  // namespace

extern "C" {

int loom_cuda_multi_token_prepare(const void* query, void* packed_query, const int32_t* sequence_lengths,
                                  int32_t* prefix_lengths, uint32_t dtype, uint32_t sequences,
                                  uint32_t query_tokens, uint32_t query_heads, uint32_t kv_heads,
                                  uint32_t head_size, void* stream) {
  if (!query || !packed_query || !sequence_lengths || !prefix_lengths || sequences == 0 || query_tokens == 0 ||
      query_heads == 0 || kv_heads == 0 || head_size == 0 || query_heads % kv_heads != 0 || dtype > 2) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const int sms = device_sms();
  if (sms <= 0) return LOOM_CUDA_UNAVAILABLE;
  const uint64_t elements = (uint64_t)sequences * query_tokens * query_heads * head_size;
  const uint64_t wanted = (elements + kThreads - 1) / kThreads;
  const uint64_t resident = (uint64_t)sms * 8u;
  const dim3 grid((uint32_t)(wanted < resident ? wanted : resident));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define LOOM_PREPARE(type)                                                                                      \
  launch_status(loom_launch::launch(multi_token_prepare_kernel<type>, grid, dim3(kThreads), 0, s,               \
                                    static_cast<const type*>(query), static_cast<type*>(packed_query),          \
                                    sequence_lengths, prefix_lengths, sequences, query_tokens, query_heads,     \
                                    kv_heads, head_size))
  if (dtype == 0) return LOOM_PREPARE(float);
  if (dtype == 1) return LOOM_PREPARE(__half);
  return LOOM_PREPARE(__nv_bfloat16);
#undef LOOM_PREPARE
}

int loom_cuda_multi_token_finish(const LoomDecodeArgs* caller_args, uint32_t query_tokens,
                                 const float* prefix_states) {
  LoomDecodeArgs current;
  if (!loom_cuda_read_decode_args(caller_args, &current)) return LOOM_CUDA_INVALID_ARGUMENT;
  const LoomDecodeArgs* args = &current;
  // a window or a soft cap per query token is not part of the multi-token forms
  if (args->sliding_window != 0 || args->logits_soft_cap != 0.0f) return LOOM_CUDA_UNSUPPORTED;
  if (prefix_states == nullptr ||
      query_tokens == 0 || !args->query || !args->key_cache || !args->value_cache || !args->block_tables ||
      !args->sequence_lengths || !args->output || args->sequences == 0 || args->query_heads == 0 ||
      args->kv_heads == 0 || args->query_heads % args->kv_heads != 0 || args->block_size == 0 ||
      args->num_blocks == 0 || args->max_blocks_per_sequence == 0 || args->dtype > 2) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const bool fp8 = args->cache_encoding == LOOM_CUDA_KV_CACHE_FP8_E4M3;
  if (fp8 && (!args->key_scales || !args->value_scales || args->scale_stride > 1)) return LOOM_CUDA_INVALID_ARGUMENT;
  if (args->head_size == 0 || args->head_size > 32u * kMaxPerLane || args->value_head_size == 0 ||
      args->value_head_size > 32u * kMaxPerLane || (fp8 && args->dtype == 0)) {
    return LOOM_CUDA_UNSUPPORTED;
  }
  FinishParams p{};
  p.query = args->query;
  p.states = prefix_states;
  p.key_cache = args->key_cache;
  p.value_cache = args->value_cache;
  p.key_scales = args->key_scales;
  p.value_scales = args->value_scales;
  p.block_tables = args->block_tables;
  p.lengths = args->sequence_lengths;
  p.output = args->output;
  p.key_block = args->key_block_stride;
  p.key_page = args->key_page_stride;
  p.key_head = args->key_head_stride;
  p.value_block = args->value_block_stride;
  p.value_page = args->value_page_stride;
  p.value_head = args->value_head_stride;
  p.sequences = args->sequences;
  p.query_tokens = query_tokens;
  p.query_heads = args->query_heads;
  p.kv_heads = args->kv_heads;
  p.head_size = args->head_size;
  p.value_head_size = args->value_head_size;
  p.num_blocks = args->num_blocks;
  p.block_size = args->block_size;
  p.max_blocks = args->max_blocks_per_sequence;
  p.scale_stride = args->scale_stride;
  p.scale = args->scale;
  const uint64_t rows = (uint64_t)args->sequences * query_tokens * args->query_heads;
  const uint64_t ctas = (rows + kFinishWarps - 1) / kFinishWarps;
  if (ctas > 0x7fffffffull) return LOOM_CUDA_INVALID_ARGUMENT;
  const dim3 grid((uint32_t)ctas), block(kFinishWarps * 32);
  cudaStream_t s = static_cast<cudaStream_t>(args->stream);
#define LOOM_FINISH(type, is_fp8) \
  launch_status(loom_launch::launch(multi_token_finish_kernel<type, is_fp8>, grid, block, 0, s, p))
  if (fp8) return args->dtype == 1 ? LOOM_FINISH(__half, true) : LOOM_FINISH(__nv_bfloat16, true);
  if (args->dtype == 0) return LOOM_FINISH(float, false);
  if (args->dtype == 1) return LOOM_FINISH(__half, false);
  return LOOM_FINISH(__nv_bfloat16, false);
#undef LOOM_FINISH
}

}  // extern "C"

// The three launches as one call. `args` describes the multi-token problem as
// loom_cuda_multi_token_finish takes it (original query, tables, lengths; output
// [sequences, query_tokens, query_heads, value_head_size]); its workspace, if
// any, serves the widened decode (size it for query_tokens * query_heads heads).
extern "C" int loom_cuda_paged_multi_token_decode(const LoomDecodeArgs* caller_args, uint32_t query_tokens,
                                                  void* packed_query, int32_t* prefix_lengths,
                                                  float* prefix_states) {
  LoomDecodeArgs current;
  if (!loom_cuda_read_decode_args(caller_args, &current) || query_tokens == 0 || !packed_query ||
      !prefix_lengths || !prefix_states) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const LoomDecodeArgs* args = &current;
  if (args->sliding_window != 0 || args->logits_soft_cap != 0.0f) return LOOM_CUDA_UNSUPPORTED;
  if ((uint64_t)args->query_heads * query_tokens > 0xffffffffull) return LOOM_CUDA_INVALID_ARGUMENT;
  int status = loom_cuda_multi_token_prepare(args->query, packed_query, args->sequence_lengths, prefix_lengths,
                                             args->dtype, args->sequences, query_tokens, args->query_heads,
                                             args->kv_heads, args->head_size, args->stream);
  if (status != LOOM_CUDA_SUCCESS) return status;
  LoomDecodeArgs prefix = *args;
  prefix.query = packed_query;
  prefix.query_heads = args->query_heads * query_tokens;
  prefix.query_token_stride = 0;
  prefix.query_head_stride = 0;
  prefix.sequence_lengths = prefix_lengths;
  prefix.output = prefix_states;
  prefix.emit_state = 1;
  status = loom_cuda_paged_decode_attention_ex(&prefix);
  if (status != LOOM_CUDA_SUCCESS) return status;
  return loom_cuda_multi_token_finish(args, query_tokens, prefix_states);
}
