// Paged MQA/GQA decode attention for sm_100a: route selection, the scalar
// fallback kernel, the log-sum-exp merge kernel and the exported symbols.
//
// Replaces crates/loom-cuda-sys/cuda/src/paged_decode_attention.cu behind the
// same `loom_cuda_paged_decode_attention_*` symbols (host gate :988-1152,
// split-K sizing :89-162,1156-1166, merge kernel :749-853) and adds the
// strided / FP8-cache / partial-state entry points declared in
// include/loom_launch.h.
//
// Kernels:
//   decode_stream_tma_kernel (decode_stream_tma.cuh) persistent CTAs that share the
//                          batch's tiles evenly, rings fed by TMA: the default
//                          whenever a workspace is given (16-bit queries, head
//                          size 64 or 128, block size a multiple of 16).
//   decode_stream_kernel   (decode_stream.cuh) the same schedule with cp.async
//                          rings, where a tensor map cannot describe the cache.
//   decode_umma_fp8_kernel (decode_umma.cuh) the same schedule on tcgen05.mma and
//                          tensor memory for FP8 caches; opt-in.
//   decode_mma_kernel      (decode_mma.cuh) one CTA per fixed partition: without
//                          workspace, odd block sizes, caller-chosen partitions.
//   decode_scalar_kernel   everything else (F32, odd head sizes, unaligned
//                          views): one query head per CTA, CUDA cores.
//   merge_*_kernel         second, light kernel: combines the partial
//                          (O, max, sum) states of a split sequence, or of
//                          several GPUs.
// A work item that one CTA finished alone is written by the first kernel, so
// the merge kernel only touches the rows that were actually split.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <type_traits>

#include "../../include/loom_launch.h"
#include "decode_block_tile.cuh"
#include "decode_common.cuh"
#include "decode_merge.cuh"
#include "decode_mma.cuh"
#include "decode_stream.cuh"
#include "decode_stream_split.cuh"
#include "decode_stream_tma.cuh"
#include "decode_umma.cuh"

namespace loom_decode {

// ============================================================ scalar path

constexpr int kScalarWarps = 4;
constexpr int kScalarThreads = kScalarWarps * 32;
constexpr int kScalarMaxValueRegs = 16;  // value_head_size <= 512

template <typename T>
__device__ __forceinline__ float widen(T value);
template <>
__device__ __forceinline__ float widen<float>(float value) { return value; }
template <>
__device__ __forceinline__ float widen<__half>(__half value) { return __half2float(value); }
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 value) { return __bfloat162float(value); }
template <>
__device__ __forceinline__ float widen<uint8_t>(uint8_t value) {
  // E4M3 byte -> F16 (exact) -> F32
  const __half_raw raw = __nv_cvt_fp8_to_halfraw(value, __NV_E4M3);
  return __half2float(__half(raw));
}

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
  return value;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
  return value;
}

// One CTA per (sequence, partition, query head); each warp walks every fourth
// token with a lane-strided dot product and keeps its own online softmax.
template <typename QT, typename CT>
__global__ void __launch_bounds__(kScalarThreads) decode_scalar_kernel(const DecodeParams p) {
  constexpr bool kFp8 = std::is_same<CT, uint8_t>::value;
  extern __shared__ __align__(16) float scalar_smem[];
  loom_launch::grid_dependency_wait();
  float* q_shared = scalar_smem;                                 // [head_size]
  float* merge_o = q_shared + p.head_size;                       // [warps][value_head_size]
  float* merge_max = merge_o + kScalarWarps * p.value_head_size; // [warps]
  float* merge_sum = merge_max + kScalarWarps;                   // [warps]

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t seq = blockIdx.x / p.max_partitions;
  const uint32_t part = blockIdx.x % p.max_partitions;
  const uint32_t query_head = blockIdx.y;
  const uint32_t kv_head = query_head / p.group;

  const uint32_t length = clamp_length(p.sequence_lengths[seq], p.max_sequence_length);
  const uint32_t visible = window_begin(length, p.sliding_window);  // first token a sliding window lets through
  const uint32_t first_part = visible / p.partition_tokens;
  if ((part * p.partition_tokens >= length && part != 0) || part < first_part) return;
  const uint32_t part_begin = max(part * p.partition_tokens, visible);
  const uint32_t part_end = min(length, (part + 1) * p.partition_tokens);
  const uint32_t n_parts =
      length == 0 ? 1u : (length + p.partition_tokens - 1) / p.partition_tokens - first_part;

  const QT* query = static_cast<const QT*>(p.query) + (uint64_t)seq * p.q_token + (uint64_t)query_head * p.q_head;
  for (uint32_t d = threadIdx.x; d < p.head_size; d += kScalarThreads) q_shared[d] = widen<QT>(query[d]);
  __syncthreads();

  const CT* keys = static_cast<const CT*>(p.key_cache);
  const CT* values = static_cast<const CT*>(p.value_cache);
  const int32_t* table = p.block_tables + (uint64_t)seq * p.max_blocks_per_sequence;
  float score_scale = p.scale_log2;
  if (kFp8) score_scale *= p.key_scales[(uint64_t)kv_head * p.scale_stride];

  float running_max = -INFINITY, running_sum = 0.0f;
  float acc[kScalarMaxValueRegs];
#pragma unroll
  for (int j = 0; j < kScalarMaxValueRegs; ++j) acc[j] = 0.0f;

  for (uint32_t token = part_begin + warp; token < part_end; token += kScalarWarps) {
    const uint32_t block = clamp_block(__ldg(table + token / p.block_size), p.num_blocks);
    const uint32_t page = token % p.block_size;
    const CT* k_row = keys + (uint64_t)block * p.k_block + (uint64_t)page * p.k_page + (uint64_t)kv_head * p.k_head;
    const CT* v_row = values + (uint64_t)block * p.v_block + (uint64_t)page * p.v_page + (uint64_t)kv_head * p.v_head;
    float dot = 0.0f;
    for (uint32_t d = lane; d < p.head_size; d += 32) dot = fmaf(q_shared[d], widen<CT>(k_row[d]), dot);
    float score = warp_sum(dot) * score_scale;
    if (p.soft_cap_log2 != 0.0f) score = soft_capped(score, p.soft_cap_log2, p.inv_soft_cap_log2);
    const float new_max = fmaxf(running_max, score);
    const float alpha = exp2f(running_max - new_max);
    const float weight = exp2f(score - new_max);
    running_max = new_max;
    running_sum = running_sum * alpha + weight;
#pragma unroll
    for (int j = 0; j < kScalarMaxValueRegs; ++j) {
      const uint32_t dv = lane + 32 * j;
      if (dv < p.value_head_size) acc[j] = acc[j] * alpha + weight * widen<CT>(v_row[dv]);
    }
  }

#pragma unroll
  for (int j = 0; j < kScalarMaxValueRegs; ++j) {
    const uint32_t dv = lane + 32 * j;
    if (dv < p.value_head_size) merge_o[warp * p.value_head_size + dv] = acc[j];
  }
  if (lane == 0) {
    merge_max[warp] = running_max;
    merge_sum[warp] = running_sum;
  }
  __syncthreads();

  float top = -INFINITY;
#pragma unroll
  for (int w = 0; w < kScalarWarps; ++w) top = fmaxf(top, merge_max[w]);
  float factor[kScalarWarps];
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < kScalarWarps; ++w) {
    factor[w] = top > -INFINITY ? exp2f(merge_max[w] - top) : 0.0f;
    total += merge_sum[w] * factor[w];
  }
  float value_scale = 1.0f;
  if (kFp8) value_scale = p.value_scales[(uint64_t)kv_head * p.scale_stride];
  const bool final_rows = n_parts == 1;
  const uint32_t stride = state_stride(p.value_head_size);
  const uint64_t query_row = (uint64_t)seq * p.query_heads + query_head;
  for (uint32_t dv = threadIdx.x; dv < p.value_head_size; dv += kScalarThreads) {
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < kScalarWarps; ++w) sum += merge_o[w * p.value_head_size + dv] * factor[w];
    sum *= value_scale;
    if (final_rows && !p.emit_state) {
      narrow_store<QT>(static_cast<QT*>(p.output) + query_row * p.value_head_size + dv,
                       total > 0.0f ? sum / total : 0.0f);
    } else {
      float* state = final_rows ? static_cast<float*>(p.output) + query_row * stride
                                : p.partials + (query_row * p.max_partitions + part) * stride;
      state[dv] = sum;
      if (dv == 0) {
        state[p.value_head_size] = top * kLn2;
        state[p.value_head_size + 1] = total;
      }
    }
  }
}

// ============================================================= merge kernel

// One CTA per output row. Part `i` of row `r` lives at
// states + r*row_stride + i*part_stride. With sequence_lengths the part count
// is ceil(length / partition_tokens) and rows with a single part are skipped
// (the decode kernel finished them); without, `fixed_parts` is used.
template <typename OT>
__global__ void __launch_bounds__(kMergeThreads)
merge_states_kernel(const float* __restrict__ states, uint64_t row_stride, uint64_t part_stride,
                    uint32_t value_head_size, uint32_t fixed_parts,
                    const int32_t* __restrict__ sequence_lengths, uint32_t rows_per_sequence,
                    uint32_t partition_tokens, uint32_t max_sequence_length, uint32_t sliding_window,
                    void* output, uint32_t emit_state) {
  loom_launch::grid_dependency_wait();
  const uint32_t row = blockIdx.x;
  uint32_t parts = fixed_parts, first_part = 0;
  if (sequence_lengths != nullptr) {
    const uint32_t length = clamp_length(sequence_lengths[row / rows_per_sequence], max_sequence_length);
    // partitions wholly before a sliding window's first token were skipped by the decode kernel
    first_part = window_begin(length, sliding_window) / partition_tokens;
    parts = (length + partition_tokens - 1) / partition_tokens - first_part;
    if (parts <= 1) return;
  }
  merge_row<OT>(states + (uint64_t)row * row_stride + (uint64_t)first_part * part_stride, parts, part_stride,
                value_head_size, row, output, emit_state);
}

// Merge after the balanced kernel: the item table says which CTAs hold parts of
// this row's work item. Rows finished by a single CTA are skipped; rows of an
// empty sequence (which no CTA visits) are written as zero.
template <typename OT>
__global__ void __launch_bounds__(kMergeThreads)
merge_stream_kernel(const float* __restrict__ slots, const uint32_t* __restrict__ item_meta,
                    const int32_t* __restrict__ sequence_lengths, uint32_t query_heads, uint32_t group,
                    uint32_t heads_per_item, uint32_t value_head_size, uint32_t max_sequence_length,
                    void* output, uint32_t emit_state, uint32_t heads_together) {
  loom_launch::grid_dependency_wait();
  const uint32_t row = blockIdx.x;
  const uint32_t seq = row / query_heads;
  const uint32_t query_head = row % query_heads;
  const uint32_t kv_head = query_head / group;
  const uint32_t head_in_group = query_head % group;
  const uint32_t head_chunks = (group + heads_per_item - 1) / heads_per_item;
  const uint32_t items_per_sequence = (query_heads / group) * head_chunks;
  const uint64_t item = (uint64_t)seq * items_per_sequence + (uint64_t)kv_head * head_chunks +
                        head_in_group / heads_per_item;
  const uint32_t stride = state_stride(value_head_size);
  // three independent loads, issued together
  const int32_t raw_length = __ldg(sequence_lengths + seq);
  const uint32_t first_cta = item_meta[2 * item];
  const uint32_t parts = item_meta[2 * item + 1];
  if (clamp_length(raw_length, max_sequence_length) == 0) {
    merge_row<OT>(slots, 0, 0, value_head_size, row, output, emit_state);
    return;
  }
  if (parts <= 1) return;
  if (heads_together != 0) {
    // the kernel whose tile holds `heads_together` KV heads: slot = heads_together * (item group + CTA) + head
    const uint64_t slot = (item / heads_together + first_cta) * heads_together + item % heads_together;
    merge_row<OT>(slots + (slot * heads_per_item + head_in_group % heads_per_item) * stride, parts,
                  (uint64_t)heads_together * heads_per_item * stride, value_head_size, row, output, emit_state);
    return;
  }
  const float* base = slots + ((item + first_cta) * heads_per_item + head_in_group % heads_per_item) * stride;
  merge_row<OT>(base, parts, (uint64_t)heads_per_item * stride, value_head_size, row, output, emit_state);
}

// ================================================================= host

thread_local const char* g_last_route = "none";

// Launch status of this library from a runtime status; the error and where it arose are kept
// for loom_cuda_last_launch_failure().
int launched(cudaError_t status, const char* where = "decode kernel launch") {
  return loom_launch::failed(status, where);
}

bool aligned16(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

// Raises a kernel's dynamic shared memory limit once per device.
template <typename Kernel>
cudaError_t ensure_smem(Kernel kernel, int bytes, std::atomic<uint64_t>& done_mask) {
  int device = 0;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) return status;
  const uint64_t bit = 1ull << (device & 63);
  if (device < 64 && (done_mask.load(std::memory_order_acquire) & bit)) return cudaSuccess;
  status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (status == cudaSuccess && device < 64) done_mask.fetch_or(bit, std::memory_order_release);
  return status;
}

// SMs of the current device (148 on a B200); 0 if no device can be queried.
uint32_t current_sm_count() {
  static std::atomic<uint32_t> cached[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (device >= 0 && device < 64) {
    const uint32_t known = cached[device].load(std::memory_order_acquire);
    if (known != 0) return known;
  }
  int count = 0;
  if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) {
    cudaGetLastError();
    return 0;
  }
  if (device >= 0 && device < 64) cached[device].store((uint32_t)count, std::memory_order_release);
  return (uint32_t)count;
}

// CTAs of the balanced kernels: two per SM, three for the TMA-fed kernel with
// eight heads per item. Workspaces are sized for the larger count and for at
// least a 148-SM device, so that a size computed before a device is current,
// or before the kernel is chosen, still fits.
constexpr uint32_t kStreamCtasPerSm = 2;
constexpr uint32_t kStreamMaxCtasPerSm = 4;
uint32_t stream_ctas_for_launch(uint32_t per_sm) { return per_sm * current_sm_count(); }
uint32_t stream_ctas_for_sizing() {
  const uint32_t sms = current_sm_count();
  return kStreamMaxCtasPerSm * (sms > 148 ? sms : 148);
}

template <typename QT, bool kFp8, int kD, int kNT>
int launch_mma(const DecodeParams& p, cudaStream_t stream) {
  static std::atomic<uint64_t> configured_masks[2];  // one per instantiation (plain, with options)
  constexpr int kBytes = mma_smem_bytes<kFp8, kD, kNT>();
  const bool options = p.sliding_window != 0 || p.soft_cap_log2 != 0.0f;
  auto kernel = options ? decode_mma_kernel<QT, kFp8, kD, kNT, true> : decode_mma_kernel<QT, kFp8, kD, kNT, false>;
  if (const cudaError_t limit = ensure_smem(kernel, kBytes, configured_masks[options ? 1 : 0]); limit != cudaSuccess) {
    return launched(limit, "shared-memory limit of a decode kernel (cudaFuncSetAttribute)");
  }
  const uint32_t head_chunks = (p.group + 8 * kNT - 1) / (8 * kNT);
  const dim3 grid(p.sequences * p.max_partitions, p.kv_heads * head_chunks, 1);
  return launched(loom_launch::launch(kernel, grid, dim3(kMmaThreads), kBytes, stream, p));
}

template <typename QT, bool kFp8, int kD, int kNT>
int launch_stream(const DecodeParams& p, uint32_t ctas, cudaStream_t stream) {
  static std::atomic<uint64_t> configured_masks[2];  // one per instantiation (plain, with options)
  constexpr int kBytes = StreamRing<kFp8, kD, kNT>::kSmemBytes;
  const bool options = p.sliding_window != 0 || p.soft_cap_log2 != 0.0f;
  auto kernel =
      options ? decode_stream_kernel<QT, kFp8, kD, kNT, true> : decode_stream_kernel<QT, kFp8, kD, kNT, false>;
  if (const cudaError_t limit = ensure_smem(kernel, kBytes, configured_masks[options ? 1 : 0]); limit != cudaSuccess) {
    return launched(limit, "shared-memory limit of a decode kernel (cudaFuncSetAttribute)");
  }
  return launched(loom_launch::launch(kernel, dim3(ctas), dim3(kMmaThreads), kBytes, stream, p));
}

// ---- tensor maps for the TMA-fed kernel ---------------------------------------

struct CacheMaps {
  CUtensorMap key, value;
  TmaAxes axes;
};

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, fetched through the runtime so that the library does
// not link against libcuda. Null if the driver does not offer it.
EncodeTiled tensor_map_encoder() {
  static const EncodeTiled encoder = [] {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      symbol = nullptr;
    }
    return reinterpret_cast<EncodeTiled>(symbol);
  }();
  return encoder;
}

// 0 = TMA where possible, 1 = always cp.async (for comparisons and as a guard).
std::atomic<uint32_t> g_copy_engine{0};

// Describes one cache as a 4-D byte tensor: (row bytes, then head / page / block
// sorted by stride). Box: up to 128 bytes of a row, 16 pages, one head, one block.
bool encode_cache_map(CUtensorMap* map, const void* base, uint32_t row_bytes, const uint64_t (&sizes)[3],
                      const uint64_t (&strides_bytes)[3], const uint32_t (&order)[3]) {
  const EncodeTiled encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  cuuint64_t dims[4] = {row_bytes, 0, 0, 0};
  cuuint64_t strides[3] = {0, 0, 0};
  cuuint32_t box[4] = {row_bytes > 128 ? 128u : row_bytes, 1, 1, 1};
  cuuint32_t element_strides[4] = {1, 1, 1, 1};
  for (int position = 0; position < 3; ++position) {
    const uint32_t which = order[position];  // 0 = head, 1 = page, 2 = block
    dims[position + 1] = sizes[which];
    strides[position] = strides_bytes[which];
    if (which == 1) box[position + 1] = 16;
    if (strides[position] % 16 != 0 || strides[position] >= (1ull << 40)) return false;
  }
  const CUtensorMapSwizzle swizzle = row_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  // L2 fetch granule no wider than a row: in an NHD cache the bytes after a
  // 128-byte row belong to another KV head, which another CTA reads at another
  // time. A 256-byte granule there cost 42 % extra DRAM reads on an FP8 cache.
  // (Rows of consecutive pages that touch, as in an HND cache, keep the wide granule.)
  const bool rows_touch = strides_bytes[1] == row_bytes;
  const CUtensorMapL2promotion promotion = (row_bytes >= 256 || rows_touch) ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                           : row_bytes >= 128               ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                                            : CU_TENSOR_MAP_L2_PROMOTION_L2_64B;
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box,
                element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promotion,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool build_cache_maps(const LoomDecodeArgs& a, bool fp8, CacheMaps* maps) {
  const uint64_t elem = fp8 ? 1 : 2;
  const uint32_t row_bytes = (uint32_t)(a.head_size * elem);
  if (row_bytes != 64 && row_bytes != 128 && row_bytes != 256) return false;
  const uint64_t sizes[3] = {a.kv_heads, a.block_size, a.num_blocks};
  const uint64_t key_strides[3] = {a.key_head_stride * elem, a.key_page_stride * elem, a.key_block_stride * elem};
  const uint64_t value_strides[3] = {a.value_head_stride * elem, a.value_page_stride * elem,
                                     a.value_block_stride * elem};
  // order the outer dimensions by the key cache's strides; the value cache must agree
  uint32_t order[3] = {0, 1, 2};
  for (int i = 0; i < 3; ++i) {
    for (int j = i + 1; j < 3; ++j) {
      if (key_strides[order[j]] < key_strides[order[i]]) {
        const uint32_t swap = order[i];
        order[i] = order[j];
        order[j] = swap;
      }
    }
  }
  for (int i = 0; i + 1 < 3; ++i) {
    if (value_strides[order[i]] > value_strides[order[i + 1]]) return false;
  }
  if (order[2] != 2) return false;  // the kernel expects the block to be the outermost coordinate
  for (uint32_t position = 0; position < 3; ++position) {
    if (order[position] == 0) maps->axes.head = position + 1;
    if (order[position] == 1) maps->axes.page = position + 1;
    if (order[position] == 2) maps->axes.block = position + 1;
  }
  return encode_cache_map(&maps->key, a.key_cache, row_bytes, sizes, key_strides, order) &&
         encode_cache_map(&maps->value, a.value_cache, row_bytes, sizes, value_strides, order);
}

// The cache as (row bytes, page, head, block) whatever the order of its strides: a box of
// [128 bytes, 16 pages, 8 heads, 1 block] then lands in shared memory as eight per-head tiles.
bool encode_block_map(CUtensorMap* map, const void* base, uint32_t row_bytes, uint64_t kv_heads,
                      uint64_t block_size, uint64_t num_blocks, uint64_t head_stride, uint64_t page_stride,
                      uint64_t block_stride) {
  const EncodeTiled encode = tensor_map_encoder();
  if (encode == nullptr || row_bytes != 128) return false;
  cuuint64_t dims[4] = {row_bytes, block_size, kv_heads, num_blocks};
  cuuint64_t strides[3] = {page_stride, head_stride, block_stride};
  cuuint32_t box[4] = {128, 16, 8, 1};
  cuuint32_t element_strides[4] = {1, 1, 1, 1};
  for (const cuuint64_t stride : strides) {
    if (stride % 16 != 0 || stride >= (1ull << 40)) return false;
  }
  // a block's rows touch along one of the two inner axes in both usual layouts
  const bool rows_touch = head_stride == row_bytes || page_stride == row_bytes;
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box,
                element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                rows_touch ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool build_block_maps(const LoomDecodeArgs& a, CacheMaps* maps) {
  return encode_block_map(&maps->key, a.key_cache, a.head_size, a.kv_heads, a.block_size, a.num_blocks,
                          a.key_head_stride, a.key_page_stride, a.key_block_stride) &&
         encode_block_map(&maps->value, a.value_cache, a.value_head_size, a.kv_heads, a.block_size, a.num_blocks,
                          a.value_head_stride, a.value_page_stride, a.value_block_stride);
}

// The balanced kernel whose tile is one 16-token block of eight KV heads (FP8 caches).
template <typename QT>
int launch_block_tile(const DecodeParams& p, uint32_t ctas, const CacheMaps& maps, cudaStream_t stream) {
  static std::atomic<uint64_t> configured{0};
  using Ring = BlockRing<128>;
  auto kernel = decode_block_tile_kernel<QT, 128>;
  if (const cudaError_t limit = ensure_smem(kernel, Ring::kSmemBytes, configured); limit != cudaSuccess) {
    return launched(limit, "shared-memory limit of a decode kernel (cudaFuncSetAttribute)");
  }
  return launched(loom_launch::launch(kernel, dim3(ctas), dim3(Ring::kThreads), Ring::kSmemBytes, stream, p, maps.key,
                                      maps.value));
}

template <typename QT, bool kFp8, int kD, int kNT>
int launch_stream_tma(const DecodeParams& p, uint32_t ctas, const CacheMaps& maps, cudaStream_t stream) {
  static std::atomic<uint64_t> configured_masks[2];  // one per instantiation (plain, with options)
  constexpr int kBytes = TmaRing<kFp8, kD, kNT>::kSmemBytes;
  const bool options = p.sliding_window != 0 || p.soft_cap_log2 != 0.0f;
  auto kernel = options ? decode_stream_tma_kernel<QT, kFp8, kD, kNT, true>
                        : decode_stream_tma_kernel<QT, kFp8, kD, kNT, false>;
  if (const cudaError_t limit = ensure_smem(kernel, kBytes, configured_masks[options ? 1 : 0]); limit != cudaSuccess) {
    return launched(limit, "shared-memory limit of a decode kernel (cudaFuncSetAttribute)");
  }
  return launched(loom_launch::launch(kernel, dim3(ctas), dim3(kMmaThreads), kBytes, stream, p, maps.key, maps.value,
                                      maps.axes));
}

// The balanced kernel with a copy-issuing warp (FP8 caches, up to 8 query heads per KV head, no options).
template <typename QT, int kD>
int launch_stream_split(const DecodeParams& p, uint32_t ctas, const CacheMaps& maps, cudaStream_t stream) {
  static std::atomic<uint64_t> configured{0};
  using Ring = SplitRing<true, kD>;
  auto kernel = decode_stream_split_kernel<QT, true, kD>;
  if (const cudaError_t limit = ensure_smem(kernel, Ring::kSmemBytes, configured); limit != cudaSuccess) {
    return launched(limit, "shared-memory limit of a decode kernel (cudaFuncSetAttribute)");
  }
  return launched(loom_launch::launch(kernel, dim3(ctas), dim3(Ring::kThreads), Ring::kSmemBytes, stream, p, maps.key,
                                      maps.value, maps.axes));
}

template <typename QT>
int launch_umma_fp8(const DecodeParams& p, uint32_t ctas, const CacheMaps& maps, cudaStream_t stream) {
  static std::atomic<uint64_t> configured{0};
  constexpr int kBytes = UmmaSmem::kBytes;
  auto kernel = decode_umma_fp8_kernel<QT>;
  if (const cudaError_t limit = ensure_smem(kernel, kBytes, configured); limit != cudaSuccess) {
    return launched(limit, "shared-memory limit of a decode kernel (cudaFuncSetAttribute)");
  }
  return launched(loom_launch::launch(kernel, dim3(ctas), dim3(kUmmaThreads), kBytes, stream, p, maps.key, maps.value,
                                      maps.axes));
}

template <typename QT, bool kFp8>
int launch_mma_shape(const DecodeParams& p, uint32_t stream_ctas, const CacheMaps* maps, cudaStream_t stream) {
  const bool wide = p.group > 8;
  if (stream_ctas != 0 && maps != nullptr) {
    if (p.head_size == 128) {
      return wide ? launch_stream_tma<QT, kFp8, 128, 2>(p, stream_ctas, *maps, stream)
                  : launch_stream_tma<QT, kFp8, 128, 1>(p, stream_ctas, *maps, stream);
    }
    return wide ? launch_stream_tma<QT, kFp8, 64, 2>(p, stream_ctas, *maps, stream)
                : launch_stream_tma<QT, kFp8, 64, 1>(p, stream_ctas, *maps, stream);
  }
  if (stream_ctas != 0) {
    if (p.head_size == 128) {
      return wide ? launch_stream<QT, kFp8, 128, 2>(p, stream_ctas, stream)
                  : launch_stream<QT, kFp8, 128, 1>(p, stream_ctas, stream);
    }
    return wide ? launch_stream<QT, kFp8, 64, 2>(p, stream_ctas, stream)
                : launch_stream<QT, kFp8, 64, 1>(p, stream_ctas, stream);
  }
  if (p.head_size == 128) {
    return wide ? launch_mma<QT, kFp8, 128, 2>(p, stream) : launch_mma<QT, kFp8, 128, 1>(p, stream);
  }
  return wide ? launch_mma<QT, kFp8, 64, 2>(p, stream) : launch_mma<QT, kFp8, 64, 1>(p, stream);
}

// Shared memory of the CUDA-core kernel: the query row, one O row per warp, (max, sum) per warp.
// One predicate for the launch and for loom_cuda_supports_paged_decode.
size_t scalar_smem_bytes(uint32_t head_size, uint32_t value_head_size) {
  return ((size_t)head_size + (size_t)kScalarWarps * value_head_size + 2 * kScalarWarps) * sizeof(float);
}
bool scalar_smem_fits(uint32_t head_size, uint32_t value_head_size) {
  return scalar_smem_bytes(head_size, value_head_size) <= 48 * 1024;
}

template <typename QT, typename CT>
int launch_scalar(const DecodeParams& p, cudaStream_t stream) {
  const size_t bytes = scalar_smem_bytes(p.head_size, p.value_head_size);
  if (!scalar_smem_fits(p.head_size, p.value_head_size)) return LOOM_CUDA_UNSUPPORTED;
  const dim3 grid(p.sequences * p.max_partitions, p.query_heads, 1);
  return launched(loom_launch::launch(decode_scalar_kernel<QT, CT>, grid, dim3(kScalarThreads), bytes, stream, p));
}

bool mma_route_fits(const LoomDecodeArgs& a, bool fp8) {
  if (a.dtype != 1 && a.dtype != 2) return false;
  if (a.head_size != a.value_head_size || (a.head_size != 64 && a.head_size != 128)) return false;
  const uint64_t elem = fp8 ? 1 : 2;
  const auto row_ok = [elem](uint64_t stride) { return (stride * elem) % 16 == 0; };
  if (!aligned16(a.query) || !aligned16(a.key_cache) || !aligned16(a.value_cache)) return false;
  if ((a.query_token_stride * 2) % 16 != 0 || (a.query_head_stride * 2) % 16 != 0) return false;
  if (!row_ok(a.key_block_stride) || !row_ok(a.key_page_stride) || !row_ok(a.key_head_stride) ||
      !row_ok(a.value_block_stride) || !row_ok(a.value_page_stride) || !row_ok(a.value_head_stride)) {
    return false;
  }
  const uint32_t group = a.query_heads / a.kv_heads;
  const uint32_t heads_per_cta = group > 8 ? 16 : 8;
  const uint64_t grid_y = (uint64_t)a.kv_heads * ((group + heads_per_cta - 1) / heads_per_cta);
  return grid_y <= 65535;
}

uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// Partition length of the fixed-partition kernels when the caller does not
// choose: the longest of {2048, ..., 64} that still yields enough CTAs to fill
// 148 SMs a few times over, assuming every sequence were as long as the maximum.
uint32_t default_partition_tokens(uint32_t sequences, uint32_t kv_heads, uint32_t max_sequence_length) {
  constexpr uint64_t kWantedCtas = 148ull * 2 * 4;
  const uint64_t heads = (uint64_t)sequences * kv_heads;
  for (uint32_t tokens = 2048; tokens > 64; tokens >>= 1) {
    if (heads * ceil_div(max_sequence_length, tokens) >= kWantedCtas) return tokens;
  }
  return 64;
}

bool mul_checked(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_mul_overflow(a, b, out); }

// F32 elements the fixed-partition path needs; 0 on bad arguments or overflow.
uint64_t fixed_workspace_elements(uint32_t sequences, uint32_t query_heads, uint32_t value_head_size,
                                  uint32_t max_sequence_length, uint32_t partition_tokens) {
  if (sequences == 0 || query_heads == 0 || value_head_size == 0 || max_sequence_length == 0 ||
      partition_tokens == 0 || partition_tokens % 16 != 0) {
    return 0;
  }
  uint64_t rows = 0, per_row = 0, total = 0;
  if (!mul_checked(sequences, query_heads, &rows) ||
      !mul_checked(ceil_div(max_sequence_length, partition_tokens), (uint64_t)value_head_size + 2, &per_row) ||
      !mul_checked(rows, per_row, &total)) {
    return 0;
  }
  return total;
}

struct StreamShape {
  uint32_t heads_per_item;  // 8 or 16 query heads per work item
  uint64_t items;           // sequences * kv_heads * head chunks
  uint64_t slot_elements;   // F32 elements of the state slots
  uint64_t total_elements;  // slots + item table
};

// Workspace of the balanced kernel: one state slot per (item + CTA), then two
// 32-bit words per item. Returns false on overflow.
bool stream_shape(uint32_t sequences, uint32_t query_heads, uint32_t kv_heads, uint32_t value_head_size,
                  uint32_t ctas, StreamShape* shape) {
  if (sequences == 0 || query_heads == 0 || kv_heads == 0 || value_head_size == 0 ||
      query_heads % kv_heads != 0) {
    return false;
  }
  const uint32_t group = query_heads / kv_heads;
  shape->heads_per_item = group > 8 ? 16 : 8;
  const uint32_t head_chunks = ceil_div(group, shape->heads_per_item);
  uint64_t per_sequence = 0, per_slot = 0, meta = 0;
  if (!mul_checked(kv_heads, head_chunks, &per_sequence) || !mul_checked(sequences, per_sequence, &shape->items) ||
      !mul_checked(shape->heads_per_item, (uint64_t)value_head_size + 2, &per_slot) ||
      shape->items > std::numeric_limits<uint64_t>::max() - ctas ||
      !mul_checked(shape->items + ctas, per_slot, &shape->slot_elements) ||
      !mul_checked(shape->items, 2, &meta) ||
      shape->slot_elements > std::numeric_limits<uint64_t>::max() - meta) {
    return false;
  }
  shape->total_elements = shape->slot_elements + meta;
  return true;
}

// Does the kernel whose tile holds eight KV heads apply to this shape? (The cache encoding and the
// layout are not part of a workspace query; the launch checks them.)
bool block_tile_shape(uint32_t query_heads, uint32_t kv_heads, uint32_t head_size, uint32_t value_head_size) {
  return kv_heads != 0 && kv_heads % 8 == 0 && query_heads % kv_heads == 0 && query_heads / kv_heads <= 8 &&
         head_size == 128 && value_head_size == 128;
}

// Its workspace: eight state slots per (group of eight items + CTA), then the item table.
bool block_tile_workspace(uint32_t sequences, uint32_t kv_heads, uint32_t value_head_size, uint32_t ctas,
                          StreamShape* shape) {
  shape->heads_per_item = 8;
  uint64_t groups = 0, per_slot = 0, slots = 0, meta = 0;
  if (!mul_checked(sequences, kv_heads / 8, &groups) || groups > std::numeric_limits<uint64_t>::max() - ctas ||
      !mul_checked(groups + ctas, 8, &slots) || !mul_checked(8, (uint64_t)value_head_size + 2, &per_slot) ||
      !mul_checked(slots, per_slot, &shape->slot_elements) || !mul_checked(sequences, kv_heads, &shape->items) ||
      !mul_checked(shape->items, 2, &meta) || shape->slot_elements > std::numeric_limits<uint64_t>::max() - meta) {
    return false;
  }
  shape->total_elements = shape->slot_elements + meta;
  return true;
}

// Size that serves whichever partitioned kernel the launch then picks.
// `every_layout` = false leaves out the (larger) layout of the eight-heads-per-tile kernel: the size
// below which no partitioned kernel can run, since the launch falls back to the other kernels when
// the workspace does not hold that layout.
uint64_t auto_workspace_elements(uint32_t sequences, uint32_t query_heads, uint32_t kv_heads,
                                 uint32_t value_head_size, uint32_t max_sequence_length,
                                 bool every_layout = true) {
  const uint64_t fixed = fixed_workspace_elements(
      sequences, query_heads, value_head_size, max_sequence_length,
      default_partition_tokens(sequences, kv_heads, max_sequence_length));
  StreamShape shape{};
  if (fixed == 0 || !stream_shape(sequences, query_heads, kv_heads, value_head_size, stream_ctas_for_sizing(), &shape)) {
    return 0;
  }
  uint64_t needed = fixed > shape.total_elements ? fixed : shape.total_elements;
  // head_size is not part of the query: the value head size stands for both (the launch checks)
  StreamShape block{};
  if (every_layout && block_tile_shape(query_heads, kv_heads, value_head_size, value_head_size)) {
    if (!block_tile_workspace(sequences, kv_heads, value_head_size, stream_ctas_for_sizing(), &block)) return 0;
    if (block.total_elements > needed) needed = block.total_elements;
  }
  return needed;
}

bool product_fits_u64(std::initializer_list<uint64_t> dims) {
  uint64_t product = 1;
  for (uint64_t d : dims) {
    if (d != 0 && product > std::numeric_limits<uint64_t>::max() / d) return false;
    product *= d;
  }
  return true;
}

int launch_decode(const LoomDecodeArgs& a) {
  const bool fp8 = a.cache_encoding == LOOM_CUDA_KV_CACHE_FP8_E4M3;
  // The argument rules of the reference launcher
  // (paged_decode_attention.cu:1018-1049) without its 1024-token cap.
  if (a.dtype > 2 || a.cache_encoding > 1 || a.query == nullptr || a.key_cache == nullptr ||
      a.value_cache == nullptr || a.block_tables == nullptr || a.sequence_lengths == nullptr ||
      a.output == nullptr || a.sequences == 0 || a.query_heads == 0 || a.kv_heads == 0 ||
      a.head_size == 0 || a.value_head_size == 0 || a.num_blocks == 0 || a.block_size == 0 ||
      a.max_blocks_per_sequence == 0 || a.query_heads % a.kv_heads != 0 ||
      a.max_sequence_length == 0 || a.max_sequence_length > (1u << 30) ||
      a.max_sequence_length > (uint64_t)a.block_size * a.max_blocks_per_sequence ||
      !std::isfinite(a.scale) || a.scale <= 0.0f ||
      (fp8 && (a.key_scales == nullptr || a.value_scales == nullptr || a.scale_stride > 1)) ||
      !product_fits_u64({a.sequences, a.query_heads, a.head_size}) ||
      !product_fits_u64({a.sequences, a.query_heads, a.value_head_size}) ||
      !product_fits_u64({a.num_blocks, a.block_size, a.kv_heads, a.head_size}) ||
      !product_fits_u64({a.num_blocks, a.block_size, a.kv_heads, a.value_head_size}) ||
      !product_fits_u64({a.sequences, a.max_blocks_per_sequence}) ||
      a.key_block_stride == 0 || a.key_page_stride == 0 || a.key_head_stride == 0 ||
      a.value_block_stride == 0 || a.value_page_stride == 0 || a.value_head_stride == 0 ||
      ((a.query_token_stride == 0) != (a.query_head_stride == 0)) ||
      (a.query_head_stride != 0 && a.query_head_stride < a.head_size) ||
      !std::isfinite(a.logits_soft_cap) || a.logits_soft_cap < 0.0f ||
      (a.flags & ~LOOM_DECODE_STABLE_METADATA) != 0 || a.reserved != 0) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }

  DecodeParams p{};
  p.query = a.query;
  p.key_cache = a.key_cache;
  p.value_cache = a.value_cache;
  p.key_scales = a.key_scales;
  p.value_scales = a.value_scales;
  p.block_tables = a.block_tables;
  p.sequence_lengths = a.sequence_lengths;
  p.output = a.output;
  p.sequences = a.sequences;
  p.query_heads = a.query_heads;
  p.kv_heads = a.kv_heads;
  p.group = a.query_heads / a.kv_heads;
  p.head_size = a.head_size;
  p.value_head_size = a.value_head_size;
  p.num_blocks = a.num_blocks;
  p.block_size = a.block_size;
  p.max_blocks_per_sequence = a.max_blocks_per_sequence;
  p.max_sequence_length = a.max_sequence_length;
  p.scale_stride = fp8 ? a.scale_stride : 0;
  p.block_shift = 32;
  if ((a.block_size & (a.block_size - 1)) == 0) p.block_shift = (uint32_t)__builtin_ctz(a.block_size);
  p.emit_state = a.emit_state ? 1 : 0;
  p.k_block = a.key_block_stride;
  p.k_page = a.key_page_stride;
  p.k_head = a.key_head_stride;
  p.v_block = a.value_block_stride;
  p.v_page = a.value_page_stride;
  p.v_head = a.value_head_stride;
  const bool dense_query = a.query_token_stride == 0 && a.query_head_stride == 0;
  p.q_head = dense_query ? a.head_size : a.query_head_stride;
  p.q_token = dense_query ? (uint64_t)a.query_heads * a.head_size : a.query_token_stride;
  p.scale_log2 = a.scale * kLog2e;
  p.sliding_window = a.sliding_window;
  p.soft_cap_log2 = a.logits_soft_cap * kLog2e;
  p.inv_soft_cap_log2 = a.logits_soft_cap > 0.0f ? 1.0f / (a.logits_soft_cap * kLog2e) : 0.0f;
  p.wait_attempts = loom_launch::wait_attempts(kDefaultWaitAttempts);
  p.wait_unmatched_bytes = loom_launch::wait_unmatched_bytes();

  const bool use_mma = mma_route_fits(a, fp8);
  const bool partitioned = a.workspace != nullptr || a.workspace_elements != 0;
  uint32_t stream_ctas = 0;  // non-zero selects the balanced kernel
  StreamShape shape{};
  CacheMaps maps;
  const CacheMaps* tma = nullptr;
  bool umma = false;
  bool split = false;  // the balanced kernel with a copy-issuing warp
  bool block_tile = false;  // the balanced kernel whose tile is one block of eight KV heads
  if (partitioned) {
    if (a.workspace == nullptr || (reinterpret_cast<uintptr_t>(a.workspace) & 3u) != 0) {
      return LOOM_CUDA_INVALID_ARGUMENT;
    }
    p.partials = a.workspace;
    uint32_t tokens = a.partition_tokens;
    if (tokens == 0 && use_mma && a.block_size % 16 == 0 && a.sequences <= kStreamMaxSequences) {
      if (a.sequences <= kTmaMaxSequences && g_copy_engine.load(std::memory_order_relaxed) != 1 &&
          build_cache_maps(a, fp8, &maps)) {
        tma = &maps;
      }
      // FP8 cache, head size 128, up to 8 query heads per KV head: the tcgen05
      // kernel applies; it is selected by copy engine 3 only, because the
      // mma.sync kernel is not slower and a little more accurate (456 vs 450-470 us on the
      // Llama-3-70B-shaped FP8 workload)
      umma = tma != nullptr && fp8 && p.group <= 8 && a.head_size == 128 && a.value_head_size == 128 &&
             g_copy_engine.load(std::memory_order_relaxed) == 3 && a.sliding_window == 0 &&
             a.logits_soft_cap == 0.0f;  // the options live in the mma.sync kernels only
      // FP8 cache, up to 8 query heads per KV head, no window or soft cap: the kernel whose copies are
      // issued by a warp of their own (copy engine 2 keeps the unsplit kernel, for comparisons)
      split = tma != nullptr && !umma && fp8 && p.group <= 8 && a.sliding_window == 0 &&
              a.logits_soft_cap == 0.0f && g_copy_engine.load(std::memory_order_relaxed) != 2;
      // ... and with KV heads in multiples of eight and head size 128 the kernel that copies a whole
      // block of eight heads at a time (copy engine 4 keeps the one-head-per-tile kernel)
      CacheMaps block_maps;
      StreamShape block_shape{};
      const uint32_t block_ctas = stream_ctas_for_launch((uint32_t)BlockRing<128>::kCtasPerSm);
      if (split && g_copy_engine.load(std::memory_order_relaxed) == 0 && block_ctas != 0 &&
          block_tile_shape(a.query_heads, a.kv_heads, a.head_size, a.value_head_size) &&
          block_tile_workspace(a.sequences, a.kv_heads, a.value_head_size, block_ctas, &block_shape) &&
          a.workspace_elements >= block_shape.total_elements && build_block_maps(a, &block_maps)) {
        block_tile = true;
        split = false;
        maps = block_maps;
        shape = block_shape;
        stream_ctas = block_ctas;
        p.item_meta = reinterpret_cast<uint32_t*>(a.workspace + shape.slot_elements);
        p.partition_tokens = 16;
        p.max_partitions = 1;
      }
      const uint32_t ctas = stream_ctas_for_launch(
          umma    ? (uint32_t)kUmmaCtasPerSm
          : split ? 2u
                  : (tma != nullptr && p.group <= 8 ? (fp8 ? 4u : 3u) : kStreamCtasPerSm));
      if (!block_tile && ctas != 0 &&
          stream_shape(a.sequences, a.query_heads, a.kv_heads, a.value_head_size, ctas, &shape) &&
          a.workspace_elements >= shape.total_elements) {
        stream_ctas = ctas;
        p.item_meta = reinterpret_cast<uint32_t*>(a.workspace + shape.slot_elements);
        p.partition_tokens = split ? (uint32_t)SplitRing<true, 128>::kTileTokens : kStreamTileTokens;
        p.max_partitions = 1;
      }
    }
    if (stream_ctas == 0) {
      if (tokens == 0) tokens = default_partition_tokens(a.sequences, a.kv_heads, a.max_sequence_length);
      const uint64_t needed = fixed_workspace_elements(a.sequences, a.query_heads, a.value_head_size,
                                                       a.max_sequence_length, tokens);
      if (needed == 0 || a.workspace_elements < needed) return LOOM_CUDA_INVALID_ARGUMENT;
      p.partition_tokens = tokens;
      p.max_partitions = ceil_div(a.max_sequence_length, tokens);
    }
  } else {
    p.partials = nullptr;
    p.partition_tokens = (a.max_sequence_length + 15u) & ~15u;
    p.max_partitions = 1;
  }
  if ((uint64_t)p.sequences * p.max_partitions > 0x7fffffffull) return LOOM_CUDA_INVALID_ARGUMENT;

  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  int status;
  if (use_mma) {
    if (stream_ctas == 0) {
      tma = nullptr;
      umma = false;
      split = false;
      block_tile = false;
    }
    // the caller's promise only matters to the balanced TMA-fed mma.sync kernel
    const bool promises_apply = tma != nullptr && !umma;
    p.early_metadata = promises_apply && (a.flags & LOOM_DECODE_STABLE_METADATA) ? 1u : 0u;
    if (umma) {
      g_last_route = "umma-fp8-balanced-tma";
      status = a.dtype == 1 ? launch_umma_fp8<__half>(p, stream_ctas, maps, stream)
                            : launch_umma_fp8<__nv_bfloat16>(p, stream_ctas, maps, stream);
    } else if (block_tile) {
      g_last_route = "mma16-fp8-balanced-block-tma";
      status = a.dtype == 1 ? launch_block_tile<__half>(p, stream_ctas, maps, stream)
                            : launch_block_tile<__nv_bfloat16>(p, stream_ctas, maps, stream);
    } else if (split) {
      g_last_route = "mma16-fp8-balanced-producer-tma";
      if (a.head_size == 128) {
        status = a.dtype == 1 ? launch_stream_split<__half, 128>(p, stream_ctas, maps, stream)
                              : launch_stream_split<__nv_bfloat16, 128>(p, stream_ctas, maps, stream);
      } else {
        status = a.dtype == 1 ? launch_stream_split<__half, 64>(p, stream_ctas, maps, stream)
                              : launch_stream_split<__nv_bfloat16, 64>(p, stream_ctas, maps, stream);
      }
    } else {
    if (stream_ctas == 0) g_last_route = fp8 ? "mma16-fp8" : "mma16";
    else if (tma != nullptr) g_last_route = fp8 ? "mma16-fp8-balanced-tma" : "mma16-balanced-tma";
    else g_last_route = fp8 ? "mma16-fp8-balanced" : "mma16-balanced";
    if (a.dtype == 1) {
      status = fp8 ? launch_mma_shape<__half, true>(p, stream_ctas, tma, stream)
                   : launch_mma_shape<__half, false>(p, stream_ctas, tma, stream);
    } else {
      status = fp8 ? launch_mma_shape<__nv_bfloat16, true>(p, stream_ctas, tma, stream)
                   : launch_mma_shape<__nv_bfloat16, false>(p, stream_ctas, tma, stream);
    }
    }
  } else {
    if (a.value_head_size > 32u * kScalarMaxValueRegs || a.query_heads > 65535u) return LOOM_CUDA_UNSUPPORTED;
    g_last_route = fp8 ? "scalar-fp8" : "scalar";
    switch (a.dtype) {
      case 0:
        status = fp8 ? launch_scalar<float, uint8_t>(p, stream) : launch_scalar<float, float>(p, stream);
        break;
      case 1:
        status = fp8 ? launch_scalar<__half, uint8_t>(p, stream) : launch_scalar<__half, __half>(p, stream);
        break;
      default:
        status = fp8 ? launch_scalar<__nv_bfloat16, uint8_t>(p, stream)
                     : launch_scalar<__nv_bfloat16, __nv_bfloat16>(p, stream);
        break;
    }
  }
  if (status != LOOM_CUDA_SUCCESS || !partitioned) return status;
  if (stream_ctas == 0 && p.max_partitions <= 1) return status;

  // Second kernel: merge the parts of every row that was split.
  const uint64_t rows = (uint64_t)p.sequences * p.query_heads;
  if (rows > 0x7fffffffull) return LOOM_CUDA_INVALID_ARGUMENT;
  const uint32_t grid = (uint32_t)rows;
  cudaError_t merge_status = cudaSuccess;
  if (stream_ctas != 0) {
#define LOOM_MERGE(type)                                                                              \
  merge_status = loom_launch::launch(                                                                 \
      merge_stream_kernel<type>, dim3(grid), dim3(kMergeThreads), 0, stream,                          \
      static_cast<const float*>(p.partials), static_cast<const uint32_t*>(p.item_meta),               \
      static_cast<const int32_t*>(p.sequence_lengths), p.query_heads, p.group, shape.heads_per_item, \
      p.value_head_size, p.max_sequence_length, p.output, p.emit_state, block_tile ? 8u : 0u)
    if (p.emit_state || a.dtype == 0) LOOM_MERGE(float);
    else if (a.dtype == 1) LOOM_MERGE(__half);
    else LOOM_MERGE(__nv_bfloat16);
#undef LOOM_MERGE
  } else {
    const uint64_t part_stride = state_stride(p.value_head_size);
    const uint64_t row_stride = part_stride * p.max_partitions;
#define LOOM_MERGE(type)                                                                          \
  merge_status = loom_launch::launch(                                                             \
      merge_states_kernel<type>, dim3(grid), dim3(kMergeThreads), 0, stream,                      \
      static_cast<const float*>(p.partials), row_stride, part_stride, p.value_head_size, 0u,      \
      static_cast<const int32_t*>(p.sequence_lengths), p.query_heads, p.partition_tokens,         \
      p.max_sequence_length, p.sliding_window, p.output, p.emit_state)
    if (p.emit_state || a.dtype == 0) LOOM_MERGE(float);
    else if (a.dtype == 1) LOOM_MERGE(__half);
    else LOOM_MERGE(__nv_bfloat16);
#undef LOOM_MERGE
  }
  return launched(merge_status, "merge kernel launch");
}

// The reference ABI: dense-inner NHD caches, block stride free.
int launch_reference_abi(uint32_t dtype, const void* query, const void* key_cache, const void* value_cache,
                         const int32_t* block_tables, const int32_t* sequence_lengths, void* output,
                         float* workspace, uint64_t workspace_elements, uint32_t sequences,
                         uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
                         uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size,
                         uint64_t key_block_stride, uint64_t value_block_stride,
                         uint32_t max_blocks_per_sequence, uint32_t max_sequence_length, float scale,
                         void* stream) {
  // paged_decode_attention.cu:1035-1048: a block stride must cover one block.
  const uint64_t key_block = (uint64_t)block_size * kv_heads * head_size;
  const uint64_t value_block = (uint64_t)block_size * kv_heads * value_head_size;
  if (key_block_stride < key_block || value_block_stride < value_block) return LOOM_CUDA_INVALID_ARGUMENT;
  LoomDecodeArgs a{};
  a.struct_size = sizeof(LoomDecodeArgs);
  a.dtype = dtype;
  a.cache_encoding = LOOM_CUDA_KV_CACHE_NATIVE;
  a.query = query;
  a.key_cache = key_cache;
  a.value_cache = value_cache;
  a.block_tables = block_tables;
  a.sequence_lengths = sequence_lengths;
  a.output = output;
  a.workspace = workspace;
  a.workspace_elements = workspace_elements;
  a.sequences = sequences;
  a.query_heads = query_heads;
  a.kv_heads = kv_heads;
  a.head_size = head_size;
  a.value_head_size = value_head_size;
  a.num_blocks = num_blocks;
  a.block_size = block_size;
  a.max_blocks_per_sequence = max_blocks_per_sequence;
  a.max_sequence_length = max_sequence_length;
  a.key_block_stride = key_block_stride;
  a.key_page_stride = (uint64_t)kv_heads * head_size;
  a.key_head_stride = head_size;
  a.value_block_stride = value_block_stride;
  a.value_page_stride = (uint64_t)kv_heads * value_head_size;
  a.value_head_stride = value_head_size;
  a.scale = scale;
  a.stream = stream;
  return launch_decode(a);
}

// ---- scratch that lives inside the library ---------------------------------------
//
// Some callers of a partitioned decode cannot hand over a workspace because they
// have no way to get device memory at that point: an engine that sized and
// claimed all of its GPU memory at start-up and treats any later allocation as a
// bug, a request handler that must not risk the device-wide stall an allocation
// can cause, or a plug-in host that gives extensions input and output buffers
// and nothing else. For them the library keeps one fixed block of device memory
// of its own. Every GPU that loads the library pays for it (16 MiB) until the
// process exits, which is why it is small and why larger shapes are refused.
constexpr uint64_t kBuiltInScratchFloats = 4ull << 20;  // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_built_in_scratch[kBuiltInScratchFloats];

// `g_built_in_scratch` in host code is only a handle for the runtime, not an
// address a kernel can use. The device address is asked for once per device,
// with that device current, and remembered.
float* built_in_scratch_address(cudaError_t* failure) {
  static std::atomic<float*> known[64];
  int device = 0;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) {
    *failure = status;
    return nullptr;
  }
  const bool cacheable = device >= 0 && device < 64;
  if (cacheable) {
    float* address = known[device].load(std::memory_order_acquire);
    if (address != nullptr) return address;
  }
  float* address = nullptr;
  status = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_built_in_scratch);
  if (status != cudaSuccess || address == nullptr) {
    *failure = status != cudaSuccess ? status : cudaErrorInvalidSymbol;
    cudaGetLastError();
    return nullptr;
  }
  if (cacheable) known[device].store(address, std::memory_order_release);
  return address;
}

void explain(char* text, uint64_t capacity, const char* format, unsigned long long a = 0,
             unsigned long long b = 0) {
  if (text != nullptr && capacity != 0) std::snprintf(text, (size_t)capacity, format, a, b);
}

void explain_text(char* text, uint64_t capacity, const char* message) {
  if (text != nullptr && capacity != 0) std::snprintf(text, (size_t)capacity, "%s", message);
}

}  // namespace loom_decode

// ================================================================ C ABI

extern "C" const char* loom_cuda_status_string(int status) {
  switch (status) {
    case LOOM_CUDA_SUCCESS: return "success";
    case LOOM_CUDA_INVALID_ARGUMENT: return "invalid argument";
    case LOOM_CUDA_UNSUPPORTED: return "unsupported";
    case LOOM_CUDA_LAUNCH_ERROR: return "CUDA launch error";
    case LOOM_CUDA_UNAVAILABLE: return "CUDA unavailable";
    default: return "unknown Loom CUDA status";
  }
}

#define LOOM_DEFINE_DECODE(suffix, scalar, code)                                                   \
  extern "C" int loom_cuda_paged_decode_attention_##suffix(                                        \
      const scalar* query, const scalar* key_cache, const scalar* value_cache,                    \
      const int32_t* block_tables, const int32_t* sequence_lengths, scalar* output,               \
      uint32_t sequences, uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,            \
      uint32_t value_head_size, uint32_t num_blocks, uint32_t block_size,                         \
      uint64_t key_block_stride, uint64_t value_block_stride, uint32_t max_blocks_per_sequence,   \
      uint32_t max_sequence_length, float scale, void* stream) {                                  \
    return loom_decode::launch_reference_abi(                                                     \
        code, query, key_cache, value_cache, block_tables, sequence_lengths, output, nullptr, 0,  \
        sequences, query_heads, kv_heads, head_size, value_head_size, num_blocks, block_size,     \
        key_block_stride, value_block_stride, max_blocks_per_sequence, max_sequence_length,       \
        scale, stream);                                                                           \
  }                                                                                               \
  extern "C" int loom_cuda_paged_decode_attention_split_k_##suffix(                                \
      const scalar* query, const scalar* key_cache, const scalar* value_cache,                    \
      const int32_t* block_tables, const int32_t* sequence_lengths, scalar* output,               \
      float* workspace, uint64_t workspace_elements, uint32_t sequences, uint32_t query_heads,    \
      uint32_t kv_heads, uint32_t head_size, uint32_t value_head_size, uint32_t num_blocks,       \
      uint32_t block_size, uint64_t key_block_stride, uint64_t value_block_stride,                \
      uint32_t max_blocks_per_sequence, uint32_t max_sequence_length, float scale,                \
      void* stream) {                                                                             \
    if (workspace == nullptr || workspace_elements == 0) return LOOM_CUDA_INVALID_ARGUMENT;       \
    return loom_decode::launch_reference_abi(                                                     \
        code, query, key_cache, value_cache, block_tables, sequence_lengths, output, workspace,   \
        workspace_elements, sequences, query_heads, kv_heads, head_size, value_head_size,         \
        num_blocks, block_size, key_block_stride, value_block_stride, max_blocks_per_sequence,    \
        max_sequence_length, scale, stream);                                                      \
  }

LOOM_DEFINE_DECODE(f32, float, 0u)
LOOM_DEFINE_DECODE(f16, uint16_t, 1u)
LOOM_DEFINE_DECODE(bf16, uint16_t, 2u)

extern "C" uint64_t loom_cuda_paged_decode_attention_split_k_workspace_elements(
    uint32_t sequences, uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t max_sequence_length) {
  if (sequences == 0 || query_heads == 0 || kv_heads == 0 || head_size == 0 || value_head_size == 0 ||
      max_sequence_length == 0 || query_heads % kv_heads != 0) {
    return 0;
  }
  // Short contexts are served by one pass per (sequence, KV head).
  if (max_sequence_length <= 256) return 0;
  return loom_decode::auto_workspace_elements(sequences, query_heads, kv_heads, value_head_size,
                                              max_sequence_length);
}

extern "C" uint32_t loom_cuda_paged_decode_default_partition_tokens(uint32_t sequences, uint32_t kv_heads,
                                                                    uint32_t max_sequence_length) {
  if (sequences == 0 || kv_heads == 0 || max_sequence_length == 0) return 0;
  return loom_decode::default_partition_tokens(sequences, kv_heads, max_sequence_length);
}

extern "C" uint64_t loom_cuda_paged_decode_workspace_elements(uint32_t sequences, uint32_t query_heads,
                                                              uint32_t kv_heads, uint32_t value_head_size,
                                                              uint32_t max_sequence_length,
                                                              uint32_t partition_tokens) {
  if (kv_heads == 0 || query_heads % kv_heads != 0) return 0;
  if (partition_tokens == 0) {
    return loom_decode::auto_workspace_elements(sequences, query_heads, kv_heads, value_head_size,
                                                max_sequence_length);
  }
  return loom_decode::fixed_workspace_elements(sequences, query_heads, value_head_size, max_sequence_length,
                                               partition_tokens);
}

// Copies a caller's LoomDecodeArgs of either known layout into the current one (options off for
// the shorter layout). False for a null pointer or an unknown struct_size.
extern "C" int loom_cuda_read_decode_args(const LoomDecodeArgs* args, LoomDecodeArgs* out) {
  if (args == nullptr || out == nullptr) return 0;
  if (args->struct_size != sizeof(LoomDecodeArgs) && args->struct_size != LOOM_DECODE_ARGS_BASE_SIZE) return 0;
  *out = LoomDecodeArgs{};
  std::memcpy(out, args, args->struct_size);
  out->struct_size = sizeof(LoomDecodeArgs);
  return 1;
}

extern "C" int loom_cuda_paged_decode_attention_ex(const LoomDecodeArgs* args) {
  LoomDecodeArgs current;
  if (!loom_cuda_read_decode_args(args, &current)) return LOOM_CUDA_INVALID_ARGUMENT;
  if (current.partition_tokens % 16 != 0) return LOOM_CUDA_INVALID_ARGUMENT;
  return loom_decode::launch_decode(current);
}

extern "C" int loom_cuda_merge_decode_states(const float* states, uint32_t parts, uint32_t rows,
                                             uint32_t value_head_size, uint32_t out_dtype, void* output,
                                             void* stream) {
  using namespace loom_decode;
  if (states == nullptr || output == nullptr || parts == 0 || rows == 0 || value_head_size == 0 ||
      out_dtype > 2 || rows > 0x7fffffffu) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const uint64_t row_stride = state_stride(value_head_size);
  const uint64_t part_stride = row_stride * rows;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  cudaError_t status = cudaSuccess;
#define LOOM_MERGE(type)                                                                               \
  status = loom_launch::launch(merge_states_kernel<type>, dim3(rows), dim3(kMergeThreads), 0,          \
                               cuda_stream, states, row_stride, part_stride, value_head_size, parts,   \
                               static_cast<const int32_t*>(nullptr), 1u, 1u, 0u, 0u, output, 0u)
  if (out_dtype == 0) LOOM_MERGE(float);
  else if (out_dtype == 1) LOOM_MERGE(__half);
  else LOOM_MERGE(__nv_bfloat16);
#undef LOOM_MERGE
  return launched(status, "merge kernel launch");
}

extern "C" int loom_cuda_supports_paged_decode(uint32_t dtype, uint32_t cache_encoding, uint32_t sequences,
                                               uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
                                               uint32_t value_head_size, uint32_t num_blocks,
                                               uint32_t block_size, uint32_t max_blocks_per_sequence,
                                               uint32_t max_sequence_length, const char** reason) {
  const char* why = nullptr;
  if (dtype > 2) {
    why = "B200 paged decode attention supports F32, FP16, and BF16 queries";
  } else if (cache_encoding > 1) {
    why = "B200 paged decode attention reads native or FP8 E4M3 caches";
  } else if (sequences == 0 || query_heads == 0 || kv_heads == 0 || head_size == 0 ||
             value_head_size == 0 || num_blocks == 0 || block_size == 0 ||
             max_blocks_per_sequence == 0 || max_sequence_length == 0 || query_heads % kv_heads != 0) {
    why = "paged decode attention contract is not well formed";
  } else if (max_sequence_length > (1u << 30) ||
             (uint64_t)sequences * query_heads > 0x7fffffffull || query_heads > 65535u) {
    why = "paged decode attention shape exceeds the CUDA ABI";
  } else if (!(head_size == value_head_size && (head_size == 64 || head_size == 128)) &&
             value_head_size > 32u * loom_decode::kScalarMaxValueRegs) {
    why = "B200 paged decode attention supports value heads of at most 512 elements";
  } else if (!loom_decode::scalar_smem_fits(head_size, value_head_size)) {
    // any shape may end on the CUDA-core route (F32, unaligned views); its shared memory bounds the head size
    why = "B200 paged decode attention head size exceeds the shared memory of its general kernel";
  }
  if (reason != nullptr) *reason = why != nullptr ? why : "supported";
  return why == nullptr ? 1 : 0;
}

extern "C" const char* loom_cuda_last_decode_route(void) { return loom_decode::g_last_route; }

extern "C" const char* loom_cuda_last_launch_failure(void) {
  const loom_launch::Failure& failure = loom_launch::last_failure();
  if (failure.error == cudaSuccess) return "none";
  static thread_local char text[192];
  std::snprintf(text, sizeof(text), "%s at %s", cudaGetErrorName(failure.error), failure.where);
  return text;
}

extern "C" uint64_t loom_cuda_plain_launch_retries(void) {
  return loom_launch::plain_retries().load(std::memory_order_relaxed);
}

extern "C" int loom_cuda_set_decode_copy_engine(uint32_t engine) {
  if (engine > 4) return LOOM_CUDA_INVALID_ARGUMENT;
  loom_decode::g_copy_engine.store(engine, std::memory_order_relaxed);
  return LOOM_CUDA_SUCCESS;
}

extern "C" int loom_cuda_set_programmatic_launch(uint32_t mode) {
  if (mode > 1) return LOOM_CUDA_INVALID_ARGUMENT;
  loom_launch::programmatic_mode().store(mode, std::memory_order_relaxed);
  return LOOM_CUDA_SUCCESS;
}

extern "C" int loom_cuda_set_wait_policy(uint32_t attempts, uint32_t unmatched_bytes) {
  // 16-byte multiples keep the armed byte count a value the copy engine could in principle deliver
  if (unmatched_bytes % 16u != 0 || unmatched_bytes > (1u << 20)) return LOOM_CUDA_INVALID_ARGUMENT;
  loom_launch::wait_policy_word().store((uint64_t)attempts | ((uint64_t)unmatched_bytes << 32),
                                        std::memory_order_relaxed);
  return LOOM_CUDA_SUCCESS;
}

extern "C" int loom_cuda_decode_timeout_flag(uint32_t* value, uint32_t reset) {
  if (value == nullptr) return LOOM_CUDA_INVALID_ARGUMENT;
  unsigned int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, loom_decode::g_decode_timeout_flag, sizeof(flag)) != cudaSuccess) {
    cudaGetLastError();
    return LOOM_CUDA_LAUNCH_ERROR;
  }
  unsigned int where = 0;
  if (cudaMemcpyFromSymbol(&where, loom_decode::g_decode_timeout_where, sizeof(where)) != cudaSuccess) {
    cudaGetLastError();
    return LOOM_CUDA_LAUNCH_ERROR;
  }
  *value = flag | where;
  if (reset != 0 && (flag | where) != 0) {
    const unsigned int zero = 0;
    if (cudaMemcpyToSymbol(loom_decode::g_decode_timeout_flag, &zero, sizeof(zero)) != cudaSuccess ||
        cudaMemcpyToSymbol(loom_decode::g_decode_timeout_where, &zero, sizeof(zero)) != cudaSuccess) {
      cudaGetLastError();
      return LOOM_CUDA_LAUNCH_ERROR;
    }
  }
  return LOOM_CUDA_SUCCESS;
}

// Partitioned decode for callers that cannot allocate: identical to
// loom_cuda_paged_decode_attention_ex, except that the partial states go into
// the library's own fixed block of device memory instead of a caller workspace
// (args->workspace and args->workspace_elements are ignored). Nothing is
// allocated or freed here or anywhere below this call.
extern "C" int loom_cuda_paged_decode_attention_built_in_scratch(const LoomDecodeArgs* args, char* error_text,
                                                                  uint64_t error_capacity) {
  using namespace loom_decode;
  explain(error_text, error_capacity, "ok");
  LoomDecodeArgs current;
  if (!loom_cuda_read_decode_args(args, &current) || current.partition_tokens % 16 != 0 ||
      current.kv_heads == 0 || current.query_heads % current.kv_heads != 0) {
    explain(error_text, error_capacity, "decode arguments are not well formed");
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  args = &current;
  const uint64_t needed =
      args->partition_tokens == 0
          ? auto_workspace_elements(args->sequences, args->query_heads, args->kv_heads, args->value_head_size,
                                    args->max_sequence_length, /*every_layout=*/false)
          : fixed_workspace_elements(args->sequences, args->query_heads, args->value_head_size,
                                     args->max_sequence_length, args->partition_tokens);
  if (needed == 0) {
    explain(error_text, error_capacity, "decode shape is empty or its scratch size overflows");
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  if (needed > kBuiltInScratchFloats) {
    explain(error_text, error_capacity,
            "this decode needs %llu F32 elements of scratch but the built-in block holds %llu; "
            "pass a workspace to loom_cuda_paged_decode_attention_ex instead",
            (unsigned long long)needed, (unsigned long long)kBuiltInScratchFloats);
    return LOOM_CUDA_UNSUPPORTED;
  }
  cudaError_t failure = cudaSuccess;
  float* scratch = built_in_scratch_address(&failure);
  if (scratch == nullptr) {
    explain(error_text, error_capacity, "the address of the built-in scratch block is unavailable (CUDA error %llu)",
            (unsigned long long)failure);
    return LOOM_CUDA_UNAVAILABLE;
  }
  // Every word of the block that the merge kernel reads is written by the decode
  // kernel of this same call, so nothing has to be cleared between calls.
  LoomDecodeArgs with_scratch = *args;
  with_scratch.workspace = scratch;
  with_scratch.workspace_elements = kBuiltInScratchFloats;
  const int status = launch_decode(with_scratch);
  if (status != LOOM_CUDA_SUCCESS) explain_text(error_text, error_capacity, loom_cuda_status_string(status));
  return status;
}
