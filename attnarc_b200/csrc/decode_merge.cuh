// Log-sum-exp merge of partial (O, max, sum) states: the arithmetic of the merge kernels.
//
// Replaces the merge of the reference's split-K path
// (crates/loom-cuda-sys/cuda/src/paged_decode_attention.cu:749-853), whose factors are computed
// by thread 0 alone.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "decode_common.cuh"

namespace loom_decode {

template <typename T>
__device__ __forceinline__ void narrow_store(T* out, float value);
template <>
__device__ __forceinline__ void narrow_store<float>(float* out, float value) { *out = value; }
template <>
__device__ __forceinline__ void narrow_store<__half>(__half* out, float value) { *out = __float2half_rn(value); }
template <>
__device__ __forceinline__ void narrow_store<__nv_bfloat16>(__nv_bfloat16* out, float value) {
  *out = __float2bfloat16_rn(value);
}

constexpr int kMergeThreads = 128;

// Merges `parts` states of one output row. Part i lives at base + i*part_stride
// and holds O (value_head_size floats), max (natural-log units) and sum. Each
// thread owns value dims and folds the parts in batches of eight whose loads
// are all issued before any is used: one round trip to memory per batch, no
// shared memory, no barrier, no shuffle. max and sum are recomputed by every
// thread from the same broadcast loads.
// Rows with many parts (one sequence far longer than a CTA's share: 40 parts on the long-context
// workload) would walk them eight at a time, one round trip to L2 after the other. They are merged by
// four groups of 32 threads instead: group q takes parts q, q + 4, ... (four per round trip, sixteen in
// flight per CTA), a thread owns four value dims (one 16-byte load per part), and the four partial
// results meet in shared memory. All threads of the CTA call this together (`parts` is CTA-uniform).
constexpr uint32_t kWideMergeParts = 17;  // from this many parts on

template <typename OT>
__device__ __forceinline__ void merge_row_wide(const float* __restrict__ base, uint32_t parts,
                                               uint64_t part_stride, uint32_t value_head_size, uint64_t row,
                                               void* output, uint32_t emit_state) {
  constexpr int kGroups = kMergeThreads / 32;
  constexpr int kBatch = 4;
  constexpr int kMaxQuads = 64;  // value head sizes up to 256
  __shared__ float group_top[kGroups], group_total[kGroups];
  __shared__ float4 group_acc[kGroups][kMaxQuads];
  const uint32_t group = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t quads = value_head_size >> 2;
  for (uint32_t quad0 = 0; quad0 < quads; quad0 += 32) {  // one pass for value head sizes up to 128
    const uint32_t quad = quad0 + lane;
    const bool owns = quad < quads;
    float top = -INFINITY, total = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t first = group; first < parts; first += kGroups * kBatch) {
      float part_max[kBatch], part_sum[kBatch];
      float4 part_o[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const uint32_t part = first + j * kGroups;
        const bool live = part < parts;
        const float* state = base + (uint64_t)(live ? part : first) * part_stride;
        part_sum[j] = live ? __ldg(state + value_head_size + 1) : 0.0f;
        part_max[j] = __ldg(state + value_head_size);
        // a state row is 8-byte, not 16-byte aligned ((value head size + 2) floats per row)
        const float2 low = owns ? __ldg(reinterpret_cast<const float2*>(state) + 2 * quad) : make_float2(0.0f, 0.0f);
        const float2 high = owns ? __ldg(reinterpret_cast<const float2*>(state) + 2 * quad + 1) : make_float2(0.0f, 0.0f);
        part_o[j] = make_float4(low.x, low.y, high.x, high.y);
      }
      float batch_top = top;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (part_sum[j] > 0.0f) batch_top = fmaxf(batch_top, part_max[j]);
      }
      if (batch_top > -INFINITY) {
        const float rescale = exp2f((top - batch_top) * kLog2e);  // 0 when top is still -inf
        total *= rescale;
        acc.x *= rescale, acc.y *= rescale, acc.z *= rescale, acc.w *= rescale;
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          if (part_sum[j] > 0.0f) {
            const float factor = exp2f((part_max[j] - batch_top) * kLog2e);
            total += part_sum[j] * factor;
            acc.x += part_o[j].x * factor, acc.y += part_o[j].y * factor;
            acc.z += part_o[j].z * factor, acc.w += part_o[j].w * factor;
          }
        }
        top = batch_top;
      }
    }
    __syncthreads();  // the previous pass has been read
    if (lane == 0) {
      group_top[group] = top;
      group_total[group] = total;
    }
    if (owns) group_acc[group][quad & (kMaxQuads - 1)] = acc;
    __syncthreads();
    if (group == 0 && owns) {
      float all_top = -INFINITY;
#pragma unroll
      for (int q = 0; q < kGroups; ++q) all_top = fmaxf(all_top, group_top[q]);
      float all_total = 0.0f;
      float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (all_top > -INFINITY) {
#pragma unroll
        for (int q = 0; q < kGroups; ++q) {
          const float factor = exp2f((group_top[q] - all_top) * kLog2e);  // 0 for a group without live parts
          const float4 o = group_acc[q][quad & (kMaxQuads - 1)];
          all_total += group_total[q] * factor;
          sum.x += o.x * factor, sum.y += o.y * factor, sum.z += o.z * factor, sum.w += o.w * factor;
        }
      }
      if (emit_state) {
        float* out = static_cast<float*>(output) + row * state_stride(value_head_size);
        *reinterpret_cast<float2*>(out + 4 * quad) = make_float2(sum.x, sum.y);
        *reinterpret_cast<float2*>(out + 4 * quad + 2) = make_float2(sum.z, sum.w);
        if (quad == 0) {
          out[value_head_size] = all_top;
          out[value_head_size + 1] = all_total;
        }
      } else {
        OT* out = static_cast<OT*>(output) + row * value_head_size + 4 * quad;
        narrow_store<OT>(out, all_total > 0.0f ? sum.x / all_total : 0.0f);
        narrow_store<OT>(out + 1, all_total > 0.0f ? sum.y / all_total : 0.0f);
        narrow_store<OT>(out + 2, all_total > 0.0f ? sum.z / all_total : 0.0f);
        narrow_store<OT>(out + 3, all_total > 0.0f ? sum.w / all_total : 0.0f);
      }
    }
  }
}

template <typename OT>
__device__ __forceinline__ void merge_row(const float* __restrict__ base, uint32_t parts,
                                          uint64_t part_stride, uint32_t value_head_size, uint64_t row,
                                          void* output, uint32_t emit_state) {
  // wide form: states that 8-byte loads can read (value head size a multiple of 4, even strides)
  if (parts >= kWideMergeParts && (value_head_size & 3u) == 0 && value_head_size <= 256 &&
      (part_stride & 1u) == 0 && (reinterpret_cast<uintptr_t>(base) & 7u) == 0) {
    merge_row_wide<OT>(base, parts, part_stride, value_head_size, row, output, emit_state);
    return;
  }
  constexpr int kBatch = 8;
  for (uint32_t dv = threadIdx.x; dv < value_head_size; dv += kMergeThreads) {
    float top = -INFINITY, total = 0.0f, acc = 0.0f;
    for (uint32_t first = 0; first < parts; first += kBatch) {
      float part_max[kBatch], part_sum[kBatch], part_o[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const bool live = first + j < parts;
        const float* state = base + (uint64_t)(live ? first + j : first) * part_stride;
        part_sum[j] = live ? __ldg(state + value_head_size + 1) : 0.0f;
        part_max[j] = __ldg(state + value_head_size);
        part_o[j] = __ldg(state + dv);
      }
      float batch_top = top;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (part_sum[j] > 0.0f) batch_top = fmaxf(batch_top, part_max[j]);
      }
      if (batch_top > -INFINITY) {
        const float rescale = exp2f((top - batch_top) * kLog2e);  // 0 when top is still -inf
        total *= rescale;
        acc *= rescale;
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          if (part_sum[j] > 0.0f) {
            const float factor = exp2f((part_max[j] - batch_top) * kLog2e);
            total += part_sum[j] * factor;
            acc += part_o[j] * factor;
          }
        }
        top = batch_top;
      }
    }
    if (emit_state) {
      float* out = static_cast<float*>(output) + row * state_stride(value_head_size);
      out[dv] = acc;
      if (dv == 0) {
        out[value_head_size] = top;
        out[value_head_size + 1] = total;
      }
    } else {
      narrow_store<OT>(static_cast<OT*>(output) + row * value_head_size + dv,
                       total > 0.0f ? acc / total : 0.0f);
    }
  }
}

}  // namespace loom_decode
