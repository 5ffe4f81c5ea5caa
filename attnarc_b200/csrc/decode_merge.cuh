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
template <typename OT>
__device__ __forceinline__ void merge_row(const float* __restrict__ base, uint32_t parts,
                                          uint64_t part_stride, uint32_t value_head_size, uint64_t row,
                                          void* output, uint32_t emit_state) {
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
