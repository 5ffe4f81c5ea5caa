// Shared pieces of the paged-decode kernels: the launch parameter block, the
// partial-state format, and the small PTX wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "launch_util.cuh"

namespace loom_decode {

// log2(e): scores are kept in base-2 units so the softmax uses ex2.
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Partial state of one (sequence, query head, partition): value_head_size
// floats of sum_i exp(s_i - max) * v_i, then max (natural-log units of the
// scaled score), then sum_i exp(s_i - max). The reference keeps the same triple
// (crates/loom-cuda-sys/cuda/src/paged_decode_attention.cu:551,685,701,743).
__host__ __device__ inline uint32_t state_stride(uint32_t value_head_size) {
  return value_head_size + 2u;
}

struct DecodeParams {
  const void* query;
  const void* key_cache;
  const void* value_cache;
  const float* key_scales;    // FP8 cache only
  const float* value_scales;  // FP8 cache only
  const int32_t* block_tables;
  const int32_t* sequence_lengths;
  void* output;      // [sequences, query_heads, Dv] of the query type, or F32 states
  float* partials;   // workspace [sequences*query_heads, max_partitions, Dv+2] or null
  uint32_t* item_meta;  // balanced kernel only: (first CTA, CTA count) per work item
  uint32_t sequences, query_heads, kv_heads, group;  // group = query_heads / kv_heads
  uint32_t head_size, value_head_size;
  uint32_t num_blocks, block_size, max_blocks_per_sequence, max_sequence_length;
  uint32_t partition_tokens;  // tokens per partition (whole context when partials == null)
  uint32_t max_partitions;
  uint32_t scale_stride;
  uint32_t block_shift;  // log2(block_size), or 32 if it is not a power of two
  uint32_t emit_state;  // final rows are F32 states instead of normalised output
  uint64_t k_block, k_page, k_head, v_block, v_page, v_head;  // element strides
  uint64_t q_token, q_head;                                   // element strides of the query
  float scale_log2;  // softmax scale * log2(e)
  // Options beyond the reference's contract (its design note lists both as later contract fields,
  // docs/design/paged-decode-attention.md:42-52). 0 = off.
  uint32_t sliding_window;  // a query sees only the last `sliding_window` tokens of its sequence
  float soft_cap_log2;      // logits soft cap * log2(e): score -> cap * tanh(score / cap)
  float inv_soft_cap_log2;
  // Balanced TMA-fed kernel only: lengths and block tables were written before the kernel
  // preceding this one in the stream started, so they may be read before that kernel has completed.
  uint32_t early_metadata;
  uint32_t wait_attempts;         // polls after which a wait on a copy barrier gives up
  uint32_t wait_unmatched_bytes;  // self-test: barriers are armed for this many bytes too many
};

// ---------------------------------------------------------------- PTX

__device__ __forceinline__ uint32_t smem_address(const void* pointer) {
  return (uint32_t)__cvta_generic_to_shared(pointer);
}

// 16-byte asynchronous global->shared copy that bypasses L1; `bytes` of 0
// writes zeros without touching global memory.
__device__ __forceinline__ void cp_async_16(uint32_t smem, const void* global, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(global), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem));
}

// Warp-wide transpose of an 8x8 matrix of 16-bit elements held one 32-bit
// register per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t value) {
  uint32_t out;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(out) : "r"(value));
  return out;
}

__device__ __forceinline__ void mma_16816_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_16816_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// How the K bytes of an FP8 cache become F16 MMA operands: by integer
// operations (true) or by the conversion instruction (false). Both are exact.
#ifndef LOOM_FP8_KEY_BY_ALU
#define LOOM_FP8_KEY_BY_ALU 0
#endif
constexpr bool kFp8KeyByAlu = LOOM_FP8_KEY_BY_ALU != 0;

// Four E4M3 bytes [b3 b2 b1 b0] -> F16 pairs (b0, b2) and (b1, b3), each value
// 2^-8 times the E4M3 value, using integer operations only. An E4M3 byte
// s eeee mmm placed as s 0eeee mmm0000000 is an F16 with the same sign and
// mantissa whose exponent field is read with bias 15 instead of 7, i.e. the
// value divided by 2^8; subnormals map to subnormals under the same factor, so
// the map is exact for every finite code. The conversion instruction
// (cvt.rn.f16x2.e4m3x2) shares a quarter-rate pipe with ex2; this form keeps
// that pipe free.
__device__ __forceinline__ uint32_t e4m3_high_bytes_to_f16x2(uint32_t x) {
  return ((x >> 1) & 0x3f803f80u) | (x & 0x80008000u);
}
__device__ __forceinline__ void e4m3x4_to_f16_by_alu(uint32_t packed, uint32_t& even, uint32_t& odd) {
  odd = e4m3_high_bytes_to_f16x2(packed);        // bytes 1 and 3
  even = e4m3_high_bytes_to_f16x2(packed << 8);  // bytes 0 and 2
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Four E4M3 bytes -> two f16x2 registers (bytes 0,1 and bytes 2,3). Exact:
// every E4M3 value is an F16 value.
__device__ __forceinline__ void e4m3x4_to_f16x2x2(uint32_t packed, uint32_t& low, uint32_t& high) {
  asm("{\n"
      ".reg .b16 lo, hi;\n"
      "mov.b32 {lo, hi}, %2;\n"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n"
      "}\n"
      : "=r"(low), "=r"(high)
      : "r"(packed));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float low, float high) {
  __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
  return *reinterpret_cast<uint32_t*>(&pair);
}

__device__ __forceinline__ uint32_t pack_f16x2(float low, float high) {
  __half2 pair = __floats2half2_rn(low, high);
  return *reinterpret_cast<uint32_t*>(&pair);
}

// First token a query sees under a sliding window of `window` tokens (0 = no window).
__device__ __forceinline__ uint32_t window_begin(uint32_t length, uint32_t window) {
  return (window != 0u && length > window) ? length - window : 0u;
}

// cap * tanh(score / cap) for a score in base-2 units (cap2 = cap * log2(e), inv_cap2 = 1 / cap2),
// as tanh(x) = 1 - 2 / (exp(2x) + 1): two special-function operations, absolute error of tanh
// below 1e-6 (the one-instruction tanh.approx is off by up to 5e-4, which a cap of 30..50
// multiplies into the exponent).
__device__ __forceinline__ float soft_capped(float score2, float cap2, float inv_cap2) {
  const float doubled = fminf(score2 * inv_cap2 * (2.0f * kLog2e), 64.0f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(doubled));
  return cap2 * (1.0f - __fdividef(2.0f, e + 1.0f));
}

// Physical block of a logical block, clamped so that a corrupt table entry can
// never turn into an address outside the cache allocation.
__device__ __forceinline__ uint32_t clamp_block(int32_t block, uint32_t num_blocks) {
  const uint32_t unsigned_block = (uint32_t)block;
  return unsigned_block < num_blocks ? unsigned_block : num_blocks - 1u;
}

// Length of a sequence, clamped into [0, max_sequence_length].
__device__ __forceinline__ uint32_t clamp_length(int32_t length, uint32_t maximum) {
  if (length <= 0) return 0u;
  return (uint32_t)length < maximum ? (uint32_t)length : maximum;
}

}  // namespace loom_decode
