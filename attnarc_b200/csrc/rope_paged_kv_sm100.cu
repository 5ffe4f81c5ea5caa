// Fused in-place RoPE on Q and K + paged write of the rotated K and of V.
//
// Replaces crates/loom-cuda-sys/cuda/src/rope_paged_kv.cu (kernel :63-212,
// launcher :214-266, exported symbols :270-406) behind the same three
// `loom_cuda_rope_paged_kv_write_*` symbols.
//
// Design for B200. The step is tiny (well under 10 MB even at the largest
// configuration) and therefore bound by launch latency and by how many bytes
// each thread moves per instruction, not by HBM bandwidth. The work of one
// token is cut into independent 16-byte "units" and spread over a flat grid,
// so 64 tokens fill dozens of CTAs instead of 64:
//   - a rotary unit owns VEC pairs of one head: two 16-byte loads of the
//     head, two of the cos/sin row, two 16-byte stores back, and for a K head
//     two vector stores into the cache;
//   - a tail unit copies 16 bytes of the non-rotated end of a K head;
//   - a value unit copies 16 bytes of V.
// A scalar kernel with one element (pair) per thread takes every shape whose
// pointers, strides or widths are not 16-byte friendly.
//
// Bit exactness. The CPU reference computes first*cos - second*sin and
// second*cos + first*sin with four separately rounded F32 operations, rounds
// to the storage type, and for an FP8 cache divides that rounded value by the
// scale in F32 before an RNE saturating E4M3 encode
// (crates/loom-kernels/src/rope_kv.rs:616-626,770-775). nvcc would contract
// the multiply-adds into FMAs, so the arithmetic below is spelled with
// __fmul_rn/__fsub_rn/__fadd_rn/__fdiv_rn, which the compiler never fuses.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <limits>
#include <type_traits>

#include "../../include/loom_launch.h"
#include "launch_util.cuh"

namespace {

constexpr int kThreads = 256;

struct RopeParams {
  void* query;
  void* key;
  const void* value;
  const int64_t* positions;
  const void* cos_sin;
  void* key_cache;
  void* value_cache;
  const float* key_scales;
  const float* value_scales;
  const int64_t* slot_mapping;
  uint32_t tokens, cache_tokens, query_heads, kv_heads, head_size;
  uint32_t value_head_size, rotary_dim, max_position, num_blocks, block_size;
  uint32_t scale_stride, is_neox;
  uint64_t q_token, q_head, k_token, k_head, v_token, v_head;
  uint64_t kc_block, kc_page, kc_head, vc_block, vc_page, vc_head;
};

template <typename T>
struct Element;

template <>
struct Element<float> {
  static __device__ __forceinline__ float widen(float value) { return value; }
  static __device__ __forceinline__ float narrow(float value) { return value; }
};

template <>
struct Element<__half> {
  static __device__ __forceinline__ float widen(__half value) { return __half2float(value); }
  static __device__ __forceinline__ __half narrow(float value) { return __float2half_rn(value); }
};

template <>
struct Element<__nv_bfloat16> {
  static __device__ __forceinline__ float widen(__nv_bfloat16 value) { return __bfloat162float(value); }
  static __device__ __forceinline__ __nv_bfloat16 narrow(float value) { return __float2bfloat16_rn(value); }
};

// One E4M3 byte from a value already rounded to the storage type.
__device__ __forceinline__ uint8_t encode_e4m3(float rounded, float scale) {
  return (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(rounded, scale), __NV_SATFINITE, __NV_E4M3);
}

// The rotation with the reference's rounding sequence.
template <typename T>
__device__ __forceinline__ void rotate_pair(T& first, T& second, T cosine, T sine) {
  const float a = Element<T>::widen(first);
  const float b = Element<T>::widen(second);
  const float c = Element<T>::widen(cosine);
  const float s = Element<T>::widen(sine);
  first = Element<T>::narrow(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
  second = Element<T>::narrow(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
}

template <typename T>
struct alignas(16) Vec16 {
  static constexpr int kCount = 16 / sizeof(T);
  T lane[kCount];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* pointer) {
  Vec16<T> out;
  *reinterpret_cast<uint4*>(&out) = *reinterpret_cast<const uint4*>(pointer);
  return out;
}

template <typename T>
__device__ __forceinline__ void store16(T* pointer, const Vec16<T>& value) {
  *reinterpret_cast<uint4*>(pointer) = *reinterpret_cast<const uint4*>(&value);
}

// Stores kCount cache elements: the vector itself for a native cache, the
// packed E4M3 bytes (8 or 4 of them) for an FP8 cache.
template <typename T, bool kFp8>
__device__ __forceinline__ void store_cache(void* cache, uint64_t offset,
                                            const Vec16<T>& value, float scale) {
  if constexpr (kFp8) {
    constexpr int kCount = Vec16<T>::kCount;
    uint32_t words[kCount / 4];
#pragma unroll
    for (int w = 0; w < kCount / 4; ++w) {
      uint32_t packed = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        packed |= (uint32_t)encode_e4m3(Element<T>::widen(value.lane[w * 4 + b]), scale) << (8 * b);
      }
      words[w] = packed;
    }
    uint8_t* target = static_cast<uint8_t*>(cache) + offset;
    if constexpr (kCount == 8) {
      *reinterpret_cast<uint2*>(target) = make_uint2(words[0], words[1]);
    } else {
      *reinterpret_cast<uint32_t*>(target) = words[0];
    }
  } else {
    store16(static_cast<T*>(cache) + offset, value);
  }
}

// Where a token's K/V row goes, or nothing to write.
struct Slot {
  bool write;
  uint64_t block, page;
};

__device__ __forceinline__ Slot resolve_slot(const RopeParams& p, uint32_t token) {
  Slot slot{false, 0, 0};
  if (token < p.cache_tokens) {
    const int64_t raw = p.slot_mapping[token];
    const uint64_t capacity = (uint64_t)p.num_blocks * p.block_size;
    if (raw >= 0 && (uint64_t)raw < capacity) {
      slot.write = true;
      slot.block = (uint64_t)raw / p.block_size;
      slot.page = (uint64_t)raw % p.block_size;
    }
  }
  return slot;
}

// ---------------------------------------------------------------- vector

template <typename T, bool kFp8>
__global__ void __launch_bounds__(kThreads)
rope_paged_kv_vector_kernel(const RopeParams p, uint32_t rotary_units_per_head,
                            uint32_t tail_units_per_head,
                            uint32_t value_units_per_head,
                            uint32_t units_per_token) {
  constexpr int kVec = Vec16<T>::kCount;
  // launched early by programmatic dependent launch: global memory is touched
  // only after the kernels before this one have completed
  loom_launch::release_dependents();  // the decode kernel of the step may set itself up meanwhile
  loom_launch::grid_dependency_wait();
  const uint64_t flat = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
  const uint64_t total = (uint64_t)p.tokens * units_per_token;
  if (flat >= total) return;
  const uint32_t token = (uint32_t)(flat / units_per_token);
  uint32_t unit = (uint32_t)(flat % units_per_token);

  const int64_t position = p.positions[token];
  // A position outside the table would read past cos_sin_cache; the reference
  // kernel drops the whole token in that case and so does this one.
  if (position < 0 || (uint64_t)position >= p.max_position) return;

  T* query = static_cast<T*>(p.query);
  T* key = static_cast<T*>(p.key);
  const T* value = static_cast<const T*>(p.value);
  const uint32_t half = p.rotary_dim / 2;
  const uint32_t heads = p.query_heads + p.kv_heads;
  const uint32_t rotary_units = heads * rotary_units_per_head;

  if (unit < rotary_units) {
    const uint32_t head = unit / rotary_units_per_head;
    const uint32_t chunk = unit % rotary_units_per_head;
    const bool is_key = head >= p.query_heads;
    const uint32_t kv_head = head - p.query_heads;
    T* row = is_key ? key + (uint64_t)token * p.k_token + (uint64_t)kv_head * p.k_head
                    : query + (uint64_t)token * p.q_token + (uint64_t)head * p.q_head;
    const T* cos_sin = static_cast<const T*>(p.cos_sin) + (uint64_t)position * p.rotary_dim;
    const Vec16<T> cosine = load16(cos_sin + chunk * kVec);
    const Vec16<T> sine = load16(cos_sin + half + chunk * kVec);
    uint32_t first_offset, second_offset;
    Vec16<T> first, second;
    if (p.is_neox) {
      first_offset = chunk * kVec;
      second_offset = half + chunk * kVec;
      first = load16(row + first_offset);
      second = load16(row + second_offset);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        rotate_pair(first.lane[i], second.lane[i], cosine.lane[i], sine.lane[i]);
      }
    } else {
      // Interleaved pairs: two adjacent vectors hold kVec pairs (even, odd).
      first_offset = chunk * 2 * kVec;
      second_offset = first_offset + kVec;
      first = load16(row + first_offset);
      second = load16(row + second_offset);
#pragma unroll
      for (int i = 0; i < kVec / 2; ++i) {
        rotate_pair(first.lane[2 * i], first.lane[2 * i + 1], cosine.lane[i], sine.lane[i]);
        rotate_pair(second.lane[2 * i], second.lane[2 * i + 1],
                    cosine.lane[kVec / 2 + i], sine.lane[kVec / 2 + i]);
      }
    }
    store16(row + first_offset, first);
    store16(row + second_offset, second);
    if (is_key) {
      const Slot slot = resolve_slot(p, token);
      if (slot.write) {
        const float scale = kFp8 ? p.key_scales[(uint64_t)kv_head * p.scale_stride] : 1.0f;
        const uint64_t base = slot.block * p.kc_block + slot.page * p.kc_page +
                              (uint64_t)kv_head * p.kc_head;
        store_cache<T, kFp8>(p.key_cache, base + first_offset, first, scale);
        store_cache<T, kFp8>(p.key_cache, base + second_offset, second, scale);
      }
    }
    return;
  }
  unit -= rotary_units;

  const Slot slot = resolve_slot(p, token);
  if (!slot.write) return;

  const uint32_t tail_units = p.kv_heads * tail_units_per_head;
  if (unit < tail_units) {
    const uint32_t kv_head = unit / tail_units_per_head;
    const uint32_t dim = p.rotary_dim + (unit % tail_units_per_head) * kVec;
    const Vec16<T> data =
        load16(key + (uint64_t)token * p.k_token + (uint64_t)kv_head * p.k_head + dim);
    const float scale = kFp8 ? p.key_scales[(uint64_t)kv_head * p.scale_stride] : 1.0f;
    store_cache<T, kFp8>(p.key_cache,
                         slot.block * p.kc_block + slot.page * p.kc_page +
                             (uint64_t)kv_head * p.kc_head + dim,
                         data, scale);
    return;
  }
  unit -= tail_units;

  const uint32_t kv_head = unit / value_units_per_head;
  const uint32_t dim = (unit % value_units_per_head) * kVec;
  const Vec16<T> data =
      load16(value + (uint64_t)token * p.v_token + (uint64_t)kv_head * p.v_head + dim);
  const float scale = kFp8 ? p.value_scales[(uint64_t)kv_head * p.scale_stride] : 1.0f;
  store_cache<T, kFp8>(p.value_cache,
                       slot.block * p.vc_block + slot.page * p.vc_page +
                           (uint64_t)kv_head * p.vc_head + dim,
                       data, scale);
}

// ---------------------------------------------------------------- scalar

template <typename T, bool kFp8>
__device__ __forceinline__ void store_cache_scalar(void* cache, uint64_t offset,
                                                   T value, float scale) {
  if constexpr (kFp8) {
    static_cast<uint8_t*>(cache)[offset] = encode_e4m3(Element<T>::widen(value), scale);
  } else {
    static_cast<T*>(cache)[offset] = value;
  }
}

// One thread per rotated pair, per K tail element, per V element.
template <typename T, bool kFp8>
__global__ void __launch_bounds__(kThreads)
rope_paged_kv_scalar_kernel(const RopeParams p, uint32_t units_per_token) {
  loom_launch::release_dependents();  // the decode kernel of the step may set itself up meanwhile
  loom_launch::grid_dependency_wait();
  const uint64_t flat = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
  const uint64_t total = (uint64_t)p.tokens * units_per_token;
  if (flat >= total) return;
  const uint32_t token = (uint32_t)(flat / units_per_token);
  uint32_t unit = (uint32_t)(flat % units_per_token);

  const int64_t position = p.positions[token];
  if (position < 0 || (uint64_t)position >= p.max_position) return;

  T* query = static_cast<T*>(p.query);
  T* key = static_cast<T*>(p.key);
  const T* value = static_cast<const T*>(p.value);
  const uint32_t half = p.rotary_dim / 2;
  const uint32_t rotary_units = (p.query_heads + p.kv_heads) * half;

  if (unit < rotary_units) {
    const uint32_t head = unit / half;
    const uint32_t pair = unit % half;
    const bool is_key = head >= p.query_heads;
    const uint32_t kv_head = head - p.query_heads;
    T* row = is_key ? key + (uint64_t)token * p.k_token + (uint64_t)kv_head * p.k_head
                    : query + (uint64_t)token * p.q_token + (uint64_t)head * p.q_head;
    const T* cos_sin = static_cast<const T*>(p.cos_sin) + (uint64_t)position * p.rotary_dim;
    const uint32_t first_dim = p.is_neox ? pair : pair * 2;
    const uint32_t second_dim = p.is_neox ? pair + half : pair * 2 + 1;
    T first = row[first_dim], second = row[second_dim];
    rotate_pair(first, second, cos_sin[pair], cos_sin[half + pair]);
    row[first_dim] = first;
    row[second_dim] = second;
    if (is_key) {
      const Slot slot = resolve_slot(p, token);
      if (slot.write) {
        const float scale = kFp8 ? p.key_scales[(uint64_t)kv_head * p.scale_stride] : 1.0f;
        const uint64_t base = slot.block * p.kc_block + slot.page * p.kc_page +
                              (uint64_t)kv_head * p.kc_head;
        store_cache_scalar<T, kFp8>(p.key_cache, base + first_dim, first, scale);
        store_cache_scalar<T, kFp8>(p.key_cache, base + second_dim, second, scale);
      }
    }
    return;
  }
  unit -= rotary_units;

  const Slot slot = resolve_slot(p, token);
  if (!slot.write) return;

  const uint32_t tail_width = p.head_size - p.rotary_dim;
  const uint32_t tail_units = p.kv_heads * tail_width;
  if (unit < tail_units) {
    const uint32_t kv_head = unit / tail_width;
    const uint32_t dim = p.rotary_dim + unit % tail_width;
    const float scale = kFp8 ? p.key_scales[(uint64_t)kv_head * p.scale_stride] : 1.0f;
    store_cache_scalar<T, kFp8>(
        p.key_cache,
        slot.block * p.kc_block + slot.page * p.kc_page + (uint64_t)kv_head * p.kc_head + dim,
        key[(uint64_t)token * p.k_token + (uint64_t)kv_head * p.k_head + dim], scale);
    return;
  }
  unit -= tail_units;

  const uint32_t kv_head = unit / p.value_head_size;
  const uint32_t dim = unit % p.value_head_size;
  const float scale = kFp8 ? p.value_scales[(uint64_t)kv_head * p.scale_stride] : 1.0f;
  store_cache_scalar<T, kFp8>(
      p.value_cache,
      slot.block * p.vc_block + slot.page * p.vc_page + (uint64_t)kv_head * p.vc_head + dim,
      value[(uint64_t)token * p.v_token + (uint64_t)kv_head * p.v_head + dim], scale);
}

// ---------------------------------------------------------------- launch

bool aligned_to(const void* pointer, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(pointer) % bytes) == 0;
}

template <typename T>
bool vector_path_fits(const RopeParams& p, bool fp8) {
  constexpr uint32_t kVec = 16 / sizeof(T);
  const uint32_t half = p.rotary_dim / 2;
  const size_t cache_vector_bytes = fp8 ? kVec : 16;
  const auto multiple = [](uint64_t value, uint64_t of) { return value % of == 0; };
  return half % kVec == 0 && p.head_size % kVec == 0 &&
         p.value_head_size % kVec == 0 && aligned_to(p.query, 16) &&
         aligned_to(p.key, 16) && aligned_to(p.value, 16) &&
         aligned_to(p.cos_sin, 16) && aligned_to(p.key_cache, cache_vector_bytes) &&
         aligned_to(p.value_cache, cache_vector_bytes) &&
         multiple(p.q_token, kVec) && multiple(p.q_head, kVec) &&
         multiple(p.k_token, kVec) && multiple(p.k_head, kVec) &&
         multiple(p.v_token, kVec) && multiple(p.v_head, kVec) &&
         multiple(p.kc_block, kVec) && multiple(p.kc_page, kVec) &&
         multiple(p.kc_head, kVec) && multiple(p.vc_block, kVec) &&
         multiple(p.vc_page, kVec) && multiple(p.vc_head, kVec);
}

template <typename T, bool kFp8>
int launch_typed(const RopeParams& p, cudaStream_t stream) {
  constexpr uint32_t kVec = 16 / sizeof(T);
  const uint32_t heads = p.query_heads + p.kv_heads;
  if (vector_path_fits<T>(p, kFp8)) {
    const uint32_t rotary_units = (p.rotary_dim / 2) / kVec;
    const uint32_t tail_units = (p.head_size - p.rotary_dim) / kVec;
    const uint32_t value_units = p.value_head_size / kVec;
    const uint64_t per_token = (uint64_t)heads * rotary_units +
                               (uint64_t)p.kv_heads * (tail_units + value_units);
    const uint64_t blocks = ((uint64_t)p.tokens * per_token + kThreads - 1) / kThreads;
    if (per_token > 0xffffffffull || blocks > 0x7fffffffull) return LOOM_CUDA_INVALID_ARGUMENT;
    return loom_launch::failed(
        loom_launch::launch(rope_paged_kv_vector_kernel<T, kFp8>, dim3((uint32_t)blocks), dim3(kThreads), 0, stream,
                            p, rotary_units, tail_units, value_units, (uint32_t)per_token),
        "RoPE + paged-KV write kernel launch");
  } else {
    const uint64_t per_token =
        (uint64_t)heads * (p.rotary_dim / 2) +
        (uint64_t)p.kv_heads * ((p.head_size - p.rotary_dim) + p.value_head_size);
    const uint64_t blocks = ((uint64_t)p.tokens * per_token + kThreads - 1) / kThreads;
    if (per_token > 0xffffffffull || blocks > 0x7fffffffull) return LOOM_CUDA_INVALID_ARGUMENT;
    // The status is this launch's own: an error that some earlier call of the process left in the
    // runtime's last-error slot is not this operator's failure and is not looked at.
    return loom_launch::failed(
        loom_launch::launch(rope_paged_kv_scalar_kernel<T, kFp8>, dim3((uint32_t)blocks), dim3(kThreads), 0, stream,
                            p, (uint32_t)per_token),
        "RoPE + paged-KV write kernel launch");
  }
}

// Argument rules of the reference launcher (rope_paged_kv.cu:231-250).
template <typename T>
int launch_rope_paged_kv_write(
    void* query, void* key, const void* value, const int64_t* positions,
    const void* cos_sin_cache, void* key_cache, void* value_cache,
    const float* key_scales, const float* value_scales,
    const int64_t* slot_mapping, uint32_t tokens, uint32_t cache_tokens,
    uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,
    uint32_t value_head_size, uint32_t rotary_dim, uint32_t max_position,
    uint32_t num_blocks, uint32_t block_size, uint32_t cache_encoding,
    uint32_t scale_stride, uint64_t query_token_stride,
    uint64_t query_head_stride, uint64_t key_token_stride,
    uint64_t key_head_stride, uint64_t value_token_stride,
    uint64_t value_head_stride, uint64_t key_cache_block_stride,
    uint64_t key_cache_page_stride, uint64_t key_cache_head_stride,
    uint64_t value_cache_block_stride, uint64_t value_cache_page_stride,
    uint64_t value_cache_head_stride, uint32_t is_neox, void* stream) {
  if (cache_encoding != LOOM_CUDA_KV_CACHE_NATIVE &&
      cache_encoding != LOOM_CUDA_KV_CACHE_FP8_E4M3) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const bool fp8 = cache_encoding == LOOM_CUDA_KV_CACHE_FP8_E4M3;
  if (query == nullptr || key == nullptr || value == nullptr ||
      positions == nullptr || cos_sin_cache == nullptr || key_cache == nullptr ||
      value_cache == nullptr || tokens == 0 ||
      (fp8 && (key_scales == nullptr || value_scales == nullptr)) ||
      (cache_tokens > 0 && slot_mapping == nullptr) || cache_tokens > tokens ||
      query_heads == 0 || kv_heads == 0 || head_size == 0 ||
      value_head_size == 0 || rotary_dim == 0 || (rotary_dim & 1u) != 0 ||
      rotary_dim > head_size || max_position == 0 || num_blocks == 0 ||
      block_size == 0 || query_token_stride == 0 || query_head_stride == 0 ||
      key_token_stride == 0 || key_head_stride == 0 || value_token_stride == 0 ||
      value_head_stride == 0 || key_cache_block_stride == 0 ||
      key_cache_page_stride == 0 || key_cache_head_stride == 0 ||
      value_cache_block_stride == 0 || value_cache_page_stride == 0 ||
      value_cache_head_stride == 0 || is_neox > 1u || scale_stride > 1u ||
      tokens > (uint32_t)std::numeric_limits<int>::max()) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  RopeParams p{};
  p.query = query;
  p.key = key;
  p.value = value;
  p.positions = positions;
  p.cos_sin = cos_sin_cache;
  p.key_cache = key_cache;
  p.value_cache = value_cache;
  p.key_scales = key_scales;
  p.value_scales = value_scales;
  p.slot_mapping = slot_mapping;
  p.tokens = tokens;
  p.cache_tokens = cache_tokens;
  p.query_heads = query_heads;
  p.kv_heads = kv_heads;
  p.head_size = head_size;
  p.value_head_size = value_head_size;
  p.rotary_dim = rotary_dim;
  p.max_position = max_position;
  p.num_blocks = num_blocks;
  p.block_size = block_size;
  p.scale_stride = scale_stride;
  p.is_neox = is_neox;
  p.q_token = query_token_stride;
  p.q_head = query_head_stride;
  p.k_token = key_token_stride;
  p.k_head = key_head_stride;
  p.v_token = value_token_stride;
  p.v_head = value_head_stride;
  p.kc_block = key_cache_block_stride;
  p.kc_page = key_cache_page_stride;
  p.kc_head = key_cache_head_stride;
  p.vc_block = value_cache_block_stride;
  p.vc_page = value_cache_page_stride;
  p.vc_head = value_cache_head_stride;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  return fp8 ? launch_typed<T, true>(p, cuda_stream)
             : launch_typed<T, false>(p, cuda_stream);
}

}  // namespace

#define LOOM_DEFINE_ROPE_WRITE(suffix, scalar, device_type)                          \
  extern "C" int loom_cuda_rope_paged_kv_write_##suffix(                             \
      scalar* query, scalar* key, const scalar* value, const int64_t* positions,    \
      const scalar* cos_sin_cache, void* key_cache, void* value_cache,              \
      const float* key_scales, const float* value_scales,                           \
      const int64_t* slot_mapping, uint32_t tokens, uint32_t cache_tokens,          \
      uint32_t query_heads, uint32_t kv_heads, uint32_t head_size,                  \
      uint32_t value_head_size, uint32_t rotary_dim, uint32_t max_position,         \
      uint32_t num_blocks, uint32_t block_size, uint32_t cache_encoding,            \
      uint32_t scale_stride, uint64_t query_token_stride,                           \
      uint64_t query_head_stride, uint64_t key_token_stride,                        \
      uint64_t key_head_stride, uint64_t value_token_stride,                        \
      uint64_t value_head_stride, uint64_t key_cache_block_stride,                  \
      uint64_t key_cache_page_stride, uint64_t key_cache_head_stride,               \
      uint64_t value_cache_block_stride, uint64_t value_cache_page_stride,          \
      uint64_t value_cache_head_stride, uint32_t is_neox, void* stream) {           \
    return launch_rope_paged_kv_write<device_type>(                                 \
        query, key, value, positions, cos_sin_cache, key_cache, value_cache,        \
        key_scales, value_scales, slot_mapping, tokens, cache_tokens, query_heads,  \
        kv_heads, head_size, value_head_size, rotary_dim, max_position, num_blocks, \
        block_size, cache_encoding, scale_stride, query_token_stride,               \
        query_head_stride, key_token_stride, key_head_stride, value_token_stride,   \
        value_head_stride, key_cache_block_stride, key_cache_page_stride,           \
        key_cache_head_stride, value_cache_block_stride, value_cache_page_stride,   \
        value_cache_head_stride, is_neox, stream);                                  \
  }

LOOM_DEFINE_ROPE_WRITE(f32, float, float)
LOOM_DEFINE_ROPE_WRITE(f16, uint16_t, __half)
LOOM_DEFINE_ROPE_WRITE(bf16, uint16_t, __nv_bfloat16)
