// Balanced persistent paged decode over an FP8 E4M3 cache on the fifth
// generation tensor cores (tcgen05.mma with the accumulators in tensor memory).
//
// Why a second compute path for FP8. With mma.sync the E4M3 bytes must be
// turned into F16 in registers first (ldmatrix, byte permute, conversion): 445
// warp instructions per 4 KB of cache, and the instruction stream, not HBM,
// bounds the kernel. tcgen05.mma of kind f8f6f4 reads E4M3 operands straight
// from the shared-memory tiles that TMA wrote, so the K and V bytes are never
// touched by a thread at all; what is left per token is the softmax.
//
// Shape of the computation, per 128-token tile of one (sequence, KV head):
//     S[128 tokens x 16] = K[128 x 128] . Qs^T          (4 MMAs, M=128 N=16 K=32)
//     O[128 dims   x 16] += V^T[128 x 128 tokens] . Ps^T (4 MMAs, A is MN-major)
// K is the K-major A operand exactly as TMA's 128-byte swizzle lays it out;
// the same kind of V tile is the MN-major A operand of the second product
// (value dims on M). The B operands must be E4M3 as well, so the 16-bit query
// and the probabilities are each split into two E4M3 planes, x = hi + lo with
// hi = e4m3(x), lo = e4m3(x - hi): columns 0-7 of S and O hold the hi plane of
// the 8 query heads, columns 8-15 the lo plane, and the two are added when the
// accumulators are read. Two planes carry 7-8 significant bits, what the BF16
// operands of the other path carry; Q is pre-scaled per head by a power of two
// so that its largest element sits near 2^8, P by 2^4 (with the reference
// allowed to lag by 2^4: p * 2^4 <= 2^8; a lag of 2^2 raised the reference, and
// rescaled O in tensor memory, on 16 % of the tiles and cost 3 %).
//
// One thread per token row: thread r reads row r of S from tensor memory
// (tcgen05.ld, lane = row), applies scale and mask, exponentiates against the
// per-head reference exponent (see chunk_softmax in decode_mma.cuh; here the
// reference is shared by the CTA and a CTA-wide vote decides when it moves),
// and writes its 16 probability bytes into the P tile. O stays in tensor memory
// for the whole work item; thread d reads row d (a value dim) at the end.
//
// Pipeline per CTA (eight warps, two CTAs per SM):
//   warps 0-3  softmax, one thread per token row;
//   warp 4     issues the QK products (and owns the tensor memory allocation);
//   warp 7     issues the PV products;
//   warps 5, 6 feed the K ring and the V ring with TMA, eight lanes at a time.
// The roles talk through mbarriers only: K / V slot landed and released, scores
// ready, P published, PV done, Q published. Scores and P have two buffers each,
// so QK of tile i + 1 runs while the softmax of tile i is busy, and PV of tile i
// runs while the softmax threads are already on tile i + 1. Barriers that are
// completed once per tile exist once per parity of the tile index: a parity
// wait cannot tell phase n from phase n - 2, and a role that lags by design
// (the softmax threads behind PV, the QK warp behind P) would otherwise hang.
//
// What measurement taught (timestamps per role and tile; 128 sequences of
// 2k-16k tokens, 8 KV heads): a thread needs about 200 ns per
// cp.async.bulk.tensor it issues and 60-90 ns per tcgen05.mma or commit, so a
// single issuing thread for the 16 copies or the 8 MMAs of a tile is the
// bottleneck (hence eight lanes and two warps); the tensor pipe itself is 3 %
// busy, and leaving out the MMAs does not change the time. What bounds the
// kernel now is the softmax threads' own chain per tile, about 1.4 us (tensor
// memory read, vote barrier, 8 exponentials, 16 byte stores, proxy fence),
// which two CTAs per SM only half hide - yet a third CTA per SM (two-slot rings,
// 80 registers) changed nothing (485 against 478 us), nor did two-slot rings at
// two CTAs per SM, so the limit is shared by the SM or lies in the memory
// system: with an HND cache (the 16 rows of a box contiguous, 2 KB) the same
// kernel takes 434 us against 479 us for NHD (128-byte rows 1 KB apart), where
// the mma.sync kernel takes 446 against 457 us. A switch of work item cost about 5 us
// (state out, Q in, first scores) and made CTAs that cover short sequences the
// last to finish; the next item's Q is therefore published before the current
// item is stored. 450-470 us on that workload against 456 us for the mma.sync
// kernel, so this kernel is opt-in (loom_cuda_set_decode_copy_engine(3)) until
// the chain is shorter.
//
// Every wait is bounded (see mbarrier_wait_prompt); after the first expiry the
// CTA stops waiting and runs to its end, and the first expired wait is
// recorded (loom_cuda_decode_timeout_flag). Tensor memory is freed on every
// path out of the kernel.
#pragma once

#include <cuda_fp8.h>

#include "decode_stream_tma.cuh"

namespace loom_decode {

constexpr uint32_t kUmmaTileTokens = 128;
constexpr int kUmmaSoftmaxThreads = 128;     // warps 0-3: one thread per token row / value dim
constexpr int kUmmaThreads = 256;            // + warp 4: QK issue, 5: K loads, 6: V loads, 7: PV issue
constexpr int kUmmaStages = 3;               // K+V tile pairs resident per CTA
constexpr uint32_t kUmmaTileBytes = 16384;   // 128 tokens x 128 bytes
// Tensor memory columns per CTA: S buffer b in columns 16 b .. 16 b + 15, O in 32-47.
// (Giving each of a product's four MMAs columns of its own, so that they do not
// accumulate one after the other, was measured and changed nothing.)
constexpr uint32_t kUmmaTmemColumns = 64;
constexpr float kUmmaSlack = 4.0f;           // p <= 2^4 before the reference moves
constexpr float kUmmaProbabilityScale = 16.0f;
constexpr int kUmmaCtasPerSm = 2;

struct UmmaSmem {
  static constexpr uint32_t kStages = 0;                                    // kUmmaStages x (K, V)
  static constexpr uint32_t kQuery = kUmmaStages * 2 * kUmmaTileBytes;      // 16 rows x 128 B
  static constexpr uint32_t kProbabilities = kQuery + 2048;                 // two buffers of 16 rows x 128 B
  static constexpr uint32_t kPrefix = kProbabilities + 4096;                // [sequences + 1]
  static constexpr uint32_t kBarriers = kPrefix + ((kTmaMaxSequences + 1) * 4 + 7) / 8 * 8;
  static constexpr uint32_t kTmemSlot = kBarriers + (4 * kUmmaStages + 7) * 8;  // K full/empty, V full/empty, scores[2], P[2], output[2], Q
  static constexpr uint32_t kHeadScale = kTmemSlot + 8;                     // [2 item parities][8]
  static constexpr uint32_t kReduce = kHeadScale + 64;                      // [4 warps][8]
  static constexpr uint32_t kWarpTotals = kReduce + 128;                    // [5]
  static constexpr uint32_t kVotes = kWarpTotals + 32;                      // [2][4]
  static constexpr uint32_t kAborted = kVotes + 32;                         // set when a wait expired
  static constexpr uint32_t kBytes = kAborted + 16;                         // the window itself is 1024-byte aligned
};

// ---- tcgen05 wrappers ---------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_slot), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void tmem_free(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

// D[tmem] (+)= A[smem desc] . B[smem desc]^T, E4M3 operands, F32 accumulate.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Makes `barrier` complete one arrival when every MMA issued so far by this
// thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t barrier) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(barrier)
               : "memory");
}

// 16 consecutive 32-bit columns of this thread's lane.
__device__ __forceinline__ void tmem_load16(float (&v)[16], uint32_t address) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_store16(uint32_t address, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(
          address),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// Shared-memory matrix descriptor of a tile whose rows are 128 bytes apart and
// which was written with the 128-byte swizzle (TMA's, or the same function by
// hand): 8-row groups 1024 bytes apart. Serves a K-major operand (rows = M or
// N index) and an MN-major operand (rows = K index) alike; the instruction
// descriptor says which it is.
__device__ __forceinline__ uint64_t umma_tile_descriptor(uint32_t smem_byte_address) {
  uint64_t descriptor = 0;
  descriptor |= (uint64_t)((smem_byte_address >> 4) & 0x3fffu);  // start address
  descriptor |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle)
  descriptor |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: next 8-row group
  descriptor |= (uint64_t)1 << 46;                               // descriptor version of this architecture
  descriptor |= (uint64_t)2 << 61;                               // 128-byte swizzle
  return descriptor;
}

// Instruction descriptor: E4M3 x E4M3 -> F32, M = 128, N = 16.
constexpr uint32_t kUmmaIdescBase = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kUmmaIdescScores = kUmmaIdescBase;               // A (keys) K-major
constexpr uint32_t kUmmaIdescValues = kUmmaIdescBase | (1u << 15);  // A (values) MN-major

// Two floats -> two E4M3 bytes (round to nearest even, saturating), low byte first.
__device__ __forceinline__ uint32_t e4m3_pair(float low, float high) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(low, high), __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float2 e4m3_pair_to_float(uint32_t pair) {
  const __half2_raw raw = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)pair, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&raw));
}

// x = hi + lo in E4M3 for two values: returns the hi pair and the lo pair.
__device__ __forceinline__ void e4m3_split_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
  hi = e4m3_pair(a, b);
  const float2 back = e4m3_pair_to_float(hi);
  lo = e4m3_pair(a - back.x, b - back.y);
}

// Byte offset of (row, byte column) inside a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t swizzled_byte(uint32_t row, uint32_t column) {
  return row * 128u + ((((column >> 4) ^ (row & 7u)) << 4) | (column & 15u));
}




// Bounded wait without a suspend hint: the handshakes between the control warp
// and the softmax warps sit on the critical path of every tile, and a sleeping
// waiter wakes up too late. Gives up after about a second of polling.
__device__ __forceinline__ bool mbarrier_wait_prompt(uint32_t barrier, uint32_t parity, uint32_t limit) {
  for (uint32_t attempt = 0; attempt < limit; ++attempt) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(barrier), "r"(parity)
        : "memory");
    if (done) return true;
  }
  atomicOr(&g_decode_timeout_flag, 1u);
  return false;
}

// Non-blocking test: has the phase with this parity completed?
__device__ __forceinline__ bool mbarrier_test(uint32_t barrier, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(barrier), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ void mbarrier_arrive(uint32_t barrier) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(barrier) : "memory");
}

// Barrier among the 128 softmax threads that also ORs a flag over them.
__device__ __forceinline__ bool softmax_threads_any(bool flag) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred pin, pout;\n"
      "setp.ne.u32 pin, %1, 0;\n"
      "bar.red.or.pred pout, 1, %2, pin;\n"
      "selp.u32 %0, 1, 0, pout;\n"
      "}\n"
      : "=r"(out)
      : "r"((uint32_t)flag), "n"(kUmmaSoftmaxThreads)
      : "memory");
  return out != 0;
}

// 16 columns of this thread's lane, without waiting for the data.
__device__ __forceinline__ void tmem_load16_start(uint32_t (&r)[16], uint32_t address) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// x = hi + lo in E4M3 for a pair of F16 values: returns the two hi bytes and the two lo bytes.
__device__ __forceinline__ void e4m3_split_half2(__half2 value, uint32_t& hi, uint32_t& lo) {
  const __half2_raw raw = *reinterpret_cast<const __half2_raw*>(&value);
  hi = (uint32_t)__nv_cvt_halfraw2_to_fp8x2(raw, __NV_SATFINITE, __NV_E4M3);
  const __half2_raw back = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)hi, __NV_E4M3);
  const __half2 rest = __hsub2(value, *reinterpret_cast<const __half2*>(&back));
  lo = (uint32_t)__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&rest), __NV_SATFINITE, __NV_E4M3);
}

// Barrier among the 128 softmax threads only (the control warp never joins it).
__device__ __forceinline__ void softmax_threads_sync() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(kUmmaSoftmaxThreads) : "memory");
}

template <typename QT>
__global__ void __launch_bounds__(kUmmaThreads, kUmmaCtasPerSm)
decode_umma_fp8_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap key_map,
                       const __grid_constant__ CUtensorMap value_map, const TmaAxes axes) {
  constexpr uint32_t kD = 128;
  constexpr uint32_t kHeads = 8;
  constexpr uint32_t kValueRing = kUmmaStages * kUmmaTileBytes;  // byte offset of the V ring

  // Three CTAs of 76 KB share an SM only without alignment slack: the window must
  // start on a 1024-byte boundary (the swizzle period) by itself.
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* smem = raw_smem;
  const uint32_t smem_base = smem_address(smem);
  if (smem_base & 1023u) {
    if (threadIdx.x == 0) {
      atomicOr(&g_decode_timeout_flag, 1u);
      atomicCAS(&g_decode_timeout_where, 0u, 31u << 20);
    }
    return;
  }
  const uint32_t query_tile = smem_base + UmmaSmem::kQuery;
  const uint32_t probability_tiles = smem_base + UmmaSmem::kProbabilities;  // tile i uses buffer i & 1
  uint32_t* prefix = reinterpret_cast<uint32_t*>(smem + UmmaSmem::kPrefix);
  // K and V tiles live in two rings of kUmmaStages slots each, fed by a warp
  // each. A K slot is released by the QK product that read it, a V slot by the
  // PV product: both loads then run about three tiles ahead of their use, where
  // a shared slot (released by PV only) left the K load a single tile of lead
  // and the latency of HBM on the critical path of every tile.
  const uint32_t full_barriers = smem_base + UmmaSmem::kBarriers;          // K slot s landed
  const uint32_t empty_barriers = full_barriers + kUmmaStages * 8;         // QK has read K slot s
  const uint32_t value_full_barriers = empty_barriers + kUmmaStages * 8;   // V slot s landed
  const uint32_t value_empty_barriers = value_full_barriers + kUmmaStages * 8;  // PV has read V slot s
  const uint32_t scores_barriers = value_empty_barriers + kUmmaStages * 8; // QK of an even / odd tile finished
  const uint32_t probabilities_barriers = scores_barriers + 16;            // 128 threads published P of an even / odd tile
  const uint32_t output_barriers = probabilities_barriers + 16;            // PV of an even / odd tile finished
  const uint32_t query_barrier = output_barriers + 16;                     // 128 threads published Q
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + UmmaSmem::kTmemSlot);
  volatile float* head_scale = reinterpret_cast<volatile float*>(smem + UmmaSmem::kHeadScale);
  volatile float* reduce = reinterpret_cast<volatile float*>(smem + UmmaSmem::kReduce);
  uint32_t* warp_totals = reinterpret_cast<uint32_t*>(smem + UmmaSmem::kWarpTotals);
  volatile uint32_t* aborted = reinterpret_cast<volatile uint32_t*>(smem + UmmaSmem::kAborted);

  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5;
  const uint32_t lane = tid & 31u;
  const bool control = warp == 4;                // issues the QK products; owns the tensor memory allocation
  const bool loader = warp == 5 || warp == 6;    // TMA loads: warp 5 feeds the K ring, warp 6 the V ring
  const bool value_issuer = warp == 7;           // issues the PV products

  if (tid == 0) {
    *aborted = 0;
#pragma unroll
    for (int i = 0; i < kUmmaStages; ++i) {
      mbarrier_init(full_barriers + i * 8, 1);
      mbarrier_init(empty_barriers + i * 8, 1);
      mbarrier_init(value_full_barriers + i * 8, 1);
      mbarrier_init(value_empty_barriers + i * 8, 1);
    }
    mbarrier_init(scores_barriers, 1);
    mbarrier_init(scores_barriers + 8, 1);
    mbarrier_init(probabilities_barriers, kUmmaSoftmaxThreads);
    mbarrier_init(probabilities_barriers + 8, kUmmaSoftmaxThreads);
    mbarrier_init(output_barriers, 1);
    mbarrier_init(output_barriers + 8, 1);
    mbarrier_init(query_barrier, kUmmaSoftmaxThreads);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  loom_launch::grid_dependency_wait();

  // ---- 128-token tiles per sequence, exclusive prefix sum ----------------------
  {
    const uint32_t per_thread = (p.sequences + kUmmaThreads - 1) / kUmmaThreads;
    const uint32_t begin = min(tid * per_thread, p.sequences);
    const uint32_t end = min(begin + per_thread, p.sequences);
    uint32_t local = 0;
    for (uint32_t s = begin; s < end; ++s) {
      const uint32_t length = clamp_length(__ldg(p.sequence_lengths + s), p.max_sequence_length);
      local += (length + kUmmaTileTokens - 1) / kUmmaTileTokens;
    }
    uint32_t inclusive = local;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if (lane >= (uint32_t)offset) inclusive += other;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    uint32_t running = inclusive - local;
    for (uint32_t w = 0; w < warp; ++w) running += warp_totals[w];
    for (uint32_t s = begin; s < end; ++s) {
      prefix[s] = running;
      const uint32_t length = clamp_length(__ldg(p.sequence_lengths + s), p.max_sequence_length);
      running += (length + kUmmaTileTokens - 1) / kUmmaTileTokens;
    }
    if (tid == kUmmaThreads - 1) prefix[p.sequences] = running;
    __syncthreads();
  }

  const uint32_t heads = p.kv_heads;  // work items per sequence (one item = one KV head, up to 8 query heads)
  const uint64_t total_tiles = (uint64_t)heads * prefix[p.sequences];
  const uint64_t ctas = gridDim.x;
  const uint64_t share = total_tiles / ctas;
  const uint64_t extra = total_tiles % ctas;
  const uint64_t range_begin = blockIdx.x * share + min((uint64_t)blockIdx.x, extra);
  const uint64_t range_end = range_begin + share + (blockIdx.x < extra ? 1u : 0u);
  if (range_begin >= range_end) return;  // nothing allocated yet
  auto cta_of = [&](uint64_t tile) -> uint32_t {
    const uint64_t boundary = extra * (share + 1);
    return tile < boundary ? (uint32_t)(tile / (share + 1)) : (uint32_t)(extra + (tile - boundary) / share);
  };
  const uint32_t my_tiles = (uint32_t)(range_end - range_begin);

  // ---- tensor memory (owned by the control warp) -----------------------------------
  if (control) tmem_alloc(smem_base + UmmaSmem::kTmemSlot, kUmmaTmemColumns);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_output = tmem_base + 32u;

  auto load_sequence = [&](StreamCursor& c) {
    c.tiles = prefix[c.seq + 1] - prefix[c.seq];
    c.length = clamp_length(__ldg(p.sequence_lengths + c.seq), p.max_sequence_length);
  };
  auto advance = [&](StreamCursor& c) {
    if (++c.tile < c.tiles) return;
    c.tile = 0;
    if (++c.head < heads) return;
    c.head = 0;
    do {
      ++c.seq;
    } while (c.seq < p.sequences && prefix[c.seq + 1] == prefix[c.seq]);
    if (c.seq < p.sequences) load_sequence(c);
  };

  StreamCursor start;
  {
    uint32_t low = 0, high = p.sequences;
    while (high - low > 1) {
      const uint32_t middle = (low + high) >> 1;
      if ((uint64_t)heads * prefix[middle] <= range_begin) low = middle;
      else high = middle;
    }
    start.seq = low;
    load_sequence(start);
    const uint64_t inside = range_begin - (uint64_t)heads * prefix[low];
    start.head = (uint32_t)(inside / start.tiles);
    start.tile = (uint32_t)(inside % start.tiles);
  }

  // After one wait has expired (the device-wide flag is set by mbarrier_wait) the
  // CTA stops waiting altogether and runs to its end on whatever it has.
  auto wait_phase = [&](uint32_t barrier, uint32_t completions) {
    // most waits find their phase complete already
    if (mbarrier_test(barrier, completions & 1u)) return;
    if (*aborted) return;
    if (!mbarrier_wait_prompt(barrier, completions & 1u, p.wait_attempts)) {
      *aborted = 1;
      const uint32_t kind = (barrier - full_barriers) >> 3;  // index into the barrier block
      atomicCAS(&g_decode_timeout_where, 0u, ((kind + 1u) << 20) | ((completions & 0x7ffffu) << 1));
    }
  };

  if (loader) {
    // ======================= load warps: each keeps one ring full =========================
    // A single thread needs about 200 ns per cp.async.bulk.tensor it issues (measured:
    // eight boxes per tile cost the loader 1.6 us, which was the kernel's whole tile
    // period). So the eight boxes of a tile are issued by eight lanes at once, each
    // with its own block id.
    {
      const bool value = warp == 6;
      const bool head_inner = axes.head < axes.page;
      const uint32_t full = value ? value_full_barriers : full_barriers;
      const uint32_t empty = value ? value_empty_barriers : empty_barriers;
      const uint32_t ring = smem_base + (value ? kValueRing : 0u);
      const CUtensorMap* map = value ? &value_map : &key_map;
      StreamCursor producer = start;
      uint32_t described = 0;
      struct TileLoad {
        uint32_t boxes;
        int32_t head, page, block;  // page and block of this lane's box
      };
      // Starts the load of this lane's block id of the next tile of the range.
      auto describe = [&](TileLoad& load) {
        const uint32_t token0 = producer.tile * kUmmaTileTokens;
        const uint32_t live = min(kUmmaTileTokens, producer.length - token0);
        load.boxes = (live + 15u) >> 4;
        load.head = (int32_t)producer.head;
        const uint32_t token = token0 + (lane & 7u) * 16u;
        const uint32_t logical = p.block_shift < 32u ? token >> p.block_shift : token / p.block_size;
        load.page = (int32_t)(token - logical * p.block_size);
        load.block = (lane & 7u) < load.boxes
                         ? __ldg(p.block_tables + (uint64_t)producer.seq * p.max_blocks_per_sequence + logical)
                         : 0;
        ++described;
        if (described < my_tiles) advance(producer);
      };
      // The block ids of tile t + 1 are in flight while tile t is copied.
      TileLoad current, next;
      describe(current);
      next = current;
      for (uint32_t tile = 0; tile < my_tiles; ++tile) {
        if (*aborted) break;  // after an expired wait no further copy is started
        if (tile + 1 < my_tiles) describe(next);
        const uint32_t slot = tile % kUmmaStages;
        // the slot's previous tile has been read by its product
        if (tile >= (uint32_t)kUmmaStages) wait_phase(empty + slot * 8, tile / kUmmaStages - 1);
        if (lane == 0) mbarrier_expect_tx(full + slot * 8, current.boxes * 2048u + p.wait_unmatched_bytes);
        __syncwarp();
        if (lane < current.boxes) {
          const int32_t block = (int32_t)clamp_block(current.block, p.num_blocks);
          const int32_t c1 = head_inner ? current.head : current.page;
          const int32_t c2 = head_inner ? current.page : current.head;
          tma_load_4d(ring + slot * kUmmaTileBytes + lane * 2048u, map, full + slot * 8, 0, c1, c2, block);
        }
        current = next;
      }
    }
  } else if (control) {
    // ======================= QK warp: one lane issues the score products ================
    // (A thread needs 60-90 ns per tcgen05.mma or commit it issues; with one thread
    // for all eight MMAs of a tile that was the tile period. QK and PV products are
    // independent of each other, so each kind has a thread of its own.)
    if (lane == 0) {
      StreamCursor cursor = start;
      uint32_t items_begun = 0;
      for (uint32_t tile = 0; tile < my_tiles; ++tile) {
        // a new item's scores need its Q; S buffer (tile & 1) was read by the softmax of tile - 2
        if (tile == 0 || cursor.tile == 0) wait_phase(query_barrier, items_begun++);
        if (tile >= 2) wait_phase(probabilities_barriers + (tile & 1u) * 8, (tile >> 1) - 1);
        const uint32_t stage = tile % kUmmaStages;
        wait_phase(full_barriers + stage * 8, tile / kUmmaStages);
        tcgen05_fence_after_sync();
        const uint64_t key_desc = umma_tile_descriptor(smem_base + stage * kUmmaTileBytes);
        const uint64_t query_desc = umma_tile_descriptor(query_tile);
        const uint32_t target = tmem_base + (tile & 1u) * 16u;
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) umma_f8(target, key_desc + 2u * k, query_desc + 2u * k, kUmmaIdescScores, k);
        umma_commit(scores_barriers + (tile & 1u) * 8);
        umma_commit(empty_barriers + stage * 8);  // the K slot may be refilled
        if (tile + 1 < my_tiles) advance(cursor);
      }
    }
  } else if (value_issuer) {
    // ======================= PV warp: one lane issues the output products ===============
    if (lane == 0) {
      StreamCursor cursor = start;
      for (uint32_t i = 0; i < my_tiles; ++i) {
        const bool first_of_item = i == 0 || cursor.tile == 0;
        // O += V^T . P^T once the 128 threads have published P
        wait_phase(probabilities_barriers + (i & 1u) * 8, i >> 1);
        const uint32_t stage = i % kUmmaStages;
        wait_phase(value_full_barriers + stage * 8, i / kUmmaStages);
        tcgen05_fence_after_sync();
        const uint64_t value_desc = umma_tile_descriptor(smem_base + kValueRing + stage * kUmmaTileBytes);
        const uint64_t probability_desc = umma_tile_descriptor(probability_tiles + (i & 1u) * 2048u);
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) {
          // 32 tokens per MMA: 32 rows of V (4096 bytes) and 32 bytes of each P row
          umma_f8(tmem_output, value_desc + 256u * k, probability_desc + 2u * k, kUmmaIdescValues,
                  (first_of_item && k == 0) ? 0u : 1u);
        }
        umma_commit(output_barriers + (i & 1u) * 8);
        umma_commit(value_empty_barriers + stage * 8);  // the V slot may be refilled
        if (i + 1 < my_tiles) advance(cursor);
      }
    }
  } else {
    // ======================= softmax warps =============================================
    const uint32_t lane_offset = (warp * 32u) << 16;  // this warp's quarter of the 128 lanes
    StreamCursor consumer = start;
    float reference[kHeads];  // exponent reference per head (base-2 units), the same in every thread
    float row_sum[kHeads];    // this thread's share of sum_i p_i
    uint32_t item_first_tile = 0;

    // Writes the two E4M3 planes of the item's queries and the per-head score scales.
    // Publishes an item's queries (two E4M3 planes) and per-head score scales, and
    // starts the load of its V scale. May run while the previous item is still
    // being finished: the Q tile is free once the previous item's last scores
    // have been read, and the scales of the two items use different slots.
    float value_scale_next = 1.0f;
    auto publish_query = [&](const StreamCursor& item_cursor, uint32_t parity) {
      const uint32_t kv_head = item_cursor.head;
      const uint32_t live_heads = min(kHeads, p.group);
      const uint32_t head = tid >> 4, piece = tid & 15u;  // 16 threads per head, 8 dims each
      float q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = 0.0f;
      if (head < live_heads) {
        const QT* row = static_cast<const QT*>(p.query) + (uint64_t)item_cursor.seq * p.q_token +
                        ((uint64_t)kv_head * p.group + head) * p.q_head + piece * 8u;
        const uint4 packed = *reinterpret_cast<const uint4*>(row);
        const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 pair = widen_pair<QT>(words[j]);
          q[2 * j] = pair.x;
          q[2 * j + 1] = pair.y;
        }
      }
      float largest = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) largest = fmaxf(largest, fabsf(q[j]));
#pragma unroll
      for (int offset = 1; offset < 16; offset <<= 1) {
        largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, offset));
      }
      // power of two that brings the largest element into [128, 256)
      int exponent = 0;
      float prescale = 1.0f;
      if (largest > 0.0f && largest < INFINITY) {
        frexpf(largest, &exponent);
        prescale = ldexpf(1.0f, 8 - exponent);
      }
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) e4m3_split_pair(q[2 * j] * prescale, q[2 * j + 1] * prescale, hi[j], lo[j]);
      const uint32_t hi_low = hi[0] | (hi[1] << 16), hi_high = hi[2] | (hi[3] << 16);
      const uint32_t lo_low = lo[0] | (lo[1] << 16), lo_high = lo[2] | (lo[3] << 16);
      asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(query_tile + swizzled_byte(head, piece * 8u)),
                   "r"(hi_low), "r"(hi_high)
                   : "memory");
      asm volatile("st.shared.v2.u32 [%0], {%1, %2};\n" ::"r"(query_tile + swizzled_byte(8u + head, piece * 8u)),
                   "r"(lo_low), "r"(lo_high)
                   : "memory");
      if (piece == 0) {
        const float key_scale = __ldg(p.key_scales + (uint64_t)kv_head * p.scale_stride);
        head_scale[parity * kHeads + head] = p.scale_log2 * key_scale / prescale;
      }
      value_scale_next = __ldg(p.value_scales + (uint64_t)kv_head * p.scale_stride);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      mbarrier_arrive(query_barrier);  // the QK warp may issue the item's first scores
    };
    float value_scale_now = 1.0f;
    uint32_t item_parity = 0;
    auto reset_item_state = [&]() {
#pragma unroll
      for (int h = 0; h < (int)kHeads; ++h) {
        reference[h] = -INFINITY;
        row_sum[h] = 0.0f;
      }
      value_scale_now = value_scale_next;
    };

    // Stores the item's result: final rows if this CTA covered the whole item,
    // else a partial state. The item's last PV product has completed.
    auto finish_item = [&](uint32_t item_seq, uint32_t item_head, uint32_t item_tiles) {
      tcgen05_fence_after_sync();
      float o[16];
      tmem_load16(o, tmem_output + lane_offset);
      tcgen05_fence_before_sync();
#pragma unroll
      for (int h = 0; h < (int)kHeads; ++h) {
        float total = row_sum[h];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
        if (lane == 0) reduce[warp * kHeads + h] = total;
      }
      softmax_threads_sync();
      const uint32_t kv_head = item_head;
      const uint32_t live_heads = min(kHeads, p.group);
      const uint64_t item = (uint64_t)item_seq * heads + item_head;
      const uint64_t item_begin = (uint64_t)heads * prefix[item_seq] + (uint64_t)item_head * item_tiles;
      const uint32_t first_cta = cta_of(item_begin);
      const uint32_t last_cta = cta_of(item_begin + item_tiles - 1);
      const uint32_t parts = last_cta - first_cta + 1;
      const float value_scale = value_scale_now * (1.0f / kUmmaProbabilityScale);
      const uint32_t stride = state_stride(kD);
      const uint64_t query_row = (uint64_t)item_seq * p.query_heads + (uint64_t)kv_head * p.group;
      const uint32_t dv = tid;
#pragma unroll
      for (int h = 0; h < (int)kHeads; ++h) {
        if ((uint32_t)h >= live_heads) break;
        const float total = reduce[h] + reduce[kHeads + h] + reduce[2 * kHeads + h] + reduce[3 * kHeads + h];
        const float acc = (o[h] + o[8 + h]) * value_scale;
        if (parts == 1 && !p.emit_state) {
          const float result = total > 0.0f ? acc / total : 0.0f;
          QT* out = static_cast<QT*>(p.output) + (query_row + h) * kD;
          if constexpr (std::is_same<QT, __nv_bfloat16>::value) out[dv] = __float2bfloat16_rn(result);
          else out[dv] = __float2half_rn(result);
        } else {
          float* row = parts == 1 ? static_cast<float*>(p.output) + (query_row + h) * stride
                                  : p.partials + ((item + blockIdx.x) * kHeads + h) * stride;
          row[dv] = acc;
          if (dv == 0) {
            row[kD] = reference[h] * kLn2;
            row[kD + 1] = total;
          }
        }
      }
      if (tid == 0 && blockIdx.x == first_cta) {
        p.item_meta[2 * item] = first_cta;
        p.item_meta[2 * item + 1] = parts;
      }
      softmax_threads_sync();  // `reduce` is reused
    };

    publish_query(consumer, item_parity);
    reset_item_state();
    softmax_threads_sync();  // the score scales are visible to the 128 threads
    // Completions of the PV products this thread has observed, per parity of the
    // tile index. A parity test cannot tell phase n from phase n - 2, so a waiter
    // must never fall two phases behind a barrier: with one barrier for the even
    // tiles and one for the odd ones, the next completion of either cannot happen
    // before this thread has published the P tile it belongs to.
    uint32_t seen_even = 0, seen_odd = 0;
    auto wait_output_of = [&](uint32_t tile) {  // the PV product of `tile` has landed
      const uint32_t wanted = (tile >> 1) + 1;
      if (tile & 1u) {
        while (seen_odd < wanted) wait_phase(output_barriers + 8, seen_odd++);
      } else {
        while (seen_even < wanted) wait_phase(output_barriers, seen_even++);
      }
    };
    auto wait_outputs_through = [&](uint32_t tile) {  // every PV product up to `tile` has landed
      if (tile >= 1) wait_output_of(tile - 1);
      wait_output_of(tile);
    };

    // byte offset of this token's column in row h of a P buffer (row 8 + h: + 1024)
    uint32_t p_offset[kHeads];
#pragma unroll
    for (int h = 0; h < (int)kHeads; ++h) p_offset[h] = swizzled_byte((uint32_t)h, tid);
    uint32_t raw_scores[16];
    bool scores_started = false;  // the tensor-memory read of this tile's scores is already under way

    for (uint32_t i = 0; i < my_tiles; ++i) {
      const uint32_t stage = i % kUmmaStages;
      const uint32_t token0 = consumer.tile * kUmmaTileTokens;
      const uint32_t live = min(kUmmaTileTokens, consumer.length - token0);
      const bool row_live = tid < live;
      const bool first_of_item = i == item_first_tile;
      const bool last_of_item = consumer.tile + 1 == consumer.tiles;
      const bool last_of_range = i + 1 == my_tiles;

      // ---- scores of this tile: row `tid` of S -------------------------------------
      if (!scores_started) {
        wait_phase(scores_barriers + (i & 1u) * 8, i >> 1);
        tcgen05_fence_after_sync();
        tmem_load16_start(raw_scores, tmem_base + (i & 1u) * 16u + lane_offset);
      }
      scores_started = false;
      tmem_load_wait();
      tcgen05_fence_before_sync();
      float s[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) s[c] = __uint_as_float(raw_scores[c]);
      float d[kHeads];
      bool over = false;
#pragma unroll
      for (int h = 0; h < (int)kHeads; ++h) {
        s[h] = (s[h] + s[8 + h]) * head_scale[item_parity * kHeads + h];  // base-2 score
        d[h] = row_live ? s[h] - reference[h] : -INFINITY;
        over |= d[h] > kUmmaSlack;
      }

      // ---- P has two buffers: the PV product of two tiles ago read this one ------------
      if (i >= 2) wait_output_of(i - 2);
      if (live < kUmmaTileTokens) {
        // rows past the end of the sequence hold whatever the page (or an older
        // tile) held: clear them in V so that 0 * garbage cannot become NaN
        wait_phase(value_full_barriers + stage * 8, i / kUmmaStages);
        if (!row_live) {
          const uint32_t row = smem_base + kValueRing + stage * kUmmaTileBytes + tid * 128u;
#pragma unroll
          for (int piece = 0; piece < 8; ++piece) {
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(row + piece * 16), "r"(0u) : "memory");
          }
        }
      }
      const bool any_over = softmax_threads_any(over);
      if (any_over) {
        // Rare: some score left the slack. Raise every head's reference to the
        // largest score of this tile and rescale what was accumulated (every PV
        // product issued so far must have landed in O first).
        if (i >= 1) wait_outputs_through(i - 1);
#pragma unroll
        for (int h = 0; h < (int)kHeads; ++h) {
          float top = row_live ? s[h] : -INFINITY;
#pragma unroll
          for (int offset = 16; offset > 0; offset >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
          if (lane == 0) reduce[warp * kHeads + h] = top;
        }
        softmax_threads_sync();
        float alpha[kHeads];
#pragma unroll
        for (int h = 0; h < (int)kHeads; ++h) {
          const float top =
              fmaxf(fmaxf(reduce[h], reduce[kHeads + h]), fmaxf(reduce[2 * kHeads + h], reduce[3 * kHeads + h]));
          const float raised = fmaxf(reference[h], top);
          alpha[h] = reference[h] == -INFINITY ? 0.0f : fast_exp2(reference[h] - raised);
          reference[h] = raised;
          row_sum[h] *= alpha[h];
          d[h] = row_live ? s[h] - raised : -INFINITY;
        }
        if (!first_of_item) {
          // O lives in tensor memory: thread = value dim
          float o[16];
          tcgen05_fence_after_sync();
          tmem_load16(o, tmem_output + lane_offset);
#pragma unroll
          for (int h = 0; h < (int)kHeads; ++h) {
            o[h] *= alpha[h];
            o[8 + h] *= alpha[h];
          }
          tmem_store16(tmem_output + lane_offset, o);
          tcgen05_fence_before_sync();
        }
        softmax_threads_sync();  // `reduce` is reused by the next slow path or item end
      }

      // ---- the next tile's scores are normally ready by now: start reading them, so
      // that the tensor-memory latency hides behind this tile's probabilities ------------
      if (!last_of_item && !last_of_range) {
        wait_phase(scores_barriers + ((i + 1) & 1u) * 8, (i + 1) >> 1);
        tcgen05_fence_after_sync();
        tmem_load16_start(raw_scores, tmem_base + ((i + 1) & 1u) * 16u + lane_offset);
        scores_started = true;
      }

      // ---- probabilities: 16 bytes of this token's column of the P tile ----------------
      {
        const uint32_t probability_tile = probability_tiles + (i & 1u) * 2048u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = fast_exp2(d[2 * j]), p1 = fast_exp2(d[2 * j + 1]);
          row_sum[2 * j] += p0;
          row_sum[2 * j + 1] += p1;
          uint32_t hi, lo;
          e4m3_split_half2(__floats2half2_rn(p0 * kUmmaProbabilityScale, p1 * kUmmaProbabilityScale), hi, lo);
          const uint32_t even = probability_tile + p_offset[2 * j], odd = probability_tile + p_offset[2 * j + 1];
          asm volatile("st.shared.u8 [%0], %1;\n" ::"r"(even), "r"(hi & 0xffu) : "memory");
          asm volatile("st.shared.u8 [%0], %1;\n" ::"r"(odd), "r"(hi >> 8) : "memory");
          asm volatile("st.shared.u8 [%0+1024], %1;\n" ::"r"(even), "r"(lo & 0xffu) : "memory");
          asm volatile("st.shared.u8 [%0+1024], %1;\n" ::"r"(odd), "r"(lo >> 8) : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      tcgen05_fence_before_sync();
      mbarrier_arrive(probabilities_barriers + (i & 1u) * 8);

      if (last_of_item || last_of_range) {
        // The next item's Q goes out first: its load, the QK warp's reaction and the
        // product itself then overlap the PV product and the store of this item.
        const StreamCursor finished = consumer;
        if (!last_of_range) {
          advance(consumer);
          publish_query(consumer, item_parity ^ 1u);
        }
        wait_outputs_through(i);
        finish_item(finished.seq, finished.head, finished.tiles);  // its barriers also publish the new scales
        if (!last_of_range) {
          item_first_tile = i + 1;
          item_parity ^= 1u;
          reset_item_state();
        }
      } else {
        advance(consumer);
      }
    }
  }

  // ---- release tensor memory -----------------------------------------------------------
  tcgen05_fence_before_sync();
  __syncthreads();
  if (*aborted) {
    // Copies started before the expiry may still be on their way into this CTA's shared memory,
    // and nobody waits for them any more: let them land before the CTA gives its memory back.
    for (int pause = 0; pause < 64; ++pause) __nanosleep(1000);
    __syncthreads();
  }
  if (control) tmem_free(tmem_base, kUmmaTmemColumns);
}

}  // namespace loom_decode
