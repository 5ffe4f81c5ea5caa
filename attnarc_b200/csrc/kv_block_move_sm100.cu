// KV block movement for a paged cache on sm_100a: move (copy, gather, scatter,
// compact), swap, and the block-table rewrite that follows a compaction.
//
// The reference lists these operators as the next ones around its paged cache
// (docs/operator-catalog.md:61 "KV block copy, swap, gather, scatter, compact,
// and remap"; roadmap item 3 at docs/operator-catalog.md:140) but ships no
// implementation or contract for them yet, so the entry points below are new,
// in the style of the launch header: plain pointers, sizes, a stream.
//
// A block is the unit the block tables name: the K bytes of one block are one
// contiguous span (block_size x kv_heads x dim elements in whatever order the
// layout puts them: NHD and HND alike), and so are its V bytes. Movement is
// therefore type- and layout-blind: spans of `block_bytes` bytes, found by a
// block id and a byte stride between blocks. The kernels are bound by HBM: every
// byte is read once and written once. Move and swap have two engines: by default
// 8 KB chunks go through shared memory on the bulk-copy engine (cp.async.bulk in
// and out, one issuing thread per CTA: the move at 0.97-1.0 of the device's copy
// bandwidth, the swap, in 4 KB chunks, at 0.98); the other engine walks 32 KB chunks with a
// grid sized to the SM count, each thread moving eight 16-byte vectors per chunk
// with all its loads issued before its stores (0.88-0.90).
//
// Block ids live on the device and are trusted engine state like block tables;
// the kernels only skip a pair that names a block outside its cache.

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "../../include/loom_launch.h"
#include "launch_util.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kVectorsPerThread = 8;
constexpr uint32_t kChunkBytes = kThreads * kVectorsPerThread * 16;  // 32 KB
constexpr int kCtasPerSm = 4;  // 64 registers per thread: eight vectors in flight and no spills

struct MoveParams {
  const uint8_t* source[2];  // K, V
  uint8_t* destination[2];
  uint64_t source_stride[2];  // bytes between blocks
  uint64_t destination_stride[2];
  const int64_t* pairs;  // [pair_count][2]: source block, destination block
  uint64_t block_bytes;
  uint32_t pair_count;
  uint32_t source_blocks;
  uint32_t destination_blocks;
  uint32_t chunks_per_block;
  uint32_t wait_attempts;         // polls after which a wait on a copy barrier gives up
  uint32_t wait_unmatched_bytes;  // self-test: barriers are armed for this many bytes too many
};

__device__ __forceinline__ uint4 load_streaming(const uint8_t* address) {
  return __ldcs(reinterpret_cast<const uint4*>(address));
}

__device__ __forceinline__ void store_streaming(uint8_t* address, uint4 value) {
  __stcs(reinterpret_cast<uint4*>(address), value);
}

// destination block <- source block, for every pair, K and V.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) kv_block_move_kernel(const MoveParams p) {
  loom_launch::grid_dependency_wait();
  const uint64_t units = (uint64_t)p.pair_count * 2u * p.chunks_per_block;
  for (uint64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    const uint32_t chunk = (uint32_t)(unit % p.chunks_per_block);
    const uint64_t rest = unit / p.chunks_per_block;
    const uint32_t which = (uint32_t)(rest & 1u);  // K and V of a pair are neighbours in the walk
    const uint64_t pair = rest >> 1;
    const int64_t from = __ldg(p.pairs + 2 * pair);
    const int64_t to = __ldg(p.pairs + 2 * pair + 1);
    if (from < 0 || from >= (int64_t)p.source_blocks || to < 0 || to >= (int64_t)p.destination_blocks) continue;
    // (selected, not indexed: indexing the parameter arrays by a run-time value copies them to local memory)
    const uint8_t* source = (which ? p.source[1] : p.source[0]) + (uint64_t)from * (which ? p.source_stride[1] : p.source_stride[0]);
    uint8_t* destination = (which ? p.destination[1] : p.destination[0]) +
                           (uint64_t)to * (which ? p.destination_stride[1] : p.destination_stride[0]);
    const uint64_t base = (uint64_t)chunk * kChunkBytes + threadIdx.x * 16u;
    uint4 held[kVectorsPerThread];
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const uint64_t offset = base + (uint64_t)j * (kThreads * 16u);
      if (offset < p.block_bytes) held[j] = load_streaming(source + offset);
    }
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const uint64_t offset = base + (uint64_t)j * (kThreads * 16u);
      if (offset < p.block_bytes) store_streaming(destination + offset, held[j]);
    }
  }
}

// ---- the same move staged through shared memory by the bulk-copy engine -------------------
//
// One thread per CTA drives a ring of kBulkStages slots of kBulkBytes: a
// cp.async.bulk load global -> shared per slot (completion counted in bytes on
// the slot's mbarrier), then a cp.async.bulk store shared -> global from the
// same slot; the slot is refilled once the store has finished READING it
// (cp.async.bulk.wait_group.read). No byte passes through a register, loads run
// kBulkStages - kBulkLag chunks ahead of the stores, and loads and stores of
// different chunks overlap freely. Every wait on a barrier is bounded; when one expires
// the thread records it, stops issuing, drains what it has issued and returns.

// Measured on 8192 and 16384 scattered 64 KB blocks of a 2 GB cache (bytes read plus
// written per second; a plain device copy of 1 GiB ran at 6.45-6.53 TB/s in the same runs):
//   8 KB x 8 slots x 3 CTAs/SM, lag 1..4   6.33-6.54 TB/s   <- chosen (lag 2)
//   16 KB x 4 x 3 (lag 1, 2), 32 KB x 3 x 2, 16 KB x 3 x 4, 8 KB x 6 x 4    5.94-6.14 TB/s
//   8 KB x 12 x 2   5.34-5.43;  4 KB x 16 x 3   4.54-4.59;  8 KB x 24 x 1   3.32-3.33
// (the last three are bound by the one issuing thread: about 150 ns per chunk).
#ifndef LOOM_BULK_BYTES
#define LOOM_BULK_BYTES 8192
#define LOOM_BULK_STAGES 8
#define LOOM_BULK_CTAS 3
#define LOOM_BULK_LAG 2
#endif
constexpr uint32_t kBulkBytes = LOOM_BULK_BYTES;
constexpr int kBulkStages = LOOM_BULK_STAGES;
constexpr int kBulkCtasPerSm = LOOM_BULK_CTAS;
constexpr int kBulkLag = LOOM_BULK_LAG;  // stores that may still be reading their slots when the next load is issued
constexpr uint32_t kBulkSharedBytes = kBulkStages * kBulkBytes + kBulkStages * 8 + kBulkStages * 16;

__device__ uint32_t g_block_move_timeout = 0;

__device__ __forceinline__ uint32_t shared_address(const void* pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

constexpr uint32_t kDefaultBulkWaitAttempts = 1u << 22;

__device__ __forceinline__ bool bulk_wait(uint32_t barrier, uint32_t parity, uint32_t limit) {
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
  atomicOr(&g_block_move_timeout, 1u);
  return false;
}

__global__ void __launch_bounds__(32, kBulkCtasPerSm) kv_block_move_bulk_kernel(const MoveParams p) {
  extern __shared__ __align__(128) uint8_t ring[];
  uint64_t* barriers = reinterpret_cast<uint64_t*>(ring + kBulkStages * kBulkBytes);
  // per slot: destination address and byte count of the chunk it holds (0 = nothing to store)
  uint64_t* targets = reinterpret_cast<uint64_t*>(ring + kBulkStages * kBulkBytes + kBulkStages * 8);
  if (threadIdx.x != 0) return;
  for (int slot = 0; slot < kBulkStages; ++slot) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(shared_address(barriers + slot)) : "memory");
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  loom_launch::grid_dependency_wait();

  const uint64_t units = (uint64_t)p.pair_count * 2u * p.chunks_per_block;
  if (blockIdx.x >= units) return;
  const uint64_t mine = (units - blockIdx.x + gridDim.x - 1) / gridDim.x;  // units blockIdx.x + k * gridDim.x
  uint32_t phases = 0;   // bit s: parity of the next completion of slot s
  uint32_t pending = 0;  // bit s: a load into slot s has been issued and not yet waited for

  // Starts the load of this CTA's k-th chunk into slot k % kBulkStages.
  auto issue_load = [&](uint64_t k) {
    const uint32_t slot = (uint32_t)(k % kBulkStages);
    const uint64_t unit = blockIdx.x + k * gridDim.x;
    const uint32_t chunk = (uint32_t)(unit % p.chunks_per_block);
    const uint64_t rest = unit / p.chunks_per_block;
    const uint32_t which = (uint32_t)(rest & 1u);
    const uint64_t pair = rest >> 1;
    const int64_t from = __ldg(p.pairs + 2 * pair);
    const int64_t to = __ldg(p.pairs + 2 * pair + 1);
    targets[2 * slot + 1] = 0;
    if (from < 0 || from >= (int64_t)p.source_blocks || to < 0 || to >= (int64_t)p.destination_blocks) return;
    const uint64_t offset = (uint64_t)chunk * kBulkBytes;
    const uint64_t left = p.block_bytes - offset;
    const uint32_t bytes = (uint32_t)(left < kBulkBytes ? left : kBulkBytes);
    const uint8_t* source = (which ? p.source[1] : p.source[0]) +
                            (uint64_t)from * (which ? p.source_stride[1] : p.source_stride[0]) + offset;
    uint8_t* destination = (which ? p.destination[1] : p.destination[0]) +
                           (uint64_t)to * (which ? p.destination_stride[1] : p.destination_stride[0]) + offset;
    targets[2 * slot] = reinterpret_cast<uint64_t>(destination);
    targets[2 * slot + 1] = bytes;
    pending |= 1u << slot;
    const uint32_t barrier = shared_address(barriers + slot);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(barrier),
                 "r"(bytes + p.wait_unmatched_bytes)
                 : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
            shared_address(ring + slot * kBulkBytes)),
        "l"(source), "r"(bytes), "r"(barrier)
        : "memory");
  };

  constexpr int kAhead = kBulkStages - kBulkLag;  // loads run this many chunks ahead of the stores
  const uint64_t ahead = mine < (uint64_t)kAhead ? mine : (uint64_t)kAhead;
  for (uint64_t k = 0; k < ahead; ++k) issue_load(k);
  for (uint64_t k = 0; k < mine; ++k) {
    const uint32_t slot = (uint32_t)(k % kBulkStages);
    const uint32_t bytes = (uint32_t)targets[2 * slot + 1];
    if (bytes != 0) {
      if (!bulk_wait(shared_address(barriers + slot), (phases >> slot) & 1u, p.wait_attempts)) break;
      phases ^= 1u << slot;
      pending &= ~(1u << slot);
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(targets[2 * slot]),
                   "r"(shared_address(ring + slot * kBulkBytes)), "r"(bytes)
                   : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    if (k + kAhead < mine) {
      // the slot to refill held chunk k - kBulkLag: every store but the kBulkLag latest has read its slot
      asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(kBulkLag) : "memory");
      issue_load(k + kAhead);
    }
  }
  // Only after an expired wait can loads still be on their way into this CTA's
  // shared memory: give each of them one more bounded wait before the CTA ends.
  for (uint32_t slot = 0; slot < (uint32_t)kBulkStages; ++slot) {
    if (pending & (1u << slot)) bulk_wait(shared_address(barriers + slot), (phases >> slot) & 1u, p.wait_attempts);
  }
  asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
}

struct SwapParams {
  uint8_t* cache[2];   // K, V
  uint64_t stride[2];  // bytes between blocks
  const int64_t* pairs;
  uint64_t block_bytes;
  uint32_t pair_count;
  uint32_t blocks;
  uint32_t chunks_per_block;
  uint32_t wait_attempts;
  uint32_t wait_unmatched_bytes;
};

// Exchanges the two blocks of every pair, K and V.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) kv_block_swap_kernel(const SwapParams p) {
  loom_launch::grid_dependency_wait();
  constexpr int kHalf = kVectorsPerThread / 2;  // two blocks are held at once
  const uint32_t chunks = p.chunks_per_block * 2u;  // chunks of 16 KB here
  const uint64_t units = (uint64_t)p.pair_count * 2u * chunks;
  for (uint64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    const uint32_t chunk = (uint32_t)(unit % chunks);
    const uint64_t rest = unit / chunks;
    const uint32_t which = (uint32_t)(rest & 1u);
    const uint64_t pair = rest >> 1;
    const int64_t left = __ldg(p.pairs + 2 * pair);
    const int64_t right = __ldg(p.pairs + 2 * pair + 1);
    if (left < 0 || left >= (int64_t)p.blocks || right < 0 || right >= (int64_t)p.blocks || left == right) continue;
    uint8_t* base_pointer = which ? p.cache[1] : p.cache[0];
    const uint64_t stride = which ? p.stride[1] : p.stride[0];
    uint8_t* first = base_pointer + (uint64_t)left * stride;
    uint8_t* second = base_pointer + (uint64_t)right * stride;
    const uint64_t base = (uint64_t)chunk * (kChunkBytes / 2) + threadIdx.x * 16u;
    uint4 a[kHalf], b[kHalf];
#pragma unroll
    for (int j = 0; j < kHalf; ++j) {
      const uint64_t offset = base + (uint64_t)j * (kThreads * 16u);
      if (offset < p.block_bytes) {
        a[j] = load_streaming(first + offset);
        b[j] = load_streaming(second + offset);
      }
    }
#pragma unroll
    for (int j = 0; j < kHalf; ++j) {
      const uint64_t offset = base + (uint64_t)j * (kThreads * 16u);
      if (offset < p.block_bytes) {
        store_streaming(first + offset, b[j]);
        store_streaming(second + offset, a[j]);
      }
    }
  }
}

// The swap on the bulk-copy engine: the ring's slots work in twins. Both blocks'
// chunks are loaded into a twin (one mbarrier counts the bytes of both loads),
// then stored crosswise, so neither store can overtake the load of what it
// overwrites. Refill rule, bounds on the waits and drain as in the move kernel.
// The swap's ring: 16 slots of 4 KB used as 8 twins. Measured (8192 / 16384 pairs of 64 KB blocks):
// 4 KB x 16 slots, twin lag 2: 6.48-6.50 TB/s; 8 KB x 8 slots, lag 1: 5.99-6.13, lag 2: 6.16-6.18;
// 8 KB x 12 slots x 2 CTAs/SM, lag 2: 6.18-6.24.
constexpr uint32_t kSwapBytes = 4096;
constexpr int kSwapStages = 16;
constexpr uint32_t kSwapSharedBytes = kSwapStages * kSwapBytes + kSwapStages * 8 + kSwapStages * 16;

__global__ void __launch_bounds__(32, kBulkCtasPerSm) kv_block_swap_bulk_kernel(const SwapParams p) {
  constexpr int kTwins = kSwapStages / 2;
  constexpr int kTwinLag = 2;                  // stores still reading when the next twin is loaded
  constexpr int kAhead = kTwins - kTwinLag;
  static_assert(kSwapStages % 2 == 0 && kAhead >= 1, "the swap needs at least two twins of slots");
  extern __shared__ __align__(128) uint8_t ring[];
  uint64_t* barriers = reinterpret_cast<uint64_t*>(ring + kSwapStages * kSwapBytes);  // one per twin
  // per twin: address of the first block's chunk, of the second block's chunk, byte count (0 = skip)
  uint64_t* targets = reinterpret_cast<uint64_t*>(ring + kSwapStages * kSwapBytes + kSwapStages * 8);
  if (threadIdx.x != 0) return;
  for (int twin = 0; twin < kTwins; ++twin) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(shared_address(barriers + twin)) : "memory");
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  loom_launch::grid_dependency_wait();

  const uint64_t units = (uint64_t)p.pair_count * 2u * p.chunks_per_block;
  if (blockIdx.x >= units) return;
  const uint64_t mine = (units - blockIdx.x + gridDim.x - 1) / gridDim.x;
  uint32_t phases = 0, pending = 0;

  auto issue_loads = [&](uint64_t k) {
    const uint32_t twin = (uint32_t)(k % kTwins);
    const uint64_t unit = blockIdx.x + k * gridDim.x;
    const uint32_t chunk = (uint32_t)(unit % p.chunks_per_block);
    const uint64_t rest = unit / p.chunks_per_block;
    const uint32_t which = (uint32_t)(rest & 1u);
    const uint64_t pair = rest >> 1;
    const int64_t left = __ldg(p.pairs + 2 * pair);
    const int64_t right = __ldg(p.pairs + 2 * pair + 1);
    targets[3 * twin + 2] = 0;
    if (left < 0 || left >= (int64_t)p.blocks || right < 0 || right >= (int64_t)p.blocks || left == right) return;
    const uint64_t offset = (uint64_t)chunk * kSwapBytes;
    const uint64_t remaining = p.block_bytes - offset;
    const uint32_t bytes = (uint32_t)(remaining < kSwapBytes ? remaining : kSwapBytes);
    uint8_t* base_pointer = which ? p.cache[1] : p.cache[0];
    const uint64_t stride = which ? p.stride[1] : p.stride[0];
    uint8_t* first = base_pointer + (uint64_t)left * stride + offset;
    uint8_t* second = base_pointer + (uint64_t)right * stride + offset;
    targets[3 * twin] = reinterpret_cast<uint64_t>(first);
    targets[3 * twin + 1] = reinterpret_cast<uint64_t>(second);
    targets[3 * twin + 2] = bytes;
    pending |= 1u << twin;
    const uint32_t barrier = shared_address(barriers + twin);
    const uint32_t slot = shared_address(ring + (2 * twin) * kSwapBytes);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(barrier), "r"(2u * bytes + p.wait_unmatched_bytes)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(slot),
                 "l"(first), "r"(bytes), "r"(barrier)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     slot + kSwapBytes),
                 "l"(second), "r"(bytes), "r"(barrier)
                 : "memory");
  };

  const uint64_t ahead = mine < (uint64_t)kAhead ? mine : (uint64_t)kAhead;
  for (uint64_t k = 0; k < ahead; ++k) issue_loads(k);
  for (uint64_t k = 0; k < mine; ++k) {
    const uint32_t twin = (uint32_t)(k % kTwins);
    const uint32_t bytes = (uint32_t)targets[3 * twin + 2];
    if (bytes != 0) {
      if (!bulk_wait(shared_address(barriers + twin), (phases >> twin) & 1u, p.wait_attempts)) break;
      phases ^= 1u << twin;
      pending &= ~(1u << twin);
      const uint32_t slot = shared_address(ring + (2 * twin) * kSwapBytes);
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(targets[3 * twin + 1]),
                   "r"(slot), "r"(bytes)
                   : "memory");  // the first block's bytes go to the second block
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(targets[3 * twin]),
                   "r"(slot + kSwapBytes), "r"(bytes)
                   : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    if (k + kAhead < mine) {
      asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(kTwinLag) : "memory");
      issue_loads(k + kAhead);
    }
  }
  for (uint32_t twin = 0; twin < (uint32_t)kTwins; ++twin) {
    if (pending & (1u << twin)) bulk_wait(shared_address(barriers + twin), (phases >> twin) & 1u, p.wait_attempts);
  }
  asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
}

// block_tables[i] <- new_ids[block_tables[i]] for ids inside the cache; other
// entries (negative sentinels of unused tail entries) stay as they are.
__global__ void __launch_bounds__(kThreads) block_table_remap_kernel(int32_t* tables, uint64_t entries,
                                                                     const int32_t* new_ids, uint32_t blocks) {
  loom_launch::grid_dependency_wait();
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < entries; i += (uint64_t)gridDim.x * kThreads) {
    const int32_t id = tables[i];
    if (id >= 0 && (uint32_t)id < blocks) tables[i] = __ldg(new_ids + id);
  }
}

// 0: bulk-copy engine through shared memory; 1: vector loads and stores through registers.
std::atomic<uint32_t> g_move_engine{0};

// Raises a bulk kernel's dynamic shared-memory limit once per device (bit d of `prepared`).
// Returns a LoomCudaStatus; a failure is recorded for loom_cuda_last_launch_failure().
template <typename Kernel>
int raise_shared_limit(Kernel kernel, uint32_t bytes, std::atomic<uint64_t>& prepared) {
  int device = 0;
  if (const cudaError_t status = cudaGetDevice(&device); status != cudaSuccess) {
    return loom_launch::failed(status, "current device query before a KV block movement launch");
  }
  if (device < 64 && (prepared.load(std::memory_order_acquire) & (1ull << device))) return LOOM_CUDA_SUCCESS;
  if (const cudaError_t status =
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
      status != cudaSuccess) {
    return loom_launch::failed(status, "shared-memory limit of a KV block movement kernel (cudaFuncSetAttribute)");
  }
  if (device < 64) prepared.fetch_or(1ull << device, std::memory_order_release);
  return LOOM_CUDA_SUCCESS;
}

// The address a kernel uses for `pointer`: itself for device or managed memory,
// the mapped device address for pinned host memory (`*host` set). False for
// memory the device cannot address (pageable host memory, unknown pointers).
bool device_view(const void* pointer, const uint8_t** view, bool* host) {
  cudaPointerAttributes attributes{};
  if (cudaPointerGetAttributes(&attributes, pointer) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (attributes.type == cudaMemoryTypeDevice || attributes.type == cudaMemoryTypeManaged) {
    *view = static_cast<const uint8_t*>(pointer);
    return true;
  }
  if (attributes.type == cudaMemoryTypeHost && attributes.devicePointer != nullptr) {
    *view = static_cast<const uint8_t*>(attributes.devicePointer);
    *host = true;
    return true;
  }
  return false;
}

int sm_count() {
  int device = 0, count = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  return count;
}

bool aligned16(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

int finish(cudaError_t launch_result) {
  return loom_launch::failed(launch_result, "KV block movement kernel launch");
}

uint32_t grid_for(uint64_t units, int sms) {
  const uint64_t resident = (uint64_t)sms * kCtasPerSm;
  return (uint32_t)(units < resident ? units : resident);
}

}  // namespace

extern "C" {

int loom_cuda_kv_block_move(const void* source_key_cache, const void* source_value_cache,
                            void* destination_key_cache, void* destination_value_cache,
                            const int64_t* block_pairs, uint32_t pair_count, uint32_t source_blocks,
                            uint32_t destination_blocks, uint64_t block_bytes, uint64_t source_key_block_stride,
                            uint64_t source_value_block_stride, uint64_t destination_key_block_stride,
                            uint64_t destination_value_block_stride, void* stream) {
  if (pair_count == 0) return LOOM_CUDA_SUCCESS;
  if (!source_key_cache || !source_value_cache || !destination_key_cache || !destination_value_cache ||
      !block_pairs || source_blocks == 0 || destination_blocks == 0 || block_bytes == 0) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const uint64_t strides[4] = {source_key_block_stride, source_value_block_stride, destination_key_block_stride,
                               destination_value_block_stride};
  for (uint64_t stride : strides) {
    if (stride < block_bytes) return LOOM_CUDA_INVALID_ARGUMENT;
    if (stride % 16u) return LOOM_CUDA_UNSUPPORTED;
  }
  if (block_bytes % 16u || !aligned16(source_key_cache) || !aligned16(source_value_cache) ||
      !aligned16(destination_key_cache) || !aligned16(destination_value_cache)) {
    return LOOM_CUDA_UNSUPPORTED;
  }
  const uint64_t chunks = (block_bytes + kChunkBytes - 1) / kChunkBytes;
  if (chunks > 0xffffffffull) return LOOM_CUDA_UNSUPPORTED;
  const int sms = sm_count();
  if (sms <= 0) return LOOM_CUDA_UNAVAILABLE;
  MoveParams p{};
  p.source[0] = static_cast<const uint8_t*>(source_key_cache);
  p.source[1] = static_cast<const uint8_t*>(source_value_cache);
  p.destination[0] = static_cast<uint8_t*>(destination_key_cache);
  p.destination[1] = static_cast<uint8_t*>(destination_value_cache);
  p.source_stride[0] = source_key_block_stride;
  p.source_stride[1] = source_value_block_stride;
  p.destination_stride[0] = destination_key_block_stride;
  p.destination_stride[1] = destination_value_block_stride;
  p.pairs = block_pairs;
  p.block_bytes = block_bytes;
  p.pair_count = pair_count;
  p.source_blocks = source_blocks;
  p.destination_blocks = destination_blocks;
  p.chunks_per_block = (uint32_t)chunks;
  p.wait_attempts = loom_launch::wait_attempts(kDefaultBulkWaitAttempts);
  p.wait_unmatched_bytes = loom_launch::wait_unmatched_bytes();
  // A cache in pinned host memory (blocks swapped out on preemption, swapped in on resume) is read
  // and written over PCIe by the vector engine; memory the device cannot address is refused.
  bool host = false;
  const uint8_t* destination_view[2] = {nullptr, nullptr};
  if (!device_view(source_key_cache, &p.source[0], &host) || !device_view(source_value_cache, &p.source[1], &host) ||
      !device_view(destination_key_cache, &destination_view[0], &host) ||
      !device_view(destination_value_cache, &destination_view[1], &host)) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  p.destination[0] = const_cast<uint8_t*>(destination_view[0]);
  p.destination[1] = const_cast<uint8_t*>(destination_view[1]);
  if (host || g_move_engine.load(std::memory_order_relaxed) == 1) {
    const uint64_t units = (uint64_t)pair_count * 2u * chunks;
    return finish(loom_launch::launch(kv_block_move_kernel, dim3(grid_for(units, sms)), dim3(kThreads), 0,
                                      static_cast<cudaStream_t>(stream), p));
  }
  const uint64_t bulk_chunks = (block_bytes + kBulkBytes - 1) / kBulkBytes;
  if (bulk_chunks > 0xffffffffull) return LOOM_CUDA_UNSUPPORTED;
  p.chunks_per_block = (uint32_t)bulk_chunks;
  static std::atomic<uint64_t> prepared{0};
  if (const int limit = raise_shared_limit(kv_block_move_bulk_kernel, kBulkSharedBytes, prepared); limit != LOOM_CUDA_SUCCESS) return limit;
  const uint64_t units = (uint64_t)pair_count * 2u * bulk_chunks;
  const uint64_t resident = (uint64_t)sms * kBulkCtasPerSm;
  return finish(loom_launch::launch(kv_block_move_bulk_kernel, dim3((uint32_t)(units < resident ? units : resident)),
                                    dim3(32), kBulkSharedBytes, static_cast<cudaStream_t>(stream), p));
}

int loom_cuda_set_kv_block_move_engine(uint32_t engine) {
  if (engine > 1) return LOOM_CUDA_INVALID_ARGUMENT;
  g_move_engine.store(engine, std::memory_order_relaxed);
  return LOOM_CUDA_SUCCESS;
}

int loom_cuda_kv_block_move_timeout_flag(uint32_t* value, uint32_t reset) {
  if (value == nullptr) return LOOM_CUDA_INVALID_ARGUMENT;
  uint32_t flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_block_move_timeout, sizeof(flag)) != cudaSuccess) {
    cudaGetLastError();
    return LOOM_CUDA_LAUNCH_ERROR;
  }
  *value = flag;
  if (reset && flag != 0) {
    const uint32_t zero = 0;
    if (cudaMemcpyToSymbol(g_block_move_timeout, &zero, sizeof(zero)) != cudaSuccess) {
      cudaGetLastError();
      return LOOM_CUDA_LAUNCH_ERROR;
    }
  }
  return LOOM_CUDA_SUCCESS;
}

int loom_cuda_kv_block_swap(void* key_cache, void* value_cache, const int64_t* block_pairs, uint32_t pair_count,
                            uint32_t num_blocks, uint64_t block_bytes, uint64_t key_block_stride,
                            uint64_t value_block_stride, void* stream) {
  if (pair_count == 0) return LOOM_CUDA_SUCCESS;
  if (!key_cache || !value_cache || !block_pairs || num_blocks == 0 || block_bytes == 0 ||
      key_block_stride < block_bytes || value_block_stride < block_bytes) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  if (block_bytes % 16u || key_block_stride % 16u || value_block_stride % 16u || !aligned16(key_cache) ||
      !aligned16(value_cache)) {
    return LOOM_CUDA_UNSUPPORTED;
  }
  const uint64_t chunks = (block_bytes + kChunkBytes - 1) / kChunkBytes;
  if (chunks > 0x7fffffffull) return LOOM_CUDA_UNSUPPORTED;
  const int sms = sm_count();
  if (sms <= 0) return LOOM_CUDA_UNAVAILABLE;
  SwapParams p{};
  p.cache[0] = static_cast<uint8_t*>(key_cache);
  p.cache[1] = static_cast<uint8_t*>(value_cache);
  p.stride[0] = key_block_stride;
  p.stride[1] = value_block_stride;
  p.pairs = block_pairs;
  p.block_bytes = block_bytes;
  p.pair_count = pair_count;
  p.blocks = num_blocks;
  p.chunks_per_block = (uint32_t)chunks;
  p.wait_attempts = loom_launch::wait_attempts(kDefaultBulkWaitAttempts);
  p.wait_unmatched_bytes = loom_launch::wait_unmatched_bytes();
  // As for a move: a cache in pinned host memory is exchanged over PCIe by the vector engine through
  // its mapped device address; memory the device cannot address is refused before any launch.
  bool host = false;
  const uint8_t* view[2] = {nullptr, nullptr};
  if (!device_view(key_cache, &view[0], &host) || !device_view(value_cache, &view[1], &host)) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  p.cache[0] = const_cast<uint8_t*>(view[0]);
  p.cache[1] = const_cast<uint8_t*>(view[1]);
  if (host || g_move_engine.load(std::memory_order_relaxed) == 1) {
    const uint64_t units = (uint64_t)pair_count * 2u * chunks * 2u;
    return finish(loom_launch::launch(kv_block_swap_kernel, dim3(grid_for(units, sms)), dim3(kThreads), 0,
                                      static_cast<cudaStream_t>(stream), p));
  }
  const uint64_t bulk_chunks = (block_bytes + kSwapBytes - 1) / kSwapBytes;
  if (bulk_chunks > 0xffffffffull) return LOOM_CUDA_UNSUPPORTED;
  p.chunks_per_block = (uint32_t)bulk_chunks;
  static std::atomic<uint64_t> prepared{0};
  if (const int limit = raise_shared_limit(kv_block_swap_bulk_kernel, kSwapSharedBytes, prepared); limit != LOOM_CUDA_SUCCESS) return limit;
  const uint64_t units = (uint64_t)pair_count * 2u * bulk_chunks;
  const uint64_t resident = (uint64_t)sms * kBulkCtasPerSm;
  return finish(loom_launch::launch(kv_block_swap_bulk_kernel, dim3((uint32_t)(units < resident ? units : resident)),
                                    dim3(32), kSwapSharedBytes, static_cast<cudaStream_t>(stream), p));
}

int loom_cuda_block_table_remap(int32_t* block_tables, uint64_t entries, const int32_t* new_block_ids,
                                uint32_t num_blocks, void* stream) {
  if (entries == 0) return LOOM_CUDA_SUCCESS;
  if (!block_tables || !new_block_ids || num_blocks == 0) return LOOM_CUDA_INVALID_ARGUMENT;
  const int sms = sm_count();
  if (sms <= 0) return LOOM_CUDA_UNAVAILABLE;
  const uint64_t wanted = (entries + kThreads - 1) / kThreads;
  const uint64_t resident = (uint64_t)sms * 8u;
  return finish(loom_launch::launch(block_table_remap_kernel, dim3((uint32_t)(wanted < resident ? wanted : resident)),
                                    dim3(kThreads), 0, static_cast<cudaStream_t>(stream), block_tables, entries,
                                    new_block_ids, num_blocks));
}

}  // extern "C"
