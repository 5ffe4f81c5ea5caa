// Exchange and merge of partial decode states between the GPUs of one node, over peer memory.
//
// The long-context mode cuts a sequence into one block range per GPU; every GPU turns its range
// into partial (O, max, sum) states and all of them need all parts (the reference has no such mode:
// docs/operator-catalog.md:109 lists distributed split-KV as planned). The parts are small
// ((Dv + 2) * 4 bytes per query head and GPU, 133 KB per GPU for 8 sequences of 32 heads) and the
// step around them takes tens of microseconds, so the exchange is bound by latency: a library
// all-gather costs a launch and a rendezvous of its own (about 12 us) before a merge kernel can
// start. Here two kernels of this library do it:
//
//   push   every GPU stores its states straight into every peer's exchange buffer (plain 16-byte
//          stores through NVLink, no load from peer memory, no multicast), fences, and adds one
//          arrival per CTA to a counter in the peer's buffer;
//   merge  every GPU waits (bounded) until the counters in its own buffer show that all parts of
//          this step have landed, merges them per row with the same log-sum-exp arithmetic as
//          loom_cuda_merge_decode_states, and stores the rows.
//
// State lives in the exchange buffer of each GPU (ExchangeHeader + two generations of parts):
//  - `epoch` counts this GPU's completed steps. Both kernels read it at their start; the merge
//    kernel's last CTA (a self-resetting ticket) increments it. Every GPU must run every step.
//  - `arrivals[src]` only ever grows: step e is complete when it reaches e * kPushCtasPerPeer, so
//    nothing is reset and nothing can be missed.
//  - parts of step e go to generation e % 2. A peer can only push step e + 2 into the generation
//    this GPU reads in step e after it has finished its own step e + 1, which waited for this
//    GPU's push of step e + 1, which is enqueued after this GPU's merge of step e: two generations
//    are enough, with no further flow control.
// A wait that runs out sets `error` in the header (read with loom_cuda_peer_exchange_status) and
// the kernel goes on with what it has; the rows of that step are then not valid.
//
// One process per GPU. Buffers are plain cudaMalloc allocations shared between the processes with
// CUDA IPC handles (peer_exchange_create / _open), so the library depends on no communication
// package; the handles travel by whatever the host program uses (torch.distributed in the Python
// layer). Kernels that wait for other GPUs must run one per GPU: never as several launches on one
// device waiting for each other (the single-GPU test enqueues all pushes before the first merge).

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "../../include/loom_launch.h"
#include "decode_merge.cuh"
#include "launch_util.cuh"

namespace {

using loom_decode::kLog2e;

constexpr uint32_t kMaxRanks = LOOM_CUDA_PEER_EXCHANGE_MAX_RANKS;
constexpr uint32_t kPushCtasPerPeer = 4;
constexpr uint32_t kPushThreads = 256;
constexpr uint32_t kMergeThreads = 128;
constexpr uint32_t kDefaultWaitPolls = 1u << 22;  // about a second of polling a counter in local memory

struct ExchangeHeader {
  unsigned long long epoch;                // completed steps of this GPU
  unsigned int ticket;                     // CTAs of the running merge kernel that have finished (wraps to 0)
  unsigned int error;                      // bit 0: a wait for a peer's parts ran out
  unsigned long long arrivals[kMaxRanks];  // arrivals[src]: CTAs of rank src that have pushed into this buffer
  unsigned long long reserved[6];
};
static_assert(sizeof(ExchangeHeader) % 16 == 0, "the parts behind the header are copied 16 bytes at a time");

struct ExchangePeers {
  uint8_t* buffer[kMaxRanks];  // base of every rank's exchange buffer as mapped into this process
};

__host__ __device__ inline uint64_t generation_floats(uint32_t world, uint32_t rows, uint32_t value_head_size) {
  return (uint64_t)world * rows * (value_head_size + 2u);
}

__device__ __forceinline__ float* parts_of(uint8_t* buffer, uint32_t generation, uint32_t world, uint32_t rows,
                                           uint32_t value_head_size) {
  return reinterpret_cast<float*>(buffer + sizeof(ExchangeHeader)) +
         generation * generation_floats(world, rows, value_head_size);
}

__device__ __forceinline__ unsigned long long load_acquire_system(const unsigned long long* address) {
  unsigned long long value;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];\n" : "=l"(value) : "l"(address) : "memory");
  return value;
}

// grid (kPushCtasPerPeer, world): CTA (c, d) copies slice c of this rank's states into rank d's
// buffer (d may be this rank: the same path, a local copy) and then reports its arrival there.
__global__ void __launch_bounds__(kPushThreads)
peer_exchange_push_kernel(const float* __restrict__ states, ExchangePeers peers, uint32_t rank, uint32_t world,
                          uint32_t rows, uint32_t value_head_size) {
  loom_launch::grid_dependency_wait();
  const uint32_t destination = blockIdx.y;
  const ExchangeHeader* mine = reinterpret_cast<const ExchangeHeader*>(peers.buffer[rank]);
  const unsigned long long step = *reinterpret_cast<const volatile unsigned long long*>(&mine->epoch) + 1ull;
  uint8_t* target = peers.buffer[destination];
  float* slot = parts_of(target, (uint32_t)(step & 1ull), world, rows, value_head_size) +
                (uint64_t)rank * rows * (value_head_size + 2u);
  // rows * (Dv + 2) floats; Dv is even on every route that emits states, so the count is even, and
  // the caller guarantees 16-byte alignment of `states` and a multiple of four floats (checked on the host)
  const uint64_t vectors = (uint64_t)rows * (value_head_size + 2u) / 4u;
  const uint4* source = reinterpret_cast<const uint4*>(states);
  uint4* sink = reinterpret_cast<uint4*>(slot);
  for (uint64_t i = (uint64_t)blockIdx.x * kPushThreads + threadIdx.x; i < vectors;
       i += (uint64_t)kPushCtasPerPeer * kPushThreads) {
    sink[i] = __ldcg(source + i);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd_system(&reinterpret_cast<ExchangeHeader*>(target)->arrivals[rank], 1ull);
  }
}

// One CTA per output row. Waits until every rank's parts of this step are in this GPU's buffer,
// merges them, stores the row; the last CTA to finish closes the step.
template <typename OT>
__global__ void __launch_bounds__(kMergeThreads)
peer_exchange_merge_kernel(uint8_t* buffer, uint32_t world, uint32_t rows, uint32_t value_head_size, void* output,
                           uint32_t wait_polls) {
  loom_launch::grid_dependency_wait();
  ExchangeHeader* header = reinterpret_cast<ExchangeHeader*>(buffer);
  const unsigned long long step = *reinterpret_cast<volatile unsigned long long*>(&header->epoch) + 1ull;
  __shared__ uint32_t complete;
  if (threadIdx.x < 32) {
    // lane r polls rank r's counter; the warp leaves when all have arrived or the polls run out
    const unsigned long long wanted = step * kPushCtasPerPeer;
    bool arrived = threadIdx.x >= world;
    uint32_t polls = 0;
    while (true) {
      if (!arrived) arrived = load_acquire_system(&header->arrivals[threadIdx.x]) >= wanted;
      if (__all_sync(0xffffffffu, arrived)) break;
      if (++polls >= wait_polls) break;
    }
    const bool all_arrived = __all_sync(0xffffffffu, arrived);
    if (threadIdx.x == 0) {
      complete = all_arrived ? 1u : 0u;
      if (!all_arrived) atomicOr(&header->error, 1u);
    }
  }
  __syncthreads();
  const uint32_t row = blockIdx.x;
  const uint32_t stride = value_head_size + 2u;
  const float* parts = parts_of(buffer, (uint32_t)(step & 1ull), world, rows, value_head_size);
  for (uint32_t dv = threadIdx.x; dv < value_head_size; dv += kMergeThreads) {
    float top = -INFINITY, total = 0.0f, acc = 0.0f;
    for (uint32_t part = 0; part < world; ++part) {
      // written by other GPUs during this kernel's lifetime: read past the L1 and the read-only path
      const float* state = parts + ((uint64_t)part * rows + row) * stride;
      const float sum = __ldcg(state + value_head_size + 1);
      if (!(sum > 0.0f)) continue;
      const float maximum = __ldcg(state + value_head_size);
      const float o = __ldcg(state + dv);
      const float new_top = fmaxf(top, maximum);
      const float keep = exp2f((top - new_top) * kLog2e);  // 0 while top is still -inf
      const float factor = exp2f((maximum - new_top) * kLog2e);
      total = total * keep + sum * factor;
      acc = acc * keep + o * factor;
      top = new_top;
    }
    loom_decode::narrow_store<OT>(static_cast<OT*>(output) + (uint64_t)row * value_head_size + dv,
                                  (complete && total > 0.0f) ? acc / total : 0.0f);
  }
  // close the step: the last CTA of this launch advances the epoch (the ticket wraps back to 0)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicInc(&header->ticket, gridDim.x - 1u) == gridDim.x - 1u) {
      atomicAdd(&header->epoch, 1ull);
    }
  }
}

bool shape_ok(uint32_t world, uint32_t rank, uint32_t rows, uint32_t value_head_size) {
  return world >= 1 && world <= kMaxRanks && rank < world && rows != 0 && rows <= 0x7fffffffu &&
         value_head_size != 0 && ((uint64_t)rows * (value_head_size + 2u)) % 4u == 0;
}

}  // namespace

extern "C" {

uint64_t loom_cuda_peer_exchange_bytes(uint32_t world, uint32_t rows, uint32_t value_head_size) {
  if (!shape_ok(world, 0, rows, value_head_size)) return 0;
  return sizeof(ExchangeHeader) + 2ull * generation_floats(world, rows, value_head_size) * sizeof(float);
}

int loom_cuda_peer_exchange_create(uint64_t bytes, void** buffer, unsigned char* handle, uint64_t handle_capacity) {
  if (buffer == nullptr || handle == nullptr || bytes < sizeof(ExchangeHeader) ||
      handle_capacity < sizeof(cudaIpcMemHandle_t)) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  void* allocation = nullptr;
  if (const cudaError_t status = cudaMalloc(&allocation, bytes); status != cudaSuccess) {
    loom_launch::failed(status, "allocating a peer exchange buffer (cudaMalloc)");
    return LOOM_CUDA_UNAVAILABLE;
  }
  cudaError_t status = cudaMemset(allocation, 0, bytes);
  cudaIpcMemHandle_t ipc{};
  if (status == cudaSuccess) status = cudaIpcGetMemHandle(&ipc, allocation);
  if (status != cudaSuccess) {
    cudaFree(allocation);
    loom_launch::failed(status, "sharing a peer exchange buffer (cudaIpcGetMemHandle)");
    return LOOM_CUDA_UNAVAILABLE;
  }
  std::memcpy(handle, &ipc, sizeof(ipc));
  *buffer = allocation;
  return LOOM_CUDA_SUCCESS;
}

int loom_cuda_peer_exchange_open(const unsigned char* handle, uint64_t handle_bytes, void** buffer) {
  if (handle == nullptr || buffer == nullptr || handle_bytes < sizeof(cudaIpcMemHandle_t)) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  cudaIpcMemHandle_t ipc{};
  std::memcpy(&ipc, handle, sizeof(ipc));
  void* mapped = nullptr;
  if (const cudaError_t status = cudaIpcOpenMemHandle(&mapped, ipc, cudaIpcMemLazyEnablePeerAccess);
      status != cudaSuccess) {
    loom_launch::failed(status, "mapping a peer's exchange buffer (cudaIpcOpenMemHandle)");
    return LOOM_CUDA_UNAVAILABLE;
  }
  *buffer = mapped;
  return LOOM_CUDA_SUCCESS;
}

int loom_cuda_peer_exchange_close(void* peer_buffer) {
  if (peer_buffer == nullptr) return LOOM_CUDA_INVALID_ARGUMENT;
  return loom_launch::failed(cudaIpcCloseMemHandle(peer_buffer), "unmapping a peer's exchange buffer");
}

int loom_cuda_peer_exchange_destroy(void* buffer) {
  if (buffer == nullptr) return LOOM_CUDA_INVALID_ARGUMENT;
  return loom_launch::failed(cudaFree(buffer), "freeing a peer exchange buffer");
}

int loom_cuda_peer_exchange_reset(void* buffer, uint64_t bytes, void* stream) {
  if (buffer == nullptr || bytes < sizeof(ExchangeHeader)) return LOOM_CUDA_INVALID_ARGUMENT;
  return loom_launch::failed(cudaMemsetAsync(buffer, 0, bytes, static_cast<cudaStream_t>(stream)),
                             "zeroing a peer exchange buffer");
}

int loom_cuda_peer_exchange_status(const void* buffer, uint64_t* completed_steps, uint32_t* error) {
  if (buffer == nullptr) return LOOM_CUDA_INVALID_ARGUMENT;
  ExchangeHeader header{};
  if (const cudaError_t status = cudaMemcpy(&header, buffer, sizeof(header), cudaMemcpyDeviceToHost);
      status != cudaSuccess) {
    return loom_launch::failed(status, "reading a peer exchange buffer's header");
  }
  if (completed_steps != nullptr) *completed_steps = header.epoch;
  if (error != nullptr) *error = header.error;
  return LOOM_CUDA_SUCCESS;
}

int loom_cuda_peer_exchange_push(const float* states, void* const* rank_buffers, uint32_t rank, uint32_t world,
                                 uint32_t rows, uint32_t value_head_size, void* stream) {
  if (states == nullptr || rank_buffers == nullptr || !shape_ok(world, rank, rows, value_head_size) ||
      (reinterpret_cast<uintptr_t>(states) & 15u) != 0) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  ExchangePeers peers{};
  for (uint32_t r = 0; r < world; ++r) {
    if (rank_buffers[r] == nullptr) return LOOM_CUDA_INVALID_ARGUMENT;
    peers.buffer[r] = static_cast<uint8_t*>(rank_buffers[r]);
  }
  return loom_launch::failed(
      loom_launch::launch(peer_exchange_push_kernel, dim3(kPushCtasPerPeer, world), dim3(kPushThreads), 0,
                          static_cast<cudaStream_t>(stream), states, peers, rank, world, rows, value_head_size),
      "peer exchange push kernel launch");
}

int loom_cuda_peer_exchange_merge(void* buffer, uint32_t world, uint32_t rows, uint32_t value_head_size,
                                  uint32_t out_dtype, void* output, void* stream) {
  if (buffer == nullptr || output == nullptr || !shape_ok(world, 0, rows, value_head_size) || out_dtype > 2) {
    return LOOM_CUDA_INVALID_ARGUMENT;
  }
  const uint32_t polls = loom_launch::wait_attempts(kDefaultWaitPolls);
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(buffer);
  cudaError_t status;
  if (out_dtype == 0) {
    status = loom_launch::launch(peer_exchange_merge_kernel<float>, dim3(rows), dim3(kMergeThreads), 0, cuda_stream,
                                 base, world, rows, value_head_size, output, polls);
  } else if (out_dtype == 1) {
    status = loom_launch::launch(peer_exchange_merge_kernel<__half>, dim3(rows), dim3(kMergeThreads), 0,
                                 cuda_stream, base, world, rows, value_head_size, output, polls);
  } else {
    status = loom_launch::launch(peer_exchange_merge_kernel<__nv_bfloat16>, dim3(rows), dim3(kMergeThreads), 0,
                                 cuda_stream, base, world, rows, value_head_size, output, polls);
  }
  return loom_launch::failed(status, "peer exchange merge kernel launch");
}

}  // extern "C"
