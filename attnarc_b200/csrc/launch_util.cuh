// Kernel launch helper shared by the decode and RoPE translation units, and the
// device side of programmatic dependent launch.
//
// With programmatic launch on (the default), every kernel of this library is
// launched with cudaLaunchAttributeProgrammaticStreamSerialization: its CTAs
// may become resident while the kernel before it in the stream drains (that
// kernel's CTAs release their dependents when they exit), which hides launch
// latency and CTA set-up. Each kernel executes griddepcontrol.wait before its
// first access to global memory, and that instruction returns only when the
// earlier kernel has completed and its writes are visible, so results do not
// depend on the mode. A kernel launched without the attribute, or after
// something that is not a kernel, passes the wait at once.
//
// Only the RoPE + KV-write kernel signals its dependents early
// (griddepcontrol.launch_dependents at its top): the decode kernel that follows
// it in a step then sets itself up, and with stable metadata runs its whole
// prologue, while the rotation is still at work. The decode and merge kernels do
// not signal early: measured on the RoPE -> decode -> merge chain, early signals
// from all three let the next step's persistent decode CTAs occupy SMs while this
// step's merge still needed them, and a 39 us step became 46 us. A signal in the
// decode kernel alone (after its last chunk, so that only the small merge kernel
// is set up early) changed nothing: 34.2 -> 34.1 us for decode + merge.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <utility>

namespace loom_launch {

// ---- what went wrong, for the caller who only sees LOOM_CUDA_LAUNCH_ERROR -----------------
//
// Every runtime call on a launch path of this library (kernel launches, the
// shared-memory limit of a kernel, device queries) reports its failure through
// `failed()`: the error and the place are remembered per thread (read with
// loom_cuda_last_launch_failure), printed when LOOM_DEBUG_LAUNCH is set, and the
// runtime's own last-error slot is cleared so that the failure cannot be
// mistaken for the result of a later call.
struct Failure {
  cudaError_t error;
  const char* where;
};
inline Failure& last_failure() {
  static thread_local Failure failure{cudaSuccess, "none"};
  return failure;
}

// Launches that the runtime refused with the programmatic-launch attribute and
// that were then issued as plain launches (process-wide count).
inline std::atomic<uint64_t>& plain_retries() {
  static std::atomic<uint64_t> count{0};
  return count;
}

// ---- bounded waits ---------------------------------------------------------------------------
//
// Every wait of a kernel on a copy barrier gives up after a number of polls and the kernel then
// records the expiry, stops copying, gives the copies still in flight one more bounded wait and
// runs to its end. The limit is a launch-time value: `attempts` polls (0 = each kernel's own
// default, about a second). `unmatched_bytes` is a self-test: every copy barrier is armed for that
// many bytes MORE than its copy delivers, so the first wait of every ring runs out although the
// data arrives; with a small `attempts` this exercises the expiry path in microseconds, without
// any fault. Process-wide; read at each launch.
inline std::atomic<uint64_t>& wait_policy_word() {
  static std::atomic<uint64_t> word{0};  // attempts | unmatched_bytes << 32
  return word;
}
inline uint32_t wait_attempts(uint32_t kernel_default) {
  const uint32_t chosen = (uint32_t)(wait_policy_word().load(std::memory_order_relaxed) & 0xffffffffu);
  return chosen != 0 ? chosen : kernel_default;
}
inline uint32_t wait_unmatched_bytes() {
  return (uint32_t)(wait_policy_word().load(std::memory_order_relaxed) >> 32);
}

// LoomCudaStatus of a runtime status: 0 (success) or 3 (launch error).
inline int failed(cudaError_t status, const char* where) {
  if (status == cudaSuccess) return 0;
  cudaGetLastError();
  last_failure() = Failure{status, where};
  static const bool verbose = std::getenv("LOOM_DEBUG_LAUNCH") != nullptr;
  if (verbose) {
    std::fprintf(stderr, "loom launch failed at %s: %s (%s)\n", where, cudaGetErrorName(status),
                 cudaGetErrorString(status));
  }
  return 3;
}

// 0 = plain launches; 1 = programmatic launch.
inline std::atomic<uint32_t>& programmatic_mode() {
  static std::atomic<uint32_t> mode{1};
  return mode;
}

template <typename... Params, typename... Args>
cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes,
                   cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  if (programmatic_mode().load(std::memory_order_relaxed) != 0) {
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
  }
  cudaError_t status = cudaLaunchKernelEx(&config, kernel, args...);
  if (status != cudaSuccess && config.numAttrs != 0) {
    // The attribute is an optimisation: a launch refused with it is tried once as a plain launch
    // (a genuine configuration error fails again and is reported).
    static const bool verbose = std::getenv("LOOM_DEBUG_LAUNCH") != nullptr;
    if (verbose) {
      std::fprintf(stderr, "loom: launch with the programmatic attribute refused (%s), retried as a plain launch\n",
                   cudaGetErrorName(status));
    }
    cudaGetLastError();
    plain_retries().fetch_add(1, std::memory_order_relaxed);
    config.attrs = nullptr;
    config.numAttrs = 0;
    status = cudaLaunchKernelEx(&config, kernel, args...);
  }
  return status;
}

#ifdef __CUDACC__
// Blocks until every kernel this one depends on has completed and flushed.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Lets the next kernel of the stream, if it was launched with the programmatic attribute, become
// resident once every CTA of this grid has got here. That kernel still sees this one's results
// only after its own grid_dependency_wait.
__device__ __forceinline__ void release_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

#endif

}  // namespace loom_launch
