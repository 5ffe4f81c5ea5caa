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
// sequences * query_tokens rows. This is the first correct path, not the fast
// one: a sequence's pages are streamed once per query token (from L2 where the
// batch's KV fits there, from HBM otherwise). The fast form packs the tokens'
// rows beside the GQA group in the MMA's N dimension over the common prefix
// and merges a short per-token tail; it is not built yet.

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
  if (status != cudaSuccess) {
    cudaGetLastError();
    return LOOM_CUDA_LAUNCH_ERROR;
  }
  return LOOM_CUDA_SUCCESS;
}
