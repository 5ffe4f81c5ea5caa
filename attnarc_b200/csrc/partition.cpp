// Multi-GPU partitioner: pure host arithmetic, see include/loom_partition.h.

#include "../../include/loom_partition.h"

#include <algorithm>
#include <numeric>
#include <vector>

namespace {

// Indices of `lengths` sorted longest first; equal lengths keep index order.
std::vector<uint32_t> longest_first(const int64_t* lengths, const std::vector<uint32_t>& subset) {
  std::vector<uint32_t> order = subset;
  std::stable_sort(order.begin(), order.end(),
                   [lengths](uint32_t a, uint32_t b) { return lengths[a] > lengths[b]; });
  return order;
}

uint32_t lightest_rank(const std::vector<uint64_t>& load) {
  return (uint32_t)(std::min_element(load.begin(), load.end()) - load.begin());
}

}  // namespace

extern "C" int loom_partition_by_sequence(const int64_t* lengths, uint32_t sequences, uint32_t ranks,
                                          uint32_t* rank_of_sequence, uint64_t* tokens_per_rank) {
  if (lengths == nullptr || rank_of_sequence == nullptr || sequences == 0 || ranks == 0) return 1;
  for (uint32_t s = 0; s < sequences; ++s) {
    if (lengths[s] < 0) return 1;
  }
  std::vector<uint32_t> all(sequences);
  std::iota(all.begin(), all.end(), 0u);
  std::vector<uint64_t> load(ranks, 0);
  for (uint32_t sequence : longest_first(lengths, all)) {
    const uint32_t rank = lightest_rank(load);
    rank_of_sequence[sequence] = rank;
    load[rank] += (uint64_t)lengths[sequence];
  }
  if (tokens_per_rank != nullptr) std::copy(load.begin(), load.end(), tokens_per_rank);
  return 0;
}

extern "C" int loom_partition_by_kv_head(uint32_t kv_heads, uint32_t ranks, uint32_t* first_head,
                                         uint32_t* head_count) {
  if (first_head == nullptr || head_count == nullptr || kv_heads == 0 || ranks == 0) return 1;
  const uint32_t base = kv_heads / ranks, extra = kv_heads % ranks;
  uint32_t next = 0;
  for (uint32_t rank = 0; rank < ranks; ++rank) {
    const uint32_t count = base + (rank < extra ? 1u : 0u);
    first_head[rank] = next;
    head_count[rank] = count;
    next += count;
  }
  return 0;
}

extern "C" int loom_partition_long_context(const int64_t* lengths, uint32_t sequences, uint32_t ranks,
                                           uint32_t block_size, uint64_t split_threshold_tokens,
                                           LoomSequenceShard* shards, uint32_t shard_capacity,
                                           uint32_t* shard_count, uint64_t* tokens_per_rank) {
  if (lengths == nullptr || shards == nullptr || shard_count == nullptr || sequences == 0 || ranks == 0 ||
      block_size == 0) {
    return 1;
  }
  uint64_t total = 0;
  for (uint32_t s = 0; s < sequences; ++s) {
    if (lengths[s] < 0) return 1;
    total += (uint64_t)lengths[s];
  }
  const uint64_t threshold =
      split_threshold_tokens != 0 ? split_threshold_tokens : (total + ranks - 1) / ranks;

  std::vector<uint64_t> load(ranks, 0);
  std::vector<std::vector<LoomSequenceShard>> per_sequence(sequences);
  std::vector<uint32_t> whole;
  for (uint32_t s = 0; s < sequences; ++s) {
    const uint64_t length = (uint64_t)lengths[s];
    if (ranks == 1 || length <= threshold) {
      whole.push_back(s);
      continue;
    }
    const uint64_t blocks = (length + block_size - 1) / block_size;
    for (uint32_t rank = 0; rank < ranks; ++rank) {
      const uint64_t first = blocks * rank / ranks;
      const uint64_t last = blocks * (rank + 1) / ranks;
      if (last == first) continue;
      LoomSequenceShard shard{};
      shard.sequence = s;
      shard.rank = rank;
      shard.first_block = (uint32_t)first;
      shard.block_count = (uint32_t)(last - first);
      shard.first_token = first * block_size;
      shard.token_count = std::min<uint64_t>(length, last * block_size) - shard.first_token;
      shard.split = 1;
      per_sequence[s].push_back(shard);
      load[rank] += shard.token_count;
    }
  }
  for (uint32_t s : longest_first(lengths, whole)) {
    const uint32_t rank = lightest_rank(load);
    const uint64_t length = (uint64_t)lengths[s];
    LoomSequenceShard shard{};
    shard.sequence = s;
    shard.rank = rank;
    shard.first_block = 0;
    shard.block_count = (uint32_t)((length + block_size - 1) / block_size);
    shard.first_token = 0;
    shard.token_count = length;
    shard.split = 0;
    per_sequence[s].push_back(shard);
    load[rank] += length;
  }
  uint32_t written = 0;
  for (uint32_t s = 0; s < sequences; ++s) {
    for (const LoomSequenceShard& shard : per_sequence[s]) {
      if (written >= shard_capacity) return 1;
      shards[written++] = shard;
    }
  }
  *shard_count = written;
  if (tokens_per_rank != nullptr) std::copy(load.begin(), load.end(), tokens_per_rank);
  return 0;
}
