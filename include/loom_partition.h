/*
 * Multi-GPU partitioner of the paged-decode path (plain C, host only).
 *
 * No counterpart exists in the reference, which runs on one device
 * (docs/operator-catalog.md:109 lists distributed split-KV as planned). The
 * decode work of a step is a set of independent (sequence, KV head) units, so
 * it shards without any exchange of data in two of the three modes:
 *   - by sequence: whole sequences go to ranks, balanced on context length;
 *   - by KV head:  each rank owns a contiguous range of KV heads and the
 *                  query heads of their groups;
 *   - long context: a sequence longer than a rank's fair share is cut into
 *                  contiguous block ranges, one per rank. Each rank produces
 *                  partial (O, max, sum) states for its range; the states are
 *                  all-gathered and merged by loom_cuda_merge_decode_states.
 *                  The remaining sequences are placed as in the first mode,
 *                  counting the shares already handed out.
 * These functions only compute the assignment. They touch no device and are
 * deterministic: ties go to the lower rank and to the lower sequence index.
 * Return value: 0 on success, 1 on an invalid argument.
 */
#ifndef LOOM_PARTITION_H_
#define LOOM_PARTITION_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Greedy longest-first assignment. rank_of_sequence has `sequences` entries,
 * tokens_per_rank has `ranks` entries (may be null). */
int loom_partition_by_sequence(const int64_t* lengths, uint32_t sequences,
                               uint32_t ranks, uint32_t* rank_of_sequence,
                               uint64_t* tokens_per_rank);

/* Contiguous KV-head ranges, sizes differing by at most one. first_head and
 * head_count have `ranks` entries; a rank beyond kv_heads gets count 0. */
int loom_partition_by_kv_head(uint32_t kv_heads, uint32_t ranks,
                              uint32_t* first_head, uint32_t* head_count);

typedef struct LoomSequenceShard {
  uint32_t sequence;    /* index into `lengths` */
  uint32_t rank;        /* owner */
  uint32_t first_block; /* first logical block of the owned range */
  uint32_t block_count;
  uint64_t first_token; /* = first_block * block_size */
  uint64_t token_count; /* tokens of the sequence inside the range */
  uint32_t split;       /* 1 if the sequence is spread over several ranks */
  uint32_t reserved;
} LoomSequenceShard;

/*
 * Long-context mode. A sequence longer than split_threshold_tokens is cut into
 * `ranks` block ranges (0 = use ceil(total tokens / ranks)). `shards` receives
 * one entry per whole sequence and one per non-empty range, ordered by
 * sequence then rank; shard_capacity >= sequences + split sequences * ranks is
 * always enough. shard_count and tokens_per_rank are outputs.
 */
int loom_partition_long_context(const int64_t* lengths, uint32_t sequences,
                                uint32_t ranks, uint32_t block_size,
                                uint64_t split_threshold_tokens,
                                LoomSequenceShard* shards,
                                uint32_t shard_capacity, uint32_t* shard_count,
                                uint64_t* tokens_per_rank);

#ifdef __cplusplus
}
#endif

#endif /* LOOM_PARTITION_H_ */
