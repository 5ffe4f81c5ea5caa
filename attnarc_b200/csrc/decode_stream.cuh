// Balanced persistent paged decode kernel.
//
// The fixed-partition kernel (decode_mma.cuh) gives every CTA one partition of
// one (sequence, KV head); with ragged context lengths the CTAs run in uneven
// waves and each one pays its own fill and drain. This kernel removes both
// costs. The K/V of the whole batch is viewed as one line of 64-token tiles,
//     sequence 0 / head 0 / tile 0..t0-1, sequence 0 / head 1 / ..., sequence 1 ...
// and CTA c of a grid of G resident CTAs (two per SM) takes a contiguous
// range of T/G (+1 for the first T mod G CTAs) tiles of it. Inside a tile warp w owns tokens
// [16w, 16w+16). Each warp keeps a private ring of K and V tiles filled by
// cp.async several tiles ahead, and the ring keeps streaming across the
// boundary between two work items, so HBM never sees a drain/fill bubble after
// the first microsecond. The 131072-token sequence of a skewed batch is spread
// over all CTAs exactly like sixty short ones are.
//
// A CTA's range may start or end inside a work item. For every item it
// touches it produces one (O, max, sum) state per query head: the final output
// if the item lies wholly inside the range, else a partial state in slot
// `item + cta` of the workspace (item and CTA numbers both only grow along the
// line, so that sum is unique). The CTA holding an item's first tile records
// (first CTA, number of CTAs) in the item table; the merge kernel reads it.
//
// The per-sequence tile counts are prefix-summed by every CTA on its own (a few
// hundred integers from L2), because lengths live in device memory and the
// launch must stay asynchronous.
#pragma once

#include "decode_mma.cuh"

namespace loom_decode {

constexpr uint32_t kStreamTileTokens = 16 * kMmaWarps;  // 64
constexpr uint32_t kStreamMaxSequences = 2048;

template <bool kFp8, int kD, int kNT>
struct StreamRing {
  using Tile = MmaTile<kFp8, kD>;
  static constexpr int kWantedBytes = kNT == 1 ? 20 * 1024 : 16 * 1024;
  static constexpr int kRaw = kWantedBytes / Tile::kTileBytes;
  static constexpr int kSlots = kRaw < 3 ? 3 : (kRaw > 9 ? 9 : kRaw);  // K and V tiles, per warp
  static constexpr int kAhead = kSlots - 1;                            // tiles in flight
  static constexpr int kRingBytes = kMmaWarps * kSlots * Tile::kTileBytes;
  static constexpr int kMergeBytes = mma_merge_bytes<kNT, kD>();
  static constexpr int kPrefixBytes = (kStreamMaxSequences + 1) * 4;
  static constexpr int kSmemBytes = kRingBytes + kMergeBytes + kPrefixBytes;
};

// Where a CTA is along the line of tiles.
struct StreamCursor {
  uint32_t seq, head, tile, tiles, length;
};

// Under a sliding window a sequence's line of tiles starts at the tile holding the first token
// the query sees; without one (window 0) that is tile 0.
__device__ __forceinline__ uint32_t stream_first_tile(uint32_t length, uint32_t window) {
  return window_begin(length, window) / kStreamTileTokens;
}
__device__ __forceinline__ uint32_t stream_tiles(uint32_t length, uint32_t window) {
  return (length + kStreamTileTokens - 1) / kStreamTileTokens - stream_first_tile(length, window);
}
// Does the 16-token chunk at token0 hold a token the query sees?
__device__ __forceinline__ bool stream_chunk_live(uint32_t token0, uint32_t length, uint32_t window) {
  return token0 < length && token0 + 16u > window_begin(length, window);
}

template <typename QT, bool kFp8, int kD, int kNT, bool kOptions>
__global__ void __launch_bounds__(kMmaThreads, 2) decode_stream_kernel(const DecodeParams p) {
  using Tile = MmaTile<kFp8, kD>;
  using Ring = StreamRing<kFp8, kD, kNT>;
  constexpr int kHeads = 8 * kNT;
  constexpr uint32_t kElem = kFp8 ? 1 : 2;

  extern __shared__ __align__(128) uint8_t smem[];
  loom_launch::grid_dependency_wait();
  uint32_t* prefix = reinterpret_cast<uint32_t*>(smem + Ring::kRingBytes + Ring::kMergeBytes);  // [sequences + 1]
  __shared__ uint32_t warp_totals[kMmaWarps];

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2;
  const uint32_t t = lane & 3u;

  // ---- tiles per sequence, exclusive prefix sum -----------------------------
  {
    const uint32_t per_thread = (p.sequences + kMmaThreads - 1) / kMmaThreads;
    const uint32_t begin = min(threadIdx.x * per_thread, p.sequences);
    const uint32_t end = min(begin + per_thread, p.sequences);
    uint32_t local = 0;
    for (uint32_t s = begin; s < end; ++s) {
      const uint32_t length = clamp_length(__ldg(p.sequence_lengths + s), p.max_sequence_length);
      local += stream_tiles(length, kOptions ? p.sliding_window : 0u);
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
      running += stream_tiles(length, kOptions ? p.sliding_window : 0u);
    }
    if (threadIdx.x == kMmaThreads - 1) prefix[p.sequences] = running;
    __syncthreads();
  }

  const uint32_t head_chunks = (p.group + kHeads - 1) / kHeads;
  const uint32_t heads = p.kv_heads * head_chunks;  // work items per sequence
  const uint64_t total_tiles = (uint64_t)heads * prefix[p.sequences];
  // The first `extra` CTAs take `share + 1` tiles, the others `share`; with
  // fewer tiles than CTAs the busy CTAs are therefore the first ones, which is
  // what lets the parts of an item sit in consecutive slots.
  const uint64_t ctas = gridDim.x;
  const uint64_t share = total_tiles / ctas;
  const uint64_t extra = total_tiles % ctas;
  const uint64_t range_begin = blockIdx.x * share + min((uint64_t)blockIdx.x, extra);
  const uint64_t range_end = range_begin + share + (blockIdx.x < extra ? 1u : 0u);
  if (range_begin >= range_end) return;
  auto cta_of = [&](uint64_t tile) -> uint32_t {
    const uint64_t boundary = extra * (share + 1);
    return tile < boundary ? (uint32_t)(tile / (share + 1)) : (uint32_t)(extra + (tile - boundary) / share);
  };
  const uint32_t my_tiles = (uint32_t)(range_end - range_begin);

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

  // ---- locate the first tile of the range -----------------------------------
  StreamCursor start;
  {
    // largest seq with heads * prefix[seq] <= range_begin
    uint32_t low = 0, high = p.sequences;  // invariant: heads*prefix[low] <= range_begin < heads*prefix[high]
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

  // ---- producer ---------------------------------------------------------------
  const uint8_t* key_bytes = static_cast<const uint8_t*>(p.key_cache);
  const uint8_t* value_bytes = static_cast<const uint8_t*>(p.value_cache);
  const uint32_t ring_base = smem_address(smem) + warp * (Ring::kSlots * Tile::kTileBytes);
  const uint32_t copy_row = lane / Tile::kSegs;
  const uint32_t copy_col = lane % Tile::kSegs;
  const uint32_t warp_token = warp * 16u;
  const uint32_t window = kOptions ? p.sliding_window : 0u;  // the plain instantiation carries no window arithmetic

  StreamCursor producer = start;
  uint32_t producer_block = 0;
  auto fetch_block = [&]() {
    // block id of the producer cursor's chunk for this warp, looked up one chunk early
    const uint32_t token0 =
        (stream_first_tile(producer.length, window) + producer.tile) * kStreamTileTokens + warp_token;
    producer_block = 0;
    if (stream_chunk_live(token0, producer.length, window)) {
      producer_block = clamp_block(
          __ldg(p.block_tables + (uint64_t)producer.seq * p.max_blocks_per_sequence + token0 / p.block_size),
          p.num_blocks);
    }
  };
  fetch_block();

  // Issues ring tile `index` (even = K, odd = V of chunk index/2) and commits.
  auto issue_tile = [&](uint32_t index) {
    if ((index >> 1) < my_tiles) {
      const bool is_value = index & 1u;
      const uint32_t token0 =
          (stream_first_tile(producer.length, window) + producer.tile) * kStreamTileTokens + warp_token;
      if (stream_chunk_live(token0, producer.length, window)) {
        const uint32_t slot = ring_base + (index % Ring::kSlots) * Tile::kTileBytes;
        const uint32_t kv_head = producer.head / head_chunks;
        const uint32_t page0 = token0 % p.block_size;
        const uint8_t* base = is_value ? value_bytes : key_bytes;
        const uint64_t block_stride = is_value ? p.v_block : p.k_block;
        const uint64_t page_stride = is_value ? p.v_page : p.k_page;
        const uint64_t head_stride = is_value ? p.v_head : p.k_head;
        const uint8_t* row = base + ((uint64_t)producer_block * block_stride +
                                     (uint64_t)(page0 + copy_row) * page_stride +
                                     (uint64_t)kv_head * head_stride) * kElem + copy_col * 16;
        const uint64_t step = (uint64_t)Tile::kRowsPerPass * page_stride * kElem;
#pragma unroll
        for (int pass = 0; pass < Tile::kPasses; ++pass) {
          const uint32_t tile_row = copy_row + pass * Tile::kRowsPerPass;
          const uint32_t bytes = (token0 + tile_row) < producer.length ? 16u : 0u;
          cp_async_16(slot + swizzled<Tile::kSegs>(tile_row, copy_col), bytes ? row + pass * step : base, bytes);
        }
      }
      if (is_value && (index >> 1) + 1 < my_tiles) {
        advance(producer);
        fetch_block();
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int index = 0; index < Ring::kAhead; ++index) issue_tile(index);

  // ---- consumer -----------------------------------------------------------------
  WarpState<kD, kNT> state;
  MergeArea<kD, kNT> area(smem + Ring::kRingBytes);
  StreamCursor consumer = start;
  const uint32_t stride = state_stride(kD);

  // current work item
  uint32_t item_seq = 0, item_head = 0, item_tiles = 0;

  auto begin_item = [&]() {
    item_seq = consumer.seq;
    item_head = consumer.head;
    item_tiles = consumer.tiles;
    const uint32_t kv_head = item_head / head_chunks;
    const uint32_t first_head = (item_head % head_chunks) * kHeads;
    const uint32_t live_heads = min((uint32_t)kHeads, p.group - first_head);
    state.reset();
    float score_scale = p.scale_log2;
    if constexpr (kFp8) score_scale *= __ldg(p.key_scales + (uint64_t)kv_head * p.scale_stride);
    load_query<QT, kFp8, kD, kNT>(
        state,
        static_cast<const QT*>(p.query) + (uint64_t)item_seq * p.q_token +
            ((uint64_t)kv_head * p.group + first_head) * p.q_head,
        p.q_head, live_heads, score_scale, g, t);
  };

  auto finish_item = [&]() {
    const uint32_t kv_head = item_head / head_chunks;
    const uint32_t first_head = (item_head % head_chunks) * kHeads;
    const uint32_t live_heads = min((uint32_t)kHeads, p.group - first_head);
    const uint64_t item = (uint64_t)item_seq * heads + item_head;
    const uint64_t item_begin = (uint64_t)heads * prefix[item_seq] + (uint64_t)item_head * item_tiles;
    const uint64_t item_end = item_begin + item_tiles;
    const uint32_t first_cta = cta_of(item_begin);
    const uint32_t last_cta = cta_of(item_end - 1);
    const uint32_t parts = last_cta - first_cta + 1;
    __syncthreads();  // the merge area may still be read by the previous item's store
    park_warp_state<kFp8, kD, kNT>(area, state, warp, g, t);
    __syncthreads();
    float value_scale = 1.0f;
    if constexpr (kFp8) value_scale = __ldg(p.value_scales + (uint64_t)kv_head * p.scale_stride);
    const uint64_t query_row = (uint64_t)item_seq * p.query_heads + (uint64_t)kv_head * p.group + first_head;
    if (parts == 1 && !p.emit_state) {
      combine_and_store<QT, kD, kNT>(area, live_heads, value_scale,
                                     static_cast<QT*>(p.output) + query_row * kD, kD, nullptr, 0);
    } else if (parts == 1) {
      combine_and_store<QT, kD, kNT>(area, live_heads, value_scale, nullptr, 0,
                                     static_cast<float*>(p.output) + query_row * stride, stride);
    } else {
      combine_and_store<QT, kD, kNT>(area, live_heads, value_scale, nullptr, 0,
                                     p.partials + (item + blockIdx.x) * kHeads * stride, stride);
    }
    if (threadIdx.x == 0 && blockIdx.x == first_cta) {
      p.item_meta[2 * item] = first_cta;
      p.item_meta[2 * item + 1] = parts;
    }
  };

  for (uint32_t chunk = 0; chunk < my_tiles; ++chunk) {
    // ---- K tile ------------------------------------------------------------
    cp_async_wait<Ring::kAhead - 1>();
    __syncwarp();
    issue_tile(2 * chunk + Ring::kAhead);
    if (chunk == 0 || consumer.tile == 0) {
      if (chunk != 0) finish_item();
      begin_item();
    }
    const uint32_t token0 =
        (stream_first_tile(consumer.length, window) + consumer.tile) * kStreamTileTokens + warp_token;
    const bool has_rows = stream_chunk_live(token0, consumer.length, window);  // warp-uniform
    uint32_t pb[kNT][2];
    if (has_rows) {
      const uint32_t k_tile = ring_base + ((2 * chunk) % Ring::kSlots) * Tile::kTileBytes;
      const uint32_t visible = window_begin(consumer.length, window);
      float s[kNT][4];
      chunk_scores<QT, kFp8, kD, kNT>(s, state, k_tile, lane);
      chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, consumer.length - token0, g,
                                       visible > token0 ? visible - token0 : 0u,
                                       kOptions ? p.soft_cap_log2 : 0.0f, kOptions ? p.inv_soft_cap_log2 : 0.0f);
    }
    // ---- V tile ------------------------------------------------------------
    cp_async_wait<Ring::kAhead - 1>();
    __syncwarp();
    issue_tile(2 * chunk + 1 + Ring::kAhead);
    if (has_rows) {
      const uint32_t v_tile = ring_base + ((2 * chunk + 1) % Ring::kSlots) * Tile::kTileBytes;
      chunk_values<QT, kFp8, kD, kNT>(state, pb, v_tile, lane);
    }
    if (chunk + 1 < my_tiles) advance(consumer);
  }
  cp_async_wait<0>();
  finish_item();
}

}  // namespace loom_decode
