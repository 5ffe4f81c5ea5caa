// Balanced persistent paged decode kernel, TMA-fed.
//
// Same schedule and arithmetic as decode_stream.cuh (even share of the batch's
// 64-token tiles per resident CTA, warp-private K/V rings, one state per work
// item and CTA), but the rings are filled by the Tensor Memory Accelerator:
// the cache is described to the hardware once per launch as a 4-D tensor
// (bytes of a row, KV head, page, block, with the caller's strides), and one
// lane per warp issues a cp.async.bulk.tensor per 16-token tile (two for a
// 256-byte row, because a 128-byte-swizzled box is at most 128 bytes wide).
// Completion is counted in bytes on an mbarrier per ring slot.
//
// Why it matters here: with cp.async every lane computes a 64-bit address and a
// predicate for each 16-byte piece, about 300 instructions per chunk on top of
// the ~250 of the MMA and softmax work, and with only eight warps per SM that
// instruction stream, not HBM, set the pace (issue slots 36 % busy at 53 % of
// DRAM peak). TMA takes the copy work out of the instruction stream.
//
// The tile of a partly filled last page is loaded whole (the page belongs to
// the sequence, so the read is in bounds); the consumer zeroes the rows of V
// beyond the sequence length before using them, and masks the matching scores,
// so stale cache contents cannot reach the output.
//
// Every wait on an mbarrier is bounded (the limit is a launch parameter). If a
// wait of a warp ever expires the kernel sets a flag in global memory (readable
// with loom_cuda_decode_timeout_flag) and that warp stops for good: it issues no
// further copy, gives each copy it still has in flight one more bounded wait,
// never waits or computes again, and only keeps walking its tiles so that it
// meets the CTA barriers of the item boundaries. The rows of the affected work
// items are then wrong, which is what the flag tells the host.
#pragma once

#include <cuda.h>

#include "decode_stream.cuh"

namespace loom_decode {

// Empty units the balanced line counts in front of every work item's tiles (decode_stream_tma_kernel).
constexpr uint32_t kItemSetupUnits = 1;

__device__ unsigned int g_decode_timeout_flag = 0;
// Which wait expired first: (wait kind + 1) << 20 | local tile index << 1; 0 if none.
__device__ unsigned int g_decode_timeout_where = 0;

// Which coordinate of the 4-D tensor map holds the KV head, the page and the
// block (coordinate 0 is always the byte offset inside a row). The outer
// dimensions are sorted by stride when the map is encoded, so NHD and HND
// caches order them differently.
struct TmaAxes {
  uint32_t head, page, block;
};

__device__ __forceinline__ void mbarrier_init(uint32_t barrier, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(barrier), "r"(count) : "memory");
}

__device__ __forceinline__ void mbarrier_expect_tx(uint32_t barrier, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(barrier), "r"(bytes) : "memory");
}

// Polls of a wait before it gives up when the launch does not say otherwise (about a second).
constexpr uint32_t kDefaultWaitAttempts = 1u << 24;

// Waits for the phase with the given parity; gives up after `limit` attempts
// and reports it.
__device__ __forceinline__ bool mbarrier_wait(uint32_t barrier, uint32_t parity,
                                              uint32_t limit = kDefaultWaitAttempts) {
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

__device__ __forceinline__ void tma_load_4d(uint32_t smem, const CUtensorMap* map, uint32_t barrier,
                                            int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::"r"(smem),
      "l"(map), "r"(barrier), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Sequences per launch of this kernel (its prefix table lives in shared memory).
constexpr uint32_t kTmaMaxSequences = 1024;

template <bool kFp8, int kD, int kNT>
struct TmaRing {
  using Tile = MmaTile<kFp8, kD>;
  static constexpr int kBoxBytes = Tile::kRowBytes > 128 ? 128 : Tile::kRowBytes;  // swizzle span
  static constexpr int kBoxes = Tile::kRowBytes / kBoxBytes;                       // per tile
  // One 8-head item per warp needs about 170 registers a thread, so three CTAs
  // fit an SM; twelve warps hide the latency of the dependent MMA and softmax
  // steps better than eight. Sixteen heads need about 240 registers: two CTAs.
  static constexpr int kCtasPerSm = kNT == 1 ? (kFp8 ? 4 : 3) : 2;
  static constexpr int kWantedBytes = kNT == 1 ? (kFp8 ? 8 * 1024 : 12 * 1024) : 16 * 1024;
  static constexpr int kRaw = kWantedBytes / Tile::kTileBytes;
  static constexpr int kSlots = kRaw < 3 ? 3 : (kRaw > 9 ? 9 : kRaw);
  static constexpr int kAhead = kSlots - 1;
  static constexpr int kRingBytes = kMmaWarps * kSlots * Tile::kTileBytes;  // 1024-byte aligned pieces
  static constexpr int kMergeBytes = mma_merge_bytes<kNT, kD>();
  static constexpr int kPrefixBytes = (kTmaMaxSequences + 1) * 4;
  static constexpr int kBarrierBytes = kMmaWarps * kSlots * 8;
  static constexpr int kSmemBytes = kRingBytes + kMergeBytes + kPrefixBytes + 4 + kBarrierBytes + 1024;
};

// kOptions: the instantiation that knows the sliding window and the logits soft cap. The plain one
// carries none of their arithmetic: an FP8 cache makes this kernel instruction-bound, and the
// window's tile bookkeeping alone cost it 12 % there.
template <typename QT, bool kFp8, int kD, int kNT, bool kOptions>
__global__ void __launch_bounds__(kMmaThreads, (TmaRing<kFp8, kD, kNT>::kCtasPerSm))
decode_stream_tma_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap key_map,
                         const __grid_constant__ CUtensorMap value_map, const TmaAxes axes) {
  using Tile = MmaTile<kFp8, kD>;
  using Ring = TmaRing<kFp8, kD, kNT>;
  constexpr int kHeads = 8 * kNT;

  extern __shared__ uint8_t raw_smem[];
  // TMA's 128-byte swizzle is a function of the shared address: tiles start on
  // 1024-byte boundaries.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023u) & ~uintptr_t(1023));
  uint8_t* merge_base = smem + Ring::kRingBytes;
  uint32_t* prefix = reinterpret_cast<uint32_t*>(merge_base + Ring::kMergeBytes);  // [sequences + 1]
  uint8_t* barrier_base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(prefix + kTmaMaxSequences + 1) + 7u) & ~uintptr_t(7));
  __shared__ uint32_t warp_totals[kMmaWarps];

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2;
  const uint32_t t = lane & 3u;

  const uint32_t ring_base = smem_address(smem) + warp * (Ring::kSlots * Tile::kTileBytes);
  const uint32_t barriers = smem_address(barrier_base) + warp * (Ring::kSlots * 8);
  if (threadIdx.x == 0) {
    // the two descriptors are fetched while the prologue runs
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&key_map) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&value_map) : "memory");
  }
  if (lane == 0) {
#pragma unroll
    for (int slot = 0; slot < Ring::kSlots; ++slot) mbarrier_init(barriers + slot * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  // Everything up to the first query load reads only lengths and block tables. When the caller
  // vouches that those were written before the preceding kernel started (early_metadata), this
  // prologue runs while that kernel (the step's RoPE + KV write) is still at work.
  if (!p.early_metadata) loom_launch::grid_dependency_wait();

  // ---- units per sequence, exclusive prefix sum -----------------------------
  // The line that is cut into equal shares counts, per work item, its tiles plus kItemSetupUnits
  // empty units in front of them: a boundary between two items costs a CTA about half a tile's
  // time (the warps' states are merged and stored, the next item's queries loaded), and a share
  // that holds a batch's shortest sequences crosses many. A unit below kItemSetupUnits of its item
  // is nothing to copy or compute, like a chunk past the end of a sequence.
  auto item_units = [](uint32_t tiles) -> uint32_t { return tiles ? tiles + kItemSetupUnits : 0u; };
  {
    const uint32_t per_thread = (p.sequences + kMmaThreads - 1) / kMmaThreads;
    const uint32_t begin = min(threadIdx.x * per_thread, p.sequences);
    const uint32_t end = min(begin + per_thread, p.sequences);
    uint32_t local = 0;
    for (uint32_t s = begin; s < end; ++s) {
      const uint32_t length = clamp_length(__ldg(p.sequence_lengths + s), p.max_sequence_length);
      local += item_units(stream_tiles(length, kOptions ? p.sliding_window : 0u));
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
      running += item_units(stream_tiles(length, kOptions ? p.sliding_window : 0u));
    }
    if (threadIdx.x == kMmaThreads - 1) prefix[p.sequences] = running;
    __syncthreads();
  }

  const uint32_t head_chunks = (p.group + kHeads - 1) / kHeads;
  const uint32_t heads = p.kv_heads * head_chunks;  // work items per sequence
  const uint64_t total_tiles = (uint64_t)heads * prefix[p.sequences];
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

  // ---- producer: lane 0 of each warp feeds that warp's ring ------------------
  // All bookkeeping below is incremental (no division or modulo per tile): the
  // instruction stream of the eight..twelve resident warps is what limits this
  // kernel once HBM is kept busy.
  const uint32_t warp_token = warp * 16u;
  // first token of this warp's 16-token chunk of a cursor's tile, and whether the chunk holds a
  // token the query sees
  auto chunk_token = [&](const StreamCursor& c) -> uint32_t {
    if (c.tile < kItemSetupUnits) return 0xffffffffu;  // a setup unit: no token, never live
    const uint32_t tile = c.tile - kItemSetupUnits;
    if constexpr (kOptions) {
      return (stream_first_tile(c.length, p.sliding_window) + tile) * kStreamTileTokens + warp_token;
    } else {
      return tile * kStreamTileTokens + warp_token;
    }
  };
  auto chunk_live = [&](uint32_t token0, const StreamCursor& c) -> bool {
    if constexpr (kOptions) return stream_chunk_live(token0, c.length, p.sliding_window);
    else return token0 < c.length;
  };
  const bool head_inner = axes.head < axes.page;  // NHD-like: the head stride is the smaller one
  StreamCursor producer = start;
  uint32_t producer_block = 0, producer_page = 0, producer_head = 0;
  auto fetch_block = [&]() {
    const uint32_t token0 = chunk_token(producer);
    producer_block = 0;
    producer_page = 0;
    producer_head = head_chunks == 1 ? producer.head : producer.head / head_chunks;
    if (chunk_live(token0, producer)) {
      // block_size is a multiple of 16 on this route, so a 16-token tile never straddles blocks
      const uint32_t logical = p.block_shift < 32u ? token0 >> p.block_shift : token0 / p.block_size;
      producer_page = token0 - logical * p.block_size;
      producer_block = clamp_block(
          __ldg(p.block_tables + (uint64_t)producer.seq * p.max_blocks_per_sequence + logical), p.num_blocks);
    }
  };
  fetch_block();

  // bit s = parity the next use of slot s completes; kAborted = a wait of this warp has expired
  constexpr uint32_t kAborted = 1u << 31;
  uint32_t phases = 0;
  uint32_t issue_left = 2 * my_tiles;  // ring tiles not yet issued (even = K, odd = V of a chunk)
  uint32_t issue_slot = 0;
  bool issue_value = false;
  auto issue_tile = [&]() {
    if (issue_left == 0) return;
    --issue_left;
    const uint32_t token0 = chunk_token(producer);
    if (chunk_live(token0, producer) && lane == 0 && !(phases & kAborted)) {
      const uint32_t destination = ring_base + issue_slot * Tile::kTileBytes;
      const uint32_t barrier = barriers + issue_slot * 8;
      const int32_t c1 = (int32_t)(head_inner ? producer_head : producer_page);
      const int32_t c2 = (int32_t)(head_inner ? producer_page : producer_head);
      // generic-proxy reads of this slot (ldmatrix of its previous tile) come
      // before the async-proxy write that refills it
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      mbarrier_expect_tx(barrier, Tile::kTileBytes + p.wait_unmatched_bytes);
      const CUtensorMap* map = issue_value ? &value_map : &key_map;
#pragma unroll
      for (int box = 0; box < Ring::kBoxes; ++box) {
        tma_load_4d(destination + box * (16 * Ring::kBoxBytes), map, barrier, box * Ring::kBoxBytes, c1, c2,
                    (int32_t)producer_block);
      }
    }
    issue_slot = issue_slot + 1 == (uint32_t)Ring::kSlots ? 0u : issue_slot + 1;
    if (issue_value && issue_left != 0) {
      advance(producer);
      fetch_block();
      // The copy side reaches a new work item one to two tiles before the computing side does:
      // its query rows are pulled into L1 now, so that begin_item finds them there instead of
      // waiting for L2 at every item boundary (one warp per CTA, a 128-byte line per lane).
      if (producer.tile == 0 && warp == 0) {
        constexpr uint32_t kLinesPerRow = (kD * sizeof(QT) + 127) / 128;
        const uint32_t kv_head = producer.head / head_chunks;
        const uint32_t first_head = (producer.head % head_chunks) * kHeads;
        const uint32_t live = min((uint32_t)kHeads, p.group - first_head);
        for (uint32_t line = lane; line < live * kLinesPerRow; line += 32) {
          const QT* row = static_cast<const QT*>(p.query) + (uint64_t)producer.seq * p.q_token +
                          ((uint64_t)kv_head * p.group + first_head + line / kLinesPerRow) * p.q_head;
          asm volatile("prefetch.global.L1 [%0];\n" ::"l"(reinterpret_cast<const char*>(row) +
                                                          (line % kLinesPerRow) * 128));
        }
      }
    }
    issue_value = !issue_value;
  };

  // ---- consumer -----------------------------------------------------------------
  WarpState<kD, kNT> state;
  MergeArea<kD, kNT> area(merge_base);
  StreamCursor consumer = start;
  const uint32_t stride = state_stride(kD);
  uint32_t consume_slot = 0;

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
    // the item's tiles on the line (its setup units lie in front of them)
    const uint64_t item_end = (uint64_t)heads * prefix[item_seq] + (uint64_t)(item_head + 1) * item_tiles;
    const uint64_t item_begin = item_end - (item_tiles - kItemSetupUnits);
    if (range_begin >= item_end || range_end <= item_begin) return;  // only setup units of it are in this share
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

  auto wait_slot = [&](uint32_t slot, uint32_t chunk) {
    if (phases & kAborted) return;
    if (!mbarrier_wait(barriers + slot * 8, (phases >> slot) & 1u, p.wait_attempts)) {
      // First expiry of this warp. The copies issued after this one may still be on their way
      // into this CTA's shared memory: each gets one more bounded wait (a slot whose tile lay
      // beyond the sequence end was never armed and just uses up its polls), then the warp stops.
      atomicCAS(&g_decode_timeout_where, 0u, (1u << 20) | ((chunk & 0x7ffffu) << 1));
      for (uint32_t other = slot + 1 == (uint32_t)Ring::kSlots ? 0u : slot + 1; other != issue_slot;
           other = other + 1 == (uint32_t)Ring::kSlots ? 0u : other + 1) {
        mbarrier_wait(barriers + other * 8, (phases >> other) & 1u, p.wait_attempts);
      }
      phases |= kAborted;
      return;
    }
    phases ^= 1u << slot;
  };

  // From here on the kernel reads what the preceding kernel wrote (the rotated Q, the new token's
  // K and V) and writes its outputs.
  if (p.early_metadata) loom_launch::grid_dependency_wait();

  // The first item's query rows are requested before the first K/V tiles: the
  // memory system answers in order of arrival, and behind the 96 KB of tiles that
  // an SM asks for at once the 2 KB of Q used to arrive 2.5 us after the first K
  // tile, with every warp waiting for it.
  begin_item();
#pragma unroll
  for (int index = 0; index < Ring::kAhead; ++index) issue_tile();

  for (uint32_t chunk = 0; chunk < my_tiles; ++chunk) {
    // refills the slot of the V tile consumed at the end of the previous round
    issue_tile();
    if (chunk != 0 && consumer.tile == 0) {
      finish_item();
      begin_item();
    }
    const uint32_t token0 = chunk_token(consumer);
    const bool has_rows = chunk_live(token0, consumer) && !(phases & kAborted);  // warp-uniform
    const uint32_t live_rows = has_rows ? min(16u, consumer.length - token0) : 0u;
    const uint32_t k_slot = consume_slot;
    const uint32_t v_slot = k_slot + 1 == (uint32_t)Ring::kSlots ? 0u : k_slot + 1;
    consume_slot = v_slot + 1 == (uint32_t)Ring::kSlots ? 0u : v_slot + 1;

    // ---- K tile ------------------------------------------------------------
    uint32_t pb[kNT][2];
    if (has_rows) {
      wait_slot(k_slot, chunk);
      float s[kNT][4];
      chunk_scores<QT, kFp8, kD, kNT, true>(s, state, ring_base + k_slot * Tile::kTileBytes, lane);
      if constexpr (kOptions) {
        const uint32_t visible = window_begin(consumer.length, p.sliding_window);
        chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, live_rows, g, visible > token0 ? visible - token0 : 0u,
                                         p.soft_cap_log2, p.inv_soft_cap_log2);
      } else {
        chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, live_rows, g);
      }
    }
    __syncwarp();
    issue_tile();  // refills the slot of the K tile just consumed

    // ---- V tile ------------------------------------------------------------
    if (has_rows) {
      wait_slot(v_slot, chunk);
      const uint32_t v_tile = ring_base + v_slot * Tile::kTileBytes;
      if (live_rows < 16u) {
        // rows past the end of the sequence hold whatever the page held: clear them
        constexpr uint32_t kPieces = 16 * Tile::kSegs;
        for (uint32_t piece = lane; piece < kPieces; piece += 32) {
          const uint32_t row = piece / Tile::kSegs;
          if (row >= live_rows) {
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(
                             v_tile + tile_offset<Tile::kSegs, true>(row, piece % Tile::kSegs)),
                         "r"(0u)
                         : "memory");
          }
        }
        __syncwarp();
      }
      chunk_values<QT, kFp8, kD, kNT, true>(state, pb, v_tile, lane);
    }
    __syncwarp();
    if (chunk + 1 < my_tiles) advance(consumer);
  }
  finish_item();
}

}  // namespace loom_decode
