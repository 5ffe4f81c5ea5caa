// Balanced persistent paged decode kernel with a copy-issuing warp (FP8 caches).
//
// Same schedule, tiles, arithmetic and workspace protocol as decode_stream_tma.cuh
// (an even share of the batch's tiles per resident CTA, warp-private K/V rings
// filled by TMA, one state per work item and CTA, merge_stream_kernel after it),
// with the roles split: seven warps only compute, an eighth only issues copies.
//
// Why. Over an FP8 cache the decode is bound by its instruction stream, not by
// HBM (E4M3 -> F16 conversion in registers; issue slots 57 % busy at 0.83 of the
// copy bandwidth). In the unsplit kernel every warp walks the producer side of
// its own ring - a second cursor over the line of tiles, the block-table
// look-up, slot and barrier bookkeeping, the copy itself - although one lane
// issues: about a quarter of the 460 instructions a warp spends on a 16-token
// chunk. Here lane r of the eighth warp does that for the ring of warp r, so the
// bookkeeping is executed once per tile of the CTA instead of once per warp and
// tile, and the computing warps shed it (and the registers it held).
//
// Hand-off. Per ring slot a `full` barrier (armed by the producer lane with the
// tile's bytes, completed by the copy) and an `empty` barrier (one arrival by
// the computing warp when it has read the tile). The producer lane waits for
// `empty` before it refills a slot; a fresh barrier passes that wait (parity
// trick), so the first lap needs no special case. Tiles of a chunk that lies
// wholly past the end of its sequence are neither copied nor waited for; both
// sides skip their slots.
//
// 256 threads at up to 128 registers, two CTAs per SM (14 computing warps per
// SM), 112-token tiles (7 warps x 16 tokens), five 2 KB slots per ring.
//
// Software pipelining inside a computing warp: the value product of a chunk is
// not issued after its softmax but together with the score product of the
// warp's next chunk (chunk_scores_and_values), the two being independent. The
// conversions of one then hide the tensor-core latency of the other; a warp
// holds the V slot of one chunk and the K slot of the next at the same time,
// which the ring order (K, V, K, V ...) allows without a deeper ring. At the
// end of a work item and of the CTA's range the deferred product runs alone.
//
// Every wait is bounded (the limit is a launch parameter). A computing warp
// whose wait expires sets the device flag and the CTA's abort word and stops
// waiting and computing; the producer then issues nothing more, the other
// computing warps stop at the expiry of their own next wait, and the CTA walks
// to its end (a pause at the end lets copies already in flight land).
#pragma once

#include "decode_stream_tma.cuh"

namespace loom_decode {

__device__ __forceinline__ void mbarrier_release(uint32_t barrier) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(barrier) : "memory");
}


// QK^T of one chunk and P.V of the chunk before it in one instruction stream (FP8 cache): the two
// products are independent of each other (the probabilities of the earlier chunk are already in
// `pb`), so the conversions of one hide the tensor-core latency of the other. Same arithmetic as
// chunk_scores followed by chunk_values.
template <typename QT, int kD>
__device__ __forceinline__ void chunk_scores_and_values(float (&s)[1][4], WarpState<kD, 1>& state, uint32_t k_tile,
                                                        const uint32_t (&pb)[1][2], uint32_t v_tile,
                                                        uint32_t lane) {
  using Tile = MmaTile<true, kD>;
  constexpr int kKSteps = kD / 16;
  const uint32_t ld_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u;
  const uint32_t ld_col = lane >> 4;
  s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.0f;
#pragma unroll
  for (int pair = 0; pair < kKSteps / 2; ++pair) {
    uint32_t rk[4], rv[4];
    ldmatrix_x4(rk, k_tile + tile_offset<Tile::kSegs, true>(ld_row, 2 * pair + ld_col));
    ldmatrix_x4_trans(rv, v_tile + tile_offset<Tile::kSegs, true>(ld_row, 2 * pair + ld_col));
    uint32_t a[4], b[4];
    e4m3x4_to_f16x2x2(rk[0], a[0], a[2]);
    e4m3x4_to_f16x2x2(rk[1], a[1], a[3]);
    e4m3x4_to_f16x2x2(__byte_perm(rv[0], 0u, 0x3120u), b[0], b[1]);
    e4m3x4_to_f16x2x2(__byte_perm(rv[1], 0u, 0x3120u), b[2], b[3]);
    mma_16816_f16(s[0], a, state.qf[0][2 * pair][0], state.qf[0][2 * pair][1]);
    mma_16816_f16(state.o[0][2 * pair], b, pb[0][0], pb[0][1]);
    e4m3x4_to_f16x2x2(rk[2], a[0], a[2]);
    e4m3x4_to_f16x2x2(rk[3], a[1], a[3]);
    e4m3x4_to_f16x2x2(__byte_perm(rv[2], 0u, 0x3120u), b[0], b[1]);
    e4m3x4_to_f16x2x2(__byte_perm(rv[3], 0u, 0x3120u), b[2], b[3]);
    mma_16816_f16(s[0], a, state.qf[0][2 * pair + 1][0], state.qf[0][2 * pair + 1][1]);
    mma_16816_f16(state.o[0][2 * pair + 1], b, pb[0][0], pb[0][1]);
  }
}

template <bool kFp8, int kD>
struct SplitRing {
  using Tile = MmaTile<kFp8, kD>;
  static constexpr int kConsumers = 7;
  static constexpr int kThreads = (kConsumers + 1) * 32;
  static constexpr int kComputeThreads = kConsumers * 32;
  static constexpr int kTileTokens = 16 * kConsumers;
  static constexpr int kCtasPerSm = 2;
  static constexpr int kBoxBytes = Tile::kRowBytes > 128 ? 128 : Tile::kRowBytes;
  static constexpr int kBoxes = Tile::kRowBytes / kBoxBytes;
  static constexpr int kSlots = (10 * 1024) / Tile::kTileBytes < 3 ? 3 : (10 * 1024) / Tile::kTileBytes;
  static constexpr int kRingBytes = kConsumers * kSlots * Tile::kTileBytes;  // 1024-byte aligned pieces
  static constexpr int kMergeBytes = mma_merge_bytes<1, kD, kConsumers>();
  static constexpr int kPrefixBytes = (kTmaMaxSequences + 1) * 4;
  static constexpr int kBarrierBytes = 2 * kConsumers * kSlots * 8;
  static constexpr int kSmemBytes = kRingBytes + kMergeBytes + kPrefixBytes + 8 + kBarrierBytes + 1024;
  static_assert(kSlots <= 16, "slot phases are kept in 16-bit halves of one register");
};

template <typename QT, bool kFp8, int kD>
__global__ void __launch_bounds__((SplitRing<kFp8, kD>::kThreads), (SplitRing<kFp8, kD>::kCtasPerSm))
decode_stream_split_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap key_map,
                           const __grid_constant__ CUtensorMap value_map, const TmaAxes axes) {
  using Tile = MmaTile<kFp8, kD>;
  using Ring = SplitRing<kFp8, kD>;
  constexpr int kNT = 1;
  constexpr int kHeads = 8;
  constexpr int kC = Ring::kConsumers;
  constexpr uint32_t kTileTokens = Ring::kTileTokens;

  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023u) & ~uintptr_t(1023));
  uint8_t* merge_base = smem + Ring::kRingBytes;
  uint32_t* prefix = reinterpret_cast<uint32_t*>(merge_base + Ring::kMergeBytes);  // [sequences + 1]
  uint8_t* barrier_base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(prefix + kTmaMaxSequences + 1) + 7u) & ~uintptr_t(7));
  __shared__ uint32_t warp_totals[kC + 1];
  __shared__ uint32_t cta_aborted;  // a wait of some warp of this CTA has expired

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2;
  const uint32_t t = lane & 3u;
  const bool producer_warp = warp == (uint32_t)kC;

  // barriers: full[ring][slot], then empty[ring][slot]
  const uint32_t full_base = smem_address(barrier_base);
  const uint32_t empty_base = full_base + kC * Ring::kSlots * 8;
  if (threadIdx.x == 0) {
    cta_aborted = 0;
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&key_map) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&value_map) : "memory");
  }
  if (!producer_warp && lane == 0) {
#pragma unroll
    for (int slot = 0; slot < Ring::kSlots; ++slot) {
      mbarrier_init(full_base + (warp * Ring::kSlots + slot) * 8, 1);
      mbarrier_init(empty_base + (warp * Ring::kSlots + slot) * 8, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  // Up to the first query load only lengths and block tables are read; with the caller's promise
  // that those are older than the preceding kernel this prologue overlaps that kernel.
  if (!p.early_metadata) loom_launch::grid_dependency_wait();

  // ---- tiles per sequence, exclusive prefix sum (all eight warps) ----------------------------
  {
    const uint32_t per_thread = (p.sequences + Ring::kThreads - 1) / Ring::kThreads;
    const uint32_t begin = min(threadIdx.x * per_thread, p.sequences);
    const uint32_t end = min(begin + per_thread, p.sequences);
    uint32_t local = 0;
    for (uint32_t s = begin; s < end; ++s) {
      const uint32_t length = clamp_length(__ldg(p.sequence_lengths + s), p.max_sequence_length);
      local += (length + kTileTokens - 1) / kTileTokens;
    }
    uint32_t inclusive = local;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if (lane >= (uint32_t)offset) inclusive += other;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();  // also: the barriers are initialised before the producer touches one
    uint32_t running = inclusive - local;
    for (uint32_t w = 0; w < warp; ++w) running += warp_totals[w];
    for (uint32_t s = begin; s < end; ++s) {
      prefix[s] = running;
      const uint32_t length = clamp_length(__ldg(p.sequence_lengths + s), p.max_sequence_length);
      running += (length + kTileTokens - 1) / kTileTokens;
    }
    if (threadIdx.x == Ring::kThreads - 1) prefix[p.sequences] = running;
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

  volatile uint32_t* aborted = &cta_aborted;

  // ================================ the copy-issuing warp ======================================
  if (producer_warp) {
    // The new token's K and V are written by the kernel before this one: no copy before it is done.
    if (p.early_metadata) loom_launch::grid_dependency_wait();
    if (lane < (uint32_t)kC) {
      const uint32_t ring = smem_address(smem) + lane * (Ring::kSlots * Tile::kTileBytes);
      const uint32_t full = full_base + lane * (Ring::kSlots * 8);
      const uint32_t empty = empty_base + lane * (Ring::kSlots * 8);
      const bool head_inner = axes.head < axes.page;  // NHD-like: the head stride is the smaller one
      StreamCursor cursor = start;
      uint32_t slot = 0;
      uint32_t empty_parity = 0xffffu;  // bit s: parity to wait for on empty[s]; a fresh barrier passes parity 1
      for (uint32_t tile = 0; tile < my_tiles; ++tile) {
        if (*aborted) break;
        const uint32_t token0 = cursor.tile * kTileTokens + lane * 16u;
        if (token0 < cursor.length) {
          // block_size is a multiple of 16 on this route, so a 16-token tile never straddles blocks
          const uint32_t logical = p.block_shift < 32u ? token0 >> p.block_shift : token0 / p.block_size;
          const int32_t page = (int32_t)(token0 - logical * p.block_size);
          const int32_t block = (int32_t)clamp_block(
              __ldg(p.block_tables + (uint64_t)cursor.seq * p.max_blocks_per_sequence + logical), p.num_blocks);
          const int32_t head = (int32_t)(head_chunks == 1 ? cursor.head : cursor.head / head_chunks);
          const int32_t c1 = head_inner ? head : page;
          const int32_t c2 = head_inner ? page : head;
#pragma unroll
          for (int kind = 0; kind < 2; ++kind) {
            if (!mbarrier_wait(empty + slot * 8, (empty_parity >> slot) & 1u, p.wait_attempts)) {
              atomicCAS(&g_decode_timeout_where, 0u, (2u << 20) | ((tile & 0x7ffffu) << 1));
              *aborted = 1;
              break;
            }
            empty_parity ^= 1u << slot;
            // the computing warp's reads of the slot (generic proxy) precede this write (async proxy)
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            mbarrier_expect_tx(full + slot * 8, Tile::kTileBytes + p.wait_unmatched_bytes);
            const CUtensorMap* map = kind ? &value_map : &key_map;
#pragma unroll
            for (int box = 0; box < Ring::kBoxes; ++box) {
              tma_load_4d(ring + slot * Tile::kTileBytes + box * (16 * Ring::kBoxBytes), map, full + slot * 8,
                          box * Ring::kBoxBytes, c1, c2, block);
            }
            slot = slot + 1 == (uint32_t)Ring::kSlots ? 0u : slot + 1;
          }
        } else {
          slot = slot + 2 >= (uint32_t)Ring::kSlots ? slot + 2 - Ring::kSlots : slot + 2;
        }
        if (tile + 1 < my_tiles) {
          advance(cursor);
          // a new work item starts with the next tile: its query rows go to L1 now, two to three tiles
          // before the computing warps ask for them (a 128-byte line per lane and pass)
          if (cursor.tile == 0) {
            constexpr uint32_t kLinesPerRow = (kD * sizeof(QT) + 127) / 128;
            const uint32_t kv_head = cursor.head / head_chunks;
            const uint32_t first_head = (cursor.head % head_chunks) * kHeads;
            const uint32_t live = min((uint32_t)kHeads, p.group - first_head);
            for (uint32_t line = lane; line < live * kLinesPerRow; line += (uint32_t)kC) {
              const QT* row = static_cast<const QT*>(p.query) + (uint64_t)cursor.seq * p.q_token +
                              ((uint64_t)kv_head * p.group + first_head + line / kLinesPerRow) * p.q_head;
              asm volatile("prefetch.global.L1 [%0];\n" ::"l"(reinterpret_cast<const char*>(row) +
                                                              (line % kLinesPerRow) * 128));
            }
          }
        }
      }
    }
    return;
  }

  // ================================ the computing warps ========================================
  const uint32_t ring_base = smem_address(smem) + warp * (Ring::kSlots * Tile::kTileBytes);
  const uint32_t full = full_base + warp * (Ring::kSlots * 8);
  const uint32_t empty = empty_base + warp * (Ring::kSlots * 8);
  auto compute_barrier = [] {
    asm volatile("bar.sync 1, %0;\n" ::"n"(Ring::kComputeThreads) : "memory");
  };

  WarpState<kD, kNT> state;
  MergeArea<kD, kNT, kC> area(merge_base);
  StreamCursor consumer = start;
  const uint32_t stride = state_stride(kD);
  constexpr uint32_t kAborted = 1u << 31;
  uint32_t phases = 0;  // bit s = parity the next use of full[s] completes; kAborted = this warp has stopped
  uint32_t consume_slot = 0;
  const uint32_t warp_token = warp * 16u;

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
    compute_barrier();  // the merge area may still be read by the previous item's store
    park_warp_state<kFp8, kD, kNT, kC>(area, state, warp, g, t);
    compute_barrier();
    float value_scale = 1.0f;
    if constexpr (kFp8) value_scale = __ldg(p.value_scales + (uint64_t)kv_head * p.scale_stride);
    const uint64_t query_row = (uint64_t)item_seq * p.query_heads + (uint64_t)kv_head * p.group + first_head;
    if (parts == 1 && !p.emit_state) {
      combine_and_store<QT, kD, kNT, kC>(area, live_heads, value_scale,
                                         static_cast<QT*>(p.output) + query_row * kD, kD, nullptr, 0);
    } else if (parts == 1) {
      combine_and_store<QT, kD, kNT, kC>(area, live_heads, value_scale, nullptr, 0,
                                         static_cast<float*>(p.output) + query_row * stride, stride);
    } else {
      combine_and_store<QT, kD, kNT, kC>(area, live_heads, value_scale, nullptr, 0,
                                         p.partials + (item + blockIdx.x) * kHeads * stride, stride);
    }
    if (threadIdx.x == 0 && blockIdx.x == first_cta) {
      p.item_meta[2 * item] = first_cta;
      p.item_meta[2 * item + 1] = parts;
    }
  };

  auto wait_slot = [&](uint32_t slot, uint32_t chunk) {
    if (phases & kAborted) return;
    // (the CTA's abort word is not polled here: a warp whose copies stop coming because another
    // warp's wait expired finds out through the expiry of its own next wait, which is bounded too)
    if (!mbarrier_wait(full + slot * 8, (phases >> slot) & 1u, p.wait_attempts)) {
      atomicCAS(&g_decode_timeout_where, 0u, (1u << 20) | ((chunk & 0x7ffffu) << 1));
      *aborted = 1;
      phases |= kAborted;
      return;
    }
    phases ^= 1u << slot;
  };
  // hands a tile's slot back to the copy-issuing warp once the whole warp has read it
  auto release_slot = [&](uint32_t slot) {
    __syncwarp();
    if (lane == 0) mbarrier_release(empty + slot * 8);
  };

  // From here on the kernel reads what the preceding kernel wrote (the rotated Q) and writes outputs.
  if (p.early_metadata) loom_launch::grid_dependency_wait();
  begin_item();

  static_assert(kFp8 && !kFp8KeyByAlu, "the merged product is written for the converted FP8 path");
  // The value product of a chunk is deferred to the next chunk's score product, so that the two run
  // as one instruction stream; `pending` says that `pb` holds probabilities whose V tile (slot
  // pending_v, pending_rows live rows) has not been used yet.
  uint32_t pb[kNT][2];
  bool pending = false;
  uint32_t pending_v = 0, pending_rows = 0;
  auto clear_dead_rows = [&](uint32_t v_tile, uint32_t live_rows) {
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
  };
  // the deferred value product on its own (end of an item, end of the range)
  auto flush_pending = [&](uint32_t chunk) {
    if (!pending) return;
    pending = false;
    wait_slot(pending_v, chunk);
    if (!(phases & kAborted)) {
      const uint32_t v_tile = ring_base + pending_v * Tile::kTileBytes;
      if (pending_rows < 16u) clear_dead_rows(v_tile, pending_rows);
      chunk_values<QT, kFp8, kD, kNT, true>(state, pb, v_tile, lane);
    }
    release_slot(pending_v);
  };

  for (uint32_t chunk = 0; chunk < my_tiles;) {
    if (chunk != 0 && consumer.tile == 0) {
      flush_pending(chunk);
      finish_item();
      begin_item();
    }
    // A run of plain tiles - same work item, inside this CTA's range, this warp's 16 tokens all
    // inside the sequence, a value product pending - goes through a loop that carries none of the
    // general case's tests (about a seventh fewer instructions per chunk).
    if (pending && !(phases & kAborted)) {
      const uint32_t full_tiles =
          consumer.length >= warp_token + 16u ? (consumer.length - warp_token - 16u) / kTileTokens + 1u : 0u;
      const uint32_t item_end = min(full_tiles, consumer.tiles);
      const uint32_t run = min(item_end > consumer.tile ? item_end - consumer.tile : 0u, my_tiles - chunk);
      if (run > 1u) {
        uint32_t done = 0;
        for (; done < run; ++done) {
          const uint32_t k_slot = consume_slot;
          const uint32_t v_slot = k_slot + 1 == (uint32_t)Ring::kSlots ? 0u : k_slot + 1;
          wait_slot(k_slot, chunk + done);
          wait_slot(pending_v, chunk + done);
          if (phases & kAborted) break;  // the general path below walks on without waiting or computing
          float s[kNT][4];
          chunk_scores_and_values<QT, kD>(s, state, ring_base + k_slot * Tile::kTileBytes, pb,
                                          ring_base + pending_v * Tile::kTileBytes, lane);
          __syncwarp();
          if (lane == 0) {
            mbarrier_release(empty + pending_v * 8);
            mbarrier_release(empty + k_slot * 8);
          }
          chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, 16u, g);
          pending_v = v_slot;
          consume_slot = v_slot + 1 == (uint32_t)Ring::kSlots ? 0u : v_slot + 1;
        }
        if (done != 0u) {
          pending_rows = 16u;
          chunk += done;
          consumer.tile += done - 1u;
          if (chunk < my_tiles) advance(consumer);
          continue;
        }
      }
    }
    const uint32_t token0 = consumer.tile * kTileTokens + warp_token;
    const bool in_sequence = token0 < consumer.length;  // warp-uniform; the copy side uses the same test
    const uint32_t live_rows = in_sequence ? min(16u, consumer.length - token0) : 0u;
    const uint32_t k_slot = consume_slot;
    const uint32_t v_slot = k_slot + 1 == (uint32_t)Ring::kSlots ? 0u : k_slot + 1;
    consume_slot = v_slot + 1 == (uint32_t)Ring::kSlots ? 0u : v_slot + 1;

    if (in_sequence) {
      wait_slot(k_slot, chunk);
      float s[kNT][4];
      if (pending) {
        wait_slot(pending_v, chunk);
        if (!(phases & kAborted)) {
          const uint32_t v_tile = ring_base + pending_v * Tile::kTileBytes;
          if (pending_rows < 16u) clear_dead_rows(v_tile, pending_rows);
          chunk_scores_and_values<QT, kD>(s, state, ring_base + k_slot * Tile::kTileBytes, pb, v_tile, lane);
        }
        __syncwarp();
        if (lane == 0) {
          mbarrier_release(empty + pending_v * 8);
          mbarrier_release(empty + k_slot * 8);
        }
      } else {
        if (!(phases & kAborted)) {
          chunk_scores<QT, kFp8, kD, kNT, true>(s, state, ring_base + k_slot * Tile::kTileBytes, lane);
        }
        release_slot(k_slot);
      }
      if (!(phases & kAborted)) chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, live_rows, g);
      pending = !(phases & kAborted);
      pending_v = v_slot;
      pending_rows = live_rows;
      if (!pending) release_slot(v_slot);
    }
    if (chunk + 1 < my_tiles) advance(consumer);
    ++chunk;
  }
  flush_pending(my_tiles);
  finish_item();
  if (*aborted) {
    // copies issued before the expiry may still be on their way into this CTA's shared memory
    for (int pause = 0; pause < 64; ++pause) __nanosleep(1000);
  }
}

}  // namespace loom_decode
