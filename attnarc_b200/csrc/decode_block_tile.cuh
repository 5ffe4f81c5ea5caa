// Balanced persistent paged decode kernel whose CTA tile is one 16-token block of eight KV heads
// (FP8 caches, head size 128, up to 8 query heads per KV head, KV heads a multiple of 8).
//
// Why. In decode_stream_split.cuh a CTA streams 112 tokens of ONE KV head per tile: seven copies
// of 16 rows of 128 bytes for K and seven for V. In an NHD cache those rows lie 1 KB apart (the
// other seven heads of the token in between), and the heads of a block are read by different CTAs
// at different times, so DRAM sees 128-byte pieces (4-5 % slower than the same bytes in an HND
// cache), and one warp waits for seven rings and issues fourteen copies per tile, which bounds the
// feed (a second copy-issuing warp at equal computing warps: 436 against 447 us on the
// Llama-3-70B-shaped workload).
//
// Here warp w of eight computing warps owns KV head 8 * group + w of the sequence, and all eight
// walk the same 16 tokens at a time. A tile's K (and V) is then ONE copy: the tensor map lists the
// cache as (row bytes, page, head, block) - strides need not be sorted - so a box of
// [128 bytes, 16 pages, 8 heads, 1 block] lands in shared memory as eight per-head tiles of
// [16 rows x 128 bytes], each swizzled exactly as the per-warp tiles of the other kernels, while
// global memory sees the block's 16 KB as one request (contiguous in an NHD cache). Two copies per
// 32 KB instead of fourteen per 28 KB, one `full` barrier per stage for the whole CTA, one `empty`
// barrier with eight arrivals.
//
// No warp ever needs another warp's state: a work item is (sequence, KV head) and belongs to one
// warp, so the end of an item is a few stores by that warp - no shared merge area, no CTA barrier
// after the prologue. Every wait is bounded as in the other kernels.
//
// Workspace protocol: as decode_stream_tma.cuh, except that the state of (sequence s, KV head
// 8 q + w) written by CTA c lives in slot 8 * (s * Q + q + c) + w (Q = KV heads / 8), because the
// eight items of a tile advance together (s * Q + q and c both only grow along the line of tiles, so
// the sum is unique); merge_stream_kernel is told so by its `heads_together` argument.
#pragma once

#include "decode_stream_split.cuh"

namespace loom_decode {

template <int kD>
struct BlockRing {
  using Tile = MmaTile<true, kD>;
  static constexpr int kWarps = 8;                   // computing warps = KV heads per tile
  static constexpr int kThreads = (kWarps + 1) * 32;
  static constexpr int kCtasPerSm = 2;
  static constexpr int kStageBytes = kWarps * Tile::kTileBytes;  // K or V of one tile: 16 KB
  static constexpr int kStages = 6;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kPrefixBytes = (kTmaMaxSequences + 1) * 4;
  static constexpr int kBarrierBytes = 2 * kStages * 8;
  static constexpr int kSmemBytes = kRingBytes + kPrefixBytes + 8 + kBarrierBytes + 1024;
  static_assert(kD == 128, "one 128-byte box per row");
  static_assert(kCtasPerSm * (kSmemBytes + 2048) <= 228 * 1024, "two CTAs per SM");
};

template <typename QT, int kD>
__global__ void __launch_bounds__((BlockRing<kD>::kThreads), (BlockRing<kD>::kCtasPerSm))
decode_block_tile_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap key_map,
                         const __grid_constant__ CUtensorMap value_map) {
  using Tile = MmaTile<true, kD>;
  using Ring = BlockRing<kD>;
  constexpr int kNT = 1;
  constexpr bool kFp8 = true;
  constexpr int kW = Ring::kWarps;
  constexpr uint32_t kTileTokens = 16;
  constexpr int kKSteps = kD / 16;
  static_assert(!kFp8KeyByAlu, "the merged product is written for the converted FP8 path");

  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023u) & ~uintptr_t(1023));
  uint32_t* prefix = reinterpret_cast<uint32_t*>(smem + Ring::kRingBytes);  // [sequences + 1]
  uint8_t* barrier_base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(prefix + kTmaMaxSequences + 1) + 7u) & ~uintptr_t(7));
  __shared__ uint32_t warp_totals[kW + 1];
  __shared__ uint32_t cta_aborted;  // a wait of some warp of this CTA has expired

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2;
  const uint32_t t = lane & 3u;
  const bool producer_warp = warp == (uint32_t)kW;

  // barriers: full[stage] (bytes of the copy), then empty[stage] (one arrival per computing warp)
  const uint32_t full = smem_address(barrier_base);
  const uint32_t empty = full + Ring::kStages * 8;
  if (threadIdx.x == 0) {
    cta_aborted = 0;
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&key_map) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&value_map) : "memory");
#pragma unroll
    for (int stage = 0; stage < Ring::kStages; ++stage) {
      mbarrier_init(full + stage * 8, 1);
      mbarrier_init(empty + stage * 8, kW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  // Up to the first query load only lengths and block tables are read; with the caller's promise
  // that those are older than the preceding kernel this prologue overlaps that kernel.
  if (!p.early_metadata) loom_launch::grid_dependency_wait();

  // ---- tiles per sequence (16 tokens each), exclusive prefix sum (all nine warps) -------------
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
    __syncthreads();  // also: the barriers are initialised before anyone touches one
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

  const uint32_t groups = p.kv_heads / kW;  // work items (of eight KV heads) per sequence
  const uint64_t total_tiles = (uint64_t)groups * prefix[p.sequences];
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
    if (++c.head < groups) return;
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
      if ((uint64_t)groups * prefix[middle] <= range_begin) low = middle;
      else high = middle;
    }
    start.seq = low;
    load_sequence(start);
    const uint64_t inside = range_begin - (uint64_t)groups * prefix[low];
    start.head = (uint32_t)(inside / start.tiles);
    start.tile = (uint32_t)(inside % start.tiles);
  }

  volatile uint32_t* aborted = &cta_aborted;
  const uint32_t ring = smem_address(smem);

  // ================================ the copy-issuing warp ======================================
  if (producer_warp) {
    // The new token's K and V are written by the kernel before this one: no copy before it is done.
    if (p.early_metadata) loom_launch::grid_dependency_wait();
    if (lane == 0) {
      StreamCursor ahead = start;
      auto lookup = [&](const StreamCursor& c) -> int32_t {
        const uint32_t token0 = c.tile * kTileTokens;
        const uint32_t logical = p.block_shift < 32u ? token0 >> p.block_shift : token0 / p.block_size;
        return (int32_t)clamp_block(
            __ldg(p.block_tables + (uint64_t)c.seq * p.max_blocks_per_sequence + logical), p.num_blocks);
      };
      int32_t ahead_block = lookup(ahead);  // a tile's block id is looked up one tile early
      uint32_t stage = 0;
      uint32_t empty_parity = 0xffffu;  // bit s: parity to wait for on empty[s]; a fresh barrier passes parity 1
      for (uint32_t tile = 0; tile < my_tiles; ++tile) {
        if (*aborted) break;
        const StreamCursor cursor = ahead;
        const int32_t block = ahead_block;
        if (tile + 1 < my_tiles) {
          advance(ahead);
          ahead_block = lookup(ahead);
        }
        // block_size is a multiple of 16 on this route, so a tile never straddles blocks
        const uint32_t token0 = cursor.tile * kTileTokens;
        const uint32_t logical = p.block_shift < 32u ? token0 >> p.block_shift : token0 / p.block_size;
        const int32_t page = (int32_t)(token0 - logical * p.block_size);
        const int32_t head = (int32_t)(cursor.head * kW);
        bool stop = false;
#pragma unroll
        for (int kind = 0; kind < 2; ++kind) {
          if (!mbarrier_wait(empty + stage * 8, (empty_parity >> stage) & 1u, p.wait_attempts)) {
            atomicCAS(&g_decode_timeout_where, 0u, (2u << 20) | ((tile & 0x7ffffu) << 1));
            *aborted = 1;
            stop = true;
            break;
          }
          empty_parity ^= 1u << stage;
          // the computing warps' reads of the stage (generic proxy) precede this write (async proxy)
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          mbarrier_expect_tx(full + stage * 8, Ring::kStageBytes + p.wait_unmatched_bytes);
          tma_load_4d(ring + stage * Ring::kStageBytes, kind ? &value_map : &key_map, full + stage * 8, 0, page,
                      head, block);
          stage = stage + 1 == (uint32_t)Ring::kStages ? 0u : stage + 1;
        }
        if (stop) break;
      }
    }
    return;
  }

  // ================================ the computing warps ========================================
  // warp w: KV head 8 * group + w; its tile inside a stage starts w * 2 KB in
  const uint32_t my_tile = ring + warp * Tile::kTileBytes;
  WarpState<kD, kNT> state;
  StreamCursor consumer = start;
  const uint32_t stride = state_stride(kD);
  constexpr uint32_t kAborted = 1u << 31;
  uint32_t phases = 0;  // bit s = parity the next use of full[s] completes; kAborted = this warp has stopped
  uint32_t consume_stage = 0;
  auto next_stage = [](uint32_t stage) { return stage + 1 == (uint32_t)Ring::kStages ? 0u : stage + 1; };

  uint32_t item_seq = 0, item_group = 0, item_tiles = 0;
  float value_scale = 1.0f;

  auto begin_item = [&]() {
    item_seq = consumer.seq;
    item_group = consumer.head;
    item_tiles = consumer.tiles;
    const uint32_t kv_head = item_group * kW + warp;
    const uint32_t live_heads = min(8u, p.group);
    state.reset();
    const float score_scale = p.scale_log2 * __ldg(p.key_scales + (uint64_t)kv_head * p.scale_stride);
    value_scale = __ldg(p.value_scales + (uint64_t)kv_head * p.scale_stride);
    load_query<QT, kFp8, kD, kNT>(
        state,
        static_cast<const QT*>(p.query) + (uint64_t)item_seq * p.q_token + (uint64_t)kv_head * p.group * p.q_head,
        p.q_head, live_heads, score_scale, g, t);
  };

  // Stores this warp's state of its work item: the final rows if this CTA covered the item, else a
  // partial state for the merge kernel. Lane (g, t) holds heads 2t, 2t+1 and value dims 16 mt + 2g, + 1.
  auto finish_item = [&]() {
    const uint32_t kv_head = item_group * kW + warp;
    const uint32_t live_heads = min(8u, p.group);
    const uint64_t super_item = (uint64_t)item_seq * groups + item_group;
    const uint64_t item_begin = (uint64_t)groups * prefix[item_seq] + (uint64_t)item_group * item_tiles;
    const uint32_t first_cta = cta_of(item_begin);
    const uint32_t last_cta = cta_of(item_begin + item_tiles - 1);
    const uint32_t parts = last_cta - first_cta + 1;
#pragma unroll
    for (int offset = 4; offset < 32; offset <<= 1) {
      state.row_sum[0][0] += __shfl_xor_sync(0xffffffffu, state.row_sum[0][0], offset);
      state.row_sum[0][1] += __shfl_xor_sync(0xffffffffu, state.row_sum[0][1], offset);
    }
    const uint64_t query_row = (uint64_t)item_seq * p.query_heads + (uint64_t)kv_head * p.group;
    const uint32_t head0 = 2 * t;
    if (parts == 1 && !p.emit_state) {
      const float inv0 = state.row_sum[0][0] > 0.0f ? value_scale / state.row_sum[0][0] : 0.0f;
      const float inv1 = state.row_sum[0][1] > 0.0f ? value_scale / state.row_sum[0][1] : 0.0f;
      QT* out0 = static_cast<QT*>(p.output) + (query_row + head0) * kD + 2 * g;
      QT* out1 = out0 + kD;
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt) {
        uint32_t pair0, pair1;
        if constexpr (std::is_same<QT, __nv_bfloat16>::value) {
          pair0 = pack_bf16x2(state.o[0][mt][0] * inv0, state.o[0][mt][2] * inv0);
          pair1 = pack_bf16x2(state.o[0][mt][1] * inv1, state.o[0][mt][3] * inv1);
        } else {
          pair0 = pack_f16x2(state.o[0][mt][0] * inv0, state.o[0][mt][2] * inv0);
          pair1 = pack_f16x2(state.o[0][mt][1] * inv1, state.o[0][mt][3] * inv1);
        }
        if (head0 < live_heads) *reinterpret_cast<uint32_t*>(out0 + mt * 16) = pair0;
        if (head0 + 1 < live_heads) *reinterpret_cast<uint32_t*>(out1 + mt * 16) = pair1;
      }
    } else {
      float* rows = parts == 1 ? static_cast<float*>(p.output) + query_row * stride
                               : p.partials + (((super_item + blockIdx.x) * kW + warp) * 8) * stride;
      float* row0 = rows + (uint64_t)head0 * stride;
      float* row1 = row0 + stride;
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt) {
        if (head0 < live_heads) {
          *reinterpret_cast<float2*>(row0 + mt * 16 + 2 * g) =
              make_float2(state.o[0][mt][0] * value_scale, state.o[0][mt][2] * value_scale);
        }
        if (head0 + 1 < live_heads) {
          *reinterpret_cast<float2*>(row1 + mt * 16 + 2 * g) =
              make_float2(state.o[0][mt][1] * value_scale, state.o[0][mt][3] * value_scale);
        }
      }
      if (g == 0) {
        if (head0 < live_heads) {
          row0[kD] = state.row_max[0][0] * kLn2;
          row0[kD + 1] = state.row_sum[0][0];
        }
        if (head0 + 1 < live_heads) {
          row1[kD] = state.row_max[0][1] * kLn2;
          row1[kD + 1] = state.row_sum[0][1];
        }
      }
    }
    if (lane == 0 && blockIdx.x == first_cta) {
      const uint64_t item = super_item * kW + warp;
      p.item_meta[2 * item] = first_cta;
      p.item_meta[2 * item + 1] = parts;
    }
  };

  auto wait_stage = [&](uint32_t stage, uint32_t chunk) {
    if (phases & kAborted) return;
    if (!mbarrier_wait(full + stage * 8, (phases >> stage) & 1u, p.wait_attempts)) {
      atomicCAS(&g_decode_timeout_where, 0u, (1u << 20) | ((chunk & 0x7ffffu) << 1));
      *aborted = 1;
      phases |= kAborted;
      return;
    }
    phases ^= 1u << stage;
  };
  // hands this warp's part of a stage back to the copy-issuing warp once the whole warp has read it
  auto release_stage = [&](uint32_t stage) {
    __syncwarp();
    if (lane == 0) mbarrier_release(empty + stage * 8);
  };
  auto clear_dead_rows = [&](uint32_t v_tile, uint32_t live_rows) {
    // rows past the end of the sequence hold whatever the page held: clear them (this warp's tile only)
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

  // From here on the kernel reads what the preceding kernel wrote (the rotated Q) and writes outputs.
  if (p.early_metadata) loom_launch::grid_dependency_wait();
  begin_item();

  // The value product of a tile is deferred into the score product of the next one (see
  // decode_stream_split.cuh): `pending` says that `pb` holds probabilities whose V stage has not been used.
  uint32_t pb[kNT][2];
  bool pending = false;
  uint32_t pending_v = 0, pending_rows = 0;
  auto flush_pending = [&](uint32_t chunk) {
    if (!pending) return;
    pending = false;
    wait_stage(pending_v, chunk);
    if (!(phases & kAborted)) {
      const uint32_t v_tile = my_tile + pending_v * Ring::kStageBytes;
      if (pending_rows < 16u) clear_dead_rows(v_tile, pending_rows);
      chunk_values<QT, kFp8, kD, kNT, true>(state, pb, v_tile, lane);
    }
    release_stage(pending_v);
  };

  for (uint32_t chunk = 0; chunk < my_tiles;) {
    if (chunk != 0 && consumer.tile == 0) {
      flush_pending(chunk);
      finish_item();
      begin_item();
    }
    // a run of full tiles of this work item inside this CTA's range: no tests inside
    if (pending && !(phases & kAborted)) {
      const uint32_t full_tiles = consumer.length / kTileTokens;
      const uint32_t run = min(full_tiles > consumer.tile ? full_tiles - consumer.tile : 0u, my_tiles - chunk);
      if (run > 1u) {
        uint32_t done = 0;
        for (; done < run; ++done) {
          const uint32_t k_stage = consume_stage;
          const uint32_t v_stage = next_stage(k_stage);
          wait_stage(k_stage, chunk + done);
          wait_stage(pending_v, chunk + done);
          if (phases & kAborted) break;  // the general path below walks on without waiting or computing
          float s[kNT][4];
          chunk_scores_and_values<QT, kD>(s, state, my_tile + k_stage * Ring::kStageBytes, pb,
                                          my_tile + pending_v * Ring::kStageBytes, lane);
          __syncwarp();
          if (lane == 0) {
            mbarrier_release(empty + pending_v * 8);
            mbarrier_release(empty + k_stage * 8);
          }
          chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, 16u, g);
          pending_v = v_stage;
          consume_stage = next_stage(v_stage);
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
    const uint32_t token0 = consumer.tile * kTileTokens;  // always inside the sequence
    const uint32_t live_rows = min(16u, consumer.length - token0);
    const uint32_t k_stage = consume_stage;
    const uint32_t v_stage = next_stage(k_stage);
    consume_stage = next_stage(v_stage);

    wait_stage(k_stage, chunk);
    float s[kNT][4];
    if (pending) {
      wait_stage(pending_v, chunk);
      if (!(phases & kAborted)) {
        const uint32_t v_tile = my_tile + pending_v * Ring::kStageBytes;
        if (pending_rows < 16u) clear_dead_rows(v_tile, pending_rows);
        chunk_scores_and_values<QT, kD>(s, state, my_tile + k_stage * Ring::kStageBytes, pb, v_tile, lane);
      }
      __syncwarp();
      if (lane == 0) {
        mbarrier_release(empty + pending_v * 8);
        mbarrier_release(empty + k_stage * 8);
      }
    } else {
      if (!(phases & kAborted)) {
        chunk_scores<QT, kFp8, kD, kNT, true>(s, state, my_tile + k_stage * Ring::kStageBytes, lane);
      }
      release_stage(k_stage);
    }
    if (!(phases & kAborted)) chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, live_rows, g);
    pending = !(phases & kAborted);
    pending_v = v_stage;
    pending_rows = live_rows;
    if (!pending) release_stage(v_stage);
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
