// Tensor-core building blocks of the paged decode kernels (16-bit queries over
// a native 16-bit or an FP8 E4M3 cache) and the fixed-partition kernel.
//
// Replaces the reference's three decode kernels
// (crates/loom-cuda-sys/cuda/src/paged_decode_attention.cu: one head per CTA
// :164-264, 2/4 packed GQA heads :269-501, split-K partials :509-747), all of
// which are scalar CUDA-core loops capped at 1024 tokens.
//
// Shape of the computation. A warp owns 16-token chunks of one (sequence, KV
// head) and ALL query heads of that KV head's group, so every K/V byte is
// fetched from HBM once however large the group is. Per chunk a warp computes,
// with m16n8k16 MMAs,
//     S^T[16 tokens x 8 heads]  = K[16 x D]   . Q^T[D x 8]
//     O^T[Dv x 8 heads]        += V^T[Dv x 16] . P^T[16 x 8]
// i.e. tokens (then value dims) ride the M side and the query heads ride N = 8,
// which is what makes a GQA group of 4..8 heads a dense tile; a group of 16
// uses two N tiles. K is the row-major A operand straight from ldmatrix, V^T is
// the same kind of shared tile read with ldmatrix.trans, Q^T lives in registers,
// and P^T is produced from the S^T accumulators by one movmatrix transpose per
// 8 tokens (no shared-memory round trip). The online softmax keeps (max, sum)
// per head in registers; max and sum cross lanes with xor shuffles.
//
// Memory. The hot loop is bound by HBM: 2*D*sizeof(cache element) bytes per
// (token, KV head). Rows are fetched as 16-byte cp.async.cg pieces (L1
// bypassed) into XOR-swizzled tiles, so both ldmatrix flavours are free of bank
// conflicts. Each warp runs its own multi-stage ring; there is no CTA-wide
// barrier in the streaming loop.
//
// FP8 cache. Bytes are staged as they are. ldmatrix moves them as 16-bit
// pairs; a byte permute plus cvt.rn.f16x2.e4m3x2 (exact) turns them into F16
// MMA operands in registers. The reduction dimension of QK^T and the row
// dimension of O^T are permuted to match what ldmatrix delivers, Q is loaded
// with the same permutation, and the epilogue un-permutes O. The K scale is
// folded into the softmax scale and the V scale into the final normalisation,
// so dequantisation costs no multiply per element.
#pragma once

#include <type_traits>

#include "decode_common.cuh"

namespace loom_decode {

constexpr int kMmaWarps = 4;
constexpr int kMmaThreads = kMmaWarps * 32;

template <bool kFp8, int kD>
struct MmaTile {
  static constexpr int kRowBytes = kD * (kFp8 ? 1 : 2);
  static constexpr int kSegs = kRowBytes / 16;       // 16-byte pieces per row
  static constexpr int kTileBytes = 16 * kRowBytes;  // one K or V chunk
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kWanted = (96 * 1024) / (kMmaWarps * kStageBytes);
  static constexpr int kStages = kWanted < 2 ? 2 : (kWanted > 8 ? 8 : kWanted);
  static constexpr int kRowsPerPass = 32 / kSegs;
  static constexpr int kPasses = 16 / kRowsPerPass;
  static_assert(kSegs >= 4 && kSegs <= 32, "row width out of range");
};

// Shared memory the cross-warp merge needs: per warp 8*kNT heads of kD + 4
// floats of O, plus one max and one sum per head.
template <int kNT, int kD, int kWarps = kMmaWarps>
constexpr int mma_merge_bytes() {
  return kWarps * (8 * kNT) * (kD + 4 + 2) * 4;
}

template <bool kFp8, int kD, int kNT>
constexpr int mma_smem_bytes() {
  constexpr int pipeline = kMmaWarps * MmaTile<kFp8, kD>::kStages * MmaTile<kFp8, kD>::kStageBytes;
  constexpr int merge = mma_merge_bytes<kNT, kD>();
  return pipeline > merge ? pipeline : merge;
}

// Byte offset of 16-byte piece `col` of row `row` inside a swizzled tile.
template <int kSegs>
__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t col) {
  if constexpr (kSegs >= 8) {
    return row * (kSegs * 16) + ((col ^ (row & 7u)) << 4);
  } else {
    return row * (kSegs * 16) + ((col ^ ((row >> 1) & 3u)) << 4);
  }
}

// The same for a tile that TMA wrote with its 128-byte (64-byte for 64-byte
// rows) swizzle: identical for rows of up to 128 bytes; a 256-byte row arrives
// as two 128-byte boxes, so the tile is two half-tiles of [16 rows x 128 B].
template <int kSegs, bool kTmaLayout>
__device__ __forceinline__ uint32_t tile_offset(uint32_t row, uint32_t col) {
  if constexpr (kTmaLayout && kSegs == 16) {
    return (col >> 3) * 2048u + row * 128u + (((col & 7u) ^ (row & 7u)) << 4);
  } else {
    return swizzled<kSegs>(row, col);
  }
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t packed) {
  const float2 wide = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
  return pack_f16x2(wide.x, wide.y);
}

// Everything one warp carries for one (sequence, KV head): the Q^T fragments and
// the running softmax state of its query heads.
template <int kD, int kNT>
struct WarpState {
  static constexpr int kKSteps = kD / 16;
  // Q^T as 16-bit MMA B fragments, one register pair per 16 head dims (F16 with
  // a permuted pairing for an FP8 cache, see load_query).
  uint32_t qf[kNT][kKSteps][2];
  float o[kNT][kKSteps][4];
  float row_max[kNT][2];
  float row_sum[kNT][2];
  // Factor that turns a raw QK^T accumulator of heads (2t, 2t+1) into a score
  // in base-2 units: softmax scale * log2(e), times the K scale and 2^8 for an
  // FP8 cache.
  float head_scale[kNT][2];

  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      row_max[nt][0] = row_max[nt][1] = -INFINITY;
      row_sum[nt][0] = row_sum[nt][1] = 0.0f;
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.0f;
    }
  }
};

// Loads the Q^T fragments of up to 8*kNT heads starting at `first_row` (a
// pointer to the first head's row; rows are `head_stride` elements apart).
// Heads at or beyond `live_heads` read as zero.
//
// FP8 cache: K bytes are turned into F16 by integer operations (see
// e4m3x4_to_f16_by_alu) that pair byte 0 with byte 2 and byte 1 with byte 3 of
// every 4-byte group and leave the values 2^-8 too small. Q is therefore loaded
// as F16 with the same pairing, and 2^8 goes into the score scale.
template <typename QT>
__device__ __forceinline__ float2 widen_pair(uint32_t packed) {
  if constexpr (std::is_same<QT, __nv_bfloat16>::value) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&packed));
  }
}

template <typename QT, bool kFp8, int kD, int kNT>
__device__ __forceinline__ void load_query(WarpState<kD, kNT>& state, const QT* first_row,
                                           uint64_t head_stride, uint32_t live_heads, float base_scale,
                                           uint32_t g, uint32_t t) {
  constexpr int kKSteps = kD / 16;
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const uint32_t head = nt * 8 + g;
    const bool live = head < live_heads;
    const QT* row = first_row + (uint64_t)(live ? head : 0u) * head_stride;
    if constexpr (kFp8) {
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        // this lane's reduction indices of step ks are dims 16 ks + 4 t + {0, 2} (b0) and {1, 3} (b1)
        uint32_t b0 = 0, b1 = 0;
        if (live) {
          const uint2 four = *reinterpret_cast<const uint2*>(row + ks * 16 + t * 4);
          const float2 low = widen_pair<QT>(four.x), high = widen_pair<QT>(four.y);
          if constexpr (kFp8KeyByAlu) {
            b0 = pack_f16x2(low.x, high.x);
            b1 = pack_f16x2(low.y, high.y);
          } else {
            b0 = pack_f16x2(low.x, low.y);
            b1 = pack_f16x2(high.x, high.y);
          }
        }
        state.qf[nt][ks][0] = b0;
        state.qf[nt][ks][1] = b1;
      }
      state.head_scale[nt][0] = state.head_scale[nt][1] = kFp8KeyByAlu ? base_scale * 256.0f : base_scale;
    } else {
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        uint32_t b0 = 0, b1 = 0;
        if (live) {
          b0 = *reinterpret_cast<const uint32_t*>(row + ks * 16 + t * 2);
          b1 = *reinterpret_cast<const uint32_t*>(row + ks * 16 + 8 + t * 2);
        }
        state.qf[nt][ks][0] = b0;
        state.qf[nt][ks][1] = b1;
      }
      state.head_scale[nt][0] = state.head_scale[nt][1] = base_scale;
    }
  }
}

// S^T = K . Q^T for one 16-token chunk staged at shared address `k_tile`.
template <typename QT, bool kFp8, int kD, int kNT, bool kTmaLayout = false>
__device__ __forceinline__ void chunk_scores(float (&s)[kNT][4], const WarpState<kD, kNT>& state,
                                             uint32_t k_tile, uint32_t lane) {
  using Tile = MmaTile<kFp8, kD>;
  constexpr bool kBf16Mma = !kFp8 && std::is_same<QT, __nv_bfloat16>::value;
  constexpr int kKSteps = kD / 16;
  // ldmatrix lane roles: matrices 0..3 = (rows 0-7, col c)(rows 8-15, col c)(rows 0-7, col c+1)(rows 8-15, col c+1)
  const uint32_t ld_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u;
  const uint32_t ld_col = lane >> 4;
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
  if constexpr (!kFp8) {
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, k_tile + tile_offset<Tile::kSegs, kTmaLayout>(ld_row, 2 * ks + ld_col));
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
        if constexpr (kBf16Mma) mma_16816_bf16(s[nt], a, state.qf[nt][ks][0], state.qf[nt][ks][1]);
        else mma_16816_f16(s[nt], a, state.qf[nt][ks][0], state.qf[nt][ks][1]);
      }
    }
  } else {
#pragma unroll
    for (int pair = 0; pair < kKSteps / 2; ++pair) {
      uint32_t r[4];
      ldmatrix_x4(r, k_tile + tile_offset<Tile::kSegs, kTmaLayout>(ld_row, 2 * pair + ld_col));
      // rows 0-7 / 8-15 of byte column c (r[0], r[1]) and of column c+1 (r[2], r[3])
      uint32_t a[4];
      if constexpr (kFp8KeyByAlu) {
        e4m3x4_to_f16_by_alu(r[0], a[0], a[2]);
        e4m3x4_to_f16_by_alu(r[1], a[1], a[3]);
      } else {
        e4m3x4_to_f16x2x2(r[0], a[0], a[2]);
        e4m3x4_to_f16x2x2(r[1], a[1], a[3]);
      }
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) mma_16816_f16(s[nt], a, state.qf[nt][2 * pair][0], state.qf[nt][2 * pair][1]);
      if constexpr (kFp8KeyByAlu) {
        e4m3x4_to_f16_by_alu(r[2], a[0], a[2]);
        e4m3x4_to_f16_by_alu(r[3], a[1], a[3]);
      } else {
        e4m3x4_to_f16x2x2(r[2], a[0], a[2]);
        e4m3x4_to_f16x2x2(r[3], a[1], a[3]);
      }
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
        mma_16816_f16(s[nt], a, state.qf[nt][2 * pair + 1][0], state.qf[nt][2 * pair + 1][1]);
      }
    }
  }
}

// Online softmax over the chunk's 16 tokens: updates the running exponent
// reference and sum, rescales O when the reference moves, and returns P^T as MMA
// B fragments. Rows at or beyond `live_rows` are masked.
//
// The reference exponent (state.row_max) is not the exact running maximum: it
// only moves when some score of the chunk exceeds it by more than kSoftmaxSlack
// (base-2 units), and then rises to the largest score of that chunk. So every
// p = 2^(score - reference) is at most 2^kSoftmaxSlack, well inside the
// range of the 16-bit P operand and of the F32 sums, and softmax is invariant
// to the choice of reference. In the common case this removes the cross-lane
// maximum (six shuffles per head pair), the correction factors and the rescale
// of the O accumulators from the chunk; one warp vote decides.
constexpr float kSoftmaxSlack = 8.0f;

//
// Options: rows below `dead_rows` are masked too (the tokens before a sliding window's first
// token); with `cap2` != 0 every score passes through the soft cap before the exponent.
template <typename QT, bool kFp8, int kD, int kNT>
__device__ __forceinline__ void chunk_softmax(uint32_t (&pb)[kNT][2], const float (&s)[kNT][4],
                                              WarpState<kD, kNT>& state, uint32_t live_rows,
                                              uint32_t g, uint32_t dead_rows = 0u, float cap2 = 0.0f,
                                              float inv_cap2 = 0.0f) {
  constexpr bool kBf16Mma = !kFp8 && std::is_same<QT, __nv_bfloat16>::value;
  constexpr int kKSteps = kD / 16;
  // score in base-2 units of a raw accumulator
  auto score = [&](float raw, float head_scale) {
    const float scaled = raw * head_scale;
    return cap2 != 0.0f ? soft_capped(scaled, cap2, inv_cap2) : scaled;
  };
  // exponents relative to the current reference
  float d[kNT][4];
  bool over = false;
  if (cap2 != 0.0f) {  // warp-uniform
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      d[nt][0] = score(s[nt][0], state.head_scale[nt][0]) - state.row_max[nt][0];
      d[nt][1] = score(s[nt][1], state.head_scale[nt][1]) - state.row_max[nt][1];
      d[nt][2] = score(s[nt][2], state.head_scale[nt][0]) - state.row_max[nt][0];
      d[nt][3] = score(s[nt][3], state.head_scale[nt][1]) - state.row_max[nt][1];
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      d[nt][0] = fmaf(s[nt][0], state.head_scale[nt][0], -state.row_max[nt][0]);
      d[nt][1] = fmaf(s[nt][1], state.head_scale[nt][1], -state.row_max[nt][1]);
      d[nt][2] = fmaf(s[nt][2], state.head_scale[nt][0], -state.row_max[nt][0]);
      d[nt][3] = fmaf(s[nt][3], state.head_scale[nt][1], -state.row_max[nt][1]);
    }
  }
  if (live_rows < 16u || dead_rows != 0u) {  // warp-uniform
    const bool low_live = g < live_rows && g >= dead_rows;
    const bool high_live = (g + 8u) < live_rows && (g + 8u) >= dead_rows;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      if (!low_live) d[nt][0] = d[nt][1] = -INFINITY;
      if (!high_live) d[nt][2] = d[nt][3] = -INFINITY;
    }
  }
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    over |= fmaxf(fmaxf(d[nt][0], d[nt][1]), fmaxf(d[nt][2], d[nt][3])) > kSoftmaxSlack;
  }
  if (__any_sync(0xffffffffu, over)) {
    // rare: move every head's reference up to the largest score of this chunk
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const bool low_dead = d[nt][0] == -INFINITY, high_dead = d[nt][2] == -INFINITY;
      const float v0 = low_dead ? -INFINITY : score(s[nt][0], state.head_scale[nt][0]);
      const float v1 = low_dead ? -INFINITY : score(s[nt][1], state.head_scale[nt][1]);
      const float v2 = high_dead ? -INFINITY : score(s[nt][2], state.head_scale[nt][0]);
      const float v3 = high_dead ? -INFINITY : score(s[nt][3], state.head_scale[nt][1]);
      float max0 = fmaxf(v0, v2), max1 = fmaxf(v1, v3);
#pragma unroll
      for (int offset = 4; offset < 32; offset <<= 1) {
        max0 = fmaxf(max0, __shfl_xor_sync(0xffffffffu, max0, offset));
        max1 = fmaxf(max1, __shfl_xor_sync(0xffffffffu, max1, offset));
      }
      const float old0 = state.row_max[nt][0], old1 = state.row_max[nt][1];
      const float new0 = fmaxf(old0, max0), new1 = fmaxf(old1, max1);
      const float alpha0 = old0 == -INFINITY ? 0.0f : fast_exp2(old0 - new0);
      const float alpha1 = old1 == -INFINITY ? 0.0f : fast_exp2(old1 - new1);
      state.row_max[nt][0] = new0;
      state.row_max[nt][1] = new1;
      d[nt][0] = v0 - new0;
      d[nt][1] = v1 - new1;
      d[nt][2] = v2 - new0;
      d[nt][3] = v3 - new1;
      state.row_sum[nt][0] *= alpha0;
      state.row_sum[nt][1] *= alpha1;
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt) {
        state.o[nt][mt][0] *= alpha0;
        state.o[nt][mt][1] *= alpha1;
        state.o[nt][mt][2] *= alpha0;
        state.o[nt][mt][3] *= alpha1;
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const float p0 = fast_exp2(d[nt][0]), p1 = fast_exp2(d[nt][1]);
    const float p2 = fast_exp2(d[nt][2]), p3 = fast_exp2(d[nt][3]);
    state.row_sum[nt][0] += p0 + p2;
    state.row_sum[nt][1] += p1 + p3;
    if constexpr (kBf16Mma) {
      pb[nt][0] = movmatrix_trans(pack_bf16x2(p0, p1));
      pb[nt][1] = movmatrix_trans(pack_bf16x2(p2, p3));
    } else {
      pb[nt][0] = movmatrix_trans(pack_f16x2(p0, p1));
      pb[nt][1] = movmatrix_trans(pack_f16x2(p2, p3));
    }
  }
}

// O^T += V^T . P^T for the chunk staged at shared address `v_tile`.
template <typename QT, bool kFp8, int kD, int kNT, bool kTmaLayout = false>
__device__ __forceinline__ void chunk_values(WarpState<kD, kNT>& state, const uint32_t (&pb)[kNT][2],
                                             uint32_t v_tile, uint32_t lane) {
  using Tile = MmaTile<kFp8, kD>;
  constexpr bool kBf16Mma = !kFp8 && std::is_same<QT, __nv_bfloat16>::value;
  constexpr int kKSteps = kD / 16;
  if constexpr (!kFp8) {
    // matrices 0..3 = (tokens 0-7, col c)(tokens 0-7, col c+1)(tokens 8-15, col c)(tokens 8-15, col c+1)
    const uint32_t ld_row = (lane & 7u) + (lane >> 4) * 8u;
    const uint32_t ld_col = (lane >> 3) & 1u;
#pragma unroll
    for (int mt = 0; mt < kKSteps; ++mt) {
      uint32_t a[4];
      ldmatrix_x4_trans(a, v_tile + tile_offset<Tile::kSegs, kTmaLayout>(ld_row, 2 * mt + ld_col));
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
        if constexpr (kBf16Mma) mma_16816_bf16(state.o[nt][mt], a, pb[nt][0], pb[nt][1]);
        else mma_16816_f16(state.o[nt][mt], a, pb[nt][0], pb[nt][1]);
      }
    }
  } else {
    // matrices 0..3 = (tokens 0-7, col c)(tokens 8-15, col c)(tokens 0-7, col c+1)(tokens 8-15, col c+1)
    const uint32_t ld_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u;
    const uint32_t ld_col = lane >> 4;
#pragma unroll
    for (int pair = 0; pair < kKSteps / 2; ++pair) {
      uint32_t r[4];
      ldmatrix_x4_trans(r, v_tile + tile_offset<Tile::kSegs, kTmaLayout>(ld_row, 2 * pair + ld_col));
      uint32_t a[4];
      e4m3x4_to_f16x2x2(__byte_perm(r[0], 0u, 0x3120u), a[0], a[1]);
      e4m3x4_to_f16x2x2(__byte_perm(r[1], 0u, 0x3120u), a[2], a[3]);
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) mma_16816_f16(state.o[nt][2 * pair], a, pb[nt][0], pb[nt][1]);
      e4m3x4_to_f16x2x2(__byte_perm(r[2], 0u, 0x3120u), a[0], a[1]);
      e4m3x4_to_f16x2x2(__byte_perm(r[3], 0u, 0x3120u), a[2], a[3]);
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) mma_16816_f16(state.o[nt][2 * pair + 1], a, pb[nt][0], pb[nt][1]);
    }
  }
}

// Layout of the cross-warp merge area (kWarps warps compute: four, unless a kernel says otherwise).
template <int kD, int kNT, int kWarps = kMmaWarps>
struct MergeArea {
  static constexpr int kHeads = 8 * kNT;
  static constexpr int kORow = kD + 4;
  float* o;    // [warps][kHeads][kORow]
  float* max;  // [warps][kHeads]
  float* sum;  // [warps][kHeads]
  __device__ __forceinline__ explicit MergeArea(void* base) {
    o = reinterpret_cast<float*>(base);
    max = o + kWarps * kHeads * kORow;
    sum = max + kWarps * kHeads;
  }
};

// Completes a warp's row sums and parks its state in the merge area. The
// caller brackets this with CTA barriers.
template <bool kFp8, int kD, int kNT, int kWarps = kMmaWarps>
__device__ __forceinline__ void park_warp_state(MergeArea<kD, kNT, kWarps> area, WarpState<kD, kNT>& state,
                                                uint32_t warp, uint32_t g, uint32_t t) {
  constexpr int kHeads = 8 * kNT;
  constexpr int kORow = kD + 4;
  constexpr int kKSteps = kD / 16;
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
#pragma unroll
    for (int offset = 4; offset < 32; offset <<= 1) {
      state.row_sum[nt][0] += __shfl_xor_sync(0xffffffffu, state.row_sum[nt][0], offset);
      state.row_sum[nt][1] += __shfl_xor_sync(0xffffffffu, state.row_sum[nt][1], offset);
    }
    const uint32_t head0 = nt * 8 + 2 * t;
    float* base0 = area.o + ((size_t)warp * kHeads + head0) * kORow;
    float* base1 = base0 + kORow;
#pragma unroll
    for (int mt = 0; mt < kKSteps; ++mt) {
      // un-permute the value dimension of the FP8 path
      const uint32_t dv_a = kFp8 ? mt * 16 + 2 * g : mt * 16 + g;
      const uint32_t dv_b = kFp8 ? dv_a + 1 : dv_a + 8;
      base0[dv_a] = state.o[nt][mt][0];
      base1[dv_a] = state.o[nt][mt][1];
      base0[dv_b] = state.o[nt][mt][2];
      base1[dv_b] = state.o[nt][mt][3];
    }
    if (g == 0) {
      area.max[warp * kHeads + head0] = state.row_max[nt][0];
      area.max[warp * kHeads + head0 + 1] = state.row_max[nt][1];
      area.sum[warp * kHeads + head0] = state.row_sum[nt][0];
      area.sum[warp * kHeads + head0 + 1] = state.row_sum[nt][1];
    }
  }
}

// Merges the parked warp states and stores, per live head, either the
// normalised output row (`final_out`, type QT) or an F32 state row
// (`state_rows` + head * state_head_stride floats). Called by the kWarps
// computing warps of the CTA (threads 0 .. 32 * kWarps - 1).
template <typename QT, int kD, int kNT, int kWarps = kMmaWarps>
__device__ __forceinline__ void combine_and_store(MergeArea<kD, kNT, kWarps> area, uint32_t live_heads,
                                                  float value_scale, QT* final_out,
                                                  uint64_t final_head_stride, float* state_rows,
                                                  uint64_t state_head_stride) {
  constexpr int kHeads = 8 * kNT;
  constexpr int kORow = kD + 4;
  for (uint32_t index = threadIdx.x; index < live_heads * kD; index += kWarps * 32) {
    const uint32_t head = index / kD;
    const uint32_t dv = index % kD;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) top = fmaxf(top, area.max[w * kHeads + head]);
    float acc = 0.0f, total = 0.0f;
    if (top > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float factor = fast_exp2(area.max[w * kHeads + head] - top);
        acc += area.o[((size_t)w * kHeads + head) * kORow + dv] * factor;
        total += area.sum[w * kHeads + head] * factor;
      }
    }
    acc *= value_scale;
    if (final_out != nullptr) {
      const float result = total > 0.0f ? acc / total : 0.0f;
      QT* out = final_out + (uint64_t)head * final_head_stride;
      if constexpr (std::is_same<QT, __nv_bfloat16>::value) out[dv] = __float2bfloat16_rn(result);
      else out[dv] = __float2half_rn(result);
    } else {
      float* row = state_rows + (uint64_t)head * state_head_stride;
      row[dv] = acc;
      if (dv == 0) {
        row[kD] = top * kLn2;
        row[kD + 1] = total;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// Fixed-partition kernel: one CTA per (sequence, KV head, partition of
// `partition_tokens`); used for the workspace-free single pass, for block sizes
// that are not a multiple of 16, and when the caller fixes the partition length.
// ----------------------------------------------------------------------------
template <typename QT, bool kFp8, int kD, int kNT, bool kOptions>
__global__ void __launch_bounds__(kMmaThreads, 2) decode_mma_kernel(const DecodeParams p) {
  using Tile = MmaTile<kFp8, kD>;
  constexpr int kHeads = 8 * kNT;

  extern __shared__ __align__(128) uint8_t smem[];
  loom_launch::grid_dependency_wait();

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2;
  const uint32_t t = lane & 3u;

  const uint32_t head_chunks = (p.group + kHeads - 1) / kHeads;
  const uint32_t seq = blockIdx.x / p.max_partitions;
  const uint32_t part = blockIdx.x % p.max_partitions;
  const uint32_t kv_head = blockIdx.y / head_chunks;
  const uint32_t first_head = (blockIdx.y % head_chunks) * kHeads;  // within the group

  const uint32_t length = clamp_length(p.sequence_lengths[seq], p.max_sequence_length);
  // Under a sliding window the sequence effectively starts at `visible`: partitions wholly before
  // it do nothing, the one holding it starts at the 16-token chunk of that token.
  const uint32_t visible = window_begin(length, kOptions ? p.sliding_window : 0u);
  const uint32_t first_part = visible / p.partition_tokens;
  if ((part * p.partition_tokens >= length && part != 0) || part < first_part) return;  // empty partition
  const uint32_t part_begin = max(part * p.partition_tokens, visible & ~15u);
  const uint32_t part_end = min(length, (part + 1) * p.partition_tokens);
  const uint32_t n_parts =
      length == 0 ? 1u : (length + p.partition_tokens - 1) / p.partition_tokens - first_part;
  const uint32_t n_chunks = part_end > part_begin ? (part_end - part_begin + 15u) / 16u : 0u;
  const uint32_t my_chunks = n_chunks > warp ? (n_chunks - warp + kMmaWarps - 1) / kMmaWarps : 0u;
  const uint32_t live_heads = min((uint32_t)kHeads, p.group - first_head);

  WarpState<kD, kNT> state;
  state.reset();
  const uint64_t first_query_head = (uint64_t)kv_head * p.group + first_head;
  float score_scale = p.scale_log2;
  if constexpr (kFp8) score_scale *= p.key_scales[(uint64_t)kv_head * p.scale_stride];
  load_query<QT, kFp8, kD, kNT>(
      state, static_cast<const QT*>(p.query) + (uint64_t)seq * p.q_token + first_query_head * p.q_head,
      p.q_head, live_heads, score_scale, g, t);

  // ---- producer side: page-table driven 16-byte copies --------------------
  const uint8_t* key_bytes = static_cast<const uint8_t*>(p.key_cache);
  const uint8_t* value_bytes = static_cast<const uint8_t*>(p.value_cache);
  constexpr uint32_t kElem = kFp8 ? 1 : 2;
  const bool page16 = (p.block_size % 16u) == 0;
  const int32_t* table = p.block_tables + (uint64_t)seq * p.max_blocks_per_sequence;
  const uint32_t smem_base = smem_address(smem) + warp * (Tile::kStages * Tile::kStageBytes);
  const uint32_t copy_row = lane / Tile::kSegs;
  const uint32_t copy_col = lane % Tile::kSegs;
  const uint64_t k_head_offset = (uint64_t)kv_head * p.k_head * kElem + copy_col * 16;
  const uint64_t v_head_offset = (uint64_t)kv_head * p.v_head * kElem + copy_col * 16;

  uint32_t cached_blocks = 0;  // block ids of 32 consecutive chunks of this warp (page16 only)

  auto issue_chunk = [&](uint32_t index) {
    // index counts this warp's chunks; the stage is index % kStages
    const uint32_t token0 = part_begin + (warp + index * kMmaWarps) * 16u;
    const uint32_t stage = smem_base + (index % Tile::kStages) * Tile::kStageBytes;
    if (page16) {
      if ((index & 31u) == 0) {
        const uint32_t ahead = part_begin + (warp + (index + lane) * kMmaWarps) * 16u;
        cached_blocks = ahead < part_end ? clamp_block(__ldg(table + ahead / p.block_size), p.num_blocks) : 0u;
      }
      const uint32_t block = __shfl_sync(0xffffffffu, cached_blocks, index & 31u);
      const uint32_t page0 = token0 % p.block_size;
      const uint8_t* k_row = key_bytes + ((uint64_t)block * p.k_block + (uint64_t)(page0 + copy_row) * p.k_page) * kElem + k_head_offset;
      const uint8_t* v_row = value_bytes + ((uint64_t)block * p.v_block + (uint64_t)(page0 + copy_row) * p.v_page) * kElem + v_head_offset;
      const uint64_t k_step = (uint64_t)Tile::kRowsPerPass * p.k_page * kElem;
      const uint64_t v_step = (uint64_t)Tile::kRowsPerPass * p.v_page * kElem;
#pragma unroll
      for (int pass = 0; pass < Tile::kPasses; ++pass) {
        const uint32_t row = copy_row + pass * Tile::kRowsPerPass;
        const uint32_t bytes = (token0 + row) < part_end ? 16u : 0u;
        cp_async_16(stage + swizzled<Tile::kSegs>(row, copy_col), bytes ? k_row + pass * k_step : key_bytes, bytes);
      }
#pragma unroll
      for (int pass = 0; pass < Tile::kPasses; ++pass) {
        const uint32_t row = copy_row + pass * Tile::kRowsPerPass;
        const uint32_t bytes = (token0 + row) < part_end ? 16u : 0u;
        cp_async_16(stage + Tile::kTileBytes + swizzled<Tile::kSegs>(row, copy_col),
                    bytes ? v_row + pass * v_step : value_bytes, bytes);
      }
    } else {
      // any block size: every row looks its own block up
#pragma unroll
      for (int pass = 0; pass < Tile::kPasses; ++pass) {
        const uint32_t row = copy_row + pass * Tile::kRowsPerPass;
        const uint32_t token = token0 + row;
        const bool live = token < part_end;
        const uint8_t* k_row = key_bytes;
        const uint8_t* v_row = value_bytes;
        if (live) {
          const uint32_t block = clamp_block(__ldg(table + token / p.block_size), p.num_blocks);
          const uint32_t page = token % p.block_size;
          k_row = key_bytes + ((uint64_t)block * p.k_block + (uint64_t)page * p.k_page) * kElem + k_head_offset;
          v_row = value_bytes + ((uint64_t)block * p.v_block + (uint64_t)page * p.v_page) * kElem + v_head_offset;
        }
        cp_async_16(stage + swizzled<Tile::kSegs>(row, copy_col), k_row, live ? 16u : 0u);
        cp_async_16(stage + Tile::kTileBytes + swizzled<Tile::kSegs>(row, copy_col), v_row, live ? 16u : 0u);
      }
    }
  };

#pragma unroll
  for (int s = 0; s < Tile::kStages - 1; ++s) {
    if ((uint32_t)s < my_chunks) issue_chunk(s);
    cp_async_commit();
  }

  for (uint32_t i = 0; i < my_chunks; ++i) {
    cp_async_wait<Tile::kStages - 2>();
    __syncwarp();
    {
      const uint32_t next = i + Tile::kStages - 1;
      if (next < my_chunks) issue_chunk(next);
      cp_async_commit();
    }
    const uint32_t stage = smem_base + (i % Tile::kStages) * Tile::kStageBytes;
    const uint32_t token0 = part_begin + (warp + i * kMmaWarps) * 16u;
    const uint32_t live_rows = part_end - token0;  // >= 1; rows beyond it are zero filled
    const uint32_t dead_rows = visible > token0 ? visible - token0 : 0u;  // tokens before the window

    float s[kNT][4];
    chunk_scores<QT, kFp8, kD, kNT>(s, state, stage, lane);
    uint32_t pb[kNT][2];
    chunk_softmax<QT, kFp8, kD, kNT>(pb, s, state, live_rows, g, dead_rows, kOptions ? p.soft_cap_log2 : 0.0f,
                                     kOptions ? p.inv_soft_cap_log2 : 0.0f);
    chunk_values<QT, kFp8, kD, kNT>(state, pb, stage + Tile::kTileBytes, lane);
  }
  cp_async_wait<0>();

  // ---- merge the four warps and store --------------------------------------
  __syncthreads();  // every warp is done with its ring; reuse the memory
  MergeArea<kD, kNT> area(smem);
  park_warp_state<kFp8, kD, kNT>(area, state, warp, g, t);
  __syncthreads();

  float value_scale = 1.0f;
  if constexpr (kFp8) value_scale = p.value_scales[(uint64_t)kv_head * p.scale_stride];
  const uint64_t query_row = (uint64_t)seq * p.query_heads + first_query_head;
  const uint32_t stride = state_stride(kD);
  if (n_parts == 1 && !p.emit_state) {
    combine_and_store<QT, kD, kNT>(area, live_heads, value_scale, static_cast<QT*>(p.output) + query_row * kD,
                                   kD, nullptr, 0);
  } else if (n_parts == 1) {
    combine_and_store<QT, kD, kNT>(area, live_heads, value_scale, nullptr, 0,
                                   static_cast<float*>(p.output) + query_row * stride, stride);
  } else {
    combine_and_store<QT, kD, kNT>(area, live_heads, value_scale, nullptr, 0,
                                   p.partials + (query_row * p.max_partitions + part) * stride,
                                   (uint64_t)p.max_partitions * stride);
  }
}

}  // namespace loom_decode
