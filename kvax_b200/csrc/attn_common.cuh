// Shared pieces of the attention kernels: the element-level mask rule derived from the
// block-mask arrays, tile-list encoding, and kernel argument structs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kvax_b200.h"

namespace kvx {

constexpr int kTile = 128;                 // native tile edge of every attention kernel
constexpr uint32_t kPartialBit = 0x80000000u;
// Element masks of partial tiles depend on (batch row, outer tile, inner tile) only, not on the head: the list builder
// works out the first kBitmapSlots of every list once -- 128 rows x 128 bits, one uint4 per outer row -- and marks
// those entries; the attention kernels then load 16 bytes per row and tile instead of comparing 128 segment ids and
// positions per row, tile and head.  Further partial entries of a list are masked by the consumer as before.
// A marked entry carries its slot: bit 31 partial, bit 30 marked, bits 27-29 the slot, bits 0-26 the inner tile.
constexpr uint32_t kBitmapBit = 0x40000000u;
constexpr int kBitmapSlotShift = 27;
constexpr uint32_t kTileIndexMask = 0x07ffffffu;
constexpr int kBitmapSlots = 8;

// Block mask plus the geometry needed to read it.
struct MaskView {
  const int32_t* lower;
  const int32_t* upper;
  const int32_t* lower_full;
  const int32_t* upper_full;
  int32_t outer_block;   // block size on the axis the mask has one row per block of
  int32_t inner_block;   // block size on the axis the bounds index
  int32_t n_outer;       // blocks per batch row
};

// Position / segment arrays of both sides.
struct TokenInfo {
  const int32_t* q_pos; const int32_t* q_seg;
  const int32_t* kv_pos; const int32_t* kv_seg;
  int32_t q_len, kv_len;
  int32_t sequential;         // assume_sequential_positions
  int32_t off_first, off_second;  // global offsets of the two halves of the local queries
};

// Bounds of one outer row, in tokens of the inner axis.
struct RowBounds { int lo, lof, uf, up; };

__device__ __forceinline__ RowBounds load_bounds(const MaskView& m, int b, int outer_token) {
  int blk = outer_token / m.outer_block;
  blk = min(blk, m.n_outer - 1);
  const long long o = (long long)b * m.n_outer + blk;
  RowBounds r;
  r.lo = __ldg(m.lower + o) * m.inner_block;
  r.lof = __ldg(m.lower_full + o) * m.inner_block;
  r.uf = __ldg(m.upper_full + o) * m.inner_block;
  r.up = __ldg(m.upper + o) * m.inner_block;
  return r;
}

// Query position used by the causal test.  With assume_sequential_positions the
// reference compares global indices: local index plus the offset of the half of the
// local sequence the token lies in (flash_attention_triton.py:101-108, 1426-1447).
__device__ __forceinline__ int query_position(const TokenInfo& t, int b, int r) {
  if (t.sequential) return r + ((2 * r >= t.q_len) ? t.off_second : t.off_first);
  return __ldg(t.q_pos + (long long)b * t.q_len + r);
}

// The reference visits inner blocks in three classes (flash_attention_triton.py:292-364
// for query-outer masks, :1067-1167 for the kv-outer mask):
//   [lo, lof)  "left"  : segment mask only   (kv-outer: causal AND segment)
//   [lof, uf)  "full"  : no mask
//   [uf, up)   "right" : causal AND segment  (kv-outer: segment only)
// `i` is the token index on the inner axis.  `seg_eq`: raw segment ids equal (PAD
// matches PAD, :32-41).  `causal`: query position >= kv position.
template <bool kKvOuter>
__device__ __forceinline__ bool element_allowed(const RowBounds& rb, int i, bool seg_eq, bool causal) {
  const bool in_left = (i >= rb.lo) && (i < rb.lof);
  const bool in_full = (i >= rb.lof) && (i < rb.uf);
  const bool in_right = (i >= rb.uf) && (i < rb.up);
  if (kKvOuter) return in_full || (seg_eq && (in_right || (in_left && causal)));
  return in_full || (seg_eq && (in_left || (in_right && causal)));
}

// Mask bits of one outer row for 32 consecutive inner tokens [i0, i0 + 32): bit j set when
// element (row, i0 + j) is allowed.  `seg` / `pos` point at the 32 inner segment ids /
// positions (global or shared memory; `pos` may be null when positions are the token
// indices).  `o_seg` / `o_pos` belong to the outer row.
// Fast path: when all four bounds of the row are multiples of 32 (mask block sizes of 32,
// 64, 128, ...) the whole chunk lies in one class, so the class is resolved once and only
// the segment and causal comparisons remain per element.
template <bool kKvOuter>
__device__ __forceinline__ uint32_t keep_bits32(const RowBounds& rb, int i0, int inner_len, bool row_valid,
                                                int o_seg, int o_pos, const int32_t* __restrict__ seg,
                                                const int32_t* __restrict__ pos) {
  if (!row_valid || i0 >= inner_len) return 0u;
  const bool whole = (i0 + 32 <= inner_len);
  if (whole && (((rb.lo | rb.lof | rb.uf | rb.up) & 31) == 0)) {
    if (i0 >= rb.lof && i0 < rb.uf) return 0xffffffffu;
    const bool in_left = (i0 >= rb.lo) && (i0 < rb.lof);
    const bool in_right = (i0 >= rb.uf) && (i0 < rb.up);
    if (!(in_left || in_right)) return 0u;
    const bool need_causal = kKvOuter ? in_left : in_right;
    uint32_t bits = 0;
    const bool vec = ((reinterpret_cast<uintptr_t>(seg) & 15) == 0) && (!pos || (reinterpret_cast<uintptr_t>(pos) & 15) == 0);
    if (vec) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int4 s4 = *reinterpret_cast<const int4*>(seg + 4 * g);
        int4 p4 = make_int4(i0 + 4 * g, i0 + 4 * g + 1, i0 + 4 * g + 2, i0 + 4 * g + 3);
        if (need_causal && pos) p4 = *reinterpret_cast<const int4*>(pos + 4 * g);
        const int sv[4] = {s4.x, s4.y, s4.z, s4.w};
        const int pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          bool ok = (sv[t] == o_seg);
          if (need_causal) ok = ok && (kKvOuter ? (pv[t] >= o_pos) : (o_pos >= pv[t]));
          bits |= (ok ? 1u : 0u) << (4 * g + t);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        bool ok = (seg[j] == o_seg);
        if (need_causal) {
          const int p = pos ? pos[j] : (i0 + j);
          ok = ok && (kKvOuter ? (p >= o_pos) : (o_pos >= p));
        }
        bits |= (ok ? 1u : 0u) << j;
      }
    }
    return bits;
  }
  // general path: class resolved per element
  uint32_t bits = 0;
#pragma unroll 4
  for (int j = 0; j < 32; ++j) {
    const int i = i0 + j;
    if (i < inner_len) {
      const int p = pos ? pos[j] : i;
      const bool causal = kKvOuter ? (p >= o_pos) : (o_pos >= p);
      bits |= (element_allowed<kKvOuter>(rb, i, seg[j] == o_seg, causal) ? 1u : 0u) << j;
    }
  }
  return bits;
}

// Mask bits of one kv row (kv-outer orientation) for the 32 queries [i0, i0 + 32) of batch row b.  `kv_pos` is the
// row's position, i.e. its index under assume_sequential_positions; the query position is then the query's index plus
// the global offset of its half of the local queries, which is folded into the kv position so that the index itself
// can be compared.  Used by the list builder (element masks of marked entries) and by the backward kernels on
// entries without one: same function, same bits.
__device__ __forceinline__ uint32_t kv_outer_keep32(const TokenInfo& tok, const RowBounds& rb, int b, bool row_valid,
                                                    int kv_seg, int kv_pos, int i0) {
  const int q_len = tok.q_len;
  const int32_t* q_seg = tok.q_seg + (long long)b * q_len;
  if (!tok.sequential)
    return keep_bits32<true>(rb, i0, q_len, row_valid, kv_seg, kv_pos, q_seg + i0, tok.q_pos + (long long)b * q_len + i0);
  const int second_from = (q_len + 1) >> 1;                 // first local query of the second half (2 r >= q_len)
  if (i0 >= second_from || i0 + 32 <= second_from || tok.off_first == tok.off_second) {
    const int off = (i0 >= second_from) ? tok.off_second : tok.off_first;
    return keep_bits32<true>(rb, i0, q_len, row_valid, kv_seg, kv_pos - off, q_seg + i0, nullptr);
  }
  uint32_t bits = 0;                                        // the chunk straddles the two halves
  if (row_valid) {
    for (int j = 0; j < 32; ++j) {
      const int i = i0 + j;
      if (i < q_len) {
        const int p = i + (i >= second_from ? tok.off_second : tok.off_first);
        bits |= (element_allowed<true>(rb, i, __ldg(q_seg + i) == kv_seg, p >= kv_pos) ? 1u : 0u) << j;
      }
    }
  }
  return bits;
}

// ---------------------------------------------------------------------------
// Tile lists (built by schedule.cu): for every (batch, outer tile) the inner tiles to
// visit, ascending; bit 31 marks tiles that need the element-level mask.
// ---------------------------------------------------------------------------
struct TileList {
  const uint32_t* tiles;   // (B, n_outer_tiles, n_inner_tiles)
  const int32_t* counts;   // (B, n_outer_tiles)
  const int32_t* order;    // (B * n_outer_tiles) launch order: row = b * n_outer_tiles + tile
  const int32_t* pair_order;   // (B * ceil(n_outer_tiles / 2)) launch order of the pairs (2p, 2p+1): row of tile 2p
  const uint4* bitmaps;        // (B * n_outer_tiles, kBitmapSlots, 128) element masks of marked entries, or null: none marked
  int32_t n_outer_tiles, n_inner_tiles;
};

// Launch geometry shared by the attention kernels: a 1-D grid over (outer tile, head).
// Outer tiles are taken in the launch order built by schedule.cu (blocks of kRowChunk
// neighbouring tiles, the blocks with the longest lists first), in chunks of kRowChunk; inside
// a chunk the heads are the slow index.  CTAs resident at the same time therefore belong to a
// few heads and neighbouring outer tiles, so they stream the same inner tiles (served by L2),
// while long work items still start early in the launch.
constexpr int kRowChunk = 32;
__device__ __forceinline__ void decode_block(int linear, int n_rows, int n_heads, int* row_rank, int* head) {
  const int per_chunk = kRowChunk * n_heads;
  const int chunk = linear / per_chunk;
  const int within = linear - chunk * per_chunk;
  const int rows_here = min(kRowChunk, n_rows - chunk * kRowChunk);
  *head = within / rows_here;
  *row_rank = chunk * kRowChunk + (within - *head * rows_here);
}

}  // namespace kvx
