// Tile-list builder: turns a block mask (four bound arrays at the caller's block sizes)
// into, for every 128-row outer tile, the ascending list of 128-column inner tiles the
// attention kernels must visit, plus a longest-first launch order of the outer tiles.
//
//   * A tile whose every element lies in the "full" range of every row is emitted as
//     unmasked.
//   * A tile in which no element survives the reference's element-level rule is dropped
//     (it contributes nothing to any row).  Most such tiles are rejected by an interval
//     test on per-tile (segment min/max, position min/max) summaries; the rest by an exact
//     128 x 128 test.
//   * Everything else is emitted as partial and masked per element by the consumer.
//
// Launches: tile_summary_kernel (one warp per 128-token tile of either side),
// schedule_kernel (one CTA of 128 threads per (outer tile, batch); thread t owns outer
// row t), order_kernel (one CTA: counting sort of the outer tiles by list length).
#include "attn_common.cuh"
#include "internal.h"

namespace kvx {

namespace {

constexpr int kChunk = 1024;   // inner tiles classified per pass

// ---- per-tile summaries ---------------------------------------------------------------
// int4 {seg_min, seg_max, pos_min, pos_max} over the valid tokens of a tile; raw segment
// ids (PAD participates: PAD matches PAD in the element rule).
__global__ void __launch_bounds__(256) tile_summary_kernel(const TokenInfo tok, int4* q_sum, int4* kv_sum,
                                                          int n_q_tiles, int n_kv_tiles, int batch) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_q = (long long)batch * n_q_tiles, n_all = n_q + (long long)batch * n_kv_tiles;
  if (warp >= n_all) return;
  const bool is_q = warp < n_q;
  const long long local = is_q ? warp : warp - n_q;
  const int n_tiles = is_q ? n_q_tiles : n_kv_tiles;
  const int b = int(local / n_tiles), t = int(local % n_tiles);
  const int len = is_q ? tok.q_len : tok.kv_len;
  int smin = INT32_MAX, smax = INT32_MIN, pmin = INT32_MAX, pmax = INT32_MIN;
  for (int i = t * kTile + lane; i < min((t + 1) * kTile, len); i += 32) {
    int seg, pos;
    if (is_q) { seg = __ldg(tok.q_seg + (long long)b * len + i); pos = query_position(tok, b, i); }
    else { seg = __ldg(tok.kv_seg + (long long)b * len + i); pos = tok.sequential ? i : __ldg(tok.kv_pos + (long long)b * len + i); }
    smin = min(smin, seg); smax = max(smax, seg); pmin = min(pmin, pos); pmax = max(pmax, pos);
  }
  smin = __reduce_min_sync(0xffffffffu, smin); smax = __reduce_max_sync(0xffffffffu, smax);
  pmin = __reduce_min_sync(0xffffffffu, pmin); pmax = __reduce_max_sync(0xffffffffu, pmax);
  if (lane == 0) (is_q ? q_sum : kv_sum)[local] = make_int4(smin, smax, pmin, pmax);
}

__device__ __forceinline__ int block_min(int v, int* s) {
  v = __reduce_min_sync(0xffffffffu, v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
  __syncthreads();
  return min(min(s[0], s[1]), min(s[2], s[3]));
}
__device__ __forceinline__ int block_max(int v, int* s) {
  v = __reduce_max_sync(0xffffffffu, v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
  __syncthreads();
  return max(max(s[0], s[1]), max(s[2], s[3]));
}

template <bool kKvOuter>
__global__ void __launch_bounds__(kTile) schedule_kernel(const ScheduleArgs a) {
  __shared__ int s_seg[kTile];
  __shared__ int s_pos[kTile];
  __shared__ int s_red[4];
  __shared__ int s_red2[4];
  __shared__ unsigned char s_code[kChunk];    // 0 drop, 1 unmasked, 2 needs the exact test, 3 partial
  __shared__ int s_count;
  __shared__ int s_partial;                   // partial entries of the list so far
  __shared__ int s_slot_tile[kBitmapSlots];   // inner tile of the partial entry that got bitmap slot i
  const int t = threadIdx.x;
  const int ot = blockIdx.x, b = blockIdx.y;
  const int o = ot * kTile + t;                       // outer token of this thread
  const bool row_valid = o < a.outer_len;

  const RowBounds rb = load_bounds(a.mask, b, min(o, a.outer_len - 1));
  int o_seg = KVAX_B200_PADDING_SEGMENT_ID, o_pos = 0;
  if (row_valid) {
    if (kKvOuter) {
      o_seg = __ldg(a.tok.kv_seg + (long long)b * a.tok.kv_len + o);
      o_pos = a.tok.sequential ? o : __ldg(a.tok.kv_pos + (long long)b * a.tok.kv_len + o);
    } else {
      o_seg = __ldg(a.tok.q_seg + (long long)b * a.tok.q_len + o);
      o_pos = query_position(a.tok, b, o);
    }
  }

  // CTA-wide ranges on the inner axis (tokens)
  const bool visits = row_valid && rb.up > rb.lo;
  const bool has_full = row_valid && rb.uf > rb.lof;
  const int vis_lo = block_min(visits ? rb.lo : INT32_MAX, s_red);
  int vis_hi = block_max(visits ? rb.up : 0, s_red);
  const int all_full_lo = block_max(row_valid ? rb.lof : 0, s_red);         // full for every row
  const int all_full_hi = min(block_min(row_valid ? rb.uf : INT32_MAX, s_red), a.inner_len);
  vis_hi = min(vis_hi, a.n_inner_tiles * kTile);

  uint32_t* out = a.tiles + ((long long)b * a.n_outer_tiles + ot) * a.n_inner_tiles;
  if (t == 0) { s_count = 0; s_partial = 0; }
  __syncthreads();
  if (vis_hi > vis_lo) {
    const int it0 = max(vis_lo, 0) / kTile;
    const int it1 = min((vis_hi + kTile - 1) / kTile, a.n_inner_tiles);
    const int4* inner_sum = a.inner_summary + (long long)b * a.n_inner_tiles;
    for (int base = it0; base < it1; base += kChunk) {
      const int n = min(kChunk, it1 - base);
      // A: interval classification.  Every thread tests its own row against the summary
      // of 32 inner tiles at a time; a tile stays a candidate when any row may hold an
      // allowed element in it.
      for (int k0 = 0; k0 < n; k0 += 32) {
        uint32_t pass = 0, sure = 0;
        if (row_valid) {
          const int kn = min(32, n - k0);
          for (int k = 0; k < kn; ++k) {
            const int c0 = (base + k0 + k) * kTile, c1 = c0 + kTile;
            const int4 s = __ldg(inner_sum + base + k0 + k);      // {smin, smax, pmin, pmax}
            const bool in_full = (c0 < rb.uf) && (c1 > rb.lof);
            const bool seg_in = (s.x <= o_seg) && (o_seg <= s.y);
            const bool left_ov = (c0 < rb.lof) && (c1 > rb.lo);
            const bool right_ov = (c0 < rb.up) && (c1 > rb.uf);
            const bool causal_ok = kKvOuter ? (s.w >= o_pos) : (o_pos >= s.z);
            const bool cls = kKvOuter ? (right_ov || (left_ov && causal_ok)) : (left_ov || (right_ov && causal_ok));
            pass |= ((in_full || (seg_in && cls)) ? 1u : 0u) << k;
            // sufficient condition for "this row has an allowed element in the tile": part of
            // the tile lies in the row's full range, or the tile is one segment equal to the
            // row's, lies inside one class of the row and (where that class is causal) every
            // position in it passes the causal test
            const bool full_hit = in_full && (max(c0, rb.lof) < a.inner_len);
            const bool single = (s.x == s.y) && (s.x == o_seg);
            const bool left_all = (c0 >= rb.lo) && (c1 <= rb.lof);
            const bool right_all = (c0 >= rb.uf) && (c1 <= rb.up);
            const bool causal_all = kKvOuter ? (s.z >= o_pos) : (o_pos >= s.w);
            const bool cls_all = kKvOuter ? (right_all || (left_all && causal_all)) : (left_all || (right_all && causal_all));
            sure |= ((full_hit || (single && cls_all)) ? 1u : 0u) << k;
          }
        }
        pass = __reduce_or_sync(0xffffffffu, pass);
        sure = __reduce_or_sync(0xffffffffu, sure);
        __syncthreads();
        if ((t & 31) == 0) { s_red[t >> 5] = int(pass); s_red2[t >> 5] = int(sure); }
        __syncthreads();
        if (t < 32 && k0 + t < n) {
          const uint32_t any = uint32_t(s_red[0] | s_red[1] | s_red[2] | s_red[3]);
          const uint32_t any_sure = uint32_t(s_red2[0] | s_red2[1] | s_red2[2] | s_red2[3]);
          const int c0 = (base + k0 + t) * kTile;
          s_code[k0 + t] = (all_full_lo <= c0 && c0 + kTile <= all_full_hi) ? 1
                           : (((any_sure >> t) & 1u) ? 3 : (((any >> t) & 1u) ? 2 : 0));
        }
      }
      __syncthreads();
      // B: exact test of the undecided tiles (CTA-wide, thread t scans the columns for row t)
      for (int k = 0; k < n; ++k) {
        if (s_code[k] != 2) continue;                       // uniform: shared memory value
        const int c0 = (base + k) * kTile;
        const int i = c0 + t;
        int seg = KVAX_B200_PADDING_SEGMENT_ID, pos = 0;
        if (i < a.inner_len) {
          if (kKvOuter) {
            seg = __ldg(a.tok.q_seg + (long long)b * a.tok.q_len + i);
            pos = query_position(a.tok, b, i);
          } else {
            seg = __ldg(a.tok.kv_seg + (long long)b * a.tok.kv_len + i);
            pos = a.tok.sequential ? i : __ldg(a.tok.kv_pos + (long long)b * a.tok.kv_len + i);
          }
        }
        s_seg[t] = seg; s_pos[t] = pos;
        __syncthreads();
        int found = 0;
        if (row_valid) {
          const int lim = min(kTile, a.inner_len - c0);
          for (int j = 0; j < lim; ++j) {
            const bool seg_eq = (s_seg[j] == o_seg);
            const bool causal = kKvOuter ? (s_pos[j] >= o_pos) : (o_pos >= s_pos[j]);
            if (element_allowed<kKvOuter>(rb, c0 + j, seg_eq, causal)) { found = 1; break; }
          }
        }
        const int any = __syncthreads_or(found);
        if (t == 0) s_code[k] = any ? 3 : 0;
      }
      __syncthreads();
      // C: ordered compaction by warp 0.  The first kBitmapSlots partial entries of a list get an element
      // mask of their own (step D) and are marked.
      const bool with_bitmaps = a.bitmaps != nullptr;
      const int partial_before = s_partial;
      if (t < 32) {
        int cnt = s_count, pcnt = partial_before;
        for (int k0 = 0; k0 < n; k0 += 32) {
          const int k = k0 + t;
          const unsigned char code = (k < n) ? s_code[k] : 0;
          const unsigned m = __ballot_sync(0xffffffffu, code != 0);
          const unsigned pm = __ballot_sync(0xffffffffu, code == 3);
          if (code != 0) {
            uint32_t e = uint32_t(base + k) | (code == 3 ? kPartialBit : 0u);
            const int slot = pcnt + __popc(pm & ((1u << t) - 1));
            if (code == 3 && with_bitmaps && slot < kBitmapSlots) { e |= kBitmapBit | (uint32_t(slot) << kBitmapSlotShift); s_slot_tile[slot] = base + k; }
            out[cnt + __popc(m & ((1u << t) - 1))] = e;
          }
          cnt += __popc(m);
          pcnt += __popc(pm);
        }
        if (t == 0) { s_count = cnt; s_partial = pcnt; }
      }
      __syncthreads();
      // D: element masks of the entries marked in this pass: thread t = outer row t, the very function the consumers
      // would call on the same arguments
      if (with_bitmaps) {
        const int slot_end = min(s_partial, kBitmapSlots);
        const int32_t* inner_seg = a.tok.kv_seg + (long long)b * a.tok.kv_len;
        const int32_t* inner_pos = a.tok.sequential ? nullptr : a.tok.kv_pos + (long long)b * a.tok.kv_len;
        for (int slot = partial_before; slot < slot_end; ++slot) {
          const int c0 = s_slot_tile[slot] * kTile;
          uint32_t w[4];
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            w[ch] = kKvOuter ? kv_outer_keep32(a.tok, rb, b, row_valid, o_seg, o_pos, c0 + ch * 32)
                             : keep_bits32<false>(rb, c0 + ch * 32, a.inner_len, row_valid, o_seg, o_pos, inner_seg + c0 + ch * 32,
                                                  inner_pos ? inner_pos + c0 + ch * 32 : nullptr);
          a.bitmaps[(((long long)b * a.n_outer_tiles + ot) * kBitmapSlots + slot) * kTile + t] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncthreads();                        // s_slot_tile is reused by the next pass
      }
    }
  }
  if (t == 0) a.counts[(long long)b * a.n_outer_tiles + ot] = s_count;
}

// Launch order.  Outer tiles are launched in blocks of kRowChunk neighbours (same batch row, consecutive tile
// indices), the blocks sorted by their mean list length, longest first: the tail of a launch is then made of short
// work items, and the CTAs that are resident together belong to neighbouring outer tiles of a few heads, which walk
// through the same inner tiles (one document) -- their loads hit in L2 and, in the fused backward, their reduce-adds
// fall on dQ accumulator lines that are still there.  (Sorting single tiles by length instead mixes the documents
// of a batch: measured 22 GB of DRAM traffic per fused-backward launch on the 32k workload for 3 GB of algorithmic bytes.)
// Counting sort of the blocks in one CTA; the order among blocks of equal key is not fixed.
constexpr int kBins = 2048;                // two per thread of order_kernel
__global__ void __launch_bounds__(1024) order_kernel(const int32_t* counts, int32_t* order, int32_t* pair_order, int n_outer,
                                                     int batch) {
  __shared__ int hist[kBins];        // rows per key, then the running start of the key's rows
  __shared__ int hist2[kBins];       // the same in units of pairs of neighbouring rows
  const int blocks_per_row = (n_outer + kRowChunk - 1) / kRowChunk;
  const int n_blocks = blocks_per_row * batch;
  auto block_info = [&](int blk, int* first_row, int* rows) -> int {     // returns the key (mean list length, clamped)
    const int b = blk / blocks_per_row, t0 = (blk - b * blocks_per_row) * kRowChunk;
    const int n = min(kRowChunk, n_outer - t0);
    *first_row = b * n_outer + t0;
    *rows = n;
    int sum = 0;
    for (int j = 0; j < n; ++j) sum += counts[*first_row + j];
    return min((sum + n - 1) / n, kBins - 1);
  };
  for (int i = threadIdx.x; i < kBins; i += blockDim.x) { hist[i] = 0; hist2[i] = 0; }
  __syncthreads();
  for (int blk = threadIdx.x; blk < n_blocks; blk += blockDim.x) {
    int first, rows;
    const int key = block_info(blk, &first, &rows);
    atomicAdd(&hist[key], rows);
    atomicAdd(&hist2[key], (rows + 1) / 2);
  }
  __syncthreads();
  // exclusive prefix over descending bins: start[bin] = number of rows in blocks with a larger key.  Thread r takes the
  // bins kBins - 1 - 2r and kBins - 2 - 2r (two per thread of the 1024), a block-wide scan of the pair sums does the rest.
  {
    __shared__ int warp_tot[32], warp_tot2[32];
    const int r = threadIdx.x, lane = r & 31, w = r >> 5;
    const int b0 = kBins - 1 - 2 * r, b1 = b0 - 1;
    const int c0 = hist[b0], c1 = hist[b1], d0 = hist2[b0], d1 = hist2[b1];
    int inc = c0 + c1, inc2 = d0 + d1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, o), t2 = __shfl_up_sync(0xffffffffu, inc2, o);
      if (lane >= o) { inc += t; inc2 += t2; }
    }
    if (lane == 31) { warp_tot[w] = inc; warp_tot2[w] = inc2; }
    __syncthreads();
    if (w == 0) {
      int t = warp_tot[lane], t2 = warp_tot2[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, t, o), u2 = __shfl_up_sync(0xffffffffu, t2, o);
        if (lane >= o) { t += u; t2 += u2; }
      }
      warp_tot[lane] = t; warp_tot2[lane] = t2;            // inclusive totals of the warps
    }
    __syncthreads();
    const int base = (w ? warp_tot[w - 1] : 0) + inc - (c0 + c1), base2 = (w ? warp_tot2[w - 1] : 0) + inc2 - (d0 + d1);
    hist[b0] = base; hist[b1] = base + c0;
    hist2[b0] = base2; hist2[b1] = base2 + d0;
  }
  __syncthreads();
  for (int blk = threadIdx.x; blk < n_blocks; blk += blockDim.x) {
    int first, rows;
    const int key = block_info(blk, &first, &rows);
    const int pos = atomicAdd(&hist[key], rows);
    for (int j = 0; j < rows; ++j) order[pos + j] = first + j;
    // a block starts at an even tile of its batch row (kRowChunk is even): its pairs are (first + 2j, first + 2j + 1)
    const int pos2 = atomicAdd(&hist2[key], (rows + 1) / 2);
    for (int j = 0; j < (rows + 1) / 2; ++j) pair_order[pos2 + j] = first + 2 * j;
  }
}

}  // namespace

void launch_tile_summaries(const TokenInfo& tok, int batch, int4* q_sum, int4* kv_sum, cudaStream_t s) {
  const int nq = (tok.q_len + kTile - 1) / kTile, nk = (tok.kv_len + kTile - 1) / kTile;
  const long long warps = (long long)batch * (nq + nk);
  tile_summary_kernel<<<int((warps + 7) / 8), 256, 0, s>>>(tok, q_sum, kv_sum, nq, nk, batch);
}

void launch_schedule(bool kv_outer, const ScheduleArgs& a, int batch, cudaStream_t s) {
  dim3 grid(a.n_outer_tiles, batch);
  if (kv_outer) schedule_kernel<true><<<grid, kTile, 0, s>>>(a);
  else schedule_kernel<false><<<grid, kTile, 0, s>>>(a);
  order_kernel<<<1, 1024, 0, s>>>(a.counts, a.order, a.pair_order, a.n_outer_tiles, batch);
}

}  // namespace kvx
