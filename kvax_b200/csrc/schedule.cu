// Tile-list builder: turns a block mask (four bound arrays at the caller's block sizes)
// into, for every 128-row outer tile, the ascending list of 128-column inner tiles the
// attention kernels must visit.  A tile whose every element lies in the "full" range of
// every row is emitted as unmasked; a tile in which no element survives the reference's
// element-level rule is dropped (it contributes nothing to any row); the rest are
// emitted as partial and masked per element by the consumer.
//
// One CTA of 128 threads per (outer tile, batch); thread t owns outer row t.
#include "attn_common.cuh"
#include "internal.h"

namespace kvx {


template <bool kKvOuter>
__global__ void __launch_bounds__(kTile) schedule_kernel(const ScheduleArgs a) {
  __shared__ int s_seg[kTile];
  __shared__ int s_pos[kTile];
  __shared__ int s_red[4][4];
  const int t = threadIdx.x;
  const int ot = blockIdx.x, b = blockIdx.y;
  const int o = ot * kTile + t;                       // outer token of this thread
  const bool row_valid = o < a.outer_len;

  RowBounds rb = load_bounds(a.mask, b, min(o, a.outer_len - 1));
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

  // CTA-wide: visited range [vis_lo, vis_hi) and the range that is "full" for all rows
  const bool visits = row_valid && rb.up > rb.lo;
  int vis_lo = visits ? rb.lo : INT32_MAX, vis_hi = visits ? rb.up : 0;
  int full_lo = row_valid ? rb.lof : 0, full_hi = row_valid ? rb.uf : INT32_MAX;
  vis_lo = __reduce_min_sync(0xffffffffu, vis_lo);
  vis_hi = __reduce_max_sync(0xffffffffu, vis_hi);
  full_lo = __reduce_max_sync(0xffffffffu, full_lo);
  full_hi = __reduce_min_sync(0xffffffffu, full_hi);
  if ((t & 31) == 0) {
    s_red[t >> 5][0] = vis_lo; s_red[t >> 5][1] = vis_hi; s_red[t >> 5][2] = full_lo; s_red[t >> 5][3] = full_hi;
  }
  __syncthreads();
  vis_lo = min(min(s_red[0][0], s_red[1][0]), min(s_red[2][0], s_red[3][0]));
  vis_hi = max(max(s_red[0][1], s_red[1][1]), max(s_red[2][1], s_red[3][1]));
  full_lo = max(max(s_red[0][2], s_red[1][2]), max(s_red[2][2], s_red[3][2]));
  full_hi = min(min(s_red[0][3], s_red[1][3]), min(s_red[2][3], s_red[3][3]));
  full_hi = min(full_hi, a.inner_len);
  vis_hi = min(vis_hi, ((a.inner_len + kTile - 1) / kTile) * kTile);

  uint32_t* out = a.tiles + ((long long)b * a.n_outer_tiles + ot) * a.n_inner_tiles;
  int count = 0;
  if (vis_hi > vis_lo) {
    const int it0 = max(vis_lo, 0) / kTile;
    const int it1 = min((vis_hi + kTile - 1) / kTile, a.n_inner_tiles);
    for (int it = it0; it < it1; ++it) {
      const int c0 = it * kTile;
      if (full_lo <= c0 && c0 + kTile <= full_hi) {     // unmasked for every row
        if (t == 0) out[count] = uint32_t(it);
        ++count;
        continue;
      }
      // stage the inner tile's segment ids and positions
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
      __syncthreads();                                   // previous iteration's readers are done
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
      if (__syncthreads_or(found)) {
        if (t == 0) out[count] = uint32_t(it) | kPartialBit;
        ++count;
      }
    }
  }
  if (t == 0) a.counts[(long long)b * a.n_outer_tiles + ot] = count;
}

void launch_schedule(bool kv_outer, const ScheduleArgs& a, int batch, cudaStream_t s) {
  dim3 grid(a.n_outer_tiles, batch);
  if (kv_outer) schedule_kernel<true><<<grid, kTile, 0, s>>>(a);
  else schedule_kernel<false><<<grid, kTile, 0, s>>>(a);
}

}  // namespace kvx
