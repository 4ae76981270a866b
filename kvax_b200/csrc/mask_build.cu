// Block-mask builder for sm_100a.
//
// Main path: ONE launch of thread-block clusters builds up to three masks (forward, dq, dkdv).  A
// cluster of up to 8 CTAs owns one batch row.  Every CTA summarises its slice of the row's blocks
// (one warp per block: coalesced 16-byte loads of positions and segment ids, warp min/max, one int4
// {seg_min, seg_max, pos_min, pos_max} per block, PAD already remapped) into its own shared memory,
// plus one summary per group of 32 blocks; sides that several masks share (same block size and PAD
// id) are summarised once, so the inputs are read from HBM exactly once.  After a cluster barrier
// every warp takes outer blocks of its slice and finds the four bounds by reading the other CTAs'
// summaries through distributed shared memory: the group summaries rule out whole groups of 32 inner
// blocks at a time, and only the first / last groups that can hold a hit are looked at block by
// block.  Masks with identical geometry (forward and dq at equal block sizes) are computed once and
// stored twice.  Nothing goes through global scratch memory.
//
// Fallback (rows whose summaries do not fit in shared memory, and the variant with built-in scratch
// memory): two launches,
//   1. mask_summary_kernel: one warp per block of either side; coalesced 16-byte loads of
//      positions and segment ids, warp min/max reductions, one int4 summary
//      {seg_min, seg_max, pos_min, pos_max} per block (PAD already remapped).
//   2. mask_bounds_kernel: one warp per outer block; lanes stride over the inner-block
//      summaries, evaluate the "may attend" / "fully attends" interval tests and fold the
//      four bounds with warp min/max reductions; lane 0 applies the host fix-ups.
//
// Semantics follow kvax/ops/mask_creator.py:26-152 (kernel) and :212-259, :317-333 (host
// steps) exactly; outputs are bit-identical with the reference's mask tensors.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <limits.h>

#include "../../include/kvax_b200.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kWarpsPerBlock = 8;

struct SideJob {           // blocks of one side (query or kv) of one mask
  const int32_t* pos;
  const int32_t* seg;
  int4* summary;           // (B, n_blocks)
  int32_t len;             // unpadded length
  int32_t block;
  int32_t n_blocks;        // ceil(len / block)
  int32_t pos_fill;        // padding value for positions beyond `len`
  int32_t pad_id;          // what PADDING_SEGMENT_ID is remapped to
  int32_t first_warp;      // global warp index of this job's first block
};

struct SummaryArgs {
  SideJob jobs[6];
  int32_t n_jobs;
  int32_t batch;
  int32_t total_warps;
};

struct BoundsJob {
  const int4* outer;       // (B, n_outer)
  const int4* inner;       // (B, n_inner)
  int32_t* lower; int32_t* upper; int32_t* lower_full; int32_t* upper_full;
  int32_t n_outer, n_inner;
  int32_t kv_outer;
  int32_t pad_id;
  int32_t first_warp;
};

struct BoundsArgs {
  BoundsJob jobs[3];
  int32_t n_jobs;
  int32_t batch;
  int32_t skip_pad;
  int32_t total_warps;
};

__device__ __forceinline__ void fold(int pos, int seg, int pad_id, int& smin, int& smax, int& pmin, int& pmax) {
  seg = (seg == KVAX_B200_PADDING_SEGMENT_ID) ? pad_id : seg;
  smin = min(smin, seg); smax = max(smax, seg);
  pmin = min(pmin, pos); pmax = max(pmax, pos);
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) mask_summary_kernel(const SummaryArgs args) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (warp >= args.total_warps) return;
  int j = 0;
#pragma unroll
  for (int t = 1; t < 6; ++t)
    if (t < args.n_jobs && warp >= args.jobs[t].first_warp) j = t;
  const SideJob& job = args.jobs[j];
  const int local = int(warp - job.first_warp);       // = b * n_blocks + blk
  const int b = local / job.n_blocks;
  const int blk = local - b * job.n_blocks;
  const long long row = (long long)b * job.len;
  const int start = blk * job.block;
  const int end = min(start + job.block, job.len);

  int smin = INT_MAX, smax = INT_MIN, pmin = INT_MAX, pmax = INT_MIN;
  const int32_t* pos = job.pos + row;
  const int32_t* seg = job.seg + row;
  // vector path when this block's first element is 16-byte aligned in both arrays
  const bool vec_ok = (((reinterpret_cast<uintptr_t>(pos + start) | reinterpret_cast<uintptr_t>(seg + start)) & 15) == 0);
  int i = start;
  if (vec_ok) {
    const int n4 = (end - start) >> 2;
    const int4* p4 = reinterpret_cast<const int4*>(pos + start);
    const int4* s4 = reinterpret_cast<const int4*>(seg + start);
    for (int v = lane; v < n4; v += 32) {
      const int4 p = __ldg(p4 + v);
      const int4 s = __ldg(s4 + v);
      fold(p.x, s.x, job.pad_id, smin, smax, pmin, pmax);
      fold(p.y, s.y, job.pad_id, smin, smax, pmin, pmax);
      fold(p.z, s.z, job.pad_id, smin, smax, pmin, pmax);
      fold(p.w, s.w, job.pad_id, smin, smax, pmin, pmax);
    }
    i = start + (n4 << 2);
  }
  for (int e = i + lane; e < end; e += 32) fold(__ldg(pos + e), __ldg(seg + e), job.pad_id, smin, smax, pmin, pmax);
  // elements added by padding to the block size (mask_creator.py:212-225)
  if (end < start + job.block && lane == 0)
    fold(job.pos_fill, KVAX_B200_PADDING_SEGMENT_ID, job.pad_id, smin, smax, pmin, pmax);

  smin = __reduce_min_sync(0xffffffffu, smin);
  smax = __reduce_max_sync(0xffffffffu, smax);
  pmin = __reduce_min_sync(0xffffffffu, pmin);
  pmax = __reduce_max_sync(0xffffffffu, pmax);
  if (lane == 0) job.summary[local] = make_int4(smin, smax, pmin, pmax);
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) mask_bounds_kernel(const BoundsArgs args) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (warp >= args.total_warps) return;
  int j = 0;
#pragma unroll
  for (int t = 1; t < 3; ++t)
    if (t < args.n_jobs && warp >= args.jobs[t].first_warp) j = t;
  const BoundsJob& job = args.jobs[j];
  const int local = int(warp - job.first_warp);       // = b * n_outer + o
  const int b = local / job.n_outer;
  const int n = job.n_inner;

  const int4 o = __ldg(job.outer + local);            // {smin, smax, pmin, pmax}
  const bool o_single = (o.x == o.y);
  int lo = n, up = 0, lof = n, upf = 0;
  const bool outer_all_pad = args.skip_pad && o_single && (o.x == job.pad_id);   // :69-76
  if (!outer_all_pad) {
    const int4* inner = job.inner + (long long)b * n;
    for (int i = lane; i < n; i += 32) {
      const int4 s = __ldg(inner + i);
      const bool seg_overlap = (s.x <= o.y) && (o.x <= s.y);                       // :98-101
      const bool both_single = o_single && (s.x == s.y);                           // :102
      bool pos_any, pos_all;
      if (!job.kv_outer) { pos_any = o.w >= s.z; pos_all = o.z >= s.w; }            // :110-112
      else               { pos_any = s.w >= o.z; pos_all = s.z >= o.w; }            // :113-115
      bool attend = pos_any && seg_overlap;
      if (args.skip_pad) attend = attend && (s.x != job.pad_id);                   // :122-124
      const bool full = both_single && pos_all && attend;                          // :139
      if (attend) { lo = min(lo, i); up = max(up, i + 1); }
      if (full)   { lof = min(lof, i); upf = max(upf, i + 1); }
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    up = __reduce_max_sync(0xffffffffu, up);
    lof = __reduce_min_sync(0xffffffffu, lof);
    upf = __reduce_max_sync(0xffffffffu, upf);
    // host fix-ups, mask_creator.py:317-333
    if (lo == n) lo = up;
    if (lof == n) lof = job.kv_outer ? up : lo;
    if (upf < lof) upf = lof;
  } else {
    lo = up = lof = upf = 0;
  }
  if (lane == 0) {
    job.lower[local] = lo;
    job.upper[local] = up;
    job.lower_full[local] = lof;
    job.upper_full[local] = upf;
  }
}

inline int cdiv(long long a, long long b) { return int((a + b - 1) / b); }
inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// ---------------------------------------------------------------------------------------
// Cluster path
// ---------------------------------------------------------------------------------------
constexpr int kMaxSets = 6;             // distinct (side, block size, PAD id) combinations of three masks
constexpr int kClusterThreads = 512;
constexpr int kGroup = 32;              // inner blocks per group summary

struct SetDesc {
  const int32_t* pos;
  const int32_t* seg;
  int32_t len, block, n_blocks;
  int32_t pos_fill, pad_id;
  int32_t per;             // blocks per CTA of the cluster (a multiple of kGroup)
  int32_t smem_off;        // int4 offset of this set's summaries in a CTA's shared memory; group summaries follow
  int32_t row_off;         // int4 offset of the CTA's private copy of the whole row's summaries (cluster * per
                           // block summaries, then cluster * per / kGroup group summaries), or -1: read remotely
};

struct ClusterMask {
  int32_t* lower; int32_t* upper; int32_t* lower_full; int32_t* upper_full;
  int32_t outer_set, inner_set, kv_outer;
  int32_t same_as;         // index of an earlier mask with the same geometry (its results are stored here too), or -1
};

struct ClusterArgs {
  SetDesc sets[kMaxSets];
  ClusterMask masks[3];
  int32_t n_sets, n_masks, batch, skip_pad, cluster;
};

__device__ __forceinline__ int4 warp_reduce_summary(int4 v) {
  v.x = __reduce_min_sync(0xffffffffu, v.x);
  v.y = __reduce_max_sync(0xffffffffu, v.y);
  v.z = __reduce_min_sync(0xffffffffu, v.z);
  v.w = __reduce_max_sync(0xffffffffu, v.w);
  return v;
}

// Summary of block `blk` of batch row `row_off` of one side; whole warp.
__device__ __forceinline__ int4 block_summary(const SetDesc& sd, long long row_off, int blk, int lane) {
  const int start = blk * sd.block;
  const int end = min(start + sd.block, sd.len);
  int smin = INT_MAX, smax = INT_MIN, pmin = INT_MAX, pmax = INT_MIN;
  const int32_t* pos = sd.pos + row_off;
  const int32_t* seg = sd.seg + row_off;
  const bool vec_ok = (((reinterpret_cast<uintptr_t>(pos + start) | reinterpret_cast<uintptr_t>(seg + start)) & 15) == 0);
  int i = start;
  if (vec_ok) {
    const int n4 = (end - start) >> 2;
    const int4* p4 = reinterpret_cast<const int4*>(pos + start);
    const int4* s4 = reinterpret_cast<const int4*>(seg + start);
    for (int v = lane; v < n4; v += 32) {
      const int4 p = __ldg(p4 + v);
      const int4 q = __ldg(s4 + v);
      fold(p.x, q.x, sd.pad_id, smin, smax, pmin, pmax);
      fold(p.y, q.y, sd.pad_id, smin, smax, pmin, pmax);
      fold(p.z, q.z, sd.pad_id, smin, smax, pmin, pmax);
      fold(p.w, q.w, sd.pad_id, smin, smax, pmin, pmax);
    }
    i = start + (n4 << 2);
  }
  for (int e = i + lane; e < end; e += 32) fold(__ldg(pos + e), __ldg(seg + e), sd.pad_id, smin, smax, pmin, pmax);
  if (end < start + sd.block && lane == 0)            // elements added by padding to the block size (mask_creator.py:212-225)
    fold(sd.pos_fill, KVAX_B200_PADDING_SEGMENT_ID, sd.pad_id, smin, smax, pmin, pmax);
  return warp_reduce_summary(make_int4(smin, smax, pmin, pmax));
}

// "may attend" / "fully attends" of outer block o against inner block s (mask_creator.py:98-139)
__device__ __forceinline__ void block_tests(const int4& o, bool o_single, const int4& s, bool kv_outer, bool skip_pad, int pad_id,
                                            bool* attend, bool* full) {
  const bool seg_overlap = (s.x <= o.y) && (o.x <= s.y);
  const bool both_single = o_single && (s.x == s.y);
  bool pos_any, pos_all;
  if (!kv_outer) { pos_any = o.w >= s.z; pos_all = o.z >= s.w; }
  else           { pos_any = s.w >= o.z; pos_all = s.z >= o.w; }
  bool att = pos_any && seg_overlap;
  if (skip_pad) att = att && (s.x != pad_id);
  *attend = att;
  *full = both_single && pos_all && att;
}


// Where the summaries of a row's inner blocks are read from: the CTA's private copy of the whole row, or the
// shared memory of the CTAs of the cluster that computed them.
struct LocalReader {
  const int4* row;         // block summaries of the whole row, then the group summaries
  int total;               // block summaries in the copy (cluster * per)
  __device__ __forceinline__ int4 inner(int i) const { return row[i]; }
  __device__ __forceinline__ int4 group(int g) const { return row[total + g]; }
};
struct RemoteReader {
  cg::cluster_group cluster;
  int4* base;              // this set's area in every CTA: `per` block summaries, then per / kGroup group summaries
  int per;
  __device__ __forceinline__ int4 inner(int i) const {
    const int rank = i / per;
    return *(cluster.map_shared_rank(base, rank) + (i - rank * per));
  }
  __device__ __forceinline__ int4 group(int g) const {
    const int gper = per / kGroup, rank = g / gper;
    return *(cluster.map_shared_rank(base, rank) + per + (g - rank * gper));
  }
};

// The four bounds of one outer block (whole warp), before the fix-ups: lower / upper over `attend`, lower_full /
// upper_full over `full`, `n` / 0 when nothing is found.  Group summaries rule out groups of 32 inner blocks: a group
// passes the interval tests whenever one of its members does (the PAD test is left to the members, it is not monotone
// under min / max).  Only the first and the last group with a hit are looked at block by block, plus -- rarely -- the
// groups between them when the `full` range does not show in those two.
template <class Reader>
__device__ __forceinline__ void find_bounds(const Reader& rd, const int4 o, const bool o_single, const int n, const int n_groups,
                                            const bool kv_outer, const bool skip_pad, const int pad_id, const int lane,
                                            int& lo, int& up, int& lof, int& upf) {
  lo = n; up = 0; lof = n; upf = 0;
  auto candidates = [&](int g0) -> unsigned {
    const int g = g0 + lane;
    bool cand = false, ful;
    if (g < n_groups) block_tests(o, o_single, rd.group(g), kv_outer, false, pad_id, &cand, &ful);
    return __ballot_sync(0xffffffffu, cand);
  };
  auto members = [&](int gi, unsigned& am, unsigned& fm) {
    const int i = gi * kGroup + lane;
    bool att = false, ful = false;
    if (i < n) block_tests(o, o_single, rd.inner(i), kv_outer, skip_pad, pad_id, &att, &ful);
    am = __ballot_sync(0xffffffffu, att);
    fm = __ballot_sync(0xffffffffu, ful);
  };
  if (n_groups <= 32) {
    const unsigned cand = candidates(0);
    unsigned am = 0, fm = 0;
    int g_first = -1;
    for (unsigned rest = cand; rest; rest &= rest - 1) {            // ascending to the first group with a hit
      const int gi = __ffs(rest) - 1;
      members(gi, am, fm);
      if (am) { g_first = gi; break; }
    }
    if (g_first < 0) return;
    const unsigned am_f = am, fm_f = fm;
    lo = g_first * kGroup + __ffs(am_f) - 1;
    int g_last = g_first;
    unsigned am_l = am_f, fm_l = fm_f;
    for (unsigned high = cand & ~((2u << g_first) - 1u); high;) {   // descending to the last group with a hit
      const int gi = 31 - __clz(high);
      high &= ~(1u << gi);
      members(gi, am, fm);
      if (am) { g_last = gi; am_l = am; fm_l = fm; break; }
    }
    up = g_last * kGroup + (31 - __clz(am_l)) + 1;
    if (!o_single) return;                                          // `full` needs a single-segment outer block
    // `full` implies `attend`: the full range lies inside [g_first, g_last]
    const unsigned mid = (g_last > g_first) ? (cand & ~((2u << g_first) - 1u) & ((1u << g_last) - 1u)) : 0u;
    int g_lof = -1;
    if (fm_f) { lof = g_first * kGroup + __ffs(fm_f) - 1; g_lof = g_first; }
    else {
      for (unsigned rest = mid; rest; rest &= rest - 1) {
        const int gi = __ffs(rest) - 1;
        members(gi, am, fm);
        if (fm) { lof = gi * kGroup + __ffs(fm) - 1; g_lof = gi; break; }
      }
      if (g_lof < 0 && g_last > g_first && fm_l) { lof = g_last * kGroup + __ffs(fm_l) - 1; g_lof = g_last; }
    }
    if (g_lof < 0) return;                                          // no full block at all
    if (g_last > g_first && fm_l) { upf = g_last * kGroup + (31 - __clz(fm_l)) + 1; return; }
    for (unsigned high = mid; high;) {                              // descending through the groups in between
      const int gi = 31 - __clz(high);
      high &= ~(1u << gi);
      if (gi < g_lof) break;
      members(gi, am, fm);
      if (fm) { upf = gi * kGroup + (31 - __clz(fm)) + 1; return; }
    }
    upf = g_first * kGroup + (31 - __clz(fm_f)) + 1;                // then the hit is in the first group (g_lof == g_first)
    return;
  }
  // rows with more than 1024 inner blocks: windows of 32 groups, ascending for the first hits, descending for the last
  bool lo_done = false, lof_done = !o_single;
  for (int g0 = 0; g0 < n_groups && !(lo_done && lof_done); g0 += 32) {
    unsigned rest = candidates(g0);
    while (rest && !(lo_done && lof_done)) {
      const int gi = g0 + __ffs(rest) - 1;
      rest &= rest - 1;
      unsigned am, fm;
      members(gi, am, fm);
      if (!lo_done && am) { lo = gi * kGroup + __ffs(am) - 1; lo_done = true; }
      if (!lof_done && fm) { lof = gi * kGroup + __ffs(fm) - 1; lof_done = true; }
    }
  }
  bool up_done = !lo_done, upf_done = !(o_single && lof != n);
  for (int g0 = ((n_groups - 1) / 32) * 32; g0 >= 0 && !(up_done && upf_done); g0 -= 32) {
    unsigned rest = candidates(g0);
    while (rest && !(up_done && upf_done)) {
      const int bit = 31 - __clz(rest);
      rest &= ~(1u << bit);
      const int gi = g0 + bit;
      unsigned am, fm;
      members(gi, am, fm);
      if (!up_done && am) { up = gi * kGroup + (31 - __clz(am)) + 1; up_done = true; }
      if (!upf_done && fm) { upf = gi * kGroup + (31 - __clz(fm)) + 1; upf_done = true; }
    }
  }
}

__global__ void __launch_bounds__(kClusterThreads, 2) mask_cluster_kernel(const ClusterArgs a) {
  extern __shared__ int4 sm[];
  cg::cluster_group cluster = cg::this_cluster();
  const int c = int(cluster.block_rank());
  const int b = blockIdx.x / a.cluster;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kClusterThreads / 32;

  // ---- phase 1: summaries of this CTA's slice of every set, then one summary per group of 32 blocks
  for (int si = 0; si < a.n_sets; ++si) {
    const SetDesc& sd = a.sets[si];
    int4* sum = sm + sd.smem_off;
    const int first = c * sd.per;
    const long long row_off = (long long)b * sd.len;
    // Fast path: blocks of at most 128 tokens whose first element is 16-byte aligned are one int4 per lane and
    // array; a warp then takes four blocks per step with all eight loads in flight before the first reduction.
    const bool fast = sd.block <= 128 && (sd.block & 3) == 0 &&
                      (((reinterpret_cast<uintptr_t>(sd.pos + row_off) | reinterpret_cast<uintptr_t>(sd.seg + row_off)) & 15) == 0);
    if (fast) {
      const int n4 = sd.block >> 2;
      for (int k0 = warp * 4; k0 < sd.per; k0 += kWarps * 4) {
        int4 pv[4], sv[4];
        bool have[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int blk = first + k0 + j;
          const int e0 = blk * sd.block + lane * 4;                  // first of this lane's four tokens
          have[j] = (k0 + j < sd.per) && (blk < sd.n_blocks) && (lane < n4) && (e0 + 4 <= sd.len);
          if (have[j]) {
            pv[j] = __ldg(reinterpret_cast<const int4*>(sd.pos + row_off + e0));
            sv[j] = __ldg(reinterpret_cast<const int4*>(sd.seg + row_off + e0));
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int blk = first + k0 + j;
          if (k0 + j >= sd.per) break;
          int smin = INT_MAX, smax = INT_MIN, pmin = INT_MAX, pmax = INT_MIN;
          if (blk < sd.n_blocks) {
            if (have[j]) {
              fold(pv[j].x, sv[j].x, sd.pad_id, smin, smax, pmin, pmax);
              fold(pv[j].y, sv[j].y, sd.pad_id, smin, smax, pmin, pmax);
              fold(pv[j].z, sv[j].z, sd.pad_id, smin, smax, pmin, pmax);
              fold(pv[j].w, sv[j].w, sd.pad_id, smin, smax, pmin, pmax);
            } else if (lane < n4) {                                   // the block is cut by the end of the row
              const int e0 = blk * sd.block + lane * 4;
              for (int e = e0; e < min(e0 + 4, sd.len); ++e)
                fold(__ldg(sd.pos + row_off + e), __ldg(sd.seg + row_off + e), sd.pad_id, smin, smax, pmin, pmax);
            }
            if (blk * sd.block + sd.block > sd.len && lane == 0)      // elements added by padding to the block size
              fold(sd.pos_fill, KVAX_B200_PADDING_SEGMENT_ID, sd.pad_id, smin, smax, pmin, pmax);
          }
          const int4 v = warp_reduce_summary(make_int4(smin, smax, pmin, pmax));
          if (lane == 0) sum[k0 + j] = v;
        }
      }
    } else {
      for (int k = warp; k < sd.per; k += kWarps) {
        const int blk = first + k;
        int4 v = make_int4(INT_MAX, INT_MIN, INT_MAX, INT_MIN);     // beyond the row: matches nothing
        if (blk < sd.n_blocks) v = block_summary(sd, row_off, blk, lane);
        if (lane == 0) sum[k] = v;
      }
    }
  }
  __syncthreads();
  for (int si = 0; si < a.n_sets; ++si) {
    const SetDesc& sd = a.sets[si];
    const int4* sum = sm + sd.smem_off;
    int4* grp = sm + sd.smem_off + sd.per;
    for (int g = warp; g < sd.per / kGroup; g += kWarps) {
      const int4 v = warp_reduce_summary(sum[g * kGroup + lane]);
      if (lane == 0) grp[g] = v;
    }
  }
  cluster.sync();

  // ---- every CTA takes a private copy of the whole row's summaries (when they fit): the scans below then only
  //      touch local shared memory and the CTAs of the cluster need each other no longer
  bool all_local = true;
  for (int si = 0; si < a.n_sets; ++si) {
    const SetDesc& sd = a.sets[si];
    if (sd.row_off < 0) { all_local = false; continue; }
    int4* base = sm + sd.smem_off;
    int4* row = sm + sd.row_off;
    const int total = a.cluster * sd.per, gper = sd.per / kGroup;
    for (int idx = threadIdx.x; idx < total; idx += kClusterThreads) {
      const int rank = idx / sd.per;
      row[idx] = *(cluster.map_shared_rank(base, rank) + (idx - rank * sd.per));
    }
    for (int idx = threadIdx.x; idx < a.cluster * gper; idx += kClusterThreads) {
      const int rank = idx / gper;
      row[total + idx] = *(cluster.map_shared_rank(base, rank) + sd.per + (idx - rank * gper));
    }
  }
  if (all_local) cluster.sync(); else __syncthreads();

  // ---- phase 2: bounds of the outer blocks of this CTA's slice
  for (int m = 0; m < a.n_masks; ++m) {
    const ClusterMask& mk = a.masks[m];
    if (mk.same_as >= 0) continue;                                  // stored together with the mask it equals
    const SetDesc& so = a.sets[mk.outer_set];
    const SetDesc& si = a.sets[mk.inner_set];
    const int n = si.n_blocks, n_groups = (n + kGroup - 1) / kGroup;
    const bool kv_outer = mk.kv_outer != 0, skip_pad = a.skip_pad != 0;
    const int pad_id = so.pad_id;
    const int4* o_sum = sm + so.smem_off;
    const LocalReader local{si.row_off >= 0 ? sm + si.row_off : nullptr, a.cluster * si.per};
    const RemoteReader remote{cluster, sm + si.smem_off, si.per};
    // results of mask m also go to the masks with the same geometry
    int32_t* out[3][4];
    int n_out = 0;
    for (int m2 = m; m2 < a.n_masks; ++m2) {
      if (m2 != m && a.masks[m2].same_as != m) continue;
      out[n_out][0] = a.masks[m2].lower; out[n_out][1] = a.masks[m2].upper;
      out[n_out][2] = a.masks[m2].lower_full; out[n_out][3] = a.masks[m2].upper_full;
      ++n_out;
    }
    for (int k = warp; k < so.per; k += kWarps) {
      const int ob = c * so.per + k;
      if (ob >= so.n_blocks) break;
      const int4 o = o_sum[k];
      const bool o_single = (o.x == o.y);
      int lo = 0, up = 0, lof = 0, upf = 0;
      const bool outer_all_pad = skip_pad && o_single && (o.x == pad_id);              // :69-76: all four stay 0
      if (!outer_all_pad) {
        if (local.row) find_bounds(local, o, o_single, n, n_groups, kv_outer, skip_pad, pad_id, lane, lo, up, lof, upf);
        else find_bounds(remote, o, o_single, n, n_groups, kv_outer, skip_pad, pad_id, lane, lo, up, lof, upf);
        // host fix-ups, mask_creator.py:317-333
        if (lo == n) lo = up;
        if (lof == n) lof = kv_outer ? up : lo;
        if (upf < lof) upf = lof;
      }
      if (lane < 4) {
        const long long idx = (long long)b * so.n_blocks + ob;
        const int val = lane == 0 ? lo : (lane == 1 ? up : (lane == 2 ? lof : upf));
        for (int t = 0; t < n_out; ++t) out[t][lane][idx] = val;
      }
    }
  }
  if (!all_local) cluster.sync();      // no CTA leaves while another may still read its summaries
}

constexpr size_t kClusterSmemLimit = 200 * 1024;
constexpr size_t kClusterRowCopyLimit = 96 * 1024;     // beyond this the scans read the other CTAs' shared memory

// KVAX_B200_EUNSUPPORTED when the row's summaries do not fit in shared memory (the caller then takes the
// two-launch path); KVAX_B200_OK after a successful launch.
int mask_build_clusters(const kvax_b200_mask_params* p, kvax_b200_stream_t stream) {
  ClusterArgs a{};
  a.batch = p->batch;
  a.skip_pad = p->skip_pad_tokens ? 1 : 0;
  a.n_masks = p->n_masks;
  int max_blocks = 1;
  auto find_set = [&](const int32_t* pos, const int32_t* seg, int len, int block, int pos_fill, int pad_id) {
    for (int i = 0; i < a.n_sets; ++i) {
      const SetDesc& sd = a.sets[i];
      if (sd.pos == pos && sd.seg == seg && sd.len == len && sd.block == block && sd.pos_fill == pos_fill && sd.pad_id == pad_id) return i;
    }
    SetDesc& sd = a.sets[a.n_sets];
    sd = SetDesc{pos, seg, len, block, cdiv(len, block), pos_fill, pad_id, 0, 0, -1};
    if (sd.n_blocks > max_blocks) max_blocks = sd.n_blocks;
    return a.n_sets++;
  };
  for (int m = 0; m < p->n_masks; ++m) {
    const kvax_b200_mask_desc& d = p->masks[m];
    const int pad_id = cdiv(p->kv_len, d.kv_block) * d.kv_block + 1;                 // :248
    const int qs = find_set(p->q_positions, p->q_segment_ids, p->q_len, d.q_block, -1, pad_id);
    const int ks = find_set(p->kv_positions, p->kv_segment_ids, p->kv_len, d.kv_block, INT_MAX, pad_id);
    ClusterMask& mk = a.masks[m];
    mk = ClusterMask{d.lower, d.upper, d.lower_full, d.upper_full, d.kv_outer ? ks : qs, d.kv_outer ? qs : ks, d.kv_outer ? 1 : 0, -1};
    for (int e = 0; e < m; ++e)
      if (a.masks[e].same_as < 0 && a.masks[e].outer_set == mk.outer_set && a.masks[e].inner_set == mk.inner_set &&
          a.masks[e].kv_outer == mk.kv_outer) { mk.same_as = e; break; }
  }
  // CTAs per row: enough that a CTA summarises about one group of blocks per set, at most the portable cluster size
  int cluster = 1;
  while (cluster < 8 && cluster * kGroup < max_blocks) cluster *= 2;
  a.cluster = cluster;
  size_t off = 0;
  for (int i = 0; i < a.n_sets; ++i) {
    SetDesc& sd = a.sets[i];
    const int per = ((cdiv(sd.n_blocks, cluster) + kGroup - 1) / kGroup) * kGroup;
    sd.per = per;
    sd.smem_off = int(off);
    off += size_t(per) + size_t(per / kGroup);
  }
  if (off * sizeof(int4) > kClusterSmemLimit || (long long)p->batch * cluster > INT_MAX) return KVAX_B200_EUNSUPPORTED;
  for (int i = 0; i < a.n_sets; ++i) {                  // private copies of the whole row, as long as they fit
    SetDesc& sd = a.sets[i];
    const size_t need = size_t(cluster) * sd.per + size_t(cluster) * sd.per / kGroup;
    if ((off + need) * sizeof(int4) <= kClusterRowCopyLimit) {
      sd.row_off = int(off);
      off += need;
    }
  }
  const size_t smem = off * sizeof(int4);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(mask_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return KVAX_B200_ELAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(p->batch) * cluster, 1, 1);
  cfg.blockDim = dim3(kClusterThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, mask_cluster_kernel, a) == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

}  // namespace

extern "C" size_t kvax_b200_mask_workspace_bytes(const kvax_b200_mask_params* p) {
  if (!p || p->n_masks < 1 || p->n_masks > 3) return 0;
  size_t total = 0;
  for (int m = 0; m < p->n_masks; ++m) {
    const kvax_b200_mask_desc& d = p->masks[m];
    if (d.q_block <= 0 || d.kv_block <= 0) return 0;
    total += align256(size_t(p->batch) * cdiv(p->q_len, d.q_block) * sizeof(int4));
    total += align256(size_t(p->batch) * cdiv(p->kv_len, d.kv_block) * sizeof(int4));
  }
  return total;
}

namespace {

int check_mask_params(const kvax_b200_mask_params* p) {
  if (!p || !p->q_positions || !p->q_segment_ids || !p->kv_positions || !p->kv_segment_ids) return KVAX_B200_EINVAL;
  if (p->batch <= 0 || p->q_len <= 0 || p->kv_len <= 0 || p->n_masks < 1 || p->n_masks > 3) return KVAX_B200_EINVAL;
  for (int m = 0; m < p->n_masks; ++m) {
    const kvax_b200_mask_desc& d = p->masks[m];
    if (d.q_block <= 0 || d.kv_block <= 0) return KVAX_B200_EINVAL;
    if (!d.lower || !d.upper || !d.lower_full || !d.upper_full) return KVAX_B200_EINVAL;
    if ((long long)cdiv(p->kv_len, d.kv_block) * d.kv_block + 1 > INT_MAX) return KVAX_B200_EUNSUPPORTED;
  }
  return KVAX_B200_OK;
}

// Two launches through a summary area in global memory (the caller's workspace or the built-in scratch).
int mask_build_two_launches(const kvax_b200_mask_params* p, void* workspace, size_t workspace_bytes,
                            kvax_b200_stream_t stream) {
  const size_t need = kvax_b200_mask_workspace_bytes(p);
  if (need == 0) return KVAX_B200_EINVAL;
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return KVAX_B200_EWORKSPACE;

  SummaryArgs sa{};
  BoundsArgs ba{};
  sa.batch = ba.batch = p->batch;
  ba.skip_pad = p->skip_pad_tokens ? 1 : 0;
  char* ws = static_cast<char*>(workspace);
  long long swarps = 0, bwarps = 0;
  for (int m = 0; m < p->n_masks; ++m) {
    const kvax_b200_mask_desc& d = p->masks[m];
    if (!d.lower || !d.upper || !d.lower_full || !d.upper_full) return KVAX_B200_EINVAL;
    const int nq = cdiv(p->q_len, d.q_block), nk = cdiv(p->kv_len, d.kv_block);
    const long long kv_padded = (long long)nk * d.kv_block;
    if (kv_padded + 1 > INT_MAX) return KVAX_B200_EUNSUPPORTED;
    const int pad_id = int(kv_padded + 1);                                         // :248
    int4* qsum = reinterpret_cast<int4*>(ws); ws += align256(size_t(p->batch) * nq * sizeof(int4));
    int4* ksum = reinterpret_cast<int4*>(ws); ws += align256(size_t(p->batch) * nk * sizeof(int4));
    SideJob& jq = sa.jobs[sa.n_jobs++];
    jq = SideJob{p->q_positions, p->q_segment_ids, qsum, p->q_len, d.q_block, nq, -1, pad_id, int(swarps)};
    swarps += (long long)p->batch * nq;
    SideJob& jk = sa.jobs[sa.n_jobs++];
    jk = SideJob{p->kv_positions, p->kv_segment_ids, ksum, p->kv_len, d.kv_block, nk, INT_MAX, pad_id, int(swarps)};
    swarps += (long long)p->batch * nk;
    BoundsJob& bj = ba.jobs[ba.n_jobs++];
    if (d.kv_outer) bj = BoundsJob{ksum, qsum, d.lower, d.upper, d.lower_full, d.upper_full, nk, nq, 1, pad_id, int(bwarps)};
    else            bj = BoundsJob{qsum, ksum, d.lower, d.upper, d.lower_full, d.upper_full, nq, nk, 0, pad_id, int(bwarps)};
    bwarps += (long long)p->batch * bj.n_outer;
    if (swarps > INT_MAX / 2 || bwarps > INT_MAX / 2) return KVAX_B200_EUNSUPPORTED;
  }
  sa.total_warps = int(swarps);
  ba.total_warps = int(bwarps);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  mask_summary_kernel<<<cdiv(swarps, kWarpsPerBlock), kWarpsPerBlock * 32, 0, s>>>(sa);
  if (cudaGetLastError() != cudaSuccess) return KVAX_B200_ELAUNCH;
  mask_bounds_kernel<<<cdiv(bwarps, kWarpsPerBlock), kWarpsPerBlock * 32, 0, s>>>(ba);
  if (cudaGetLastError() != cudaSuccess) return KVAX_B200_ELAUNCH;
  return KVAX_B200_OK;
}

}  // namespace

extern "C" int kvax_b200_mask_build(const kvax_b200_mask_params* p, void* workspace, size_t workspace_bytes,
                                    kvax_b200_stream_t stream) {
  int rc = check_mask_params(p);
  if (rc) return rc;
  const size_t need = kvax_b200_mask_workspace_bytes(p);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return KVAX_B200_EWORKSPACE;
  rc = mask_build_clusters(p, stream);
  if (rc != KVAX_B200_EUNSUPPORTED) return rc;          // built, or a real error
  return mask_build_two_launches(p, workspace, workspace_bytes, stream);
}

// ---------------------------------------------------------------------------------------
// Variant with built-in scratch memory, for callers that cannot provide a workspace.
// ---------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;
constexpr int kMaxDevices = 64;

// Lives in the library's device image: every GPU that loads the library holds it.
static __device__ __align__(256) unsigned char g_mask_scratch[kStaticScratchBytes];

// Device address of g_mask_scratch per device.  In host code the symbol's name is only a
// stand-in; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device while that device is current.  The cache is keyed by device ordinal, i.e. it
// assumes the device's primary context (the one the CUDA runtime uses).
void* g_scratch_addr[kMaxDevices] = {};

}  // namespace

extern "C" int kvax_b200_mask_build_static(const kvax_b200_mask_params* p, kvax_b200_stream_t stream) {
  // arguments first: a size computed from a non-positive batch or length means nothing
  if (!p || !p->q_positions || !p->q_segment_ids || !p->kv_positions || !p->kv_segment_ids) return KVAX_B200_EINVAL;
  if (p->batch <= 0 || p->q_len <= 0 || p->kv_len <= 0 || p->n_masks < 1 || p->n_masks > 3) return KVAX_B200_EINVAL;
  const size_t need = kvax_b200_mask_workspace_bytes(p);
  if (need == 0) return KVAX_B200_EINVAL;
  if (need > kStaticScratchBytes) return KVAX_B200_ESCRATCH;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return KVAX_B200_ENODEVICE;
  void* ptr = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {   // first call on this device (two racing first calls obtain the same address)
    if (cudaGetSymbolAddress(&ptr, g_mask_scratch) != cudaSuccess || !ptr) return KVAX_B200_ENODEVICE;
    __atomic_store_n(&g_scratch_addr[dev], ptr, __ATOMIC_RELEASE);
  }
  return mask_build_two_launches(p, ptr, kStaticScratchBytes, stream);
}
