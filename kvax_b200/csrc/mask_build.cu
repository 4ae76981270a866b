// Block-mask builder for sm_100a.
//
// Two launches build up to three masks (forward, dq, dkdv):
//   1. mask_summary_kernel: one warp per block of either side; coalesced 16-byte loads of
//      positions and segment ids, warp min/max reductions, one int4 summary
//      {seg_min, seg_max, pos_min, pos_max} per block (PAD already remapped).
//   2. mask_bounds_kernel: one warp per outer block; lanes stride over the inner-block
//      summaries, evaluate the "may attend" / "fully attends" interval tests and fold the
//      four bounds with warp min/max reductions; lane 0 applies the host fix-ups.
//
// Semantics follow kvax/ops/mask_creator.py:26-152 (kernel) and :212-259, :317-333 (host
// steps) exactly; outputs are bit-identical with the reference's mask tensors.
#include <cuda_runtime.h>
#include <stdint.h>
#include <limits.h>

#include "../../include/kvax_b200.h"

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

extern "C" int kvax_b200_mask_build(const kvax_b200_mask_params* p, void* workspace, size_t workspace_bytes,
                                    kvax_b200_stream_t stream) {
  if (!p || !p->q_positions || !p->q_segment_ids || !p->kv_positions || !p->kv_segment_ids) return KVAX_B200_EINVAL;
  if (p->batch <= 0 || p->q_len <= 0 || p->kv_len <= 0 || p->n_masks < 1 || p->n_masks > 3) return KVAX_B200_EINVAL;
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
  return kvax_b200_mask_build(p, ptr, kStaticScratchBytes, stream);
}
