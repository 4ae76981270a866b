// C-ABI layer: argument checks, workspace layout, TMA tensor maps, launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include "../../include/kvax_b200.h"
#include "internal.h"

namespace {

using namespace kvx;

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
inline int cdiv(long long a, long long b) { return int((a + b - 1) / b); }

// cuTensorMapEncodeTiled is fetched through the runtime so that the library does not
// link against libcuda (it has to load on machines without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 tensor (batch, seq, heads, D) with element strides {batch, seq, head}; boxes of
// 128 rows x 64 columns of one head, 128-byte swizzle, out-of-range rows read as zero.
int make_tmap(CUtensorMap* map, const void* base, int batch, int seq, int heads, int d, const int64_t* strides, int dtype) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return KVAX_B200_ENODEVICE;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((strides[0] | strides[1] | strides[2]) & 7)) return KVAX_B200_EUNSUPPORTED;
  cuuint64_t dims[4] = {cuuint64_t(d), cuuint64_t(heads), cuuint64_t(seq), cuuint64_t(batch)};
  cuuint64_t gstr[3] = {cuuint64_t(strides[2]) * 2, cuuint64_t(strides[1]) * 2, cuuint64_t(strides[0]) * 2};
  cuuint32_t box[4] = {64, 1, cuuint32_t(kTile), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType elem = dtype == KVAX_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, elem, 4, const_cast<void*>(base), dims, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

// fp32 accumulator (batch, seq, heads, D) contiguous; boxes of 32 rows x 32 columns of one head (128-byte rows),
// 128-byte swizzle: the shared-memory source of the fused backward's reduce-adds.
int make_tmap_acc(CUtensorMap* map, float* base, int batch, int seq, int heads, int d) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return KVAX_B200_ENODEVICE;
  cuuint64_t dims[4] = {cuuint64_t(d), cuuint64_t(heads), cuuint64_t(seq), cuuint64_t(batch)};
  cuuint64_t gstr[3] = {cuuint64_t(d) * 4, cuuint64_t(heads) * d * 4, cuuint64_t(seq) * heads * d * 4};
  cuuint32_t box[4] = {32, 1, 32, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

int check_shape(const kvax_b200_attn_shape& s) {
  if (s.batch <= 0 || s.q_len <= 0 || s.kv_len <= 0 || s.q_heads <= 0 || s.kv_heads <= 0) return KVAX_B200_EINVAL;
  if (s.q_heads % s.kv_heads) return KVAX_B200_EINVAL;
  if (s.dtype != KVAX_B200_BF16 && s.dtype != KVAX_B200_F16) return KVAX_B200_EUNSUPPORTED;
  if (s.head_dim != 64 && s.head_dim != 128) return KVAX_B200_EUNSUPPORTED;
  if (!s.q_segment_ids || !s.kv_segment_ids) return KVAX_B200_EINVAL;
  if (!s.assume_sequential_positions && (!s.q_positions || !s.kv_positions)) return KVAX_B200_EINVAL;
  if (!(s.scale > 0.f) || !isfinite(s.scale)) return KVAX_B200_EUNSUPPORTED;
  return KVAX_B200_OK;
}

TokenInfo token_info(const kvax_b200_attn_shape& s) {
  TokenInfo t;
  t.q_pos = s.q_positions; t.q_seg = s.q_segment_ids; t.kv_pos = s.kv_positions; t.kv_seg = s.kv_segment_ids;
  t.q_len = s.q_len; t.kv_len = s.kv_len;
  t.sequential = s.assume_sequential_positions ? 1 : 0;
  t.off_first = s.q_global_offset_first; t.off_second = s.q_global_offset_second;
  return t;
}

int mask_view(const kvax_b200_block_mask& m, bool kv_outer, int q_len, int kv_len, MaskView* v) {
  if (!m.lower || !m.upper || !m.lower_full || !m.upper_full || m.q_block <= 0 || m.kv_block <= 0) return KVAX_B200_EINVAL;
  v->lower = m.lower; v->upper = m.upper; v->lower_full = m.lower_full; v->upper_full = m.upper_full;
  v->outer_block = kv_outer ? m.kv_block : m.q_block;
  v->inner_block = kv_outer ? m.q_block : m.kv_block;
  v->n_outer = kv_outer ? cdiv(kv_len, m.kv_block) : cdiv(q_len, m.q_block);
  return KVAX_B200_OK;
}

struct ListLayout { size_t tiles_off, counts_off, order_off, bitmaps_off, total; int n_outer, n_inner, batch; bool bitmaps; };

ListLayout list_layout(int batch, int outer_len, int inner_len, size_t base, bool bitmaps = false) {
  ListLayout l;
  l.batch = batch;
  l.n_outer = cdiv(outer_len, kTile); l.n_inner = cdiv(inner_len, kTile);
  l.tiles_off = base;
  l.counts_off = l.tiles_off + align256(size_t(batch) * l.n_outer * l.n_inner * sizeof(uint32_t));
  l.order_off = l.counts_off + align256(size_t(batch) * l.n_outer * sizeof(int32_t));
  // launch order of the single tiles, then of the pairs of neighbouring tiles (the forward's work items)
  l.bitmaps_off = l.order_off + align256(size_t(batch) * (l.n_outer + (l.n_outer + 1) / 2) * sizeof(int32_t));
  l.bitmaps = bitmaps;
  // element masks of the first partial entries of every list (attn_common.cuh)
  l.total = l.bitmaps_off + (bitmaps ? align256(size_t(batch) * l.n_outer * kBitmapSlots * kTile * sizeof(uint4)) : 0);
  return l;
}

// per-tile summaries of both sides: query tiles first, kv tiles after
struct SummaryLayout { size_t q_off, kv_off, total; };
SummaryLayout summary_layout(int batch, int q_len, int kv_len, size_t base) {
  SummaryLayout l;
  l.q_off = base;
  l.kv_off = l.q_off + align256(size_t(batch) * cdiv(q_len, kTile) * sizeof(int4));
  l.total = l.kv_off + align256(size_t(batch) * cdiv(kv_len, kTile) * sizeof(int4));
  return l;
}

void fill_schedule(ScheduleArgs* sa, const MaskView& mv, const TokenInfo& tok, char* ws, const ListLayout& ll,
                   const int4* inner_summary, int outer_len, int inner_len) {
  sa->mask = mv; sa->tok = tok;
  sa->tiles = reinterpret_cast<uint32_t*>(ws + ll.tiles_off);
  sa->counts = reinterpret_cast<int32_t*>(ws + ll.counts_off);
  sa->order = reinterpret_cast<int32_t*>(ws + ll.order_off);
  sa->pair_order = sa->order + size_t(ll.batch) * ll.n_outer;
  sa->inner_summary = inner_summary;
  sa->bitmaps = ll.bitmaps ? reinterpret_cast<uint4*>(ws + ll.bitmaps_off) : nullptr;
  sa->n_outer_tiles = ll.n_outer; sa->n_inner_tiles = ll.n_inner;
  sa->outer_len = outer_len; sa->inner_len = inner_len;
}

void fill_list(TileList* l, const ScheduleArgs& sa) {
  l->tiles = sa.tiles; l->counts = sa.counts; l->order = sa.order; l->pair_order = sa.pair_order; l->bitmaps = sa.bitmaps;
  l->n_outer_tiles = sa.n_outer_tiles; l->n_inner_tiles = sa.n_inner_tiles;
}

}  // namespace

extern "C" const char* kvax_b200_version(void) { return "kvax_b200 0.2 (sm_100a)"; }

extern "C" int kvax_b200_host_word_device_pointer(void* host_ptr, void** device_ptr) {
  if (!host_ptr || !device_ptr) return KVAX_B200_EINVAL;
  return cudaHostGetDevicePointer(device_ptr, host_ptr, 0) == cudaSuccess ? KVAX_B200_OK : KVAX_B200_EUNSUPPORTED;
}

extern "C" const char* kvax_b200_error_string(int code) {
  switch (code) {
    case KVAX_B200_OK: return "ok";
    case KVAX_B200_EINVAL: return "invalid argument";
    case KVAX_B200_EUNSUPPORTED: return "unsupported shape, dtype or alignment";
    case KVAX_B200_EWORKSPACE: return "workspace too small or misaligned";
    case KVAX_B200_ELAUNCH: return "CUDA launch or tensor-map creation failed";
    case KVAX_B200_ENODEVICE: return "no usable device or driver entry point";
    case KVAX_B200_ESCRATCH: return "problem exceeds the library's built-in 4 MiB scratch area; use the workspace variant";
    default: return "unknown error";
  }
}

extern "C" size_t kvax_b200_attn_fwd_workspace_bytes(const kvax_b200_attn_fwd_params* p) {
  if (!p || check_shape(p->shape) != KVAX_B200_OK) return 0;
  const ListLayout ll = list_layout(p->shape.batch, p->shape.q_len, p->shape.kv_len, 0, true);
  return summary_layout(p->shape.batch, p->shape.q_len, p->shape.kv_len, ll.total).total;
}

extern "C" int kvax_b200_attn_fwd(const kvax_b200_attn_fwd_params* p, void* workspace, size_t workspace_bytes,
                                  kvax_b200_stream_t stream) {
  if (!p || !p->q || !p->k || !p->v || !p->out || !p->lse) return KVAX_B200_EINVAL;
  const kvax_b200_attn_shape& s = p->shape;
  int rc = check_shape(s);
  if (rc) return rc;
  const ListLayout ll = list_layout(s.batch, s.q_len, s.kv_len, 0, true);
  const SummaryLayout sl = summary_layout(s.batch, s.q_len, s.kv_len, ll.total);
  if (!workspace || workspace_bytes < sl.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return KVAX_B200_EWORKSPACE;
  if ((s.o_strides[0] | s.o_strides[1] | s.o_strides[2]) & 7 || (reinterpret_cast<uintptr_t>(p->out) & 15)) return KVAX_B200_EUNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);

  MaskView mv;
  rc = mask_view(p->mask, false, s.q_len, s.kv_len, &mv);
  if (rc) return rc;

  ScheduleArgs sa;
  int4* q_sum = reinterpret_cast<int4*>(ws + sl.q_off);
  int4* kv_sum = reinterpret_cast<int4*>(ws + sl.kv_off);
  fill_schedule(&sa, mv, token_info(s), ws, ll, kv_sum, s.q_len, s.kv_len);
  const int stages = p->stages ? p->stages : 3;
  if (stages & 1) {
    launch_tile_summaries(sa.tok, s.batch, q_sum, kv_sum, st);
    launch_schedule(false, sa, s.batch, st);
    if (cudaGetLastError() != cudaSuccess) return KVAX_B200_ELAUNCH;
  }
  if (!(stages & 2)) return KVAX_B200_OK;

  FwdLaunch L;
  rc = make_tmap(&L.tmap_q, p->q, s.batch, s.q_len, s.q_heads, s.head_dim, s.q_strides, s.dtype);  if (rc) return rc;
  rc = make_tmap(&L.tmap_k, p->k, s.batch, s.kv_len, s.kv_heads, s.head_dim, s.k_strides, s.dtype); if (rc) return rc;
  rc = make_tmap(&L.tmap_v, p->v, s.batch, s.kv_len, s.kv_heads, s.head_dim, s.v_strides, s.dtype); if (rc) return rc;
  FwdArgs& a = L.args;
  fill_list(&a.list, sa);
  a.mask = mv; a.tok = sa.tok;
  a.out = static_cast<__nv_bfloat16*>(p->out); a.lse = p->lse; a.status = p->status;
  for (int i = 0; i < 3; ++i) a.o_strides[i] = s.o_strides[i];
  a.scale_log2e = s.scale * 1.4426950408889634f;
  a.q_heads = s.q_heads; a.group = s.q_heads / s.kv_heads; a.batch = s.batch;
  L.batch = s.batch; L.head_dim = s.head_dim; L.dtype = s.dtype;
  // Two work items per CTA that share their K / V tiles halve the K / V traffic and pay on long sequences; short ones
  // have too few and too uneven CTAs that way (measured: 8k tokens 20 % slower, 16k dense 7-14 % faster).  With
  // grouped-query attention the two items are one query tile of two heads of a kv group (identical tile lists), else
  // two neighbouring query tiles of one head.
  bool pairs = s.kv_len >= 16384;
  // Head pairs have no one-sided entries and pay on shorter sequences too, as soon as the halved number of CTAs still
  // fills the SMs twice over (measured, 32/8 heads: 8k tokens B=1 0.292 against 0.301 ms, B=4 0.97 / 1.06, 4k B=8 0.77 / 0.89).
  if (s.q_heads / s.kv_heads % 2 == 0 && (long long)cdiv(s.q_len, kTile) * s.batch * (s.q_heads / 2) >= 2 * 148) pairs = true;
  if (p->flags & KVAX_B200_FWD_ONE_TILE) pairs = false;
  if (p->flags & (KVAX_B200_FWD_TILE_PAIRS | KVAX_B200_FWD_HEAD_PAIRS)) pairs = true;
  a.empty_lse = (p->flags & KVAX_B200_FWD_EMPTY_LSE_INF) ? INFINITY : 0.f;
  a.pair_heads = (a.group % 2 == 0) ? 1 : 0;
  if (p->flags & KVAX_B200_FWD_TILE_PAIRS) a.pair_heads = 0;
  if ((p->flags & KVAX_B200_FWD_HEAD_PAIRS) && a.group % 2) return KVAX_B200_EUNSUPPORTED;
  return pairs ? launch_attn_fwd(L, st) : launch_attn_fwd_one(L, st);
}

namespace {

struct BwdLayout { ListLayout dq, dkdv; SummaryLayout sum; size_t delta_off, acc_off, kv_acc_off, kv_acc_bytes, total; bool fused; int head_split; };

bool use_fused(const kvax_b200_attn_bwd_params& p) {
  return !(p.flags & KVAX_B200_BWD_TWO_KERNEL) && attn_bwd_fused_supports(p.shape.head_dim);
}

// Fused backward: CTAs per (kv tile, kv head).  One CTA walks every query head of the kv head; when that gives few CTAs
// (short sequences, few kv heads: one long CTA then holds up a whole launch) the query heads are divided over 2, 4, ...
// CTAs whose dK / dV parts are summed in fp32 accumulators.
int fused_head_split(const kvax_b200_attn_shape& s) {
  const int group = s.q_heads / s.kv_heads;
  const long long ctas = (long long)cdiv(s.kv_len, kTile) * s.batch * s.kv_heads;
  int split = 1;
  // Measured: below 16 CTAs per SM the split pays whatever the group; up to 32 per SM it pays for CTAs that walk eight
  // or more heads (128k tokens, 32/4 heads: 86.6 -> 82.9 ms) and costs 3 % for four (32k, 32/8 heads: the zero fill
  // and the final pass over dK / dV outweigh the shorter tail).
  while (group % (2 * split) == 0 && (ctas * split < 16 * 148 || (ctas * split < 32 * 148 && group / split >= 8))) split *= 2;
  return split;
}

BwdLayout bwd_layout(const kvax_b200_attn_bwd_params& p) {
  const kvax_b200_attn_shape& s = p.shape;
  BwdLayout l;
  l.fused = use_fused(p);
  l.head_split = l.fused ? fused_head_split(s) : 1;
  l.dq = list_layout(s.batch, s.q_len, s.kv_len, 0);
  l.dkdv = list_layout(s.batch, s.kv_len, s.q_len, l.dq.total, true);
  l.sum = summary_layout(s.batch, s.q_len, s.kv_len, l.dkdv.total);
  l.delta_off = l.sum.total;
  l.acc_off = l.delta_off + align256(size_t(s.batch) * s.q_heads * s.q_len * sizeof(float));
  l.kv_acc_off = l.acc_off + (l.fused ? align256(size_t(s.batch) * s.q_len * s.q_heads * s.head_dim * sizeof(float)) : 0);
  l.kv_acc_bytes = l.head_split > 1 ? align256(size_t(s.batch) * s.kv_len * s.kv_heads * s.head_dim * sizeof(float)) : 0;
  l.total = l.kv_acc_off + 2 * l.kv_acc_bytes;      // dK and dV accumulators of the split fused backward
  return l;
}

}  // namespace

extern "C" size_t kvax_b200_attn_bwd_workspace_bytes(const kvax_b200_attn_bwd_params* p) {
  if (!p || check_shape(p->shape) != KVAX_B200_OK) return 0;
  return bwd_layout(*p).total;
}

extern "C" int kvax_b200_attn_bwd(const kvax_b200_attn_bwd_params* p, void* workspace, size_t workspace_bytes,
                                  kvax_b200_stream_t stream) {
  if (!p || !p->q || !p->k || !p->v || !p->out || !p->dout || !p->lse || !p->dq || !p->dk || !p->dv) return KVAX_B200_EINVAL;
  const kvax_b200_attn_shape& s = p->shape;
  int rc = check_shape(s);
  if (rc) return rc;
  const BwdLayout bl = bwd_layout(*p);
  if (!workspace || workspace_bytes < bl.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return KVAX_B200_EWORKSPACE;
  long long dq_strides[3] = {p->dq_strides[0], p->dq_strides[1], p->dq_strides[2]};
  if ((dq_strides[0] | dq_strides[1] | dq_strides[2]) == 0)          // not given: dq laid out like q
    for (int i = 0; i < 3; ++i) dq_strides[i] = s.q_strides[i];
  if ((s.o_strides[0] | s.o_strides[1] | s.o_strides[2] | dq_strides[0] | dq_strides[1] | dq_strides[2]) & 7) return KVAX_B200_EUNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(p->dq) | reinterpret_cast<uintptr_t>(p->dk) | reinterpret_cast<uintptr_t>(p->dv) |
       reinterpret_cast<uintptr_t>(p->out) | reinterpret_cast<uintptr_t>(p->dout)) & 15) return KVAX_B200_EUNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  float* delta = reinterpret_cast<float*>(ws + bl.delta_off);
  float* dq_acc = bl.fused ? reinterpret_cast<float*>(ws + bl.acc_off) : nullptr;
  float* dk_acc = bl.head_split > 1 ? reinterpret_cast<float*>(ws + bl.kv_acc_off) : nullptr;
  float* dv_acc = bl.head_split > 1 ? reinterpret_cast<float*>(ws + bl.kv_acc_off + bl.kv_acc_bytes) : nullptr;
  const TokenInfo tok = token_info(s);

  MaskView mv_dq, mv_dkdv;
  rc = mask_view(p->mask_dq, false, s.q_len, s.kv_len, &mv_dq);     if (rc) return rc;
  rc = mask_view(p->mask_dkdv, true, s.q_len, s.kv_len, &mv_dkdv);  if (rc) return rc;

  int4* q_sum = reinterpret_cast<int4*>(ws + bl.sum.q_off);
  int4* kv_sum = reinterpret_cast<int4*>(ws + bl.sum.kv_off);
  ScheduleArgs sq, sk;
  fill_schedule(&sq, mv_dq, tok, ws, bl.dq, kv_sum, s.q_len, s.kv_len);
  fill_schedule(&sk, mv_dkdv, tok, ws, bl.dkdv, q_sum, s.kv_len, s.q_len);
  const int all = bl.fused ? (1 | 2 | 16 | 32) : (1 | 2 | 4 | 8);
  const int stages = p->stages ? (p->stages & all) : all;
  if (stages & 1) {
    launch_tile_summaries(tok, s.batch, q_sum, kv_sum, st);
    if (!bl.fused) launch_schedule(false, sq, s.batch, st);       // the fused kernel only walks the kv-outer lists
    launch_schedule(true, sk, s.batch, st);
  }
  if (cudaGetLastError() != cudaSuccess) return KVAX_B200_ELAUNCH;

  long long ostr[3] = {s.o_strides[0], s.o_strides[1], s.o_strides[2]};
  if (stages & 2) {
    rc = launch_attn_bwd_delta(static_cast<const __nv_bfloat16*>(p->out), static_cast<const __nv_bfloat16*>(p->dout), delta,
                               dq_acc, ostr, s.batch, s.q_len, s.q_heads, s.head_dim, s.dtype, st);
    if (rc) return rc;
    if (dk_acc && cudaMemsetAsync(dk_acc, 0, 2 * bl.kv_acc_bytes, st) != cudaSuccess) return KVAX_B200_ELAUNCH;
  }
  if (!(stages & (4 | 8 | 16 | 32))) return KVAX_B200_OK;

  CUtensorMap tq, tk, tv, tdo;
  rc = make_tmap(&tq, p->q, s.batch, s.q_len, s.q_heads, s.head_dim, s.q_strides, s.dtype);     if (rc) return rc;
  rc = make_tmap(&tk, p->k, s.batch, s.kv_len, s.kv_heads, s.head_dim, s.k_strides, s.dtype);   if (rc) return rc;
  rc = make_tmap(&tv, p->v, s.batch, s.kv_len, s.kv_heads, s.head_dim, s.v_strides, s.dtype);   if (rc) return rc;
  rc = make_tmap(&tdo, p->dout, s.batch, s.q_len, s.q_heads, s.head_dim, s.o_strides, s.dtype); if (rc) return rc;

  BwdArgs a;
  a.tok = tok; a.lse = p->lse; a.delta = delta;
  a.dq = static_cast<__nv_bfloat16*>(p->dq); a.dq_acc = dq_acc; a.dk = p->dk; a.dv = p->dv; a.status = p->status;
  a.dkdv_16bit = (p->flags & KVAX_B200_BWD_DKDV_16BIT) ? 1 : 0;
  for (int i = 0; i < 3; ++i) a.dq_strides[i] = dq_strides[i];
  a.scale = s.scale; a.scale_log2e = s.scale * 1.4426950408889634f;
  a.q_heads = s.q_heads; a.kv_heads = s.kv_heads; a.group = s.q_heads / s.kv_heads;
  a.batch = s.batch;
  a.head_split = 1; a.dkdv_accumulate = 0;

  if (bl.fused) {
    if (stages & 16) {
      FusedBwdLaunch F;
      F.args = a;
      if (dk_acc) {
        F.args.head_split = bl.head_split; F.args.dkdv_accumulate = 1; F.args.dkdv_16bit = 0;
        F.args.dk = dk_acc; F.args.dv = dv_acc;
      }
      fill_list(&F.args.list, sk);
      F.args.mask = mv_dkdv;
      F.tmap_k = tk; F.tmap_v = tv; F.tmap_q = tq; F.tmap_do = tdo;
      rc = make_tmap_acc(&F.tmap_dq, dq_acc, s.batch, s.q_len, s.q_heads, s.head_dim);
      if (rc) return rc;
      F.batch = s.batch; F.head_dim = s.head_dim; F.dtype = s.dtype;
      rc = launch_attn_bwd_fused(F, st);
      if (rc) return rc;
    }
    if (stages & 32) {
      rc = launch_attn_bwd_dq_cast(dq_acc, a.dq, dq_strides, s.batch, s.q_len, s.q_heads, s.head_dim, s.scale, s.dtype, st);
      if (rc) return rc;
      if (dk_acc) {                 // the summed dK / dV parts go to the caller's arrays: fp32 copy or rounded to the operand type
        const size_t n = size_t(s.batch) * s.kv_len * s.kv_heads * s.head_dim;
        if (a.dkdv_16bit) {
          const long long kstr[3] = {(long long)s.kv_len * s.kv_heads * s.head_dim, (long long)s.kv_heads * s.head_dim, s.head_dim};
          rc = launch_attn_bwd_dq_cast(dk_acc, reinterpret_cast<__nv_bfloat16*>(p->dk), kstr, s.batch, s.kv_len, s.kv_heads, s.head_dim, 1.f, s.dtype, st);
          if (rc) return rc;
          rc = launch_attn_bwd_dq_cast(dv_acc, reinterpret_cast<__nv_bfloat16*>(p->dv), kstr, s.batch, s.kv_len, s.kv_heads, s.head_dim, 1.f, s.dtype, st);
          if (rc) return rc;
        } else {
          if (cudaMemcpyAsync(p->dk, dk_acc, n * sizeof(float), cudaMemcpyDeviceToDevice, st) != cudaSuccess ||
              cudaMemcpyAsync(p->dv, dv_acc, n * sizeof(float), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            return KVAX_B200_ELAUNCH;
        }
      }
    }
    return KVAX_B200_OK;
  }

  BwdLaunch L;
  L.args = a;
  L.batch = s.batch; L.head_dim = s.head_dim; L.dtype = s.dtype;
  // dQ: resident Q, dO of one query tile; streams K, V
  fill_list(&L.args.list, sq);
  L.args.mask = mv_dq;
  L.tmap_x1 = tq; L.tmap_x2 = tdo; L.tmap_y1 = tk; L.tmap_y2 = tv;
  if (stages & 4) {
    rc = launch_attn_bwd(L, false, st);
    if (rc) return rc;
  }
  if (!(stages & 8)) return KVAX_B200_OK;
  // dK/dV: resident K, V of one kv tile; streams Q, dO of every query head of the group
  fill_list(&L.args.list, sk);
  L.args.mask = mv_dkdv;
  L.tmap_x1 = tk; L.tmap_x2 = tv; L.tmap_y1 = tq; L.tmap_y2 = tdo;
  return launch_attn_bwd(L, true, st);
}
