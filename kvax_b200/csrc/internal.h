// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attn_common.cuh"

namespace kvx {

struct ScheduleArgs {
  MaskView mask;
  TokenInfo tok;
  uint32_t* tiles;     // (B, n_outer_tiles, n_inner_tiles)
  int32_t* counts;     // (B, n_outer_tiles)
  int32_t* order;      // (B * n_outer_tiles) launch order of the rows (blocks of neighbours, longest lists first)
  int32_t* pair_order; // (B * ceil(n_outer_tiles / 2)) the same order for pairs (2p, 2p+1): row of the even tile
  const int4* inner_summary;  // (B, n_inner_tiles) {seg_min, seg_max, pos_min, pos_max}
  uint4* bitmaps;      // (B * n_outer_tiles, kBitmapSlots, 128) element masks of the first partial entries of a list, or null
  int32_t n_outer_tiles, n_inner_tiles;
  int32_t outer_len, inner_len;
};
void launch_tile_summaries(const TokenInfo& tok, int batch, int4* q_sum, int4* kv_sum, cudaStream_t s);
void launch_schedule(bool kv_outer, const ScheduleArgs& a, int batch, cudaStream_t s);

struct FwdArgs {
  TileList list;            // one row per query tile
  MaskView mask;            // forward mask (query-outer)
  TokenInfo tok;
  __nv_bfloat16* out;       // Q, K and V reach the kernel through their tensor maps
  float* lse;               // (B, Hq, Sq)
  int32_t* status;
  long long o_strides[3];   // batch, seq, head (elements)
  float scale_log2e;
  int32_t q_heads, group;   // group = Hq / Hkv
  int32_t batch;
  float empty_lse;          // log-sum-exp written for the rows of query tiles without any key tile (0, or +inf on request)
  int32_t pair_heads;       // pair kernel: a CTA takes one query tile of two heads of a kv group instead of two tiles of one head
};

struct FwdLaunch {
  CUtensorMap tmap_q, tmap_k, tmap_v;
  FwdArgs args;
  int batch, head_dim, dtype;   // dtype: KVAX_B200_BF16 / KVAX_B200_F16 operands (and outputs)
};
// CTAs of two neighbouring query tiles that share their K / V tiles (attn_fwd.cu), or of one query tile (attn_fwd_one.cu).
int launch_attn_fwd(const FwdLaunch& L, cudaStream_t stream);
int launch_attn_fwd_one(const FwdLaunch& L, cudaStream_t stream);

struct BwdArgs {
  TileList list;            // dQ kernel: one row per query tile; dK/dV kernel: per kv tile
  MaskView mask;            // dq mask (query-outer) or dkdv mask (kv-outer)
  TokenInfo tok;
  const float* lse;         // (B, Hq, Sq) base-2 log-sum-exp from the forward
  const float* delta;       // (B, Hq, Sq) rowsum(O * dO)
  __nv_bfloat16* dq;        // dQ kernel output, strides dq_strides
  float* dq_acc;            // fused kernel: fp32 dQ accumulator (B, Sq, Hq, D) contiguous, zero on entry
  float* dk;                // dK/dV kernel outputs, (B, Skv, Hkv, D) contiguous: fp32, or (dkdv_16bit) the operand type
  float* dv;
  int32_t dkdv_16bit;
  int32_t dkdv_accumulate;  // fused kernel: dk / dv are fp32 accumulators (zero on entry) that every CTA adds its part to
  int32_t head_split;       // fused kernel: CTAs per (kv tile, kv head), each with group / head_split query heads
  int32_t* status;
  long long dq_strides[3];  // element strides (batch, seq, head) of dq
  float scale_log2e, scale;
  int32_t q_heads, kv_heads, group;
  int32_t batch;
};

struct BwdLaunch {
  CUtensorMap tmap_x1, tmap_x2, tmap_y1, tmap_y2;
  BwdArgs args;
  int batch, head_dim, dtype;
};
int launch_attn_bwd(const BwdLaunch& L, bool kv_outer, cudaStream_t stream);
// delta = rowsum(O * dO); when `dq_acc` is given, the (B, Sq, Hq, D) fp32 dQ accumulator of the fused
// backward is zero-filled by the same pass.
int launch_attn_bwd_delta(const __nv_bfloat16* o, const __nv_bfloat16* d_o, float* delta, float* dq_acc,
                          const long long* strides, int batch, int seq, int heads, int head_dim, int dtype, cudaStream_t stream);

// Fused backward (attn_bwd_fused.cu): K, V, Q, dO tensor maps as for the dK/dV kernel plus the map of the
// fp32 dQ accumulator (B, Sq, Hq, D), boxes of 32 rows x 32 columns, 128-byte swizzle.
struct FusedBwdLaunch {
  CUtensorMap tmap_k, tmap_v, tmap_q, tmap_do, tmap_dq;
  BwdArgs args;             // list / mask: the kv-outer ones
  int batch, head_dim, dtype;
};
bool attn_bwd_fused_supports(int head_dim);
int launch_attn_bwd_fused(const FusedBwdLaunch& L, cudaStream_t stream);
int launch_attn_bwd_dq_cast(const float* acc, __nv_bfloat16* dq, const long long* dq_strides, int batch, int seq, int heads,
                            int dim, float scale, int dtype, cudaStream_t stream);

}  // namespace kvx
