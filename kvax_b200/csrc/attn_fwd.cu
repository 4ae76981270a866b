// Flash-attention forward for sm_100a (B200).
//
// One CTA per (head, 128-row query tile, batch); six warps:
//   warps 0-3  softmax: thread t owns query row t (TMEM lane t).  Reads the score tile
//              from TMEM, applies the element mask on partial tiles, runs the online
//              softmax in registers, writes P (bf16) back over the score columns,
//              rescales the output accumulator when a row maximum moved, and runs the
//              epilogue (normalise, cast, store O and the base-2 log-sum-exp).
//   warp 4     producer: TMA loads of the Q tile once and of the K and V tile of every
//              list entry (128-byte-swizzled shared-memory tiles, no multicast).
//   warp 5     MMA issuer: one thread issues S = Q K^T (both operands from shared
//              memory) and O += P V (P from TMEM, V from shared memory, N-major) as
//              tcgen05.mma with fp32 accumulators in TMEM.
// TMEM: 128 columns S/P + D columns O = 256 columns, shared memory 3 x 32 KB, so two
// CTAs are resident per SM and one CTA's softmax overlaps the other's MMAs.
// Which kv tiles are visited, and which of them need the element mask, comes from the
// tile list built by schedule.cu from the caller's block mask.
//
// Semantics follow flash_attention_forward_kernel (kvax/ops/flash_attention_triton.py:
// 137-370): scores scaled by scale*log2(e), exp2-domain online softmax, P rounded to the
// input dtype before P V, O = acc / l, LSE2 = m + log2(l); query tiles with no work get
// O = 0 and LSE2 = 0 (:253-258).
#include "attn_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace kvx {

namespace {

constexpr int kThreads = 192;
constexpr int kTmemCols = 256;

enum FwdBar { B_QFULL = 0, B_KFULL, B_KEMPTY, B_VFULL, B_VEMPTY, B_SFULL, B_PFULL, B_OFULL, B_COUNT };

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;     // one 128 x D bf16 tile
  static constexpr int kBoxBytes = kTile * 64 * 2;     // one TMA box: 128 rows x 64 columns
  static constexpr int kQ = 0, kK = kTileBytes, kV = 2 * kTileBytes;
  static constexpr int kBars = 3 * kTileBytes;
  static constexpr int kTmemSlot = kBars + 8 * B_COUNT;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4 + 1024;     // + slack for 1024-byte alignment
};

template <int D>
__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdArgs a) {
  using L = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kQ;
  uint8_t* sK = smem + L::kK;
  uint8_t* sV = smem + L::kV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbort);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int row_rank, h;
  decode_block(blockIdx.x, a.list.n_outer_tiles * a.batch, a.q_heads, &row_rank, &h);
  const long long list_row = __ldg(a.list.order + row_rank);       // longest lists first
  const int b = int(list_row / a.list.n_outer_tiles), qt = int(list_row % a.list.n_outer_tiles);
  const int kvh = h / a.group;
  const int count = __ldg(a.list.counts + list_row);
  const uint32_t* list = a.list.tiles + list_row * a.list.n_inner_tiles;

  const int r = qt * kTile + tid;                        // query row of a softmax thread
  const bool row_valid = (tid < kTile) && (r < a.tok.q_len);
  __nv_bfloat16* o_row = a.out + (long long)b * a.o_strides[0] + (long long)r * a.o_strides[1] + (long long)h * a.o_strides[2];
  float* lse_row = a.lse + ((long long)b * a.q_heads + h) * a.tok.q_len + r;

  if (count == 0) {                                      // nothing to attend: zeros (:253-258)
    if (row_valid) {
      uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(o_row)[i] = z;
      *lse_row = 0.f;
    }
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(&bars[i], i == B_PFULL ? kTile : 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;                         // scores, later P (bf16 pairs)
  const uint32_t tO = tmem_base + kTile;                 // output accumulator

  if (warp == 4) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(&bars[B_QFULL], L::kTileBytes);
#pragma unroll
      for (int x = 0; x < D / 64; ++x) tma_load_4d(sQ + x * L::kBoxBytes, &tmap_q, &bars[B_QFULL], x * 64, h, qt * kTile, b);
      bool ok = true;
      for (int it = 0; it < count && ok; ++it) {
        const int u = int(__ldg(list + it) & ~kPartialBit);
        if (it > 0) ok = mbar_wait(&bars[B_KEMPTY], (it - 1) & 1, abort_flag, a.status, B_KEMPTY);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[B_KFULL], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x) tma_load_4d(sK + x * L::kBoxBytes, &tmap_k, &bars[B_KFULL], x * 64, kvh, u * kTile, b);
        if (it > 0) ok = mbar_wait(&bars[B_VEMPTY], (it - 1) & 1, abort_flag, a.status, B_VEMPTY);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[B_VFULL], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x) tma_load_4d(sV + x * L::kBoxBytes, &tmap_v, &bars[B_VFULL], x * 64, kvh, u * kTile, b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(kTile, D, 0, 1);       // P (TMEM)    x V (N-major)
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(&bars[B_QFULL], 0, abort_flag, a.status, B_QFULL);
      for (int it = 0; it < count && ok; ++it) {
        ok = mbar_wait(&bars[B_KFULL], it & 1, abort_flag, a.status, B_KFULL);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * L::kBoxBytes + (kk & 3) * 32;   // 16 bf16 = 32 B inside a 128 B row
          umma_ss(tS, make_sdesc_sw128(q_addr + off, 16, 1024), make_sdesc_sw128(k_addr + off, 16, 1024), idesc_s, kk > 0);
        }
        umma_commit(&bars[B_KEMPTY]);
        umma_commit(&bars[B_SFULL]);
        ok = mbar_wait(&bars[B_PFULL], it & 1, abort_flag, a.status, B_PFULL);
        if (!ok) break;
        ok = mbar_wait(&bars[B_VFULL], it & 1, abort_flag, a.status, B_VFULL);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          // 16 kv rows per step: rows are 128 B apart, d columns 0-63 / 64-127 in separate boxes
          const uint64_t vdesc = make_sdesc_sw128(v_addr + kk * 16 * 128, L::kBoxBytes, 1024);
          umma_ts(tO, tS + kk * 8, vdesc, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars[B_VEMPTY]);
        if (it == count - 1) umma_commit(&bars[B_OFULL]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const uint32_t lane_base = uint32_t(warp * 32) << 16;
    const float c = a.scale_log2e;
    RowBounds rb = load_bounds(a.mask, b, min(r, a.tok.q_len - 1));
    int q_seg = KVAX_B200_PADDING_SEGMENT_ID, q_pos = 0;
    if (row_valid) {
      q_seg = __ldg(a.tok.q_seg + (long long)b * a.tok.q_len + r);
      q_pos = query_position(a.tok, b, r);
    }
    const int32_t* kv_seg = a.tok.kv_seg + (long long)b * a.tok.kv_len;
    const int32_t* kv_pos = a.tok.kv_pos + (long long)b * a.tok.kv_len;

    // Online softmax state.  `m` is the reference maximum the exponentials use.  It only
    // follows the true running maximum when that has grown by more than kLazy (log2
    // units): P then stays below 2^kLazy, and the accumulator in TMEM needs no rescaling
    // for small increases.  O / l and LSE2 = m + log2(l) do not depend on the choice.
    constexpr float kLazy = 8.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < count && ok; ++it) {
      const uint32_t e = __ldg(list + it);
      const int c0 = int(e & ~kPartialBit) * kTile;
      const bool partial = (e & kPartialBit) != 0;

      // element mask of partial tiles (computed before the scores arrive)
      uint32_t keep[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (partial) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t bits = 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = c0 + ch * 32 + j;
            bool al = false;
            if (col < a.tok.kv_len) {
              const int ks = __ldg(kv_seg + col);
              const int kp = a.tok.sequential ? col : __ldg(kv_pos + col);
              al = row_valid && element_allowed<false>(rb, col, ks == q_seg, q_pos >= kp);
            }
            bits |= (al ? 1u : 0u) << j;
          }
          keep[ch] = bits;
        }
      }

      ok = mbar_wait(&bars[B_SFULL], it & 1, abort_flag, a.status, B_SFULL);
      if (!ok) break;
      tc_fence_after();

      // pass 1: row maximum of the raw scores (scaled afterwards: scale > 0)
      float mx = -INFINITY;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t v[32];
        tmem_ld32(tS + lane_base + ch * 32, v);
        tmem_ld_wait(v);
        if (partial) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = ((keep[ch] >> j) & 1u) ? v[j] : 0xff800000u;   // -inf
        }
#pragma unroll
        for (int j = 0; j < 32; j += 2) mx = fmax3(mx, __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
      }
      mx *= c;
      float alpha = 1.f;
      if (mx - m > kLazy) {                     // also taken when m is still -inf
        alpha = fast_exp2(m - mx);              // 0 when m was -inf
        m = mx;
      }
      const float neg_m = (m == -INFINITY) ? 0.f : -m;

      // pass 2: p = exp2(s*c - m), row sum, P (bf16 pairs) back into the score columns
      float rowsum = 0.f;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t v[32];
        tmem_ld32(tS + lane_base + ch * 32, v);
        tmem_ld_wait(v);
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(v[j]), c, neg_m));
          float p1 = fast_exp2(fmaf(__uint_as_float(v[j + 1]), c, neg_m));
          if (partial) {
            p0 = ((keep[ch] >> j) & 1u) ? p0 : 0.f;
            p1 = ((keep[ch] >> (j + 1)) & 1u) ? p1 : 0.f;
          }
          rowsum += p0 + p1;
          pk[j >> 1] = pack_bf16(p0, p1);
        }
        tmem_st16(tS + lane_base + ch * 16, pk);
      }
      l = l * alpha + rowsum;

      // rescale the accumulator when some row of this warp moved its reference maximum
      if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t v[32];
          tmem_ld32(tO + lane_base + ch * 32, v);
          tmem_ld_wait(v);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
          tmem_st32(tO + lane_base + ch * 32, v);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[B_PFULL]);
    }

    if (ok) ok = mbar_wait(&bars[B_OFULL], 0, abort_flag, a.status, B_OFULL);
    if (ok) {
      tc_fence_after();
      const float inv = (l > 0.f) ? (1.f / l) : 0.f;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t v[32];
        tmem_ld32(tO + lane_base + ch * 32, v);
        tmem_ld_wait(v);
        if (row_valid) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[j + 0]) * inv, __uint_as_float(v[j + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
            reinterpret_cast<uint4*>(o_row)[(ch * 32 + j) >> 3] = w;
          }
        }
      }
      // A row that saw no unmasked key keeps O = 0 and gets LSE2 = +inf, so that the
      // backward pass computes exp2(s - LSE2) = 0 for it.
      if (row_valid) *lse_row = (l > 0.f) ? (m + __log2f(l)) : INFINITY;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    // After an aborted run a TMA copy may still be in flight: give it a bounded moment
    // before the CTA (and its shared memory) goes away.
    if (*abort_flag && lane == 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) { }
    }
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

int launch_attn_fwd(const FwdLaunch& L, cudaStream_t stream) {
  const FwdArgs& a = L.args;
  dim3 grid(a.list.n_outer_tiles * L.batch * a.q_heads, 1, 1);
  cudaError_t err;
  if (L.head_dim == 128) {
    constexpr int smem = FwdSmem<128>::kTotal;
    err = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return KVAX_B200_ELAUNCH;
    attn_fwd_kernel<128><<<grid, kThreads, smem, stream>>>(L.tmap_q, L.tmap_k, L.tmap_v, a);
  } else if (L.head_dim == 64) {
    constexpr int smem = FwdSmem<64>::kTotal;
    err = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return KVAX_B200_ELAUNCH;
    attn_fwd_kernel<64><<<grid, kThreads, smem, stream>>>(L.tmap_q, L.tmap_k, L.tmap_v, a);
  } else {
    return KVAX_B200_EUNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

}  // namespace kvx
