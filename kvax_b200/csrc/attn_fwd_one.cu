// Flash-attention forward for sm_100a (B200), one query tile per CTA: the variant for short sequences, where
// CTAs of two query tiles (attn_fwd.cu) are too few and too uneven to fill 148 SMs.
//
// One CTA per (head, 128-row query tile, batch), one CTA per SM, eleven warps:
//   warps 0-3  softmax group 0: even entries of the tile list.
//   warps 4-7  softmax group 1: odd entries of the tile list.
//              In both groups thread t owns query row (t % 128) = TMEM lane.  The groups run
//              two independent online softmaxes (own running maximum, own row sum, own
//              output accumulator in TMEM) that are merged in the epilogue, so they never
//              wait for one another: while one group is in its softmax (TMEM reads, exp2,
//              TMEM writes) the tensor pipe serves the MMAs of the other.
//   warp 8     Q and K producer (and TMEM allocation): three-stage TMA ring for K.
//   warp 9     MMA issuer: one thread issues S = Q K^T (both operands from shared memory)
//              and O += P V (P from TMEM, V from shared memory, N-major) as tcgen05.mma
//              with fp32 accumulators in TMEM, in the order
//              QK(0) QK(1) | PV(0) QK(2) | PV(1) QK(3) | ...
//              QK(j+2) may overwrite the columns of P(j) because tcgen05.mma instructions of
//              one thread execute in issue order and PV(j), the reader of P(j), is issued first.
//   warp 10    V producer: three-stage TMA ring.
// TMEM (512 columns): S0 | S1 | O0 | O1 (P(j) is written as bf16 pairs over S(j & 1)).
// Shared memory: Q 32 KB + K 3 x 32 KB + V 3 x 32 KB, 128-byte-swizzled TMA tiles loaded
// without multicast straight from the (batch, seq, head, dim) layout.  Which kv tiles are
// visited, and which of them need the element mask, comes from the tile list built by
// schedule.cu from the caller's block mask.
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

constexpr int kSoftmaxThreads = 256;                 // two groups of 128
constexpr int kKWarp = 8, kMmaWarp = 9, kVWarp = 10;
constexpr int kThreads = 11 * 32;
constexpr int kTmemCols = 512;
constexpr int kKStages = 3, kVStages = 3;

enum FwdBar {
  B_QFULL = 0,
  B_KFULL0, B_KFULL1, B_KFULL2, B_KEMPTY0, B_KEMPTY1, B_KEMPTY2,
  B_VFULL0, B_VFULL1, B_VFULL2, B_VEMPTY0, B_VEMPTY1, B_VEMPTY2,
  B_SFULL0, B_SFULL1,
  B_PFULL0, B_PFULL1,                        // kv columns 0-63 of P(j) are in TMEM (group j & 1)
  B_PREST0, B_PREST1,                        // kv columns 64-127 too
  B_ALLDONE,                                 // the last P V of the CTA (and with it every MMA) has completed: completes once
  B_LFULL, B_COUNT
};

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;     // one 128 x D bf16 tile
  static constexpr int kBoxBytes = kTile * 64 * 2;     // one TMA box: 128 rows x 64 columns
  static constexpr int kQ = 0;
  static constexpr int kK = kTileBytes;
  static constexpr int kV = kK + kKStages * kTileBytes;
  static constexpr int kBars = kV + kVStages * kTileBytes;
  static constexpr int kTmemSlot = kBars + 8 * B_COUNT;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4 + 1024;     // + slack for 1024-byte alignment
  static_assert(kTotal <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

template <int D, bool kF16>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_one_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
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

  const int row = tid & (kTile - 1);
  const int wg = (tid >> 7) & 1;                         // softmax group; in the epilogue also the column half
  const int r = qt * kTile + row;                        // query row of a softmax thread
  const bool is_softmax = tid < kSoftmaxThreads;
  const bool row_valid = is_softmax && (r < a.tok.q_len);
  // the epilogue stores D/2 output columns per thread
  __nv_bfloat16* o_row = a.out + (long long)b * a.o_strides[0] + (long long)r * a.o_strides[1] +
                         (long long)h * a.o_strides[2] + wg * (D / 2);
  float* lse_row = a.lse + ((long long)b * a.q_heads + h) * a.tok.q_len + r;

  if (count == 0) {                                      // nothing to attend: zeros (:253-258)
    if (row_valid) {
      uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < D / 16; ++i) reinterpret_cast<uint4*>(o_row)[i] = z;
      if (wg == 0) *lse_row = a.empty_lse;
    }
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) {
      const int n = (i >= B_PFULL0 && i <= B_PREST1) ? kTile : (i == B_LFULL ? kSoftmaxThreads : 1);
      mbar_init(&bars[i], n);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kKWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;                 // scores of list entry j: tmem_base + 128 * (j & 1)
  const uint32_t tO = tmem_base + 2 * kTile;             // accumulator of group g: tO + 128 * g

  if (warp == kKWarp) {
    // ------------------------------------------------------------------ Q and K producer
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k);
      mbar_arrive_expect_tx(&bars[B_QFULL], L::kTileBytes);
#pragma unroll
      for (int x = 0; x < D / 64; ++x) tma_load_4d(sQ + x * L::kBoxBytes, &tmap_q, &bars[B_QFULL], x * 64, h, qt * kTile, b);
      bool ok = true;
      uint32_t e_next = __ldg(list);               // list entries are fetched one iteration ahead
      for (int it = 0; it < count && ok; ++it) {
        const int st = it % kKStages, use = it / kKStages;
        const int u = int(e_next & kTileIndexMask);
        if (it + 1 < count) e_next = ldg_pinned(list + it + 1);
        if (use > 0) ok = mbar_wait(&bars[B_KEMPTY0 + st], (use - 1) & 1, abort_flag, a.status, B_KEMPTY0 + st);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[B_KFULL0 + st], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sK + st * L::kTileBytes + x * L::kBoxBytes, &tmap_k, &bars[B_KFULL0 + st], x * 64, kvh, u * kTile, b);
      }
    }
  } else if (warp == kVWarp) {
    // ------------------------------------------------------------------ V producer
    if (lane == 0) {
      prefetch_tmap(&tmap_v);
      bool ok = true;
      uint32_t e_next = __ldg(list);
      for (int it = 0; it < count && ok; ++it) {
        const int st = it % kVStages, use = it / kVStages;
        const int u = int(e_next & kTileIndexMask);
        if (it + 1 < count) e_next = ldg_pinned(list + it + 1);
        if (use > 0) ok = mbar_wait(&bars[B_VEMPTY0 + st], (use - 1) & 1, abort_flag, a.status, B_VEMPTY0 + st);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[B_VFULL0 + st], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sV + st * L::kTileBytes + x * L::kBoxBytes, &tmap_v, &bars[B_VFULL0 + st], x * 64, kvh, u * kTile, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one elected lane issues)
    constexpr uint32_t idesc_s = make_idesc_16(kTile, kTile, 0, 0, kF16);   // Q (K-major) x K (K-major)
    constexpr uint32_t idesc_o = make_idesc_16(kTile, D, 0, 1, kF16);       // P (TMEM)    x V (N-major)
    const uint32_t q_lo = sdesc_lo_sw128(smem_u32(sQ), 16);
    const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
    const int n = __shfl_sync(0xffffffffu, count, 0);
    bool ok = true;
    // `tmem_sync`: the barrier orders TMEM loads / stores of other threads before the MMAs that follow; barriers
    // completed by TMA alone need no tcgen05 fence.
    auto wait = [&](int bar, uint32_t parity, bool tmem_sync) {
      ok = mbar_wait(&bars[bar], parity, abort_flag, a.status, bar);
      ok = __all_sync(0xffffffffu, ok);
      if (tmem_sync) tc_fence_after();
    };
    auto issue_qk = [&](int it) {            // scores of list entry `it` into buffer it & 1
      const int st = it % kKStages, use = it / kKStages;
      wait(B_KFULL0 + st, use & 1, false);
      if (!ok) return;
      const uint32_t ts = tmem_base + (it & 1) * kTile;
      const uint32_t k_lo = sdesc_lo_sw128(k_addr + st * L::kTileBytes, 16);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * L::kBoxBytes + (kk & 3) * 32) >> 4;   // 16 bf16 = 32 B inside a 128 B row
          umma_ss_lo(ts, q_lo + off, k_lo + off, idesc_s, kk > 0);
        }
        umma_commit(&bars[B_SFULL0 + (it & 1)]);
        umma_commit(&bars[B_KEMPTY0 + st]);           // the K producer may refill the stage
      }
      __syncwarp();
    };
    wait(B_QFULL, 0, false);
    if (ok) issue_qk(0);
    if (ok && n > 1) issue_qk(1);
    for (int it = 0; it < n && ok; ++it) {
      const int g = it & 1, vs = it % kVStages, vuse = it / kVStages;
      wait(B_VFULL0 + vs, vuse & 1, false);
      if (!ok) break;
      wait(B_PFULL0 + g, (it >> 1) & 1, true);
      if (!ok) break;
      const uint32_t tp = tmem_base + g * kTile;
      // 16 kv rows per step: rows are 128 B apart, d columns 0-63 / 64-127 in separate boxes
      const uint32_t v_lo = sdesc_lo_sw128(v_addr + vs * L::kTileBytes, L::kBoxBytes);
      // P arrives in two halves: the first four k-steps run while the group still exponentiates the second half
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < kTile / 32; ++kk)
          umma_ts_lo(tO + g * kTile, tp + kk * 8, v_lo + ((kk * 16 * 128) >> 4), idesc_o, (it > 1 || kk > 0) ? 1u : 0u);
      }
      __syncwarp();
      wait(B_PREST0 + g, (it >> 1) & 1, true);
      if (!ok) break;
      if (elect_one()) {
#pragma unroll
        for (int kk = kTile / 32; kk < kTile / 16; ++kk)
          umma_ts_lo(tO + g * kTile, tp + kk * 8, v_lo + ((kk * 16 * 128) >> 4), idesc_o, 1u);
        umma_commit(&bars[B_VEMPTY0 + vs]);           // V stage free; P V(it) done (rescale)
        if (it + 1 == n) umma_commit(&bars[B_ALLDONE]);
      }
      __syncwarp();
      if (it + 2 < n) issue_qk(it + 2);   // reuses buffer g: issued after PV(it), which read P(it)
    }
  } else {
    // ------------------------------------------------------------------ softmax groups + epilogue
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + wg * kTile + lane_base;
    const uint32_t tOg = tO + wg * kTile + lane_base;
    const float c = a.scale_log2e;
    RowBounds rb = load_bounds(a.mask, b, min(r, a.tok.q_len - 1));
    int q_seg = KVAX_B200_PADDING_SEGMENT_ID, q_pos = 0;
    if (row_valid) {
      q_seg = __ldg(a.tok.q_seg + (long long)b * a.tok.q_len + r);
      q_pos = query_position(a.tok, b, r);
    }
    const int32_t* kv_seg = a.tok.kv_seg + (long long)b * a.tok.kv_len;
    const int32_t* kv_pos = a.tok.kv_pos + (long long)b * a.tok.kv_len;

    // Online softmax state of this group.  `m` is the reference maximum the exponentials
    // use.  It only follows the true running maximum when that has grown by more than kLazy
    // (log2 units): P then stays below 2^kLazy and the accumulator in TMEM needs no rescaling
    // for small increases.  The merged result does not depend on the choice.
    constexpr float kLazy = 8.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // element masks of this list that the list builder worked out (slot in the entry)
    const uint4* bitmap_row = a.list.bitmaps + (list_row * kBitmapSlots) * kTile + row;
    uint32_t e_next = (wg < count) ? __ldg(list + wg) : 0u;   // list entries are fetched one iteration ahead
    for (int it = wg; it < count && ok; it += 2) {
      const uint32_t e = e_next;
      if (it + 2 < count) e_next = ldg_pinned(list + it + 2);
      const int c0 = int(e & kTileIndexMask) * kTile;
      const bool partial = (e & kPartialBit) != 0;

      // element mask of partial tiles (computed before the scores arrive)
      uint32_t keep[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (partial) {
        if (e & kBitmapBit) {                   // worked out once by the list builder for every head: 16 bytes per row
          const uint4 w = __ldg(bitmap_row + ((e >> kBitmapSlotShift) & (kBitmapSlots - 1)) * kTile);
          keep[0] = w.x; keep[1] = w.y; keep[2] = w.z; keep[3] = w.w;
        } else {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            keep[ch] = keep_bits32<false>(rb, c0 + ch * 32, a.tok.kv_len, row_valid, q_seg, q_pos, kv_seg + c0 + ch * 32,
                                          a.tok.sequential ? nullptr : kv_pos + c0 + ch * 32);
        }
      }
      ok = mbar_wait(&bars[B_SFULL0 + wg], (it >> 1) & 1, abort_flag, a.status, B_SFULL0 + wg);
      if (!ok) break;
      tc_fence_after();

      // All 128 scores of the row are read into registers with four back-to-back TMEM loads
      // (one round trip), reduced to the row maximum, exponentiated in place and written back
      // as P (bf16 pairs) over the first 64 score columns.
      uint32_t v[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld32(tS + ch * 32, v[ch]);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains: no serial dependency
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        tmem_ld_wait(v[ch]);
        if (partial) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[ch][j] = ((keep[ch] >> j) & 1u) ? v[ch][j] : 0xff800000u;   // -inf
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
#pragma unroll
          for (int t = 0; t < 4; ++t)
            mx4[t] = fmax3(mx4[t], __uint_as_float(v[ch][j + 2 * t]), __uint_as_float(v[ch][j + 2 * t + 1]));
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= c;                                  // scale > 0
      float alpha = 1.f;
      if (mx - m > kLazy) {                     // also taken when m is still -inf
        alpha = fast_exp2(m - mx);              // 0 when m was -inf
        m = mx;
      }
      // rescale this group's accumulator when some row of the warp moved its reference maximum.  The group's
      // previous P V, PV(it-2), was issued before QK(it), whose scores are here: it has completed.
      if (it > 1 && __any_sync(0xffffffffu, alpha != 1.f)) {
        const int pv = it - 2;
        ok = mbar_wait(&bars[B_VEMPTY0 + pv % kVStages], (pv / kVStages) & 1, abort_flag, a.status, B_VEMPTY0 + pv % kVStages);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < D / 16; ++ch) {     // rare: kept small, the 128 scores of the row stay in registers
          uint32_t o[16];
          tmem_ld16(tOg + ch * 16, o);
          tmem_ld_wait16(o);
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st16(tOg + ch * 16, o);
        }
      }
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[ch][j]), c, neg_m));       // exp2(-inf) = 0 on masked columns
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[ch][j + 1]), c, neg_m));
          rs4[(j >> 1) & 3] += p0 + p1;
          pk[j >> 1] = pack16<kF16>(p0, p1);
        }
        if (ch == 2) {                          // the first half of P (and the rescaled accumulator) is in TMEM by now
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(&bars[B_PFULL0 + wg]);
        }
        tmem_st16(tS + ch * 16, pk);
      }
      const float rowsum = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      l = l * alpha + rowsum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[B_PREST0 + wg]);
    }

    // ---- epilogue: merge the two groups, normalise, store.  The (m, l) pairs are exchanged
    // through the (now idle) Q tile in shared memory; every thread then handles D/2 columns.
    float2* xl = reinterpret_cast<float2*>(sQ);              // [group][row]
    // All MMAs done: the last P V has completed.  A barrier of its own that completes once: a group that finishes
    // early would otherwise wait for a phase of a ring barrier that may lie more than one phase ahead, which a
    // parity wait cannot tell from the phase before.
    if (ok) ok = mbar_wait(&bars[B_ALLDONE], 0, abort_flag, a.status, B_ALLDONE);
    if (ok) {
      xl[wg * kTile + row] = make_float2(m, l);
      mbar_arrive(&bars[B_LFULL]);
      ok = mbar_wait(&bars[B_LFULL], 0, abort_flag, a.status, B_LFULL);
    }
    if (ok) {
      tc_fence_after();
      const float2 other = xl[(wg ^ 1) * kTile + row];
      const float m0 = wg ? other.x : m, l0 = wg ? other.y : l;     // group 0 / group 1 state
      const float m1 = wg ? m : other.x, l1 = wg ? l : other.y;
      const float mt = fmaxf(m0, m1);
      const float a0 = (l0 > 0.f) ? fast_exp2(m0 - mt) : 0.f;       // a group that saw nothing contributes nothing
      const float a1 = (l1 > 0.f) ? fast_exp2(m1 - mt) : 0.f;
      const float lt = l0 * a0 + l1 * a1;
      const float inv = (lt > 0.f) ? (1.f / lt) : 0.f;
      const float w0 = a0 * inv, w1 = a1 * inv;
      const uint32_t col0 = wg * (D / 2);
#pragma unroll
      for (int ch = 0; ch < D / 64; ++ch) {
        uint32_t v0[32], v1[32];
        tmem_ld32(tO + lane_base + col0 + ch * 32, v0);
        tmem_ld32(tO + kTile + lane_base + col0 + ch * 32, v1);
        tmem_ld_wait(v0);
        tmem_ld_wait(v1);
        if (row_valid) {
          float o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float x0 = (w0 != 0.f) ? __uint_as_float(v0[j]) * w0 : 0.f;   // an unused accumulator holds garbage
            const float x1 = (w1 != 0.f) ? __uint_as_float(v1[j]) * w1 : 0.f;
            o[j] = x0 + x1;
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack16<kF16>(o[j + 0], o[j + 1]);
            w.y = pack16<kF16>(o[j + 2], o[j + 3]);
            w.z = pack16<kF16>(o[j + 4], o[j + 5]);
            w.w = pack16<kF16>(o[j + 6], o[j + 7]);
            reinterpret_cast<uint4*>(o_row)[(ch * 32 + j) >> 3] = w;
          }
        }
      }
      // A row that saw no unmasked key keeps O = 0 and gets LSE2 = +inf, so that the
      // backward pass computes exp2(s - LSE2) = 0 for it.
      if (row_valid && wg == 0) *lse_row = (lt > 0.f) ? (mt + __log2f(lt)) : INFINITY;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kKWarp) {
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

namespace {
template <int D, bool kF16>
int launch_one(const FwdLaunch& L, cudaStream_t stream) {
  const FwdArgs& a = L.args;
  dim3 grid(a.list.n_outer_tiles * L.batch * a.q_heads, 1, 1);
  constexpr int smem = FwdSmem<D>::kTotal;
  auto kern = attn_fwd_one_kernel<D, kF16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return KVAX_B200_ELAUNCH;
  kern<<<grid, kThreads, smem, stream>>>(L.tmap_q, L.tmap_k, L.tmap_v, a);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
}  // namespace

int launch_attn_fwd_one(const FwdLaunch& L, cudaStream_t stream) {
  const bool f16 = L.dtype == KVAX_B200_F16;
  if (L.head_dim == 128) return f16 ? launch_one<128, true>(L, stream) : launch_one<128, false>(L, stream);
  if (L.head_dim == 64) return f16 ? launch_one<64, true>(L, stream) : launch_one<64, false>(L, stream);
  return KVAX_B200_EUNSUPPORTED;
}

}  // namespace kvx
