// Fused flash-attention backward for sm_100a (B200): dK, dV and dQ from ONE kv-outer kernel,
// five matrix products per tile pair (S, dP, dV, dK, dQ) and one exponential per score, instead
// of the seven products and two exponentials of the dQ kernel + dK/dV kernel pair in attn_bwd.cu.
//
// CTA = (128-row kv tile, kv head, batch); K and V of the tile stay in shared memory; the Q tiles
// (with the 128 LSE2 / delta values of their queries) of every query head of the GQA group x every
// listed query tile stream through a two-stage TMA ring, the dO tiles through a single buffer (dO is
// dead once dV has run, long before the next dP needs its successor).  Fourteen warps:
//   warps 0-7   register math.  Thread t owns kv row t % 128 (= TMEM lane) and the 64-column half
//               t / 128 of every 128 x 128 tile:
//                 A: P^T = exp2(S^T * scale*log2e - LSE2), masked, -> bf16 -> TMEM (over S^T)
//                 B: dS^T = P^T * (dP^T - delta) -> bf16 -> a shared-memory tile of its own, written
//                    in the 128-byte-swizzled layout TMA produces, so the one copy serves as the
//                    K-major A operand of dK and as the MN-major A operand of dQ.
//   warps 8-11  dQ drain.  Warp w owns TMEM lanes 32 (w % 4) ... = 32 query rows of the finished
//               128 x D fp32 dQ tile.  It pulls them into registers (which frees the TMEM columns for
//               the next dP^T), stages them through a private double-buffered 4 KB area and adds them
//               to the fp32 dQ accumulator in global memory with TMA tile reduce-adds
//               (cp.reduce.async.bulk.tensor, this GPU's own memory, no multicast) -- asynchronously,
//               beside the register math of the next item.  (Plain red.global.add from registers was
//               measured three times slower: the SM issues one 128-byte reduction every ~20 cycles.)
//   warp 12     TMA producer and TMEM allocation.
//   warp 13     MMA issuer (whole warp runs the loop, one elected lane issues):
//                 S^T(0) dP^T(0) | dV(i) S^T(i+1) | dQ(i) dK(i) | dP^T(i+1) | ...
//               S^T  = K Q^T        (SS)            -> T1
//               dP^T = V dO^T       (SS)            -> T2
//               dV  += P^T dO       (A = P^T in TMEM over T1, B = dO N-major)
//               dQ   = dS K         (A = dS^T tile read MN-major, B = K tile read MN-major) -> T2, over dP^T
//               dK  += dS^T Q       (A = dS^T tile read K-major,  B = Q N-major)
// TMEM (512 columns): T1 | T2 | dV | dK.  dQ shares its columns with dP^T: that makes
// dP^T(i) -> dS^T(i) -> dQ(i) -> drain -> dP^T(i+1) one serial chain, which the other chain
// S^T(i+1) -> P^T(i+1) -> dV(i+1) overlaps.
// Shared memory (D = 128): K, V 64 KB + 2 x Q 64 KB + dO 32 KB + dS^T 32 KB + drain staging 32 KB +
// LSE2 / delta 2 KB.
//
// dQ is accumulated with fp32 atomics at L2, so its summation order (and last bits) vary from run
// to run; dK and dV are accumulated in TMEM in a fixed order.
//
// Semantics follow flash_attention_backward_kernel_dquery (kvax/ops/flash_attention_triton.py:620-871)
// and flash_attention_backward_kernel_dkdv (:874-1191); the element mask of partial tiles is the
// kv-outer rule of :1067-1167.
#include <cuda_runtime.h>

#include "attn_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace kvx {

// Optional phase clocks (compiled in with -DKVAX_PHASE_CLOCKS only): lane 0 of one warp per role sums
// the clock64 cycles it spends in each phase of its loop and stores the sums per CTA, so that a run
// shows which waits and which work make up an item.  Off in the shipped library.
#ifdef KVAX_PHASE_CLOCKS
__device__ unsigned int* g_phase_clocks = nullptr;       // (grid, 4 roles, 12 slots)
#define PH_BEGIN() unsigned int ph_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long ph_t = clock64();
#define PH(slot) { const long long ph_now = clock64(); ph_acc[slot] += (unsigned int)(ph_now - ph_t); ph_t = ph_now; }
#define PH_END(role, items) \
  if (g_phase_clocks && lane == 0) { \
    ph_acc[11] = (unsigned int)(items); \
    for (int s_ = 0; s_ < 12; ++s_) g_phase_clocks[((long long)blockIdx.x * 4 + (role)) * 12 + s_] = ph_acc[s_]; \
  }
#else
#define PH_BEGIN()
#define PH(slot)
#define PH_END(role, items)
#endif

namespace {

constexpr int kTmemCols = 512;
constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kDrainWarp0 = kComputeWarps;             // 8 % 4 == 0: drain warp w owns TMEM lane quarter w % 4
constexpr int kDrainWarps = 4;
constexpr int kProducerWarp = kDrainWarp0 + kDrainWarps, kMmaWarp = kProducerWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;          // 448
constexpr int kSlice = kTile / 2;                      // columns per register-math thread
constexpr int kStageBuf = 32 * 32 * 4;                 // one drain staging buffer: 32 rows x 32 fp32

enum FBar { F_XFULL = 0, F_QFULL0, F_QFULL1, F_QEMPTY0, F_QEMPTY1, F_DOFULL, F_DOEMPTY, F_SFULL, F_PFULL, F_DPFULL,
            F_DSFULL, F_DQFULL, F_DRAINED, F_ACCFULL, F_COUNT };

template <int D>
struct FusedSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kBoxBytes = kTile * 64 * 2;
  static constexpr int kX1 = 0, kX2 = kTileBytes;
  static constexpr int kQ = 2 * kTileBytes;                       // Q stage s at kQ + s * tile
  static constexpr int kDO = 4 * kTileBytes;                      // dO, single buffer
  static constexpr int kDS = 5 * kTileBytes;                      // dS^T tile: 128 kv rows x 128 queries bf16 (two boxes)
  static constexpr int kStage = kDS + kTile * kTile * 2;          // drain warp w, buffer u: kStage + (2 w + u) * kStageBuf
  static constexpr int kCols = kStage + kDrainWarps * 2 * kStageBuf;   // Q stage s: lse2[128] | delta[128]
  static constexpr int kColBytes = kTile * 4;
  static constexpr int kBars = kCols + 2 * 2 * kColBytes;
  static constexpr int kTmemSlot = kBars + 8 * F_COUNT;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4;
  static_assert(kTotal <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

// Mask bits of kv row r for the 64 queries [i0, i0 + 64) of a partial list entry that carries no element mask from the
// list builder (more than kBitmapSlots partial entries in one list: rare).  Deliberately not inlined: what it needs --
// the row's bounds, its segment id and position, the query arrays -- then lives in no register of the item loop (a
// build of the loop that took every mask from the list builder ran 4 % faster than one that could also compute them).
__device__ __noinline__ uint2 fused_keep_slow(const BwdArgs* a, int b, int r, int i0) {
  const bool row_valid = r < a->tok.kv_len;
  const RowBounds rb = load_bounds(a->mask, b, min(r, a->tok.kv_len - 1));
  int kv_seg = KVAX_B200_PADDING_SEGMENT_ID, kv_pos = 0;
  if (row_valid) {
    kv_seg = __ldg(a->tok.kv_seg + (long long)b * a->tok.kv_len + r);
    kv_pos = a->tok.sequential ? r : __ldg(a->tok.kv_pos + (long long)b * a->tok.kv_len + r);
  }
  return make_uint2(kv_outer_keep32(a->tok, rb, b, row_valid, kv_seg, kv_pos, i0),
                    kv_outer_keep32(a->tok, rb, b, row_valid, kv_seg, kv_pos, i0 + 32));
}

template <int D, bool kF16>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                      const __grid_constant__ CUtensorMap tmap_dq, const __grid_constant__ BwdArgs a) {
  using L = FusedSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbort);
  float* s_cols = reinterpret_cast<float*>(smem + L::kCols);

  // The swizzled tiles need a 1024-byte aligned base and the layout leaves no slack to round up.
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) report_status(a.status, ST_SMEM_MISALIGNED);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // With `head_split` > 1 the query heads of a kv head are divided over that many CTAs (short or few lists would
  // otherwise leave SMs idle behind a few long CTAs); their dK / dV parts meet in fp32 accumulators by atomic adds.
  int row_rank, hh;
  decode_block(blockIdx.x, a.list.n_outer_tiles * a.batch, a.kv_heads * a.head_split, &row_rank, &hh);
  const int kvh = hh / a.head_split;
  const long long list_row = __ldg(a.list.order + row_rank);     // longest lists first
  const int b = int(list_row / a.list.n_outer_tiles), kt = int(list_row % a.list.n_outer_tiles);
  const int group = a.group / a.head_split;                      // query heads of this CTA
  const int first_head = kvh * a.group + (hh % a.head_split) * group;
  const int count = __ldg(a.list.counts + list_row);
  const uint32_t* list = a.list.tiles + list_row * a.list.n_inner_tiles;
  const int n_items = count * group;           // item i: query head kvh*group + i / count, query tile list[i % count]
  const int q_len = a.tok.q_len;

  const int row = tid & (kTile - 1);           // kv row / TMEM lane of a register-math thread
  const int half = (tid >> 7) & 1;             // its column half; in the epilogue its half of the D columns
  const int r = kt * kTile + row;
  const bool is_compute = tid < kComputeThreads;
  const bool row_valid = is_compute && (r < a.tok.kv_len);
  // dK / dV rows of this thread: fp32, or 16-bit elements of the operand type when the caller asked for that
  const long long dkv_off = (((long long)b * a.tok.kv_len + r) * a.kv_heads + kvh) * D + half * (D / 2);
  float* dk_row = a.dk + dkv_off;
  float* dv_row = a.dv + dkv_off;
  uint16_t* dk_row16 = reinterpret_cast<uint16_t*>(a.dk) + dkv_off;
  uint16_t* dv_row16 = reinterpret_cast<uint16_t*>(a.dv) + dkv_off;

  if (n_items == 0) {                          // no contributing tile: zero gradients (nothing to add to accumulators)
    if (row_valid && !a.dkdv_accumulate) {
      if (a.dkdv_16bit) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < D / 16; ++i) { reinterpret_cast<uint4*>(dk_row16)[i] = z; reinterpret_cast<uint4*>(dv_row16)[i] = z; }
      } else {
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { reinterpret_cast<float4*>(dk_row)[i] = z; reinterpret_cast<float4*>(dv_row)[i] = z; }
      }
    }
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < F_COUNT; ++i) {
      const int n = (i == F_PFULL || i == F_DSFULL) ? kComputeThreads : (i == F_DRAINED ? kDrainWarps * 32 : 1);
      mbar_init(&bars[i], n);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tT1 = tmem_base, tT2 = tmem_base + kTile;
  const uint32_t tDV = tmem_base + 2 * kTile, tDK = tmem_base + 2 * kTile + D;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer (whole warp; one elected lane issues)
    const int n = __shfl_sync(0xffffffffu, n_items, 0);
    const int cnt = __shfl_sync(0xffffffffu, count, 0);
    if (elect_one()) {
      prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do);
      mbar_arrive_expect_tx(&bars[F_XFULL], 2 * L::kTileBytes);
#pragma unroll
      for (int x = 0; x < D / 64; ++x) {
        tma_load_4d(smem + L::kX1 + x * L::kBoxBytes, &tmap_k, &bars[F_XFULL], x * 64, kvh, kt * kTile, b);
        tma_load_4d(smem + L::kX2 + x * L::kBoxBytes, &tmap_v, &bars[F_XFULL], x * 64, kvh, kt * kTile, b);
      }
    }
    __syncwarp();
    bool ok = true;
    uint32_t e_next = __ldg(list);                 // list entries are fetched one iteration ahead
    int li = 0, qh = first_head;                  // index into the list, query head
    PH_BEGIN()
    for (int i = 0; i < n && ok; ++i) {
      const int st = i & 1;
      const int u = int(e_next & kTileIndexMask);
      const int yh = qh;
      if (++li == cnt) { li = 0; ++qh; }
      if (i + 1 < n) e_next = __ldg(list + li);
      PH(1)
      // ---- Q(i) with LSE2 / delta: its stage is free once dK(i-2) has completed
      if (i >= 2) {
        ok = mbar_wait(&bars[F_QEMPTY0 + st], ((i >> 1) - 1) & 1, abort_flag, a.status, F_QEMPTY0 + st);
        ok = __all_sync(0xffffffffu, ok);
      }
      PH(0)
      if (!ok) break;
      uint8_t* yq = smem + L::kQ + st * L::kTileBytes;
      float* cs = s_cols + st * 2 * kTile;
      const int col0 = u * kTile;
      const float* lse_src = a.lse + ((long long)b * a.q_heads + yh) * q_len + col0;
      const float* dl_src = a.delta + ((long long)b * a.q_heads + yh) * q_len + col0;
      const bool bulk = (col0 + kTile <= q_len) &&
                        (((reinterpret_cast<uintptr_t>(lse_src) | reinterpret_cast<uintptr_t>(dl_src)) & 15) == 0);
      if (!bulk) {                                 // tile cut by the end of the sequence, or unaligned rows
#pragma unroll
        for (int k = 0; k < kTile / 32; ++k) {
          const int j = lane + 32 * k;
          const bool valid = col0 + j < q_len;
          cs[j] = valid ? __ldg(lse_src + j) : INFINITY;            // exp2(-inf) = 0
          cs[kTile + j] = valid ? __ldg(dl_src + j) : 0.f;
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (elect_one()) {
        mbar_arrive_expect_tx(&bars[F_QFULL0 + st], L::kTileBytes + (bulk ? 2 * L::kColBytes : 0));
#pragma unroll
        for (int x = 0; x < D / 64; ++x) tma_load_4d(yq + x * L::kBoxBytes, &tmap_q, &bars[F_QFULL0 + st], x * 64, yh, u * kTile, b);
        if (bulk) {
          bulk_load_1d(cs, lse_src, L::kColBytes, &bars[F_QFULL0 + st]);
          bulk_load_1d(cs + kTile, dl_src, L::kColBytes, &bars[F_QFULL0 + st]);
        }
      }
      __syncwarp();
      // ---- dO(i): the single buffer is free once dV(i-1) has completed
      if (i >= 1) {
        ok = mbar_wait(&bars[F_DOEMPTY], uint32_t((i - 1) & 1), abort_flag, a.status, F_DOEMPTY);
        ok = __all_sync(0xffffffffu, ok);
      }
      PH(2)
      if (!ok) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&bars[F_DOFULL], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(smem + L::kDO + x * L::kBoxBytes, &tmap_do, &bars[F_DOFULL], x * 64, yh, u * kTile, b);
      }
      __syncwarp();
    }
    PH_END(3, n)
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one elected lane issues)
    constexpr uint32_t idesc_t = make_idesc_16(kTile, kTile, 0, 0, kF16);    // X (K-major) x Y (K-major)
    constexpr uint32_t idesc_dv = make_idesc_16(kTile, D, 0, 1, kF16);       // P^T (TMEM) x dO (N-major)
    constexpr uint32_t idesc_dq = make_idesc_16(kTile, D, 1, 1, kF16);       // dS^T tile (MN-major A) x K tile (MN-major B)
    constexpr uint32_t idesc_dk = make_idesc_16(kTile, D, 0, 1, kF16);       // dS^T tile (K-major A) x Q (N-major B)
    const uint32_t x1_lo = sdesc_lo_sw128(smem_u32(smem + L::kX1), 16), x2_lo = sdesc_lo_sw128(smem_u32(smem + L::kX2), 16);
    const uint32_t kmn_lo = sdesc_lo_sw128(smem_u32(smem + L::kX1), L::kBoxBytes);   // K tile with kv as the contraction index
    const uint32_t qbase = smem_u32(smem + L::kQ);
    const uint32_t do_k_lo = sdesc_lo_sw128(smem_u32(smem + L::kDO), 16);            // dO, head dimension contracted (dP^T)
    const uint32_t do_n_lo = sdesc_lo_sw128(smem_u32(smem + L::kDO), L::kBoxBytes);  // dO, queries contracted (dV)
    const uint32_t ds_addr = smem_u32(smem + L::kDS);
    const uint32_t ds_mn_lo = sdesc_lo_sw128(ds_addr, L::kBoxBytes), ds_k_lo = sdesc_lo_sw128(ds_addr, 16);
    const int n = __shfl_sync(0xffffffffu, n_items, 0);
    bool ok = true;
    // `tmem_sync`: the barrier orders TMEM loads / stores of other threads before the MMAs that follow; barriers
    // completed by TMA alone need no tcgen05 fence.
    auto wait = [&](int bar, uint32_t parity, bool tmem_sync) {
      ok = mbar_wait(&bars[bar], parity, abort_flag, a.status, bar);
      ok = __all_sync(0xffffffffu, ok);
      if (tmem_sync) tc_fence_after();
    };
    auto issue_t = [&](uint32_t t_addr, uint32_t x_lo, uint32_t y_lo) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = ((kk >> 2) * L::kBoxBytes + (kk & 3) * 32) >> 4;
        umma_ss_lo(t_addr, x_lo + off, y_lo + off, idesc_t, kk > 0);
      }
    };
    wait(F_XFULL, 0, false);
    if (ok) wait(F_QFULL0, 0, false);
    if (ok) wait(F_DOFULL, 0, false);
    if (ok) {
      if (elect_one()) {
        issue_t(tT1, x1_lo, sdesc_lo_sw128(qbase, 16));
        umma_commit(&bars[F_SFULL]);
        issue_t(tT2, x2_lo, do_k_lo);
        umma_commit(&bars[F_DPFULL]);
      }
      __syncwarp();
    }
    PH_BEGIN()
    for (int i = 0; i < n && ok; ++i) {
      const int st = i & 1;
      const uint32_t ph = uint32_t(i & 1);
      const uint32_t yq = qbase + st * L::kTileBytes, yqn = qbase + (st ^ 1) * L::kTileBytes;
      const uint32_t acc_on = (i > 0) ? 1u : 0u;
      const bool more = (i + 1 < n);
      wait(F_PFULL, ph, true);                                                      // P^T(i) written, S^T(i) consumed
      PH(0)
      if (!ok) break;
      if (elect_one()) {
        // dV += P^T dO: the half h of the register-math threads wrote its four K-steps at column offset 64 h
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts_lo(tDV, tT1 + (kk >> 2) * kSlice + (kk & 3) * 8, do_n_lo + ((kk * 16 * 128) >> 4), idesc_dv, acc_on | (kk > 0));
        umma_commit(&bars[F_DOEMPTY]);                                              // dO(i) is dead: its buffer may take dO(i+1)
      }
      __syncwarp();
      PH(1)
      if (more) {
        wait(F_QFULL0 + (st ^ 1), ((i + 1) >> 1) & 1, false);
        PH(2)
        if (!ok) break;
        if (elect_one()) {
          issue_t(tT1, x1_lo, sdesc_lo_sw128(yqn, 16));                             // scores of item i+1
          umma_commit(&bars[F_SFULL]);
        }
        __syncwarp();
        PH(3)
      }
      wait(F_DSFULL, ph, true);                                                     // dS^T(i) in its tile, dP^T(i) consumed
      PH(4)
      if (!ok) break;
      if (elect_one()) {
        // dQ(i) = dS K over the dP^T columns: both operands read with kv as the contraction index (16 kv rows per
        // step = 16 lines of 128 bytes)
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ss_lo(tT2, ds_mn_lo + ((kk * 16 * 128) >> 4), kmn_lo + ((kk * 16 * 128) >> 4), idesc_dq, kk > 0);
        umma_commit(&bars[F_DQFULL]);
        // dK(i) += dS^T(i) Q(i)
        const uint32_t q_lo = sdesc_lo_sw128(yq, L::kBoxBytes);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * L::kBoxBytes + (kk & 3) * 32) >> 4;
          umma_ss_lo(tDK, ds_k_lo + off, q_lo + ((kk * 16 * 128) >> 4), idesc_dk, acc_on | (kk > 0));
        }
        umma_commit(&bars[F_QEMPTY0 + st]);                                         // Q(i) is dead; also: the dS^T tile may be rewritten
        if (!more) umma_commit(&bars[F_ACCFULL]);
      }
      __syncwarp();
      PH(5)
      if (more) {
        wait(F_DRAINED, ph, true);                                                  // dQ(i) has left the T2 columns
        PH(6)
        if (ok) wait(F_DOFULL, uint32_t((i + 1) & 1), false);
        if (!ok) break;
        if (elect_one()) {
          issue_t(tT2, x2_lo, do_k_lo);                                             // dP^T of item i+1
          umma_commit(&bars[F_DPFULL]);
        }
        __syncwarp();
        PH(7)
      }
    }
    PH_END(1, n)
  } else if (is_compute) {
    // ------------------------------------------------------------------ register math
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const int cb = half * kSlice;                             // first column (within the tile) of this thread
    const uint32_t my_t1 = tT1 + lane_base + cb;              // fp32 columns of this thread; P^T goes to the first 32 of them
    const uint32_t my_t2 = tT2 + lane_base + cb;
    const float c = a.scale_log2e;
    // Mask bits of this thread's 64 queries of partial list entry e: the element mask the list builder worked out for
    // the first partial entries of every list (one 8-byte load), else computed by the function above.
    const uint2* bitmap_row = reinterpret_cast<const uint2*>(a.list.bitmaps + (list_row * kBitmapSlots) * kTile + row) + half;
    auto item_keep = [&](uint32_t e, uint32_t* k2) {
      const uint2 w = (e & kBitmapBit) ? __ldg(bitmap_row + ((e >> kBitmapSlotShift) & (kBitmapSlots - 1)) * (kTile * 2))
                                       : fused_keep_slow(&a, b, r, int(e & kTileIndexMask) * kTile + cb);
      k2[0] = w.x; k2[1] = w.y;
    };

    bool ok = true;
    uint32_t e_next = ldg_pinned(list);
    int li = 0;
    // mask bits of the coming item are fetched one item ahead (in the gap while dP^T of the current item is
    // awaited), so that their global loads never sit in front of the exponentials
    uint32_t keep_next[2] = {0xffffffffu, 0xffffffffu};
    if (e_next & kPartialBit) item_keep(e_next, keep_next);
    uint8_t* ds_row = smem + L::kDS + half * L::kBoxBytes + row * 128;   // this thread's 128-byte row of the dS^T tile
    PH_BEGIN()
    for (int i = 0; i < n_items && ok; ++i) {
      const uint32_t e = e_next;
      if (++li == count) li = 0;
      if (i + 1 < n_items) e_next = ldg_pinned(list + li);
      const bool partial = (e & kPartialBit) != 0;
      const int st = i & 1;
      const uint32_t ph = uint32_t(i & 1);
      const float* cs = s_cols + st * 2 * kTile;
      const float4* cs_lse = reinterpret_cast<const float4*>(cs + cb);
      const float4* cs_dl = reinterpret_cast<const float4*>(cs + kTile + cb);
      const uint32_t keep[2] = {keep_next[0], keep_next[1]};

      // LSE2 / delta of this item have landed together with its Q tile
      ok = mbar_wait(&bars[F_QFULL0 + st], (i >> 1) & 1, abort_flag, a.status, F_QFULL0 + st);
      PH(1)
      if (!ok) break;

      // ---- A: P^T = exp2(S^T * scale*log2e - LSE2); the 64 values of this thread stay in registers for B
      ok = mbar_wait(&bars[F_SFULL], ph, abort_flag, a.status, F_SFULL);
      PH(2)
      if (!ok) break;
      tc_fence_after();
      uint32_t v[2][32];
      tmem_ld32(my_t1, v[0]);
      tmem_ld32(my_t1 + 32, v[1]);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        tmem_ld_wait(v[ch]);
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
          const float4 ls = cs_lse[(ch * 32 + jj) >> 2];
          const float l4[4] = {ls.x, ls.y, ls.z, ls.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float pv = fast_exp2(fmaf(__uint_as_float(v[ch][jj + t]), c, -l4[t]));
            if (partial) pv = ((keep[ch] >> (jj + t)) & 1u) ? pv : 0.f;
            v[ch][jj + t] = __float_as_uint(pv);
          }
        }
        uint32_t pk[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 2) pk[jj >> 1] = pack16<kF16>(__uint_as_float(v[ch][jj]), __uint_as_float(v[ch][jj + 1]));
        tmem_st16(my_t1 + ch * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[F_PFULL]);
      PH(3)

      keep_next[0] = keep_next[1] = 0xffffffffu;
      if (i + 1 < n_items && (e_next & kPartialBit)) item_keep(e_next, keep_next);
      PH(0)

      // ---- B: dS^T = P^T * (dP^T - delta) -> bf16 -> the dS^T tile in shared memory
      ok = mbar_wait(&bars[F_DPFULL], ph, abort_flag, a.status, F_DPFULL);
      PH(4)
      if (!ok) break;
      tc_fence_after();
      uint32_t dp[2][16];                                     // 16 columns at a time, the next request in flight
      tmem_ld16(my_t2, dp[0]);
      if (i > 0) {      // dQ(i-1) and dK(i-1), the readers of the tile, have completed (the commit that frees Q stage (i-1) & 1)
        ok = mbar_wait(&bars[F_QEMPTY0 + ((i - 1) & 1)], ((i - 1) >> 1) & 1, abort_flag, a.status, F_QEMPTY0 + ((i - 1) & 1));
        if (!ok) break;
      }
      PH(5)
      {
        // kv row `row`, queries [64 half, 64 half + 64) = one 128-byte row of box `half`: eight 16-byte chunks at the
        // positions the 128-byte swizzle assigns them
        uint8_t* slot = ds_row;
#pragma unroll
        for (int sc = 0; sc < 4; ++sc) {                      // columns [16 sc, 16 sc + 16) of this thread's 64
          if (sc + 1 < 4) tmem_ld16(my_t2 + (sc + 1) * 16, dp[(sc + 1) & 1]);
          tmem_ld_wait16(dp[sc & 1]);
          const int ch = sc >> 1, j0 = (sc & 1) * 16;
#pragma unroll
          for (int jj = 0; jj < 16; jj += 8) {
            const float4 dl0 = cs_dl[(sc * 16 + jj) >> 2], dl1 = cs_dl[((sc * 16 + jj) >> 2) + 1];
            const float dl[8] = {dl0.x, dl0.y, dl0.z, dl0.w, dl1.x, dl1.y, dl1.z, dl1.w};
            float d[8];
#pragma unroll
            for (int t = 0; t < 8; ++t)
              d[t] = __uint_as_float(v[ch][j0 + jj + t]) * (__uint_as_float(dp[sc & 1][jj + t]) - dl[t]);
            const int ck = sc * 2 + (jj >> 3);                // 16-byte chunk: 8 queries
            *reinterpret_cast<uint4*>(slot + ((ck ^ (row & 7)) << 4)) =
                make_uint4(pack16<kF16>(d[0], d[1]), pack16<kF16>(d[2], d[3]), pack16<kF16>(d[4], d[5]), pack16<kF16>(d[6], d[7]));
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars[F_DSFULL]);
      PH(6)
    }
    if (warp == 0) { PH_END(0, n_items) }

    if (ok) ok = mbar_wait(&bars[F_ACCFULL], 0, abort_flag, a.status, F_ACCFULL);
    if (ok) {
      tc_fence_after();
      // every thread stores D/2 columns of its row: columns [half*D/2, (half+1)*D/2)
#pragma unroll
      for (int ch = 0; ch < D / 64; ++ch) {
        uint32_t v1[32], v2[32];
        tmem_ld32(tDV + lane_base + half * (D / 2) + ch * 32, v1);
        tmem_ld32(tDK + lane_base + half * (D / 2) + ch * 32, v2);
        tmem_ld_wait(v1);
        tmem_ld_wait(v2);
        if (row_valid && a.dkdv_accumulate) {
#pragma unroll
          for (int jj = 0; jj < 32; jj += 4) {
            red_add_f32x4(dv_row + ch * 32 + jj, __uint_as_float(v1[jj]), __uint_as_float(v1[jj + 1]), __uint_as_float(v1[jj + 2]),
                          __uint_as_float(v1[jj + 3]));
            red_add_f32x4(dk_row + ch * 32 + jj, __uint_as_float(v2[jj]) * a.scale, __uint_as_float(v2[jj + 1]) * a.scale,
                          __uint_as_float(v2[jj + 2]) * a.scale, __uint_as_float(v2[jj + 3]) * a.scale);
          }
        } else if (row_valid) {
          if (a.dkdv_16bit) {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 8) {
              uint4 w1, w2;
              w1.x = pack16<kF16>(__uint_as_float(v1[jj + 0]), __uint_as_float(v1[jj + 1]));
              w1.y = pack16<kF16>(__uint_as_float(v1[jj + 2]), __uint_as_float(v1[jj + 3]));
              w1.z = pack16<kF16>(__uint_as_float(v1[jj + 4]), __uint_as_float(v1[jj + 5]));
              w1.w = pack16<kF16>(__uint_as_float(v1[jj + 6]), __uint_as_float(v1[jj + 7]));
              w2.x = pack16<kF16>(__uint_as_float(v2[jj + 0]) * a.scale, __uint_as_float(v2[jj + 1]) * a.scale);
              w2.y = pack16<kF16>(__uint_as_float(v2[jj + 2]) * a.scale, __uint_as_float(v2[jj + 3]) * a.scale);
              w2.z = pack16<kF16>(__uint_as_float(v2[jj + 4]) * a.scale, __uint_as_float(v2[jj + 5]) * a.scale);
              w2.w = pack16<kF16>(__uint_as_float(v2[jj + 6]) * a.scale, __uint_as_float(v2[jj + 7]) * a.scale);
              reinterpret_cast<uint4*>(dv_row16)[(ch * 32 + jj) >> 3] = w1;
              reinterpret_cast<uint4*>(dk_row16)[(ch * 32 + jj) >> 3] = w2;
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 4) {
              reinterpret_cast<float4*>(dv_row)[(ch * 32 + jj) >> 2] =
                  make_float4(__uint_as_float(v1[jj]), __uint_as_float(v1[jj + 1]), __uint_as_float(v1[jj + 2]), __uint_as_float(v1[jj + 3]));
              reinterpret_cast<float4*>(dk_row)[(ch * 32 + jj) >> 2] =
                  make_float4(__uint_as_float(v2[jj]) * a.scale, __uint_as_float(v2[jj + 1]) * a.scale,
                              __uint_as_float(v2[jj + 2]) * a.scale, __uint_as_float(v2[jj + 3]) * a.scale);
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ dQ drain (warps 8-11)
    const int dw = warp - kDrainWarp0;                        // = TMEM lane quarter of this warp
    const uint32_t lane_base = uint32_t(dw * 32) << 16;
    uint8_t* stage = smem + L::kStage + dw * 2 * kStageBuf;
    uint8_t* my_row = stage + lane * 128;                     // this lane's query row in staging buffer 0: 32 fp32, swizzled
    if (lane == 0) prefetch_tmap(&tmap_dq);
    bool ok = true;
    uint32_t e_next = ldg_pinned(list);
    int li = 0, qh = first_head;
    PH_BEGIN()
    for (int i = 0; i < n_items && ok; ++i) {
      const int q0 = int(e_next & kTileIndexMask) * kTile + dw * 32;    // first query row this warp drains
      const int yh = qh;
      if (++li == count) { li = 0; ++qh; }
      if (i + 1 < n_items) e_next = ldg_pinned(list + li);
      const bool live = q0 < q_len;                           // rows beyond the sequence are clipped by TMA; skip all-out boxes
      ok = mbar_wait(&bars[F_DQFULL], uint32_t(i & 1), abort_flag, a.status, F_DQFULL);
      PH(0)
      if (!ok) break;
      tc_fence_after();
      // Registers hold three 32-column chunks at a time (the register file leaves 128 per thread): chunks 0-2 are
      // requested at once; chunk 0 is written to its staging buffer as soon as it arrives and chunk 3 is requested
      // into its registers right behind those stores; the T2 columns are released as soon as all chunks are in
      // registers, and everything else (proxy fence, reduce-add, the other chunks) happens after that.
      auto put = [&](int ch, const uint32_t (&x)[32]) {       // registers -> staging buffer ch & 1
        uint8_t* dst = my_row + (ch & 1) * kStageBuf;
#pragma unroll
        for (int ck = 0; ck < 8; ++ck)
          *reinterpret_cast<uint4*>(dst + ((ck ^ (lane & 7)) << 4)) = make_uint4(x[4 * ck], x[4 * ck + 1], x[4 * ck + 2], x[4 * ck + 3]);
      };
      auto reduce = [&](int ch) {                             // staging buffer ch & 1 -> += accumulator
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (live) tma_reduce_add_4d(&tmap_dq, stage + (ch & 1) * kStageBuf, ch * 32, yh, q0, b);
          // a group is committed for skipped boxes too (it is empty and complete at once): `buffer_free` counts groups,
          // and a skipped one must not let the group before it, which may still read the other buffer, fall out of the count
          bulk_commit_group();
        }
      };
      auto buffer_free = [&]() {                              // the reduce-add issued from the buffer two chunks ago has read it
        if (lane == 0) bulk_wait_group_read<1>();
        __syncwarp();
      };
      static_assert(D == 128, "drain schedule written for four 32-column chunks");
      uint32_t x0[32], x1[32], x2[32];
      tmem_ld32(tT2 + lane_base, x0);
      tmem_ld32(tT2 + lane_base + 32, x1);
      tmem_ld32(tT2 + lane_base + 64, x2);
      buffer_free();                                          // buffer 0: chunk 2 of the previous item, long gone
      tmem_ld_wait(x0);
      put(0, x0);
      tmem_ld32(tT2 + lane_base + 96, x0);                    // chunk 3 takes the registers of chunk 0
      tmem_ld_wait(x1);
      tmem_ld_wait(x2);
      tmem_ld_wait(x0);
      tc_fence_before();
      mbar_arrive(&bars[F_DRAINED]);                          // the T2 columns may take dP^T(i+1)
      PH(1)
      reduce(0);
      buffer_free(); put(1, x1); reduce(1);
      buffer_free(); put(2, x2); reduce(2);
      buffer_free(); put(3, x0); reduce(3);
      PH(2)
    }
    if (dw == 0) { PH_END(2, n_items) }
    if (lane == 0) bulk_wait_group<0>();                      // all reduce-adds performed before the CTA goes away
    __syncwarp();
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
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

// dq[b, s, h, :] = scale * acc[b, s, h, :] rounded to bf16 (or fp16); acc is (B, Sq, Hq, D) fp32 contiguous, dq has its own strides.
template <bool kF16>
__global__ void __launch_bounds__(256) attn_bwd_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                              long long s0, long long s1, long long s2, int seq, int heads, int dim,
                                                              float scale, long long n_vec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 8;
    const int d = int(e % dim);
    const long long t = e / dim;
    const int h = int(t % heads);
    const long long t2 = t / heads;
    const int s = int(t2 % seq);
    const long long b = t2 / seq;
    const float4 x = __ldcs(reinterpret_cast<const float4*>(acc + e)), y = __ldcs(reinterpret_cast<const float4*>(acc + e) + 1);
    uint4 w;
    w.x = pack16<kF16>(x.x * scale, x.y * scale); w.y = pack16<kF16>(x.z * scale, x.w * scale);
    w.z = pack16<kF16>(y.x * scale, y.y * scale); w.w = pack16<kF16>(y.z * scale, y.w * scale);
    *reinterpret_cast<uint4*>(dq + b * s0 + s * s1 + h * s2 + d) = w;
  }
}

template <int D, bool kF16>
int launch_fused(const FusedBwdLaunch& L, cudaStream_t stream) {
  static_assert(D == 128, "the drain is written for four 32-column chunks");
  constexpr int smem = FusedSmem<D>::kTotal;
  auto kern = attn_bwd_fused_kernel<D, kF16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return KVAX_B200_ELAUNCH;
  dim3 grid(L.args.list.n_outer_tiles * L.batch * L.args.kv_heads * L.args.head_split, 1, 1);
  kern<<<grid, kThreads, smem, stream>>>(L.tmap_k, L.tmap_v, L.tmap_q, L.tmap_do, L.tmap_dq, L.args);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

}  // namespace

bool attn_bwd_fused_supports(int head_dim) { return head_dim == 128; }

#ifdef KVAX_PHASE_CLOCKS
// profiling builds only: where the phase clocks go ((grid, 4, 12) uint32 in device memory), or null
extern "C" int kvax_b200_debug_set_phase_buffer(unsigned int* buf) {
  return cudaMemcpyToSymbol(g_phase_clocks, &buf, sizeof(buf)) == cudaSuccess ? 0 : -4;
}
#endif

int launch_attn_bwd_fused(const FusedBwdLaunch& L, cudaStream_t stream) {
  if (L.head_dim == 128) return L.dtype == KVAX_B200_F16 ? launch_fused<128, true>(L, stream) : launch_fused<128, false>(L, stream);
  return KVAX_B200_EUNSUPPORTED;
}

int launch_attn_bwd_dq_cast(const float* acc, __nv_bfloat16* dq, const long long* dq_strides, int batch, int seq, int heads,
                            int dim, float scale, int dtype, cudaStream_t stream) {
  const long long n_vec = (long long)batch * seq * heads * dim / 8;
  const long long want = (n_vec + 255) / 256;
  const int blocks = int(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
  if (dtype == KVAX_B200_F16)
    attn_bwd_dq_cast_kernel<true><<<blocks, 256, 0, stream>>>(acc, dq, dq_strides[0], dq_strides[1], dq_strides[2], seq, heads, dim, scale, n_vec);
  else
    attn_bwd_dq_cast_kernel<false><<<blocks, 256, 0, stream>>>(acc, dq, dq_strides[0], dq_strides[1], dq_strides[2], seq, heads, dim, scale, n_vec);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

}  // namespace kvx
