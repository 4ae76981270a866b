// Flash-attention forward for sm_100a (B200).
//
// One CTA per (head, PAIR of neighbouring 128-row query tiles, batch), one CTA per SM, eleven warps:
//   warps 0-3  softmax group 0: query tile 2p.
//   warps 4-7  softmax group 1: query tile 2p + 1.
//              In both groups thread t owns query row (t % 128) = TMEM lane of its tile.  Each group has its
//              own scores and its own output accumulator in TMEM and its own tile list; the two tiles share
//              every K / V tile that both lists name (neighbouring query tiles of one document name almost
//              the same ones), so a K / V tile is brought into shared memory once for two score tiles:
//              half the L2 -> SM traffic and half the shared-memory fill of a one-tile CTA, and while one
//              group is in its softmax the tensor pipe serves the MMAs of the other.
//   warp 8     Q and K producer (and TMEM allocation): three-stage TMA ring for K.
//   warp 9     MMA issuer: one thread issues S_g = Q_g K^T (both operands from shared memory) and
//              O_g += P_g V (P from TMEM, V from shared memory, N-major) as tcgen05.mma with fp32
//              accumulators in TMEM.  It walks the union of the two tile lists; with both tiles on every
//              entry the order is
//              QK(0,0) QK(1,0) | PV(0,0) QK(0,1) | PV(1,0) QK(1,1) | PV(0,1) QK(0,2) | ...
//              QK(g,u+1) may overwrite the columns of P(g,u) because tcgen05.mma instructions of one thread
//              execute in issue order and PV(g,u), the reader of P(g,u), is issued first.  The scores of
//              union entry u+1 are never issued before step u, so a K stage is never waited for more than
//              one entry ahead of the oldest unfinished one.
//   warp 10    V producer: two-stage TMA ring.
// TMEM (512 columns): S0 | S1 | O0 | O1 (P_g is written as bf16 pairs over S_g).
// Shared memory: Q 2 x 32 KB + K 3 x 32 KB + V 2 x 32 KB, 128-byte-swizzled TMA tiles loaded without
// multicast straight from the (batch, seq, head, dim) layout.  Which kv tiles a query tile visits, and
// which of them need the element mask, comes from the tile lists built by schedule.cu from the caller's
// block mask.
//
// Semantics follow flash_attention_forward_kernel (kvax/ops/flash_attention_triton.py:
// 137-370): scores scaled by scale*log2(e), exp2-domain online softmax, P rounded to the
// input dtype before P V, O = acc / l, LSE2 = m + log2(l); query tiles with no work get
// O = 0 and LSE2 = 0 (:253-258).
#include "attn_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace kvx {

// Optional phase clocks (compiled in with -DKVAX_PHASE_CLOCKS only): lane 0 of one warp per role sums the
// clock64 cycles it spends in each phase of its loop and stores the sums per CTA.  Off in the shipped library.
#ifdef KVAX_PHASE_CLOCKS
__device__ unsigned int* g_fwd_phase_clocks = nullptr;   // (grid, 4 roles, 12 slots)
#define FPH_BEGIN() unsigned int ph_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long ph_t = clock64();
#define FPH(slot) { const long long ph_now = clock64(); ph_acc[slot] += (unsigned int)(ph_now - ph_t); ph_t = ph_now; }
#define FPH_END(role, items) \
  if (g_fwd_phase_clocks && lane == 0) { \
    ph_acc[11] = (unsigned int)(items); \
    for (int s_ = 0; s_ < 12; ++s_) g_fwd_phase_clocks[((long long)blockIdx.x * 4 + (role)) * 12 + s_] = ph_acc[s_]; \
  }
#else
#define FPH_BEGIN()
#define FPH(slot)
#define FPH_END(role, items)
#endif

namespace {

constexpr int kSoftmaxThreads = 256;                 // two groups of 128
constexpr int kKWarp = 8, kMmaWarp = 9, kVWarp = 10;
constexpr int kThreads = 11 * 32;
constexpr int kTmemCols = 512;
constexpr int kKStages = 3, kVStages = 2;

enum FwdBar {
  B_QFULL0 = 0, B_QFULL1,
  B_KFULL0, B_KFULL1, B_KFULL2, B_KEMPTY0, B_KEMPTY1, B_KEMPTY2,
  B_VFULL0, B_VFULL1, B_VEMPTY0, B_VEMPTY1,
  B_SFULL0, B_SFULL1,                        // scores of group g's next list entry are in TMEM
  B_PFULL0, B_PFULL1,                        // kv columns 0-63 of group g's P are in TMEM
  B_PREST0, B_PREST1,                        // kv columns 64-127 too
  B_DONE0, B_DONE1,                          // the last P V of group g has completed: completes once
  B_COUNT
};

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;     // one 128 x D bf16 tile
  static constexpr int kBoxBytes = kTile * 64 * 2;     // one TMA box: 128 rows x 64 columns
  static constexpr int kQ = 0;                         // two query tiles
  static constexpr int kK = 2 * kTileBytes;
  static constexpr int kV = kK + kKStages * kTileBytes;
  static constexpr int kBars = kV + kVStages * kTileBytes;
  static constexpr int kTmemSlot = kBars + 8 * B_COUNT;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kDesc = kAbort + 4;             // one word per K stage: what the MMA issuer does with the entry
  static constexpr int kTotal = kDesc + 4 * kKStages + 1024;   // + slack for 1024-byte alignment
  static_assert(kTotal <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

// Walk over the union of two ascending tile lists (entries: tile index, bit 31 = needs the element mask).
// Every role that touches K / V stages (both producers, the MMA issuer) walks it the same way.  The entry
// after the cursor of each list is fetched when the cursor moves, one step before it is looked at (with a load
// the compiler cannot sink to its first use).
struct PairWalk {
  static constexpr uint32_t kEnd = 0x7fffffffu;
  const uint32_t* l0; const uint32_t* l1;
  int n0, n1, i0, i1;
  uint32_t e0, e1;
  __device__ __forceinline__ void init(const uint32_t* a, int na, const uint32_t* b, int nb) {
    l0 = a; l1 = b; n0 = na; n1 = nb; i0 = 0; i1 = 0;
    e0 = (n0 > 0) ? ldg_pinned(l0) : kEnd;
    e1 = (n1 > 0) ? ldg_pinned(l1) : kEnd;
  }
  __device__ __forceinline__ bool more() const { return i0 < n0 || i1 < n1; }
  // takes the next union entry: its kv tile and which of the two lists hold it
  __device__ __forceinline__ void next(int* tile, bool* m0, bool* m1) {
    const uint32_t t0 = (i0 < n0) ? (e0 & kTileIndexMask) : kEnd;
    const uint32_t t1 = (i1 < n1) ? (e1 & kTileIndexMask) : kEnd;
    const uint32_t t = min(t0, t1);
    *tile = int(t); *m0 = (t0 == t); *m1 = (t1 == t);
    if (*m0) { ++i0; if (i0 < n0) e0 = ldg_pinned(l0 + i0); }
    if (*m1) { ++i1; if (i1 < n1) e1 = ldg_pinned(l1 + i1); }
  }
  // membership of the entry after the one `next` returned last (only meaningful while more())
  __device__ __forceinline__ void peek(bool* m0, bool* m1) const {
    const uint32_t t0 = (i0 < n0) ? (e0 & kTileIndexMask) : kEnd;
    const uint32_t t1 = (i1 < n1) ? (e1 & kTileIndexMask) : kEnd;
    const uint32_t t = min(t0, t1);
    *m0 = (t0 == t); *m1 = (t1 == t);
  }
};

// What the MMA issuer needs to know about union entry u, worked out by the K producer (which walks the lists
// anyway) and handed over in shared memory with the K stage: the issuer's loop then holds no list arithmetic.
constexpr uint32_t kDescM0 = 1u, kDescM1 = 2u;            // entry u is in the list of tile 0 / tile 1
constexpr uint32_t kDescMore = 4u;                        // there is an entry u + 1 ...
constexpr uint32_t kDescN0 = 8u, kDescN1 = 16u;           // ... in the list of tile 0 / tile 1
constexpr uint32_t kDescLast1 = 32u;                      // ... whose scores group 1 issues last (else group 0)
constexpr uint32_t kDescFin0 = 64u, kDescFin1 = 128u;     // entry u is the last one of tile 0 / tile 1

template <int D, bool kF16>
__global__ void __launch_bounds__(kThreads, 1)
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
  volatile uint32_t* step_desc = reinterpret_cast<volatile uint32_t*>(smem + L::kDesc);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_outer = a.list.n_outer_tiles;
  // The two work items of the CTA are either two neighbouring query tiles of one head, or -- `pair_heads`, for
  // grouped-query attention -- one query tile of two query heads that read the same kv head: then both items have
  // the same tile list, every K / V tile serves both and no union entry is ever one-sided.
  const int ph = a.pair_heads ? 1 : 0;
  int pair_rank, hh;
  decode_block(blockIdx.x, (ph ? n_outer : (n_outer + 1) / 2) * a.batch, ph ? a.q_heads / 2 : a.q_heads, &pair_rank, &hh);
  const long long row0 = __ldg((ph ? a.list.order : a.list.pair_order) + pair_rank);     // list row of item 0
  const int b = int(row0 / n_outer), qt0 = int(row0 % n_outer);
  const bool has1 = ph || qt0 + 1 < n_outer;
  const int h0 = ph ? 2 * hh : hh;                       // query head of item 0; item 1: h0 + ph
  const int kvh = h0 / a.group;
  const int n0 = __ldg(a.list.counts + row0);
  const int n1 = ph ? n0 : (has1 ? __ldg(a.list.counts + row0 + 1) : 0);
  const uint32_t* list0 = a.list.tiles + row0 * a.list.n_inner_tiles;
  const uint32_t* list1 = ph ? list0 : list0 + a.list.n_inner_tiles;

  const int row = tid & (kTile - 1);
  const int wg = (tid >> 7) & 1;                         // softmax group = work item of the CTA
  const int qt = qt0 + (ph ? 0 : wg);
  const int h = h0 + (ph ? wg : 0);                      // query head of this thread's item
  const int r = qt * kTile + row;                        // query row of a softmax thread
  const bool is_softmax = tid < kSoftmaxThreads;
  const bool row_valid = is_softmax && (r < a.tok.q_len);
  const int count = wg ? n1 : n0;                        // list length of this thread's tile
  const uint32_t* list = wg ? list1 : list0;
  __nv_bfloat16* o_row = a.out + (long long)b * a.o_strides[0] + (long long)r * a.o_strides[1] + (long long)h * a.o_strides[2];
  float* lse_row = a.lse + ((long long)b * a.q_heads + h) * a.tok.q_len + r;

  if (is_softmax && count == 0 && row_valid) {           // nothing to attend: zeros (:253-258)
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(o_row)[i] = z;
    *lse_row = a.empty_lse;
  }
  if (n0 == 0 && n1 == 0) return;

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(&bars[i], (i >= B_PFULL0 && i <= B_PREST1) ? kTile : 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kKWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;                 // scores of group g: tmem_base + 128 g
  const uint32_t tO = tmem_base + 2 * kTile;             // accumulator of group g: tO + 128 g

  if (warp == kKWarp) {
    // ------------------------------------------------------------------ Q and K producer
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if ((g ? n1 : n0) == 0) continue;
        mbar_arrive_expect_tx(&bars[B_QFULL0 + g], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sQ + g * L::kTileBytes + x * L::kBoxBytes, &tmap_q, &bars[B_QFULL0 + g], x * 64, h0 + (ph ? g : 0),
                      (qt0 + (ph ? 0 : g)) * kTile, b);
      }
      PairWalk w;
      w.init(list0, n0, list1, n1);
      bool ok = true;
      for (int u = 0; w.more() && ok; ++u) {
        int tile; bool m0, m1;
        w.next(&tile, &m0, &m1);
        const int st = u % kKStages, use = u / kKStages;
        uint32_t desc = (m0 ? kDescM0 : 0u) | (m1 ? kDescM1 : 0u);
        if (m0 && w.i0 == w.n0) desc |= kDescFin0;
        if (m1 && w.i1 == w.n1) desc |= kDescFin1;
        if (w.more()) {
          bool x0, x1;
          w.peek(&x0, &x1);
          desc |= kDescMore | (x0 ? kDescN0 : 0u) | (x1 ? kDescN1 : 0u);
          // scores of entry u + 1 are issued by the members of entry u first (in group order), then by the rest
          int last_g = -1;
          if (x0 && m0) last_g = 0;
          if (x1 && m1) last_g = 1;
          if (x0 && !m0) last_g = 0;
          if (x1 && !m1) last_g = 1;
          if (last_g == 1) desc |= kDescLast1;
        }
        if (use > 0) ok = mbar_wait(&bars[B_KEMPTY0 + st], (use - 1) & 1, abort_flag, a.status, B_KEMPTY0 + st);
        if (!ok) break;
        step_desc[st] = desc;                                   // published by the arrive below
        mbar_arrive_expect_tx(&bars[B_KFULL0 + st], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sK + st * L::kTileBytes + x * L::kBoxBytes, &tmap_k, &bars[B_KFULL0 + st], x * 64, kvh, tile * kTile, b);
      }
    }
  } else if (warp == kVWarp) {
    // ------------------------------------------------------------------ V producer
    if (lane == 0) {
      prefetch_tmap(&tmap_v);
      PairWalk w;
      w.init(list0, n0, list1, n1);
      bool ok = true;
      for (int u = 0; w.more() && ok; ++u) {
        int tile; bool m0, m1;
        w.next(&tile, &m0, &m1);
        const int st = u % kVStages, use = u / kVStages;
        if (use > 0) ok = mbar_wait(&bars[B_VEMPTY0 + st], (use - 1) & 1, abort_flag, a.status, B_VEMPTY0 + st);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[B_VFULL0 + st], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(sV + st * L::kTileBytes + x * L::kBoxBytes, &tmap_v, &bars[B_VFULL0 + st], x * 64, kvh, tile * kTile, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one elected lane issues)
    constexpr uint32_t idesc_s = make_idesc_16(kTile, kTile, 0, 0, kF16);   // Q (K-major) x K (K-major)
    constexpr uint32_t idesc_o = make_idesc_16(kTile, D, 0, 1, kF16);       // P (TMEM)    x V (N-major)
    const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
    const int cnt0 = __shfl_sync(0xffffffffu, n0, 0), cnt1 = __shfl_sync(0xffffffffu, n1, 0);
    bool ok = true;
    FPH_BEGIN()
    // `tmem_sync`: the barrier orders TMEM loads / stores of other threads before the MMAs that follow; barriers
    // completed by TMA alone need no tcgen05 fence.
    auto wait = [&](int bar, uint32_t parity, bool tmem_sync) {
      ok = mbar_wait(&bars[bar], parity, abort_flag, a.status, bar);
      ok = __all_sync(0xffffffffu, ok);
      if (tmem_sync) tc_fence_after();
    };
    uint32_t ph0 = 0, ph1 = 0;               // phase of group g's P barriers = number of its P V products so far, mod 2
    uint32_t acc0 = 0, acc1 = 0;             // group g's accumulator holds something
    uint32_t d_next = 0;                     // descriptor of the entry whose K stage was waited for last
    // K stage of union entry u: waits for the tile and fetches the entry's descriptor
    auto wait_k = [&](int u) {
      const int st = u % kKStages, use = u / kKStages;
      FPH(6)
      wait(B_KFULL0 + st, use & 1, false);
      d_next = step_desc[st];
      FPH(0)
    };
    // scores of group g for union entry u; `last`: no other group will read this K stage afterwards
    auto issue_qk = [&](int g, int u, bool last) {
      const int st = u % kKStages;
      const uint32_t ts = tmem_base + g * kTile;
      const uint32_t q_lo = sdesc_lo_sw128(q_addr + g * L::kTileBytes, 16);
      const uint32_t k_lo = sdesc_lo_sw128(k_addr + st * L::kTileBytes, 16);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * L::kBoxBytes + (kk & 3) * 32) >> 4;   // 16 bf16 = 32 B inside a 128 B row
          umma_ss_lo(ts, q_lo + off, k_lo + off, idesc_s, kk > 0);
        }
        umma_commit(&bars[B_SFULL0 + g]);
        if (last) umma_commit(&bars[B_KEMPTY0 + st]);     // the K producer may refill the stage
      }
      __syncwarp();
      FPH(1)
    };
    // O_g += P_g V for union entry u (V stage vs); `release`: the last reader of the V stage; `fin`: the group's last product
    auto issue_pv = [&](int g, int vs, uint32_t ph, uint32_t acc, bool release, bool fin) {
      wait(B_PFULL0 + g, ph, true);
      FPH(3)
      if (!ok) return;
      const uint32_t tp = tmem_base + g * kTile;
      // 16 kv rows per step: rows are 128 B apart, d columns 0-63 / 64-127 in separate boxes
      const uint32_t v_lo = sdesc_lo_sw128(v_addr + vs * L::kTileBytes, L::kBoxBytes);
      // P arrives in two halves: the first four k-steps run while the group still exponentiates the second half
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < kTile / 32; ++kk)
          umma_ts_lo(tO + g * kTile, tp + kk * 8, v_lo + ((kk * 16 * 128) >> 4), idesc_o, (kk > 0) ? 1u : acc);
      }
      __syncwarp();
      FPH(5)
      wait(B_PREST0 + g, ph, true);
      FPH(4)
      if (!ok) return;
      if (elect_one()) {
#pragma unroll
        for (int kk = kTile / 32; kk < kTile / 16; ++kk)
          umma_ts_lo(tO + g * kTile, tp + kk * 8, v_lo + ((kk * 16 * 128) >> 4), idesc_o, 1u);
        if (release) umma_commit(&bars[B_VEMPTY0 + vs]);     // V stage free
        if (fin) umma_commit(&bars[B_DONE0 + g]);
      }
      __syncwarp();
      FPH(5)
    };
    if (cnt0 > 0) wait(B_QFULL0, 0, false);
    if (ok && cnt1 > 0) wait(B_QFULL1, 0, false);
    if (ok) wait_k(0);
    uint32_t d = d_next;
    if (ok && (d & kDescM0)) issue_qk(0, 0, !(d & kDescM1));
    if (ok && (d & kDescM1)) issue_qk(1, 0, true);
    int n_pv = 0;
    for (int u = 0; ok; ++u) {
      const int vs = u % kVStages, vuse = u / kVStages;
      const bool more = (d & kDescMore) != 0;
      const bool last1 = (d & kDescLast1) != 0;
      FPH(6)
      wait(B_VFULL0 + vs, vuse & 1, false);
      FPH(2)
      if (!ok) break;
      bool k_ready = false;
      if (d & kDescM0) {
        issue_pv(0, vs, ph0, acc0, !(d & kDescM1), (d & kDescFin0) != 0);
        if (!ok) break;
        ph0 ^= 1u; acc0 = 1u; ++n_pv;
        if (more && (d & kDescN0)) {              // reuses S_0: issued after PV(0, u), which read P_0
          if (!k_ready) { wait_k(u + 1); k_ready = true; if (!ok) break; }
          issue_qk(0, u + 1, !last1);
        }
      }
      if (d & kDescM1) {
        issue_pv(1, vs, ph1, acc1, true, (d & kDescFin1) != 0);
        if (!ok) break;
        ph1 ^= 1u; acc1 = 1u; ++n_pv;
        if (more && (d & kDescN1)) {
          if (!k_ready) { wait_k(u + 1); k_ready = true; if (!ok) break; }
          issue_qk(1, u + 1, last1);
        }
      }
      if (!more) break;
      if (!k_ready) { wait_k(u + 1); if (!ok) break; }
      if ((d & kDescN0) && !(d & kDescM0)) issue_qk(0, u + 1, !last1);
      if ((d & kDescN1) && !(d & kDescM1)) issue_qk(1, u + 1, last1);
      d = d_next;
    }
    FPH_END(2, n_pv)
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
    // for small increases.
    constexpr float kLazy = 8.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // element masks of this item's list that the list builder worked out (slot in the entry)
    const uint4* bitmap_row = a.list.bitmaps + ((row0 + (ph ? 0 : wg)) * kBitmapSlots) * kTile + row;
    uint32_t e_next = (count > 0) ? ldg_pinned(list) : 0u;     // list entries are fetched one iteration ahead
    FPH_BEGIN()
    for (int it = 0; it < count && ok; ++it) {
      const uint32_t e = e_next;
      if (it + 1 < count) e_next = ldg_pinned(list + it + 1);
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

      FPH(0)
      ok = mbar_wait(&bars[B_SFULL0 + wg], it & 1, abort_flag, a.status, B_SFULL0 + wg);
      ok = __all_sync(0xffffffffu, ok);         // the warp leaves the loop together (warp-wide votes below)
      FPH(1)
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
      // Rescale this group's accumulator when some row of the warp moved its reference maximum.  The group's
      // previous P V was issued before the scores that have just arrived and tcgen05.commit covers everything
      // issued before it: that product has completed.
      if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
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
      FPH(2)
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
          FPH(3)
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(&bars[B_PFULL0 + wg]);
          FPH(4)
        }
        tmem_st16(tS + ch * 16, pk);
      }
      const float rowsum = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      l = l * alpha + rowsum;
      FPH(5)
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[B_PREST0 + wg]);
      FPH(6)
    }
    if ((warp & 3) == 0) { FPH_END(wg, count) }

    // ---- epilogue of this group: normalise and store its tile.  A barrier of its own that completes once
    // tells that the group's last P V (and with it every MMA into its accumulator) has completed.
    if (count > 0) {
      if (ok) ok = mbar_wait(&bars[B_DONE0 + wg], 0, abort_flag, a.status, B_DONE0 + wg);
      if (ok) {
        tc_fence_after();
        const float inv = (l > 0.f) ? (1.f / l) : 0.f;     // a row that saw no unmasked key: O = 0
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t o[32];
          tmem_ld32(tOg + ch * 32, o);
          tmem_ld_wait(o);
          if (row_valid) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 w4;
              w4.x = pack16<kF16>(__uint_as_float(o[j + 0]) * inv, __uint_as_float(o[j + 1]) * inv);
              w4.y = pack16<kF16>(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
              w4.z = pack16<kF16>(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
              w4.w = pack16<kF16>(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
              reinterpret_cast<uint4*>(o_row)[(ch * 32 + j) >> 3] = w4;
            }
          }
        }
        // A row that saw no unmasked key gets LSE2 = +inf, so that the backward pass computes
        // exp2(s - LSE2) = 0 for it.
        if (row_valid) *lse_row = (l > 0.f) ? (m + __log2f(l)) : INFINITY;
      }
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

#ifdef KVAX_PHASE_CLOCKS
// profiling builds only: where the phase clocks go ((grid, 4, 12) uint32 in device memory), or null
extern "C" int kvax_b200_debug_set_fwd_phase_buffer(unsigned int* buf) {
  return cudaMemcpyToSymbol(g_fwd_phase_clocks, &buf, sizeof(buf)) == cudaSuccess ? 0 : -4;
}
#endif

namespace {
template <int D, bool kF16>
int launch_pairs(const FwdLaunch& L, cudaStream_t stream) {
  const FwdArgs& a = L.args;
  // one CTA per pair of query tiles and head, or per query tile and pair of heads
  dim3 grid(a.pair_heads ? a.list.n_outer_tiles * L.batch * (a.q_heads / 2) : ((a.list.n_outer_tiles + 1) / 2) * L.batch * a.q_heads, 1, 1);
  constexpr int smem = FwdSmem<D>::kTotal;
  auto kern = attn_fwd_kernel<D, kF16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return KVAX_B200_ELAUNCH;
  kern<<<grid, kThreads, smem, stream>>>(L.tmap_q, L.tmap_k, L.tmap_v, a);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
}  // namespace

int launch_attn_fwd(const FwdLaunch& L, cudaStream_t stream) {
  const bool f16 = L.dtype == KVAX_B200_F16;
  if (L.head_dim == 128) return f16 ? launch_pairs<128, true>(L, stream) : launch_pairs<128, false>(L, stream);
  if (L.head_dim == 64) return f16 ? launch_pairs<64, true>(L, stream) : launch_pairs<64, false>(L, stream);
  return KVAX_B200_EUNSUPPORTED;
}

}  // namespace kvx
