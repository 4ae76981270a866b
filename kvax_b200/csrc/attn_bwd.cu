// Flash-attention backward for sm_100a (B200): delta preprocess, dQ kernel, dK/dV kernel.
//
// Both main kernels keep an "outer" 128-row tile resident in shared memory (dQ kernel: the
// Q and dO tiles of one query tile and head; dK/dV kernel: the K and V tiles of one kv tile
// and kv head) while "inner" tiles stream through TMA rings (dQ kernel: K and V tiles of the
// list of kv tiles; dK/dV kernel: Q and dO tiles of every query head of the group times the
// list of query tiles).  Per inner tile:
//     T1 = X1 * Y1^T   (scores:  Q K^T   or  K Q^T)        tcgen05, both operands smem
//     T2 = X2 * Y2^T   (dP:      dO V^T  or  V dO^T)       tcgen05, both operands smem
//     P  = exp2(T1 * scale*log2e - LSE2), masked;  dS = P * (T2 - delta)   (registers)
//     P, dS -> bf16 -> TMEM
//     dV += P^T dO (dK/dV kernel);  dQ += dS K  or  dK += dS^T Q   tcgen05, A from TMEM
// The first warps do the register math (thread t: outer row t % 128 = TMEM lane and a column
// slice t / 128 of every tile: halves with 8 warps in the dQ kernel, quarters with 16 warps in
// the dK/dV kernel), the next warp is the TMA producer and the last one issues the MMAs: the
// whole warp runs the issue loop and one elected lane executes the tcgen05 instructions.  The MMA
// order is software-pipelined so that the tensor pipe has work while the register math of
// the neighbouring step runs; tcgen05.mma instructions of one thread execute in issue
// order, which is what lets a later MMA overwrite TMEM columns an earlier one reads.
// The query heads of a GQA group are accumulated on chip by the dK/dV kernel, so dK/dV
// leave the kernel already summed over the group (the reference sums a (B, Hq, Skv, D) fp32
// temporary afterwards, kvax/ops/flash_attention_triton.py:1855-1868).
//
// Semantics follow flash_attention_backward_kernel_dquery (:620-871),
// flash_attention_backward_kernel_dkdv (:874-1191) and attn_bwd_preprocess (:373-410).
#include <cuda_fp16.h>

#include "attn_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace kvx {

namespace {

constexpr int kComputeWarps = 8;                    // two per SM sub-partition
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kProducerWarp = kComputeWarps, kMmaWarp = kComputeWarps + 1;
constexpr int kThreads = (kComputeWarps + 2) * 32;
constexpr int kTmemCols = 512;
constexpr int kHalf = kTile / 2;                    // columns handled by one compute thread

// ---------------------------------------------------------------------------------------
// dK/dV kernel (kv-outer).  TMEM is full (T1 | T2 | dV | dK), so there is one score buffer:
//     T1(0) T2(0) | dV(0), T1(1) | dK(0), T2(1) | dV(1), T1(2) | ...
// P(i) is written over S(i) in T1 and dS(i) over dP(i) in T2.  LSE2 and delta are per
// column here (one query per column): the producer warp brings the 128 values of each into
// shared memory with two 512-byte bulk copies per item, on the same barrier as the Q and dO
// tiles (plus segment ids and positions for partial tiles), so the register math never
// waits on a global load.  A tile that crosses the end of the sequence, or rows that are
// not 16-byte aligned, are copied by the producer's lanes instead.
// Shared memory: K, V 2 x 32 KB + 2 stages x (Q, dO 64 KB + column info 2 KB).
// ---------------------------------------------------------------------------------------
// Sixteen register-math warps here (four per SM sub-partition: thread t owns kv row t % 128 and the 32-column quarter
// t / 128 of every tile): the math of a tile splits by columns without any exchange between threads, and four warps
// per scheduler hide the TMEM round trips and the shared-memory reads of LSE2 / delta that two warps left exposed.
constexpr int kKvComputeWarps = 16;
constexpr int kKvComputeThreads = kKvComputeWarps * 32;
constexpr int kKvProducerWarp = kKvComputeWarps, kKvMmaWarp = kKvComputeWarps + 1;
constexpr int kKvThreads = (kKvComputeWarps + 2) * 32;
constexpr int kQuarter = kTile / 4;                 // columns handled by one compute thread

enum KvBar { K_XFULL = 0, K_YFULL0, K_YFULL1, K_YEMPTY0, K_YEMPTY1, K_SFULL0, K_SFULL1, K_DPFULL, K_PFULL0, K_PFULL1, K_DSFULL, K_ACCFULL, K_COUNT };

template <int D>
struct KvSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kBoxBytes = kTile * 64 * 2;
  static constexpr int kX1 = 0, kX2 = kTileBytes;
  static constexpr int kY = 2 * kTileBytes;              // stage s: Q at kY + s*2*tile, dO right after
  static constexpr int kCols = 6 * kTileBytes;           // stage s: seg | pos | lse2 | delta, 128 x 4 B each
  static constexpr int kColBytes = kTile * 4;
  static constexpr int kBars = kCols + 2 * 4 * kColBytes;
  static constexpr int kTmemSlot = kBars + 8 * K_COUNT;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4 + 1024;
  static_assert(kTotal <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

template <int D, bool kF16>
__global__ void __launch_bounds__(kKvThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                     const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                     const BwdArgs a) {
  using L = KvSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbort);
  int* s_cols = reinterpret_cast<int*>(smem + L::kCols);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int row_rank, kvh;
  decode_block(blockIdx.x, a.list.n_outer_tiles * a.batch, a.kv_heads, &row_rank, &kvh);
  const long long list_row = __ldg(a.list.order + row_rank);     // longest lists first
  const int b = int(list_row / a.list.n_outer_tiles), kt = int(list_row % a.list.n_outer_tiles);
  const int group = a.group;
  const int count = __ldg(a.list.counts + list_row);
  const uint32_t* list = a.list.tiles + list_row * a.list.n_inner_tiles;
  const int n_items = count * group;           // item i: query head kvh*group + i / count, query tile list[i % count]
  const int q_len = a.tok.q_len;

  const int row = tid & (kTile - 1);           // kv row / TMEM lane of a compute thread
  const int quarter = tid >> 7;                 // column quarter of a compute thread
  const int half = quarter & 1;                // epilogue: quarters 0 and 1 store D/2 columns each
  const int r = kt * kTile + row;
  const bool is_compute = tid < kKvComputeThreads;
  const bool row_valid = is_compute && (r < a.tok.kv_len);
  // dK / dV rows of this thread: fp32, or 16-bit elements of the operand type when the caller asked for that
  const long long dkv_off = (((long long)b * a.tok.kv_len + r) * a.kv_heads + kvh) * D + half * (D / 2);
  float* dk_row = a.dk + dkv_off;
  float* dv_row = a.dv + dkv_off;
  uint16_t* dk_row16 = reinterpret_cast<uint16_t*>(a.dk) + dkv_off;
  uint16_t* dv_row16 = reinterpret_cast<uint16_t*>(a.dv) + dkv_off;

  if (n_items == 0) {                          // no contributing tile: zero gradients
    if (row_valid && quarter < 2) {
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
    for (int i = 0; i < K_COUNT; ++i)
      mbar_init(&bars[i], (i == K_PFULL0 || i == K_PFULL1 || i == K_DSFULL) ? kKvComputeThreads : 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kKvProducerWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tT1 = tmem_base, tT2 = tmem_base + kTile;
  const uint32_t tAcc1 = tmem_base + 2 * kTile, tAcc2 = tmem_base + 3 * kTile;

  if (warp == kKvProducerWarp) {
    // ------------------------------------------------------------------ producer (whole warp; one elected lane issues)
    const int n = __shfl_sync(0xffffffffu, n_items, 0);
    const int cnt = __shfl_sync(0xffffffffu, count, 0);
    if (elect_one()) {
      prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do);
      mbar_arrive_expect_tx(&bars[K_XFULL], 2 * L::kTileBytes);
#pragma unroll
      for (int x = 0; x < D / 64; ++x) {
        tma_load_4d(smem + L::kX1 + x * L::kBoxBytes, &tmap_k, &bars[K_XFULL], x * 64, kvh, kt * kTile, b);
        tma_load_4d(smem + L::kX2 + x * L::kBoxBytes, &tmap_v, &bars[K_XFULL], x * 64, kvh, kt * kTile, b);
      }
    }
    __syncwarp();
    bool ok = true;
    uint32_t e_next = __ldg(list);                 // list entries are fetched one iteration ahead
    int li = 0, qh = kvh * group;                  // index into the list, query head
    for (int i = 0; i < n && ok; ++i) {
      const int st = i & 1;
      const uint32_t e = e_next;
      const int u = int(e & kTileIndexMask);
      const bool partial = (e & kPartialBit) != 0;
      const int yh = qh;
      if (++li == cnt) { li = 0; ++qh; }
      if (i + 1 < n) e_next = __ldg(list + li);
      if (i >= 2) {
        ok = mbar_wait(&bars[K_YEMPTY0 + st], ((i >> 1) - 1) & 1, abort_flag, a.status, K_YEMPTY0 + st);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (!ok) break;
      uint8_t* y1 = smem + L::kY + st * 2 * L::kTileBytes;
      uint8_t* y2 = y1 + L::kTileBytes;
      int* cs = s_cols + st * 4 * kTile;
      const int col0 = u * kTile;
      const float* lse_src = a.lse + ((long long)b * a.q_heads + yh) * q_len + col0;
      const float* dl_src = a.delta + ((long long)b * a.q_heads + yh) * q_len + col0;
      const int32_t* seg_src = a.tok.q_seg + (long long)b * q_len + col0;
      const int32_t* pos_src = a.tok.sequential ? nullptr : a.tok.q_pos + (long long)b * q_len + col0;
      uintptr_t align = reinterpret_cast<uintptr_t>(lse_src) | reinterpret_cast<uintptr_t>(dl_src);
      if (partial) align |= reinterpret_cast<uintptr_t>(seg_src) | reinterpret_cast<uintptr_t>(pos_src);
      const bool bulk = (col0 + kTile <= q_len) && ((align & 15) == 0);
      uint32_t extra = 0;
      if (bulk) {
        extra = 2 * L::kColBytes;
        if (partial) {
          extra += L::kColBytes;
          if (pos_src) {
            extra += L::kColBytes;
          } else {
#pragma unroll
            for (int k = 0; k < kTile / 32; ++k) cs[kTile + lane + 32 * k] = query_position(a.tok, b, col0 + lane + 32 * k);
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < kTile / 32; ++k) {
          const int j = lane + 32 * k;
          const bool valid = col0 + j < q_len;
          reinterpret_cast<float*>(cs)[2 * kTile + j] = valid ? __ldg(lse_src + j) : INFINITY;   // exp2(-inf) = 0
          reinterpret_cast<float*>(cs)[3 * kTile + j] = valid ? __ldg(dl_src + j) : 0.f;
          if (partial) {
            cs[j] = valid ? __ldg(seg_src + j) : KVAX_B200_PADDING_SEGMENT_ID;
            cs[kTile + j] = valid ? query_position(a.tok, b, col0 + j) : 0;
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (elect_one()) {
        mbar_arrive_expect_tx(&bars[K_YFULL0 + st], 2 * L::kTileBytes + extra);
#pragma unroll
        for (int x = 0; x < D / 64; ++x) {
          tma_load_4d(y1 + x * L::kBoxBytes, &tmap_q, &bars[K_YFULL0 + st], x * 64, yh, u * kTile, b);
          tma_load_4d(y2 + x * L::kBoxBytes, &tmap_do, &bars[K_YFULL0 + st], x * 64, yh, u * kTile, b);
        }
        if (bulk) {
          bulk_load_1d(cs + 2 * kTile, lse_src, L::kColBytes, &bars[K_YFULL0 + st]);
          bulk_load_1d(cs + 3 * kTile, dl_src, L::kColBytes, &bars[K_YFULL0 + st]);
          if (partial) {
            bulk_load_1d(cs, seg_src, L::kColBytes, &bars[K_YFULL0 + st]);
            if (pos_src) bulk_load_1d(cs + kTile, pos_src, L::kColBytes, &bars[K_YFULL0 + st]);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp == kKvMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one elected lane issues)
    constexpr uint32_t idesc_t = make_idesc_16(kTile, kTile, 0, 0, kF16);
    constexpr uint32_t idesc_acc = make_idesc_16(kTile, D, 0, 1, kF16);
    const uint32_t x1_lo = sdesc_lo_sw128(smem_u32(smem + L::kX1), 16), x2_lo = sdesc_lo_sw128(smem_u32(smem + L::kX2), 16);
    const uint32_t ybase = smem_u32(smem + L::kY);
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
    // A operand (bf16 pairs in TMEM): quarter q wrote its two K-steps at column offset 32 q
    auto issue_acc = [&](uint32_t acc_addr, uint32_t a_addr, uint32_t y_lo, uint32_t acc_on) {
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk)
        umma_ts_lo(acc_addr, a_addr + (kk >> 1) * kQuarter + (kk & 1) * 8, y_lo + ((kk * 16 * 128) >> 4), idesc_acc, acc_on | (kk > 0));
    };
    wait(K_XFULL, 0, false);
    if (ok) wait(K_YFULL0, 0, false);
    if (ok) {
      if (elect_one()) {
        issue_t(tT1, x1_lo, sdesc_lo_sw128(ybase, 16));
        umma_commit(&bars[K_SFULL0]);
        issue_t(tT2, x2_lo, sdesc_lo_sw128(ybase + L::kTileBytes, 16));
        umma_commit(&bars[K_DPFULL]);
      }
      __syncwarp();
    }
    for (int i = 0; i < n && ok; ++i) {
      const int st = i & 1;
      const uint32_t y1 = ybase + st * 2 * L::kTileBytes, y2 = y1 + L::kTileBytes;
      const uint32_t y1n = ybase + (st ^ 1) * 2 * L::kTileBytes, y2n = y1n + L::kTileBytes;
      const uint32_t acc_on = (i > 0) ? 1u : 0u;
      const bool more = (i + 1 < n);
      wait(K_PFULL0 + st, (i >> 1) & 1, true);                                      // P(i) written, S(i) consumed
      if (!ok) break;
      if (elect_one()) issue_acc(tAcc1, tT1, sdesc_lo_sw128(y2, L::kBoxBytes), acc_on);   // dV += P^T dO
      __syncwarp();
      if (more) {
        wait(K_YFULL0 + (st ^ 1), ((i + 1) >> 1) & 1, false);
        if (!ok) break;
        if (elect_one()) {
          issue_t(tT1, x1_lo, sdesc_lo_sw128(y1n, 16));                             // scores of item i+1
          umma_commit(&bars[K_SFULL0 + (st ^ 1)]);
        }
        __syncwarp();
      }
      wait(K_DSFULL, i & 1, true);                                                  // dS(i) written
      if (!ok) break;
      if (elect_one()) {
        issue_acc(tAcc2, tT2, sdesc_lo_sw128(y1, L::kBoxBytes), acc_on);            // dK += dS^T Q
        umma_commit(&bars[K_YEMPTY0 + st]);
        if (more) {
          issue_t(tT2, x2_lo, sdesc_lo_sw128(y2n, 16));                             // dP of item i+1
          umma_commit(&bars[K_DPFULL]);
        } else {
          umma_commit(&bars[K_ACCFULL]);
        }
      }
      __syncwarp();
    }
  } else if (is_compute) {
    // ------------------------------------------------------------------ register math
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const int cb = quarter * kQuarter;                        // first column (within the tile) of this thread
    const uint32_t my_t1 = tT1 + lane_base + cb;              // fp32 columns of this thread; P goes to the first 16 of them
    const uint32_t my_t2 = tT2 + lane_base + cb;
    const float c = a.scale_log2e;
    const RowBounds rb = load_bounds(a.mask, b, min(r, a.tok.kv_len - 1));
    int kv_seg = KVAX_B200_PADDING_SEGMENT_ID, kv_pos = 0;
    if (row_valid) {
      kv_seg = __ldg(a.tok.kv_seg + (long long)b * a.tok.kv_len + r);
      kv_pos = a.tok.sequential ? r : __ldg(a.tok.kv_pos + (long long)b * a.tok.kv_len + r);
    }
    bool ok = true;
    uint32_t e_next = __ldg(list);
    int li = 0;
    for (int i = 0; i < n_items && ok; ++i) {
      const uint32_t e = e_next;
      if (++li == count) li = 0;
      if (i + 1 < n_items) e_next = __ldg(list + li);
      const int c0 = int(e & kTileIndexMask) * kTile;
      const bool partial = (e & kPartialBit) != 0;
      const int st = i & 1;                                   // Y stage, column-info buffer and barrier pair of this item
      const int* cs = s_cols + st * 4 * kTile;
      const float4* cs_lse = reinterpret_cast<const float4*>(cs + 2 * kTile + cb);
      const float4* cs_dl = reinterpret_cast<const float4*>(cs + 3 * kTile + cb);

      // column info of this item has landed together with its Q and dO tiles
      ok = mbar_wait(&bars[K_YFULL0 + st], (i >> 1) & 1, abort_flag, a.status, K_YFULL0 + st);
      if (!ok) break;

      // element mask of partial tiles, one bit per column of this thread's quarter
      uint32_t keep = 0xffffffffu;
      if (partial) keep = keep_bits32<true>(rb, c0 + cb, q_len, row_valid, kv_seg, kv_pos, cs + cb, cs + kTile + cb);

      // ---- P = exp2(S * scale*log2e - LSE2): the 32 values of this thread stay in registers
      ok = mbar_wait(&bars[K_SFULL0 + st], (i >> 1) & 1, abort_flag, a.status, K_SFULL0 + st);
      if (!ok) break;
      tc_fence_after();
      uint32_t v[32];
      tmem_ld32(my_t1, v);
      tmem_ld_wait(v);
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4) {
        const float4 ls = cs_lse[jj >> 2];
        const float l4[4] = {ls.x, ls.y, ls.z, ls.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float pv = fast_exp2(fmaf(__uint_as_float(v[jj + t]), c, -l4[t]));
          if (partial) pv = ((keep >> (jj + t)) & 1u) ? pv : 0.f;
          v[jj + t] = __float_as_uint(pv);
        }
      }
      {
        uint32_t pk[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 2) pk[jj >> 1] = pack16<kF16>(__uint_as_float(v[jj]), __uint_as_float(v[jj + 1]));
        tmem_st16(my_t1, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[K_PFULL0 + st]);

      // ---- dS = P * (dP - delta)
      ok = mbar_wait(&bars[K_DPFULL], i & 1, abort_flag, a.status, K_DPFULL);
      if (!ok) break;
      tc_fence_after();
      uint32_t dp[32];
      tmem_ld32(my_t2, dp);
      tmem_ld_wait(dp);
      {
        uint32_t ds[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
          const float4 dl = cs_dl[jj >> 2];
          const float d0 = __uint_as_float(v[jj + 0]) * (__uint_as_float(dp[jj + 0]) - dl.x);
          const float d1 = __uint_as_float(v[jj + 1]) * (__uint_as_float(dp[jj + 1]) - dl.y);
          const float d2 = __uint_as_float(v[jj + 2]) * (__uint_as_float(dp[jj + 2]) - dl.z);
          const float d3 = __uint_as_float(v[jj + 3]) * (__uint_as_float(dp[jj + 3]) - dl.w);
          ds[jj >> 1] = pack16<kF16>(d0, d1);
          ds[(jj >> 1) + 1] = pack16<kF16>(d2, d3);
        }
        tmem_st16(my_t2, ds);      // over the first 16 of this thread's 32 dP columns, all of which are in registers
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[K_DSFULL]);
    }

    if (ok) ok = mbar_wait(&bars[K_ACCFULL], 0, abort_flag, a.status, K_ACCFULL);
    if (ok && quarter < 2) {
      tc_fence_after();
      // threads of quarters 0 and 1 store D/2 columns of their row: columns [half*D/2, (half+1)*D/2)
#pragma unroll
      for (int ch = 0; ch < D / 64; ++ch) {
        uint32_t v1[32], v2[32];
        tmem_ld32(tAcc1 + lane_base + half * (D / 2) + ch * 32, v1);
        tmem_ld32(tAcc2 + lane_base + half * (D / 2) + ch * 32, v2);
        tmem_ld_wait(v1);
        tmem_ld_wait(v2);
        if (row_valid) {
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kKvProducerWarp) {
    if (*abort_flag && lane == 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) { }
    }
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// dQ kernel (query-outer).  Same building blocks as the template above, with a pipeline of
// its own that the free TMEM columns make possible:
//   * K runs through a three-stage ring, V through a two-stage ring (V is only needed for dP);
//   * the scores are double-buffered (T1a / T1b) and issued two items ahead;
//   * dS(i) is written over the consumed scores S(i) instead of over dP(i), so dP(i+1) does
//     not wait for the dQ MMAs of item i:
//         T1(0) T2(0) T1(1) | T2(1), dQ(0), T1(2) | T2(2), dQ(1), T1(3) | ...
//   * LSE2 and delta are per-row scalars here, and the segment ids / positions of partial
//     tiles are read straight from global memory, so there is no per-item staging barrier.
// TMEM: T1a | T2 | T1b | dQ.  Shared memory: Q, dO 2 x 32 KB + K 3 x 32 KB + V 2 x 32 KB.
// ---------------------------------------------------------------------------------------
constexpr int kDqKStages = 3, kDqVStages = 2;
enum DqBar {
  Q_XFULL = 0, Q_KFULL0, Q_KFULL1, Q_KFULL2, Q_KEMPTY0, Q_KEMPTY1, Q_KEMPTY2,
  Q_VFULL0, Q_VFULL1, Q_VEMPTY0, Q_VEMPTY1, Q_SFULL0, Q_SFULL1, Q_DPFULL, Q_DSFULL, Q_ACCFULL, Q_COUNT
};

template <int D>
struct DqSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kBoxBytes = kTile * 64 * 2;
  static constexpr int kX1 = 0, kX2 = kTileBytes;
  static constexpr int kK = 2 * kTileBytes;
  static constexpr int kV = kK + kDqKStages * kTileBytes;
  static constexpr int kBars = kV + kDqVStages * kTileBytes;
  static constexpr int kTmemSlot = kBars + 8 * Q_COUNT;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4 + 1024;
  static_assert(kTotal <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

template <int D, bool kF16>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const BwdArgs a) {
  using L = DqSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbort);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int row_rank, h;
  decode_block(blockIdx.x, a.list.n_outer_tiles * a.batch, a.q_heads, &row_rank, &h);
  const long long list_row = __ldg(a.list.order + row_rank);     // longest lists first
  const int b = int(list_row / a.list.n_outer_tiles), qt = int(list_row % a.list.n_outer_tiles);
  const int kvh = h / a.group;
  const int n_items = __ldg(a.list.counts + list_row);
  const uint32_t* list = a.list.tiles + list_row * a.list.n_inner_tiles;

  const int row = tid & (kTile - 1);
  const int half = (tid >> 7) & 1;
  const int r = qt * kTile + row;
  const bool is_compute = tid < kComputeThreads;
  const bool row_valid = is_compute && (r < a.tok.q_len);
  __nv_bfloat16* dq_row = a.dq + (long long)b * a.dq_strides[0] + (long long)r * a.dq_strides[1] + (long long)h * a.dq_strides[2] + half * (D / 2);

  if (n_items == 0) {
    if (row_valid) {
      uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < D / 16; ++i) reinterpret_cast<uint4*>(dq_row)[i] = z;
    }
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < Q_COUNT; ++i) mbar_init(&bars[i], i == Q_DSFULL ? kComputeThreads : 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tT1a = tmem_base, tT2 = tmem_base + kTile, tT1b = tmem_base + 2 * kTile, tAcc = tmem_base + 3 * kTile;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(&bars[Q_XFULL], 2 * L::kTileBytes);
#pragma unroll
      for (int x = 0; x < D / 64; ++x) {
        tma_load_4d(smem + L::kX1 + x * L::kBoxBytes, &tmap_q, &bars[Q_XFULL], x * 64, h, qt * kTile, b);
        tma_load_4d(smem + L::kX2 + x * L::kBoxBytes, &tmap_do, &bars[Q_XFULL], x * 64, h, qt * kTile, b);
      }
      bool ok = true;
      uint32_t e_next = ldg_pinned(list);
      for (int i = 0; i < n_items && ok; ++i) {
        const int u = int(e_next & kTileIndexMask);
        if (i + 1 < n_items) e_next = ldg_pinned(list + i + 1);
        const int ks = i % kDqKStages, kuse = i / kDqKStages;
        if (kuse > 0) ok = mbar_wait(&bars[Q_KEMPTY0 + ks], (kuse - 1) & 1, abort_flag, a.status, Q_KEMPTY0 + ks);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[Q_KFULL0 + ks], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(smem + L::kK + ks * L::kTileBytes + x * L::kBoxBytes, &tmap_k, &bars[Q_KFULL0 + ks], x * 64, kvh, u * kTile, b);
        const int vs = i % kDqVStages, vuse = i / kDqVStages;
        if (vuse > 0) ok = mbar_wait(&bars[Q_VEMPTY0 + vs], (vuse - 1) & 1, abort_flag, a.status, Q_VEMPTY0 + vs);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[Q_VFULL0 + vs], L::kTileBytes);
#pragma unroll
        for (int x = 0; x < D / 64; ++x)
          tma_load_4d(smem + L::kV + vs * L::kTileBytes + x * L::kBoxBytes, &tmap_v, &bars[Q_VFULL0 + vs], x * 64, kvh, u * kTile, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one elected lane issues)
    constexpr uint32_t idesc_t = make_idesc_16(kTile, kTile, 0, 0, kF16);
    constexpr uint32_t idesc_acc = make_idesc_16(kTile, D, 0, 1, kF16);
    const uint32_t x1_lo = sdesc_lo_sw128(smem_u32(smem + L::kX1), 16), x2_lo = sdesc_lo_sw128(smem_u32(smem + L::kX2), 16);
    const uint32_t kbase = smem_u32(smem + L::kK), vbase = smem_u32(smem + L::kV);
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
    auto issue_t1 = [&](int i) {               // scores of item i into buffer i & 1
      const int ks = i % kDqKStages;
      wait(Q_KFULL0 + ks, (i / kDqKStages) & 1, false);
      if (!ok) return;
      const uint32_t k_lo = sdesc_lo_sw128(kbase + ks * L::kTileBytes, 16);
      if (elect_one()) {
        issue_t((i & 1) ? tT1b : tT1a, x1_lo, k_lo);
        umma_commit(&bars[Q_SFULL0 + (i & 1)]);
      }
      __syncwarp();
    };
    auto issue_t2 = [&](int i) {               // dP of item i
      const int vs = i % kDqVStages;
      wait(Q_VFULL0 + vs, (i / kDqVStages) & 1, false);
      if (!ok) return;
      const uint32_t v_lo = sdesc_lo_sw128(vbase + vs * L::kTileBytes, 16);
      if (elect_one()) {
        issue_t(tT2, x2_lo, v_lo);
        umma_commit(&bars[Q_DPFULL]);
        umma_commit(&bars[Q_VEMPTY0 + vs]);
      }
      __syncwarp();
    };
    wait(Q_XFULL, 0, false);
    if (ok) issue_t1(0);
    if (ok) issue_t2(0);
    if (ok && n > 1) issue_t1(1);
    for (int i = 0; i < n && ok; ++i) {
      wait(Q_DSFULL, i & 1, true);                   // dS(i) written; dP(i), S(i) consumed
      if (!ok) break;
      if (i + 1 < n) issue_t2(i + 1);
      if (!ok) break;
      const int ks = i % kDqKStages;
      const uint32_t ds_addr = (i & 1) ? tT1b : tT1a;
      const uint32_t k_lo = sdesc_lo_sw128(kbase + ks * L::kTileBytes, L::kBoxBytes);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)                                      // dQ += dS K
          umma_ts_lo(tAcc, ds_addr + (kk >> 2) * kHalf + (kk & 3) * 8, k_lo + ((kk * 16 * 128) >> 4), idesc_acc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bars[Q_KEMPTY0 + ks]);
        if (i + 1 >= n) umma_commit(&bars[Q_ACCFULL]);
      }
      __syncwarp();
      if (i + 2 < n) issue_t1(i + 2);          // over dS(i): after the dQ MMAs of item i in issue order
    }
  } else {
    // ------------------------------------------------------------------ register math
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const int cb = half * kHalf;
    const float c = a.scale_log2e;
    const RowBounds rb = load_bounds(a.mask, b, min(r, a.tok.q_len - 1));
    int q_seg = KVAX_B200_PADDING_SEGMENT_ID, q_pos = 0;
    float neg_lse = 0.f, delta = 0.f;
    if (row_valid) {
      q_seg = __ldg(a.tok.q_seg + (long long)b * a.tok.q_len + r);
      q_pos = query_position(a.tok, b, r);
      neg_lse = -__ldg(a.lse + ((long long)b * a.q_heads + h) * a.tok.q_len + r);
      delta = __ldg(a.delta + ((long long)b * a.q_heads + h) * a.tok.q_len + r);
    }
    const int32_t* kv_seg = a.tok.kv_seg + (long long)b * a.tok.kv_len;
    const int32_t* kv_pos = a.tok.kv_pos + (long long)b * a.tok.kv_len;
    bool ok = true;
    uint32_t e_next = ldg_pinned(list);
    for (int i = 0; i < n_items && ok; ++i) {
      const uint32_t e = e_next;
      if (i + 1 < n_items) e_next = ldg_pinned(list + i + 1);
      const int c0 = int(e & kTileIndexMask) * kTile;
      const bool partial = (e & kPartialBit) != 0;
      uint32_t keep[2] = {0xffffffffu, 0xffffffffu};
      if (partial) {
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
          keep[ch] = keep_bits32<false>(rb, c0 + cb + ch * 32, a.tok.kv_len, row_valid, q_seg, q_pos, kv_seg + c0 + cb + ch * 32,
                                        a.tok.sequential ? nullptr : kv_pos + c0 + cb + ch * 32);
      }
      const int sbuf = i & 1;
      const uint32_t my_t1 = (sbuf ? tT1b : tT1a) + lane_base + cb;
      const uint32_t my_t2 = tT2 + lane_base + cb;

      // ---- P = exp2(S * scale*log2e - LSE2)
      ok = mbar_wait(&bars[Q_SFULL0 + sbuf], (i >> 1) & 1, abort_flag, a.status, Q_SFULL0 + sbuf);
      if (!ok) break;
      tc_fence_after();
      uint32_t v[2][32], dp[2][32];
      tmem_ld32(my_t1, v[0]);
      tmem_ld32(my_t1 + 32, v[1]);
      tmem_ld_wait(v[0]);
      tmem_ld_wait(v[1]);
      auto exp_chunk = [&](int ch) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          float pv = fast_exp2(fmaf(__uint_as_float(v[ch][jj]), c, neg_lse));
          if (partial) pv = ((keep[ch] >> jj) & 1u) ? pv : 0.f;
          v[ch][jj] = __float_as_uint(pv);
        }
      };
      exp_chunk(0);
      // dP of this item was issued a whole item ago: its TMEM round trip overlaps the second
      // half of the exponentials
      ok = mbar_wait(&bars[Q_DPFULL], i & 1, abort_flag, a.status, Q_DPFULL);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(my_t2, dp[0]);
      tmem_ld32(my_t2 + 32, dp[1]);
      exp_chunk(1);

      // ---- dS = P * (dP - delta), written over the consumed scores of this item
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        tmem_ld_wait(dp[ch]);
        uint32_t ds[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 2) {
          const float d0 = __uint_as_float(v[ch][jj]) * (__uint_as_float(dp[ch][jj]) - delta);
          const float d1 = __uint_as_float(v[ch][jj + 1]) * (__uint_as_float(dp[ch][jj + 1]) - delta);
          ds[jj >> 1] = pack16<kF16>(d0, d1);
        }
        tmem_st16(my_t1 + ch * 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[Q_DSFULL]);
    }

    if (ok) ok = mbar_wait(&bars[Q_ACCFULL], 0, abort_flag, a.status, Q_ACCFULL);
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int ch = 0; ch < D / 64; ++ch) {
        uint32_t v[32];
        tmem_ld32(tAcc + lane_base + half * (D / 2) + ch * 32, v);
        tmem_ld_wait(v);
        if (row_valid) {
#pragma unroll
          for (int jj = 0; jj < 32; jj += 8) {
            uint4 w;
            w.x = pack16<kF16>(__uint_as_float(v[jj + 0]) * a.scale, __uint_as_float(v[jj + 1]) * a.scale);
            w.y = pack16<kF16>(__uint_as_float(v[jj + 2]) * a.scale, __uint_as_float(v[jj + 3]) * a.scale);
            w.z = pack16<kF16>(__uint_as_float(v[jj + 4]) * a.scale, __uint_as_float(v[jj + 5]) * a.scale);
            w.w = pack16<kF16>(__uint_as_float(v[jj + 6]) * a.scale, __uint_as_float(v[jj + 7]) * a.scale);
            reinterpret_cast<uint4*>(dq_row)[(ch * 32 + jj) >> 3] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
    if (*abort_flag && lane == 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) { }
    }
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[b, h, s] = sum_d O[b, s, h, d] * dO[b, s, h, d]   (fp32), HBM-bound.
// D/8 lanes per row (16-byte loads), 32 / (D/8) rows per warp.  With `dq_acc` the same lanes zero
// their eight elements of the row's fp32 dQ accumulator ((B, Sq, Hq, D) contiguous).
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                            const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                                            float* __restrict__ dq_acc, long long sb, long long ss,
                                                            long long sh, int batch, int seq, int heads, int f16) {
  constexpr int kLanes = D / 8, kRowsPerWarp = 32 / kLanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / kLanes, li = lane % kLanes;
  const long long n_rows = (long long)batch * seq * heads;
  const long long warps_total = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w * kRowsPerWarp < n_rows; w += warps_total) {
    const long long row = w * kRowsPerWarp + sub;            // = (b * seq + s) * heads + h
    float acc = 0.f;
    long long b = 0, s = 0, h = 0;
    if (row < n_rows) {
      h = row % heads; s = (row / heads) % seq; b = row / ((long long)heads * seq);
      const long long off = b * sb + s * ss + h * sh + li * 8;
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(o + off));
      const uint4 y = __ldg(reinterpret_cast<const uint4*>(d_o + off));
      if (dq_acc) {
        float4* z = reinterpret_cast<float4*>(dq_acc + row * D + li * 8);
        z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float2 xf, yf;
        if (f16) {
          xf = __half22float2(*reinterpret_cast<const __half2*>(&xw[t]));
          yf = __half22float2(*reinterpret_cast<const __half2*>(&yw[t]));
        } else {
          xf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[t]));
          yf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yw[t]));
        }
        acc = fmaf(xf.x, yf.x, acc);
        acc = fmaf(xf.y, yf.y, acc);
      }
    }
#pragma unroll
    for (int m = kLanes / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (row < n_rows && li == 0) delta[(b * heads + h) * seq + s] = acc;
  }
}

template <int D, bool kF16>
int launch_dkdv(const BwdLaunch& L, cudaStream_t stream) {
  constexpr int smem = KvSmem<D>::kTotal;
  auto kern = attn_bwd_dkdv_kernel<D, kF16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return KVAX_B200_ELAUNCH;
  dim3 grid(L.args.list.n_outer_tiles * L.batch * L.args.kv_heads, 1, 1);
  kern<<<grid, kKvThreads, smem, stream>>>(L.tmap_x1, L.tmap_x2, L.tmap_y1, L.tmap_y2, L.args);   // K, V, Q, dO
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

template <int D, bool kF16>
int launch_dq(const BwdLaunch& L, cudaStream_t stream) {
  constexpr int smem = DqSmem<D>::kTotal;
  auto kern = attn_bwd_dq_kernel<D, kF16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return KVAX_B200_ELAUNCH;
  dim3 grid(L.args.list.n_outer_tiles * L.batch * L.args.q_heads, 1, 1);
  kern<<<grid, kThreads, smem, stream>>>(L.tmap_x1, L.tmap_x2, L.tmap_y1, L.tmap_y2, L.args);   // Q, dO, K, V
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

}  // namespace

int launch_attn_bwd(const BwdLaunch& L, bool kv_outer, cudaStream_t stream) {
  if (L.dtype == KVAX_B200_F16) {
    if (L.head_dim == 128) return kv_outer ? launch_dkdv<128, true>(L, stream) : launch_dq<128, true>(L, stream);
    if (L.head_dim == 64) return kv_outer ? launch_dkdv<64, true>(L, stream) : launch_dq<64, true>(L, stream);
    return KVAX_B200_EUNSUPPORTED;
  }
  if (L.head_dim == 128) return kv_outer ? launch_dkdv<128, false>(L, stream) : launch_dq<128, false>(L, stream);
  if (L.head_dim == 64) return kv_outer ? launch_dkdv<64, false>(L, stream) : launch_dq<64, false>(L, stream);
  return KVAX_B200_EUNSUPPORTED;
}

int launch_attn_bwd_delta(const __nv_bfloat16* o, const __nv_bfloat16* d_o, float* delta, float* dq_acc,
                          const long long* strides, int batch, int seq, int heads, int head_dim, int dtype,
                          cudaStream_t stream) {
  const int f16 = dtype == KVAX_B200_F16;
  const long long rows = (long long)batch * seq * heads;
  const int rows_per_warp = 32 / (head_dim / 8);
  long long blocks = (rows / rows_per_warp + 7) / 8 + 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (head_dim == 128)
    attn_bwd_delta_kernel<128><<<int(blocks), 256, 0, stream>>>(o, d_o, delta, dq_acc, strides[0], strides[1], strides[2], batch, seq, heads, f16);
  else if (head_dim == 64)
    attn_bwd_delta_kernel<64><<<int(blocks), 256, 0, stream>>>(o, d_o, delta, dq_acc, strides[0], strides[1], strides[2], batch, seq, heads, f16);
  else
    return KVAX_B200_EUNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

}  // namespace kvx
