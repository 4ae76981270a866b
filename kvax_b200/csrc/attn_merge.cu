// Merge of two partial attention results over disjoint sets of keys -- the step that lets the all-gather
// schedule of context parallelism start on the keys a rank already holds while the others are still on
// their way (the reference leaves that overlap to XLA's asynchronous collectives around
// kvax/ops/flash_attention_triton.py:2107-2154).
//
// Each part is a normalised output row with the base-2 log-sum-exp of its scores (what attn_fwd writes;
// +inf marks a row without any allowed key).  With w_x = 2^(lse_x - lse), lse = log2(2^lse_a + 2^lse_b):
//     out = w_a * out_a + w_b * out_b
// 16 bytes per thread and transfer, four transfers in flight per thread: reads both parts once, writes one; HBM bound.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/kvax_b200.h"

namespace {

template <bool kF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if (kF16) return __half22float2(*reinterpret_cast<const __half2*>(&u));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}
template <bool kF16>
__device__ __forceinline__ uint32_t pack2(float x, float y) {
  if (kF16) { __half2 h = __floats2half2_rn(x, y); return *reinterpret_cast<uint32_t*>(&h); }
  __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<uint32_t*>(&h);
}

// out_a, out_b: (batch, seq, heads, head_dim) dense; lse_a, lse_b: (batch, heads, seq) fp32.  Result in out_a, lse_a.
// A thread owns 16-byte vectors; the `row_vecs` (a power of two <= 32) vectors of a row sit in one warp.  Four
// independent vectors per thread and step, every load issued before the first use.
template <bool kF16>
__global__ void __launch_bounds__(256, 3) attn_merge_kernel(uint4* __restrict__ out_a, float* __restrict__ lse_a,
                                                        const uint4* __restrict__ out_b, const float* __restrict__ lse_b,
                                                        long long total_vecs, int seq, int heads, int row_shift) {
  constexpr int kUnroll = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // the loop bound is the same for the 32 lanes of a warp (they meet in __syncwarp below); lanes past the end idle inside
  for (long long w0 = (long long)blockIdx.x * blockDim.x + (threadIdx.x - lane); w0 < total_vecs; w0 += stride * kUnroll) {
    const long long i0 = w0 + lane;
    uint4 va[kUnroll], vb[kUnroll];
    float la[kUnroll], lb[kUnroll];
    uint32_t li[kUnroll];                                 // index of the row's log-sum-exp (the row count fits 31 bits)
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      const long long i = i0 + k * stride;
      li[k] = 0xffffffffu;
      if (i >= total_vecs) continue;
      // 32-bit index arithmetic (the host checks the row count): 64-bit divisions would make the kernel issue bound
      const uint32_t row = uint32_t(i >> row_shift);
      const uint32_t bs = row / uint32_t(heads), h = row - bs * uint32_t(heads);
      const uint32_t bb = bs / uint32_t(seq), sq = bs - bb * uint32_t(seq);
      li[k] = (bb * uint32_t(heads) + h) * uint32_t(seq) + sq;
      la[k] = lse_a[li[k]];
      lb[k] = __ldg(lse_b + li[k]);
      va[k] = out_a[i];
      vb[k] = __ldg(out_b + i);
    }
    __syncwarp();                                         // every lane of a row has read lse_a before one of them replaces it
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      if (li[k] == 0xffffffffu) continue;
      const long long i = i0 + k * stride;
      const bool has_a = la[k] != INFINITY, has_b = lb[k] != INFINITY;
      float wa = 0.f, wb = 0.f, l = INFINITY;
      if (has_a || has_b) {
        const float m = has_a ? (has_b ? fmaxf(la[k], lb[k]) : la[k]) : lb[k];
        const float ea = has_a ? exp2f(la[k] - m) : 0.f, eb = has_b ? exp2f(lb[k] - m) : 0.f;
        const float inv = __fdividef(1.f, ea + eb);
        wa = ea * inv; wb = eb * inv;
        l = m + __log2f(ea + eb);
      }
      const uint32_t* a = reinterpret_cast<const uint32_t*>(&va[k]);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(&vb[k]);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = unpack2<kF16>(a[j]), y = unpack2<kF16>(b[j]);
        ow[j] = pack2<kF16>(wa * x.x + wb * y.x, wa * x.y + wb * y.y);
      }
      out_a[i] = o;
      if ((i & ((1LL << row_shift) - 1)) == 0) lse_a[li[k]] = l;
    }
  }
}

}  // namespace

extern "C" int kvax_b200_attn_merge(void* out_a, float* lse_a, const void* out_b, const float* lse_b, int64_t batch, int64_t seq,
                                    int32_t heads, int32_t head_dim, int32_t dtype, kvax_b200_stream_t stream) {
  if (!out_a || !lse_a || !out_b || !lse_b || batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0) return KVAX_B200_EINVAL;
  if (dtype != KVAX_B200_BF16 && dtype != KVAX_B200_F16) return KVAX_B200_EUNSUPPORTED;
  // a row is 1, 2, 4, ... 32 vectors of 16 bytes (head_dim 8 ... 256 at 16 bits), so that it never straddles two warps
  const int row_vecs = head_dim / 8;
  if ((head_dim & 7) || row_vecs > 32 || (row_vecs & (row_vecs - 1)) ||
      ((reinterpret_cast<uintptr_t>(out_a) | reinterpret_cast<uintptr_t>(out_b)) & 15) || seq > INT32_MAX ||
      batch * seq * heads > (int64_t)INT32_MAX)
    return KVAX_B200_EUNSUPPORTED;
  int row_shift = 0;
  while ((1 << row_shift) < row_vecs) ++row_shift;
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long total = (long long)batch * seq * heads * row_vecs;
  long long blocks = (total + 256 * 4 - 1) / (256 * 4);
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == KVAX_B200_F16)
    attn_merge_kernel<true><<<int(blocks), 256, 0, s>>>(static_cast<uint4*>(out_a), lse_a, static_cast<const uint4*>(out_b), lse_b,
                                                       total, int(seq), heads, row_shift);
  else
    attn_merge_kernel<false><<<int(blocks), 256, 0, s>>>(static_cast<uint4*>(out_a), lse_a, static_cast<const uint4*>(out_b), lse_b,
                                                        total, int(seq), heads, row_shift);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
