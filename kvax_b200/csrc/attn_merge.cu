// Merge of two partial attention results over disjoint sets of keys -- the step that lets the all-gather
// schedule of context parallelism start on the keys a rank already holds while the others are still on
// their way (the reference leaves that overlap to XLA's asynchronous collectives around
// kvax/ops/flash_attention_triton.py:2107-2154).
//
// Each part is a normalised output row with the base-2 log-sum-exp of its scores (what attn_fwd writes;
// +inf marks a row without any allowed key).  With w_x = 2^(lse_x - lse), lse = log2(2^lse_a + 2^lse_b):
//     out = w_a * out_a + w_b * out_b
// One warp per (token, head) row, 8 or 16 bytes per lane: reads both parts once, writes one; HBM bound.
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
template <bool kF16>
__global__ void __launch_bounds__(256) attn_merge_kernel(uint2* __restrict__ out_a, float* __restrict__ lse_a,
                                                        const uint2* __restrict__ out_b, const float* __restrict__ lse_b,
                                                        long long rows, int seq, int heads, int row_vecs) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int h = int(r % heads);
    const long long bs = r / heads;
    const int s = int(bs % seq);
    const long long b = bs / seq;
    const long long li = (b * heads + h) * seq + s;
    const float la = lse_a[li], lb = lse_b[li];
    const bool has_a = la != INFINITY, has_b = lb != INFINITY;
    float wa = 0.f, wb = 0.f, l = INFINITY;
    if (has_a || has_b) {
      const float m = has_a ? (has_b ? fmaxf(la, lb) : la) : lb;
      const float ea = has_a ? exp2f(la - m) : 0.f, eb = has_b ? exp2f(lb - m) : 0.f;
      const float inv = 1.f / (ea + eb);
      wa = ea * inv; wb = eb * inv;
      l = m + log2f(ea + eb);
    }
    for (int v = lane; v < row_vecs; v += 32) {
      const long long i = r * row_vecs + v;
      const uint2 a = out_a[i], bq = __ldg(out_b + i);
      const float2 a0 = unpack2<kF16>(a.x), a1 = unpack2<kF16>(a.y), b0 = unpack2<kF16>(bq.x), b1 = unpack2<kF16>(bq.y);
      uint2 o;
      o.x = pack2<kF16>(wa * a0.x + wb * b0.x, wa * a0.y + wb * b0.y);
      o.y = pack2<kF16>(wa * a1.x + wb * b1.x, wa * a1.y + wb * b1.y);
      out_a[i] = o;
    }
    if (lane == 0) lse_a[li] = l;
  }
}

}  // namespace

extern "C" int kvax_b200_attn_merge(void* out_a, float* lse_a, const void* out_b, const float* lse_b, int64_t batch, int64_t seq,
                                    int32_t heads, int32_t head_dim, int32_t dtype, kvax_b200_stream_t stream) {
  if (!out_a || !lse_a || !out_b || !lse_b || batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0) return KVAX_B200_EINVAL;
  if (dtype != KVAX_B200_BF16 && dtype != KVAX_B200_F16) return KVAX_B200_EUNSUPPORTED;
  if ((head_dim & 3) || ((reinterpret_cast<uintptr_t>(out_a) | reinterpret_cast<uintptr_t>(out_b)) & 7) || seq > INT32_MAX)
    return KVAX_B200_EUNSUPPORTED;
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long rows = (long long)batch * seq * heads;
  long long blocks = (rows + 7) / 8;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == KVAX_B200_F16)
    attn_merge_kernel<true><<<int(blocks), 256, 0, s>>>(static_cast<uint2*>(out_a), lse_a, static_cast<const uint2*>(out_b), lse_b,
                                                       rows, int(seq), heads, head_dim / 4);
  else
    attn_merge_kernel<false><<<int(blocks), 256, 0, s>>>(static_cast<uint2*>(out_a), lse_a, static_cast<const uint2*>(out_b), lse_b,
                                                        rows, int(seq), heads, head_dim / 4);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
