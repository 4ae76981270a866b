// Context-parallel token permutation: chunk gather along the sequence axis.
// Pure data movement (HBM-bound): each CTA streams 16-byte vectors of one chunk;
// the grid is sized in multiples of the SM count and strides over the whole array.
// Index rule follows kvax/utils/permutation.py:9-42.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kvax_b200.h"

namespace {

__device__ __forceinline__ int source_chunk(int c, int cp, int reverse) {
  const int n = 2 * cp;
  if (!reverse) return (c & 1) ? (n - 1 - (c >> 1)) : (c >> 1);   // [0, n-1, 1, n-2, ...]
  return (c < cp) ? (2 * c) : (2 * (n - 1 - c) + 1);               // argsort of the above
}

template <typename V>
__global__ void __launch_bounds__(256) permute_chunks_kernel(const V* __restrict__ src, V* __restrict__ dst,
                                                            long long total_vecs, long long chunk_vecs, int cp,
                                                            int reverse) {
  const int n = 2 * cp;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs;
       i += (long long)gridDim.x * blockDim.x) {
    const long long chunk = i / chunk_vecs;
    const long long off = i - chunk * chunk_vecs;
    const long long b = chunk / n;
    const int c = int(chunk - b * n);
    const long long s = (b * n + source_chunk(c, cp, reverse)) * chunk_vecs + off;
    dst[i] = __ldg(src + s);
  }
}

}  // namespace

extern "C" int kvax_b200_permute_tokens(const void* src, void* dst, int64_t batch, int64_t seq_len, int64_t row_bytes,
                                        int32_t cp, int32_t reverse, kvax_b200_stream_t stream) {
  if (!src || !dst || batch <= 0 || seq_len <= 0 || row_bytes <= 0 || cp <= 0) return KVAX_B200_EINVAL;
  if (src == dst) return KVAX_B200_EINVAL;
  if (seq_len % (2 * cp) != 0) return KVAX_B200_EINVAL;
  const long long chunk_bytes = (seq_len / (2 * cp)) * row_bytes;
  const long long total_bytes = batch * seq_len * row_bytes;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool a16 = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0 && chunk_bytes % 16 == 0;
  const bool a4 = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 3) == 0 && chunk_bytes % 4 == 0;
  auto grid_for = [&](long long vecs) {
    long long blocks = (vecs + 255) / 256;
    long long cap = (long long)sms * 8;
    return int(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
  };
  if (a16) {
    const long long v = total_bytes / 16;
    permute_chunks_kernel<int4><<<grid_for(v), 256, 0, s>>>(static_cast<const int4*>(src), static_cast<int4*>(dst), v,
                                                            chunk_bytes / 16, cp, reverse);
  } else if (a4) {
    const long long v = total_bytes / 4;
    permute_chunks_kernel<int><<<grid_for(v), 256, 0, s>>>(static_cast<const int*>(src), static_cast<int*>(dst), v,
                                                           chunk_bytes / 4, cp, reverse);
  } else {
    permute_chunks_kernel<char><<<grid_for(total_bytes), 256, 0, s>>>(static_cast<const char*>(src),
                                                                      static_cast<char*>(dst), total_bytes, chunk_bytes,
                                                                      cp, reverse);
  }
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

// ---------------------------------------------------------------------------------------
// Head regrouping for the head-exchange schedule of context parallelism: one pass that
// turns (B, S, cp * Hl, D) into the all-to-all send layout (cp, B, S, Hl, D) -- group r =
// the heads rank r will own -- or back (`to_groups` = 0: (cp, B, S, Hl, D) -> (B, S, cp * Hl, D)).
// Pure data movement, 16-byte vectors; `head_bytes` = D * element size (a multiple of 16).
// ---------------------------------------------------------------------------------------
namespace {

__global__ void __launch_bounds__(256) regroup_heads_kernel(const int4* __restrict__ src, int4* __restrict__ dst,
                                                           long long tokens, int cp, int hl, int head_vecs, int to_groups) {
  // token-major view: grouped[r][t][h][v], flat[t][r][h][v]
  const long long group_vecs = tokens * hl * head_vecs;      // vectors per group
  const long long total = group_vecs * cp;
  const int per_tok = hl * head_vecs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    // i indexes the grouped layout
    const long long r = i / group_vecs;
    const long long rem = i - r * group_vecs;
    const long long t = rem / per_tok;
    const long long within = rem - t * per_tok;
    const long long flat = (t * cp + r) * per_tok + within;
    if (to_groups) dst[i] = __ldg(src + flat);
    else dst[flat] = __ldg(src + i);
  }
}

}  // namespace

extern "C" int kvax_b200_regroup_heads(const void* src, void* dst, int64_t tokens, int32_t cp, int32_t heads_per_group,
                                       int64_t head_bytes, int32_t to_groups, kvax_b200_stream_t stream) {
  if (!src || !dst || src == dst || tokens <= 0 || cp <= 0 || heads_per_group <= 0 || head_bytes <= 0) return KVAX_B200_EINVAL;
  if ((head_bytes & 15) || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return KVAX_B200_EUNSUPPORTED;
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long total = tokens * cp * heads_per_group * (head_bytes / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)sms * 8) blocks = (long long)sms * 8;
  regroup_heads_kernel<<<int(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const int4*>(src), static_cast<int4*>(dst), tokens, cp, heads_per_group, int(head_bytes / 16), to_groups);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
