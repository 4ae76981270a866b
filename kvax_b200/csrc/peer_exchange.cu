// Head exchange of context parallelism over peer memory (NVLink / NVSwitch), one kernel per tensor and
// direction: the regrouping by destination rank, the placement in natural token order and the transfer
// itself are one pass of plain 16-byte loads from this GPU's memory and stores into the landing buffers of
// the peers (no NCCL copy, no send layout, no gather buffer).
//
// The reference reaches the same data movement through XLA's all-gather of K / V
// (kvax/ops/flash_attention_triton.py:2064-2115); the head exchange replaces it with an all-to-all between
// sequence sharding and head sharding, see kvax_b200/ops/flash_attention.py.
//
// Landing buffers are plain cudaMalloc allocations shared between the processes of one node with CUDA IPC
// handles.  The kernels never wait for another GPU: the callers order them with collectives on the stream
// (every rank has finished reading its landing buffer before anyone writes it again; every rank has
// finished writing before anyone reads).
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/kvax_b200.h"

namespace {

struct PeerBases { char* p[KVAX_B200_MAX_PEERS]; };

// Natural position of local token t of rank `rank`: with the load-balancing permutation rank r holds the
// chunks r and 2 cp - 1 - r of 2 cp chunks (kvax/utils/permutation.py:9-42), else chunks 2r and 2r + 1.
__device__ __forceinline__ long long natural_token(int rank, long long t, long long half, int cp, int permuted) {
  const int second = t >= half;
  const long long chunk = permuted ? (second ? (2 * cp - 1 - rank) : rank) : (2 * rank + second);
  return chunk * half + (t - (second ? half : 0));
}

// to_heads = 1: src (local_tokens, cp * hl, head) -> peer r's buffer (cp * local_tokens, hl, head) in natural order
// to_heads = 0: src (cp * local_tokens, hl, head) natural order -> peer r's buffer (local_tokens, cp * hl, head)
__global__ void __launch_bounds__(256) head_exchange_kernel(const int4* __restrict__ src, const __grid_constant__ PeerBases dst, long long dst_offset_vecs,
                                                            long long local_tokens, int cp, int me, int hl, int head_vecs,
                                                            int permuted, int to_heads) {
  const int row_vecs = hl * head_vecs;                       // one token's heads for one rank
  const long long per_rank = local_tokens * row_vecs;
  const long long total = per_rank * cp;
  const long long half = local_tokens / 2;
  // four independent 16-byte transfers per thread and step: enough stores in flight to fill the links
  constexpr int kUnroll = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += stride * kUnroll) {
    int4 val[kUnroll];
    int4* out[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      const long long i = i0 + k * stride;
      out[k] = nullptr;
      if (i >= total) continue;
      // the destinations rotate with the rank so that the ranks do not all write to the same peer at once
      const int rr = int(i / per_rank);
      const int r = (rr + me) % cp;
      const long long rem = i - (long long)rr * per_rank;
      const long long t = rem / row_vecs;
      const int w = int(rem - t * row_vecs);
      long long s, d;
      if (to_heads) {
        s = (t * cp + r) * row_vecs + w;
        d = natural_token(me, t, half, cp, permuted) * row_vecs + w;
      } else {
        s = natural_token(r, t, half, cp, permuted) * row_vecs + w;
        d = (t * cp + me) * row_vecs + w;
      }
      val[k] = __ldg(src + s);
      out[k] = reinterpret_cast<int4*>(dst.p[r]) + dst_offset_vecs + d;
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k)
      if (out[k]) *out[k] = val[k];
  }
  __threadfence_system();
}

}  // namespace

extern "C" int kvax_b200_peer_buffer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes == 0) return KVAX_B200_EINVAL;
  return cudaMalloc(ptr, bytes) == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

extern "C" int kvax_b200_peer_buffer_free(void* ptr) {
  return cudaFree(ptr) == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

extern "C" int kvax_b200_peer_buffer_export(void* ptr, unsigned char handle[KVAX_B200_PEER_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == KVAX_B200_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle) return KVAX_B200_EINVAL;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) { cudaGetLastError(); return KVAX_B200_EUNSUPPORTED; }
  memcpy(handle, &h, sizeof(h));
  return KVAX_B200_OK;
}

extern "C" int kvax_b200_peer_buffer_open(const unsigned char handle[KVAX_B200_PEER_HANDLE_BYTES], void** peer_ptr) {
  if (!handle || !peer_ptr) return KVAX_B200_EINVAL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  if (cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return KVAX_B200_EUNSUPPORTED; }
  return KVAX_B200_OK;
}

extern "C" int kvax_b200_peer_buffer_close(void* peer_ptr) {
  return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}

extern "C" int kvax_b200_head_exchange(const void* src, void* const* peer_buffers, int64_t dst_offset_bytes, int64_t local_tokens,
                                       int32_t cp, int32_t rank, int32_t heads_per_rank, int64_t head_bytes, int32_t permuted,
                                       int32_t to_heads, kvax_b200_stream_t stream) {
  if (!src || !peer_buffers || local_tokens <= 0 || cp <= 0 || cp > KVAX_B200_MAX_PEERS || rank < 0 || rank >= cp ||
      heads_per_rank <= 0 || head_bytes <= 0 || dst_offset_bytes < 0)
    return KVAX_B200_EINVAL;
  if ((head_bytes & 15) || (dst_offset_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (local_tokens & 1))
    return KVAX_B200_EUNSUPPORTED;
  PeerBases b;
  for (int r = 0; r < cp; ++r) {
    if (!peer_buffers[r] || (reinterpret_cast<uintptr_t>(peer_buffers[r]) & 15)) return KVAX_B200_EINVAL;
    b.p[r] = static_cast<char*>(peer_buffers[r]);
  }
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long total = local_tokens * cp * heads_per_rank * (head_bytes / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  head_exchange_kernel<<<int(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const int4*>(src), b, dst_offset_bytes / 16, local_tokens, cp, rank, heads_per_rank, int(head_bytes / 16),
      permuted, to_heads);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
