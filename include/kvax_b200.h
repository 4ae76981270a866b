/*
 * kvax_b200 — C ABI of the B200 (sm_100a) attention hot path.
 *
 * Every entry point only enqueues work on the caller's stream.  The caller owns all
 * buffers (inputs, outputs, workspace); nothing here allocates, frees, synchronises or
 * throws.  Return value: 0 on success, a negative KVAX_B200_E* code for a rejected
 * call.  Device-side protocol failures (a bounded wait that gave up) are reported
 * through the optional int32 `status` word in device memory: 0 = ok.
 *
 * Each declaration cites the call site in the reference (nebius/kvax) whose
 * `jt.triton_call(...)` custom call it replaces.
 *
 * Tensors use the public layout of the reference API: q/o/do/dq are (B, Sq, Hq, D),
 * k/v/dk/dv are (B, Skv, Hkv, D), element strides given explicitly so that the
 * (B, H, S, D) layout the reference uses internally can be passed as well.  The head
 * dimension must be contiguous.
 */
#ifndef KVAX_B200_H_
#define KVAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* kvax_b200_stream_t; /* == cudaStream_t */

enum {
  KVAX_B200_OK = 0,
  KVAX_B200_EINVAL = -1,      /* bad argument (null pointer, non-positive size, ...) */
  KVAX_B200_EUNSUPPORTED = -2,/* shape or dtype outside what the kernels cover        */
  KVAX_B200_EWORKSPACE = -3,  /* workspace too small or misaligned                    */
  KVAX_B200_ELAUNCH = -4,     /* the CUDA runtime refused a launch or a tensor map    */
  KVAX_B200_ENODEVICE = -5,   /* no usable sm_100 device / driver entry point missing */
  KVAX_B200_ESCRATCH = -6     /* problem needs more than the library's built-in scratch area */
};

enum { KVAX_B200_BF16 = 0, KVAX_B200_F16 = 1 };   /* operand (and output) type of the attention kernels */

#define KVAX_B200_PADDING_SEGMENT_ID (-1) /* kvax/utils/common.py:9 */

const char* kvax_b200_version(void);
const char* kvax_b200_error_string(int code);

/* The `status` word of the attention entry points may live in page-locked host memory, so
 * that the host can look at it at any time without synchronising the stream.  This returns
 * the address under which the current device reaches such a word (KVAX_B200_EUNSUPPORTED
 * when the memory is not page-locked and mapped).  Allocates nothing.  (No counterpart in
 * the reference, whose custom calls have no status channel.) */
int kvax_b200_host_word_device_pointer(void* host_ptr, void** device_ptr);

/* ------------------------------------------------------------------------------------
 * Block-mask builder.
 * Replaces compute_attention_mask_kernel (kvax/ops/mask_creator.py:26-152) together with
 * the host steps around its launch that belong to the bit-exact contract: padding to the
 * block size (:212-225), the PAD -> kv_len_padded+1 remap (:247-259), and the
 * "nothing found" fix-ups (:317-333).  One call builds up to three masks (forward, dq,
 * dkdv — mask_creator.py:438-488) with two kernel launches in total.
 * ---------------------------------------------------------------------------------- */
typedef struct kvax_b200_mask_desc {
  int32_t q_block;        /* query block size of this mask                               */
  int32_t kv_block;       /* kv block size of this mask                                  */
  int32_t kv_outer;       /* 0: one row per query block (forward / dq masks);
                             1: one row per kv block (dkdv mask, calculate_dkdv_mask)    */
  int32_t reserved;
  int32_t* lower;         /* out, (B, n_outer) int32                                     */
  int32_t* upper;         /* out                                                         */
  int32_t* lower_full;    /* out                                                         */
  int32_t* upper_full;    /* out                                                         */
} kvax_b200_mask_desc;

typedef struct kvax_b200_mask_params {
  const int32_t* q_positions;    /* (B, Sq)  */
  const int32_t* q_segment_ids;  /* (B, Sq)  */
  const int32_t* kv_positions;   /* (B, Skv) */
  const int32_t* kv_segment_ids; /* (B, Skv) */
  int32_t batch, q_len, kv_len;
  int32_t skip_pad_tokens;
  int32_t n_masks;               /* 1..3 */
  int32_t reserved;
  kvax_b200_mask_desc masks[3];
} kvax_b200_mask_params;

size_t kvax_b200_mask_workspace_bytes(const kvax_b200_mask_params* p);
/* `workspace`: device memory, 256-byte aligned, at least kvax_b200_mask_workspace_bytes(p). */
int kvax_b200_mask_build(const kvax_b200_mask_params* p, void* workspace, size_t workspace_bytes,
                         kvax_b200_stream_t stream);

/* Block-mask builder for callers that cannot hand over device memory of their own.
 * (No counterpart in the reference: its custom calls get every buffer from XLA.)
 *
 * Some hosts of this library may only pass the buffers their framework gave them and
 * have no way to obtain extra device memory at call time: a custom-call handler that
 * runs while the framework owns the allocator (its arena is fixed once a program is
 * compiled), code running inside a region where allocation is forbidden, or a binding
 * that simply did not declare a workspace result.  For them this entry point does what
 * kvax_b200_mask_build does, with the per-block summaries kept in a fixed 4 MiB area
 * inside the library's own device image instead of a caller workspace.  It never calls
 * cudaMalloc / cudaFree or any allocating routine.
 *
 * Limit: kvax_b200_mask_workspace_bytes(p) must not exceed 4 MiB (4194304 bytes), i.e.
 * the masks of one call may cover at most 262144 blocks counted over both sides and all
 * masks (batch * (ceil(Sq/q_block) + ceil(Skv/kv_block)) summed over the masks, with
 * 256-byte rounding per array); beyond that the call returns KVAX_B200_ESCRATCH and
 * launches nothing.  Every GPU that loads the library holds the 4 MiB until exit.
 *
 * The first call on each device looks up the device address of the area (with that
 * device current); make that first call outside any stream capture.  The address is
 * remembered per device ordinal: only the device's primary context (the CUDA runtime's)
 * is supported.  All calls on a
 * device share the one area and nothing in it has to start at zero (every summary is
 * rewritten before it is read), but two calls whose kernels overlap on the GPU — different
 * streams, no ordering between them — race on it: order them.                          */
int kvax_b200_mask_build_static(const kvax_b200_mask_params* p, kvax_b200_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Context-parallel token permutation (pure data movement, bit-exact).
 * Replaces the XLA gather behind apply_permutation (kvax/utils/permutation.py:18-42):
 * axis 1 of a (B, S, inner) array is cut into 2*cp chunks, chunk order becomes
 * [0, 2cp-1, 1, 2cp-2, ...] (reverse = 0) or its inverse (reverse = 1).
 * `row_bytes` is the size of one token (product of the trailing dims times the element
 * size).
 * ---------------------------------------------------------------------------------- */
int kvax_b200_permute_tokens(const void* src, void* dst, int64_t batch, int64_t seq_len, int64_t row_bytes,
                             int32_t cp, int32_t reverse, kvax_b200_stream_t stream);

/* Head regrouping for the head-exchange schedule of context parallelism (no counterpart in
 * the reference, which only has the all-gather schedule, flash_attention_triton.py:2107-2154):
 * one pass from (tokens, cp * heads_per_group, D) to the all-to-all send layout
 * (cp, tokens, heads_per_group, D) -- group r holds the heads rank r will own -- or back
 * (to_groups = 0).  `tokens` = batch * local sequence length, `head_bytes` = D * element size,
 * a multiple of 16; both pointers 16-byte aligned. */
int kvax_b200_regroup_heads(const void* src, void* dst, int64_t tokens, int32_t cp, int32_t heads_per_group,
                            int64_t head_bytes, int32_t to_groups, kvax_b200_stream_t stream);

/* Merge of two partial attention results over disjoint key sets, for the all-gather schedule of
 * context parallelism when its collectives overlap the kernels (the reference leaves that overlap
 * to XLA's asynchronous collectives around the shard_map body, flash_attention_triton.py:2107-2154):
 * `out_a` / `out_b` are (batch, seq, heads, head_dim) dense outputs of kvax_b200_attn_fwd in `dtype`,
 * `lse_a` / `lse_b` their (batch, heads, seq) base-2 log-sum-exps (+inf: row without keys).  The merged
 * output and log-sum-exp replace `out_a` and `lse_a`.  head_dim 8, 16, 32, 64, 128 or 256, pointers 16-byte aligned. */
int kvax_b200_attn_merge(void* out_a, float* lse_a, const void* out_b, const float* lse_b, int64_t batch, int64_t seq,
                         int32_t heads, int32_t head_dim, int32_t dtype, kvax_b200_stream_t stream);

/* Head exchange over peer memory (no counterpart in the reference; it moves the data the
 * reference's all-gather of K / V moves, flash_attention_triton.py:2064-2115, for the
 * head-exchange schedule): one kernel reads a tensor of this GPU and stores every token's heads
 * straight into the landing buffers of the ranks that own them, over NVLink, already in the layout
 * the attention kernels read.
 *
 * Landing buffers are allocated by `peer_buffer_alloc` (cudaMalloc), made known to the other
 * processes of the node with `peer_buffer_export` (a CUDA IPC handle of
 * KVAX_B200_PEER_HANDLE_BYTES bytes, carried by the caller, e.g. through torch.distributed) and
 * `peer_buffer_open`.  `peer_buffers[r]` is rank r's buffer as this process addresses it
 * (`peer_buffers[rank]` the own one), `dst_offset_bytes` the place of this tensor inside every
 * buffer.  The batch is 1 and `local_tokens` even (two half-sequences per rank).
 *   to_heads = 1: src (local_tokens, cp * heads_per_rank, D) -> rank r gets heads
 *                 [r * heads_per_rank, ...) of these tokens at their natural token position
 *                 in its (cp * local_tokens, heads_per_rank, D) buffer;
 *   to_heads = 0: src (cp * local_tokens, heads_per_rank, D) in natural token order -> rank r
 *                 gets its tokens into heads [rank * heads_per_rank, ...) of its
 *                 (local_tokens, cp * heads_per_rank, D) buffer.
 * `permuted`: the local tokens of rank r are chunks r and 2 cp - 1 - r of the natural order
 * (kvax/utils/permutation.py:9-42), else chunks 2r and 2r + 1.
 * The kernel waits for nobody.  The caller orders it on the stream against the peers: nobody
 * may still read the destination region when it starts, and a rank may read its own buffer once
 * all ranks' kernels have completed (a collective on the same stream on both sides). */
#define KVAX_B200_MAX_PEERS 16
#define KVAX_B200_PEER_HANDLE_BYTES 64
int kvax_b200_peer_buffer_alloc(size_t bytes, void** ptr);
int kvax_b200_peer_buffer_free(void* ptr);
int kvax_b200_peer_buffer_export(void* ptr, unsigned char handle[KVAX_B200_PEER_HANDLE_BYTES]);
int kvax_b200_peer_buffer_open(const unsigned char handle[KVAX_B200_PEER_HANDLE_BYTES], void** peer_ptr);
int kvax_b200_peer_buffer_close(void* peer_ptr);
int kvax_b200_head_exchange(const void* src, void* const* peer_buffers, int64_t dst_offset_bytes, int64_t local_tokens,
                            int32_t cp, int32_t rank, int32_t heads_per_rank, int64_t head_bytes, int32_t permuted,
                            int32_t to_heads, kvax_b200_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Flash attention, forward and backward.
 * ---------------------------------------------------------------------------------- */
typedef struct kvax_b200_block_mask {   /* one AttentionMask (kvax/utils/typing.py:15-37) */
  const int32_t* lower;
  const int32_t* upper;
  const int32_t* lower_full;
  const int32_t* upper_full;
  int32_t q_block;   /* block sizes the mask was built with */
  int32_t kv_block;
} kvax_b200_block_mask;

typedef struct kvax_b200_attn_shape {
  int32_t batch, q_len, kv_len;
  int32_t q_heads, kv_heads;
  int32_t head_dim;        /* Dqk == Dv; 64 or 128                                       */
  int32_t dtype;           /* KVAX_B200_BF16 or KVAX_B200_F16: q, k, v, out, dout, dq            */
  int32_t assume_sequential_positions; /* causal test on indices + query_global_offset   */
  float scale;
  int32_t reserved;
  /* element strides (batch, seq, head); head_dim stride is 1 */
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3];
  const int32_t* q_positions;    /* (B, Sq)  */
  const int32_t* q_segment_ids;  /* (B, Sq)  */
  const int32_t* kv_positions;   /* (B, Skv) */
  const int32_t* kv_segment_ids; /* (B, Skv) */
  /* Global index of local query token 0 / of the first token of the second half of the
     local queries (context parallelism with the load-balancing permutation,
     flash_attention_triton.py:1426-1447).  Both 0 without context parallelism; only read
     when assume_sequential_positions != 0. */
  int32_t q_global_offset_first, q_global_offset_second;
} kvax_b200_attn_shape;

/* Forward.  Replaces flash_attention_forward_kernel (flash_attention_triton.py:137-370,
 * launched at :1517-1540): out (B, Sq, Hq, D) in the input dtype and the base-2
 * log-sum-exp (B, Hq, Sq) fp32.  The workspace holds the per-query-tile list of kv tiles
 * to visit (tiles of the block mask that are entirely masked are dropped from it). */
typedef struct kvax_b200_attn_fwd_params {
  kvax_b200_attn_shape shape;
  const void* q; const void* k; const void* v;
  kvax_b200_block_mask mask;      /* forward mask */
  void* out;                      /* (B, Sq, Hq, D), strides = shape.o_strides */
  float* lse;                     /* (B, Hq, Sq) */
  int32_t* status;                /* optional device int32, must be 0 on entry */
  /* 0 = everything; else bit set: 1 tile list, 2 attention kernel (see the backward). */
  int32_t stages;
  int32_t flags;                  /* KVAX_B200_FWD_*; 0: the library picks the kernel by shape */
} kvax_b200_attn_fwd_params;

/* Forward kernels: a CTA works on one 128-row query tile, or on two work items that share
 * every K / V tile brought on chip: two neighbouring query tiles of one head, or (grouped-query
 * attention, an even number of query heads per kv head) one query tile of two query heads of a
 * kv group.  Same results either way.  Default: head pairs when the group is even and at least two CTAs per SM
 * remain (or from 16k kv tokens on), tile pairs for other shapes from 16k kv tokens on, else one tile. */
enum { KVAX_B200_FWD_ONE_TILE = 1, KVAX_B200_FWD_TILE_PAIRS = 2, KVAX_B200_FWD_HEAD_PAIRS = 4,
       /* query tiles without any key tile get lse = +inf instead of the reference's 0 (flash_attention_triton.py:253-258),
          so that kvax_b200_attn_merge can tell them from rows that have keys */
       KVAX_B200_FWD_EMPTY_LSE_INF = 8 };

size_t kvax_b200_attn_fwd_workspace_bytes(const kvax_b200_attn_fwd_params* p);
int kvax_b200_attn_fwd(const kvax_b200_attn_fwd_params* p, void* workspace, size_t workspace_bytes,
                       kvax_b200_stream_t stream);

/* Backward.  Replaces attn_bwd_preprocess (:373-410, launched :1692-1704),
 * flash_attention_backward_kernel_dquery (:620-871, launched :1740-1766) and
 * flash_attention_backward_kernel_dkdv (:874-1191, launched :1778-1807), plus the
 * GQA group sum (:1855-1868).  dk/dv are fp32 (B, Skv, Hkv, D) contiguous, already
 * summed over the query heads of each group, as the reference returns them before the
 * context-parallel reduction; dq is in the input dtype with its own strides.
 *
 * Two schedules produce the gradients:
 *   fused (default, head_dim 128): one kv-outer kernel computes dK, dV and dQ with five
 *     matrix products per tile pair; partial dQ tiles are summed into an fp32 accumulator in
 *     the workspace with bulk reduce-adds (the order of those fp32 additions varies from run
 *     to run, so dq is reproducible to rounding, not bit for bit) and a last kernel scales
 *     and casts it;
 *   two-kernel (KVAX_B200_BWD_TWO_KERNEL in `flags`, and every head_dim the fused kernel does
 *     not cover): a query-outer dQ kernel and a kv-outer dK/dV kernel, seven products per
 *     tile pair, bit-reproducible. */
enum {
  KVAX_B200_BWD_TWO_KERNEL = 1,
  /* dk and dv point to (B, Skv, Hkv, D) tensors of the operand type (shape.dtype) instead of fp32: for callers
     that need no fp32 reduction over ranks afterwards; saves the cast pass and half the bytes */
  KVAX_B200_BWD_DKDV_16BIT = 2
};

typedef struct kvax_b200_attn_bwd_params {
  kvax_b200_attn_shape shape;
  const void* q; const void* k; const void* v;
  const void* out; const void* dout;   /* strides = shape.o_strides for both */
  const float* lse;                    /* (B, Hq, Sq) from the forward */
  kvax_b200_block_mask mask_dq;        /* one row per query block */
  kvax_b200_block_mask mask_dkdv;      /* one row per kv block    */
  void* dq;                            /* (B, Sq, Hq, D) input dtype, strides = dq_strides */
  float* dk;                           /* (B, Skv, Hkv, D) contiguous, fp32 (or see KVAX_B200_BWD_DKDV_16BIT) */
  float* dv;                           /* (B, Skv, Hkv, D) contiguous, fp32 (or see KVAX_B200_BWD_DKDV_16BIT) */
  int32_t* status;
  /* 0 = everything.  Otherwise a bit set of the parts to launch, for timing or profiling
     one kernel on a workspace a full call has already filled: 1 tile lists, 2 delta (and the
     zero fill of the dQ accumulator), 4 dQ kernel, 8 dK/dV kernel, 16 fused kernel,
     32 dQ scale-and-cast.  Bits that do not belong to the chosen schedule are ignored. */
  int32_t stages;
  int32_t flags;                       /* KVAX_B200_BWD_* */
  int64_t dq_strides[3];               /* element strides (batch, seq, head) of dq */
} kvax_b200_attn_bwd_params;

size_t kvax_b200_attn_bwd_workspace_bytes(const kvax_b200_attn_bwd_params* p);
int kvax_b200_attn_bwd(const kvax_b200_attn_bwd_params* p, void* workspace, size_t workspace_bytes,
                       kvax_b200_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Self-test of the bounded device waits.  (No counterpart in the reference.)
 * Every wait on a barrier inside the attention kernels gives up after a time budget, writes
 * 100 + barrier id to the status word and lets the kernel run to its end.  This entry point
 * launches one warp that waits, with the same routine, on a barrier nobody ever arrives on,
 * with a budget of `budget_ns` (clamped to [1 us, 100 ms]).  Afterwards *status is
 * 100 + bar_id and *done is 2 ("gave up and returned").  `status` and `done` are int32 words
 * the device can address (device memory or mapped page-locked host memory), zero on entry.
 * ---------------------------------------------------------------------------------- */
int kvax_b200_wait_probe(int32_t* status, int32_t* done, int64_t budget_ns, int32_t bar_id,
                         kvax_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KVAX_B200_H_ */
