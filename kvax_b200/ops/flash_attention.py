"""`flash_attention`: document-masked causal GQA attention, forward and backward.

API of kvax/ops/flash_attention_triton.py:2027-2178.  Tensors are torch CUDA tensors in
the public layout (batch, sequence, heads, head_dim); the kernels read that layout
directly through strided TMA descriptors, so the four layout transposes of the reference
(:2158-2160, :2176) do not exist here.

Execution model: one process per GPU.  With context parallelism (the query sequence
axis of `query_specs` names a mesh axis of size > 1) every process passes its own slice
of the permuted sequence for query, key and value — what a device sees of the
reference's global arrays — and the full, un-permuted kv positions / segment ids.

Two context-parallel schedules produce the same results:

* "all_gather" (the reference's, flash_attention_triton.py:2064-2115): K and V are
  all-gathered over NCCL into natural order, the kernels run on the local queries, and the
  backward pass reduce-scatters fp32 dK/dV back to their owners before the cast to the
  input dtype.  Under document masks the work per rank is uneven, because the
  load-balancing permutation only balances a plain causal mask.  With
  `set_context_parallel_overlap(True)` the kernels run on the rank's own keys while the
  rest is gathered, and the reduce-scatter of the remote keys' gradients runs under the
  kernels of the local keys.
* "head_exchange": an all-to-all turns the sequence sharding into a head sharding
  (every rank receives the whole sequence for heads/CP of the heads), the kernels run the
  single-device problem in natural token order on those heads, and a second all-to-all
  brings the output (and, in the backward pass, dQ/dK/dV) back to sequence sharding.  The
  work per rank is exactly 1/CP of the whole, whatever the mask, and no gradient reduction
  is needed: every dK/dV element is complete on one rank.  It needs kv_heads % CP == 0; with fewer
  kv heads than ranks (CP a multiple of kv_heads, q_heads % CP == 0) K / V are all-gathered instead, every rank
  keeps the kv head its query heads read, and dK / dV are reduce-scattered over the ranks that share a head.

`set_context_parallel_mode("auto")` (the default) picks "head_exchange" when the head
counts allow it.
"""
from __future__ import annotations

import contextlib
import math

import torch
import torch.distributed

from kvax_b200 import _lib
from kvax_b200._status import check_last_status, status_word
from kvax_b200.utils.common import FlashAttentionParamsConfig, get_default_flash_attention_params
from kvax_b200.utils.sharding import Mesh, _check_mesh_or_get_global, get_query_context_mesh_axis_name
from kvax_b200.utils.typing import AttentionMask

_CP_MODES = ("auto", "all_gather", "head_exchange")
_cp_mode = "auto"


def set_context_parallel_mode(mode: str) -> None:
    """Chooses the context-parallel schedule: "auto", "all_gather" or "head_exchange"."""
    global _cp_mode
    if mode not in _CP_MODES:
        raise ValueError(f"unknown context-parallel mode {mode!r}; expected one of {_CP_MODES}")
    _cp_mode = mode


def get_context_parallel_mode() -> str:
    return _cp_mode


_cp_overlap = False


def set_context_parallel_overlap(on: bool) -> None:
    """All-gather schedule only: with `on`, the attention kernels first run on the keys and values the rank already
    holds (its own two chunks, which contain the causal diagonal) while K and V of the other ranks are gathered on a
    second stream, then on the gathered rest, and the two partial results are merged; in the backward pass the
    gradients of the remote keys are computed first and their reduce-scatter runs under the kernels of the local
    keys.  Needs position arrays (not `assume_sequential_positions`) and self-attention lengths; other calls
    take the serial schedule."""
    global _cp_overlap
    _cp_overlap = bool(on)


def get_context_parallel_overlap() -> bool:
    return _cp_overlap


_FWD_KERNELS = ("auto", "one_tile", "tile_pairs", "head_pairs")
_fwd_kernel = "auto"


def set_forward_kernel(kernel: str) -> None:
    """Which forward kernel runs: a CTA per 128-row query tile ("one_tile"); a CTA per two work items that share
    their K / V tiles -- two neighbouring query tiles of one head ("tile_pairs") or one query tile of two query heads
    of a kv group ("head_pairs", grouped-query attention with an even group); or the library's choice ("auto",
    default: head pairs when the group is even and at least two CTAs per SM remain, else pairs from 16k kv tokens
    on, else one tile).  Same results to rounding either way."""
    global _fwd_kernel
    if kernel not in _FWD_KERNELS:
        raise ValueError(f"unknown forward kernel {kernel!r}; expected one of {_FWD_KERNELS}")
    _fwd_kernel = kernel


def get_forward_kernel() -> str:
    return _fwd_kernel


_FP32_OPERANDS = ("auto", "float16", "bfloat16")
_fp32_operands = "auto"


def set_fp32_operand_dtype(mode: str) -> None:
    """Which 16-bit type fp32 inputs are rounded to.  "float16": the 10-bit fraction of the tf32 arithmetic the
    reference uses on fp32 tensors, range up to 65504; "bfloat16": 7-bit fraction, the range of fp32; "auto"
    (default): float16 when the largest magnitude of query, key and value is at most 2^14 (one device-to-host
    read per call), else bfloat16."""
    global _fp32_operands
    if mode not in _FP32_OPERANDS:
        raise ValueError(f"unknown operand type {mode!r}; expected one of {_FP32_OPERANDS}")
    _fp32_operands = mode


def get_fp32_operand_dtype() -> str:
    return _fp32_operands


def _fp32_operand_dtype(q, k, v) -> torch.dtype:
    if _fp32_operands != "auto":
        return torch.float16 if _fp32_operands == "float16" else torch.bfloat16
    amax = torch.stack([t.detach().abs().amax() for t in (q, k, v)]).max().item()
    return torch.float16 if amax <= 16384.0 else torch.bfloat16


class _GradScaleBox:
    """Shared by the casts around one call on fp32 tensors: the power of two the output gradient was multiplied
    with on its way into fp16, which the input gradients are divided by on their way out."""

    def __init__(self):
        self.inv = None


class _ToOperand(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dtype, box):
        ctx.box, ctx.in_dtype = box, x.dtype
        return x.to(dtype)

    @staticmethod
    def backward(ctx, g):
        g = g.to(ctx.in_dtype)
        if ctx.box.inv is not None:
            g = g * ctx.box.inv
        return g, None, None


class _FromOperand(torch.autograd.Function):
    @staticmethod
    def forward(ctx, out, dtype, box):
        ctx.box, ctx.op_dtype = box, out.dtype
        return out.to(dtype)

    @staticmethod
    def backward(ctx, g):
        if ctx.op_dtype == torch.float16:
            # largest magnitude -> [1, 2): small gradients keep their bits, nothing overflows; exact (power of two)
            amax = g.abs().amax().clamp_min(1e-30)
            s = torch.exp2(-torch.floor(torch.log2(amax)))
            ctx.box.inv = 1.0 / s
            g = g * s
        return g.to(ctx.op_dtype), None, None


_HX_TRANSPORTS = ("auto", "peer", "nccl")
_hx_transport = "auto"


def set_head_exchange_transport(mode: str) -> None:
    """How the head exchange moves data between the GPUs of a node.  "peer": one kernel per tensor that stores
    straight into landing buffers in the peers' memory (CUDA IPC, NVLink); "nccl": grouped NCCL sends and
    receives; "auto" (default): peer memory when the buffers can be shared, else NCCL."""
    global _hx_transport
    if mode not in _HX_TRANSPORTS:
        raise ValueError(f"unknown head-exchange transport {mode!r}; expected one of {_HX_TRANSPORTS}")
    _hx_transport = mode


def get_head_exchange_transport() -> str:
    return _hx_transport


def _exchange(tensors, to_heads: bool, cp: int, rank: int, group, permuted: bool):
    """Zero-copy head exchange of batch-1 tensors by the chosen transport."""
    if _hx_transport != "nccl":
        from kvax_b200.ops import _peer
        outs = _peer.exchange(tensors, to_heads, cp, rank, group, permuted, _phase)
        if outs is not None:
            return outs
        if _hx_transport == "peer":
            raise RuntimeError("head-exchange transport \"peer\": the landing buffers cannot be shared between the ranks")
    fn = _exchange_seq_to_heads if to_heads else _exchange_heads_to_seq
    return fn(tensors, cp, rank, group, permuted)


# Optional phase timing of the context-parallel schedules: CUDA events around the exchange, mask and kernel
# phases of a call, summed per name.  Off by default (no events are recorded).
_phase_log: list | None = None


def enable_phase_timing(on: bool = True) -> None:
    """Starts (or stops and discards) the recording of per-phase CUDA events in the context-parallel paths."""
    global _phase_log
    _phase_log = [] if on else None


def phase_times_ms() -> dict[str, float]:
    """Milliseconds per phase name summed over everything recorded since `enable_phase_timing()`."""
    out: dict[str, float] = {}
    if _phase_log:
        torch.cuda.synchronize()
        for name, e0, e1 in _phase_log:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
    return out


@contextlib.contextmanager
def _phase(name: str):
    if _phase_log is None:
        yield
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    try:
        yield
    finally:
        e1.record()
        _phase_log.append((name, e0, e1))


_BWD_MODES = ("fused", "two_kernel")
_bwd_mode = "fused"


def set_backward_mode(mode: str) -> None:
    """Chooses the backward schedule.  "fused" (default): one kv-outer kernel computes dK, dV
    and dQ with five matrix products per tile pair; dQ is summed with fp32 atomics, so its last
    bits vary from run to run.  "two_kernel": a dQ kernel and a dK/dV kernel, seven products per
    tile pair, bit-reproducible.  Head dims the fused kernel does not cover always take the
    two-kernel path."""
    global _bwd_mode
    if mode not in _BWD_MODES:
        raise ValueError(f"unknown backward mode {mode!r}; expected one of {_BWD_MODES}")
    _bwd_mode = mode


def get_backward_mode() -> str:
    return _bwd_mode


# Workspaces (tile lists, delta, the fp32 dQ accumulator) are scratch that only lives during one call's
# kernels; calls on one stream run in order, so one buffer per (device, stream, kind) is reused.
_workspaces: dict[tuple, torch.Tensor] = {}


def _workspace(kind: str, nbytes: int, device: torch.device) -> torch.Tensor:
    key = (kind, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


_SUPPORTED_HEAD_DIMS = (16, 32, 64, 128, 192, 256)   # what the reference accepts
_KERNEL_HEAD_DIMS = (64, 128)                         # what the sm_100a kernels cover today


def _i32(x):
    return x.to(torch.int32).contiguous()


def _block_mask(mask: AttentionMask, q_block: int, kv_block: int) -> tuple[_lib.BlockMask, list]:
    keep = [t.to(torch.int32).contiguous() for t in mask.flatten()]
    bm = _lib.BlockMask()
    bm.lower, bm.upper, bm.lower_full, bm.upper_full = (t.data_ptr() for t in keep)
    bm.q_block, bm.kv_block = int(q_block), int(kv_block)
    return bm, keep


def _fill_shape(s: _lib.AttnShape, q, k, v, o, q_pos, q_seg, kv_pos, kv_seg, scale, sequential, offsets):
    B, Sq, Hq, D = q.shape
    s.batch, s.q_len, s.kv_len = B, Sq, k.shape[1]
    s.q_heads, s.kv_heads, s.head_dim = Hq, k.shape[2], D
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise _lib.KvaxB200Error(f"the kernels take bf16 or fp16 operands of one type, got {q.dtype}, {k.dtype}, {v.dtype}")
    s.dtype = _lib.DTYPE_F16 if q.dtype == torch.float16 else _lib.DTYPE_BF16
    s.assume_sequential_positions = int(bool(sequential))
    s.scale = float(scale)
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        if t.stride(3) != 1:
            raise AssertionError("head_dim must be contiguous")
        arr = getattr(s, name)
        arr[0], arr[1], arr[2] = t.stride(0), t.stride(1), t.stride(2)
    s.q_positions, s.q_segment_ids = q_pos.data_ptr(), q_seg.data_ptr()
    s.kv_positions, s.kv_segment_ids = kv_pos.data_ptr(), kv_seg.data_ptr()
    s.q_global_offset_first, s.q_global_offset_second = offsets


def attention_forward(q, k, v, q_pos, q_seg, kv_pos, kv_seg, mask_fwd: AttentionMask, fwd_blocks, scale,
                      assume_sequential_positions=False, offsets=(0, 0), workspace=None, stages=0, out=None, lse=None,
                      kernel=None, empty_lse_inf=False):
    """Direct wrapper of kvax_b200_attn_fwd.  Returns (out, lse2, status) with lse2 (B, Hq, Sq)
    fp32, the base-2 log-sum-exp of the scaled scores, and the device's status word (a pinned
    host tensor; see `check_status`).  With `workspace` or `stages` the workspace is returned too.
    `empty_lse_inf`: query tiles without any key tile get lse2 = +inf (what `attention_merge` needs) instead of 0."""
    lib = _lib.load()
    B, Sq, Hq, D = q.shape
    out = torch.empty_like(q) if out is None else out
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device) if lse is None else lse
    status, status_ptr = status_word(q.device)
    p = _lib.AttnFwdParams()
    p.stages = int(stages)
    p.flags = {"auto": 0, "one_tile": _lib.FWD_ONE_TILE, "tile_pairs": _lib.FWD_TILE_PAIRS,
               "head_pairs": _lib.FWD_HEAD_PAIRS}[kernel or _fwd_kernel] | (_lib.FWD_EMPTY_LSE_INF if empty_lse_inf else 0)
    _fill_shape(p.shape, q, k, v, out, q_pos, q_seg, kv_pos, kv_seg, scale, assume_sequential_positions, offsets)
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.mask, keep = _block_mask(mask_fwd, *fwd_blocks)
    p.out, p.lse, p.status = out.data_ptr(), lse.data_ptr(), status_ptr
    ws_bytes = lib.kvax_b200_attn_fwd_workspace_bytes(p)
    if ws_bytes == 0:
        raise _lib.KvaxB200Error("kvax_b200_attn_fwd_workspace_bytes rejected the arguments "
                                 f"(head_dim={D}, dtype={q.dtype})")
    ws = _workspace("fwd", ws_bytes, q.device) if workspace is None else workspace
    with torch.cuda.device(q.device):
        rc = lib.kvax_b200_attn_fwd(p, ws.data_ptr(), ws.numel(), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "kvax_b200_attn_fwd")
    if workspace is not None or stages:
        return out, lse, status, ws
    return out, lse, status


def attention_backward(q, k, v, out, dout, lse, q_pos, q_seg, kv_pos, kv_seg, mask_dq: AttentionMask,
                       mask_dkdv: AttentionMask, bwd_blocks, scale, assume_sequential_positions=False,
                       offsets=(0, 0), workspace=None, stages=0, grads=None, mode=None, dkdv_in_operand_dtype=False):
    """Direct wrapper of kvax_b200_attn_bwd.  Returns (dq in the input dtype, dk fp32,
    dv fp32, status); dk/dv are summed over the query heads of each kv head.  `mode`:
    "fused" / "two_kernel" (default: `get_backward_mode()`).  `dkdv_in_operand_dtype`: dk / dv come out of the
    kernels in the dtype of q instead of fp32 (no cast pass afterwards; for callers without a reduction over ranks)."""
    lib = _lib.load()
    if grads is None:
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)     # dense, whatever the strides of q
        kv_grad_dtype = q.dtype if dkdv_in_operand_dtype else torch.float32
        dk = torch.empty(k.shape, dtype=kv_grad_dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=kv_grad_dtype, device=v.device)
    else:
        dq, dk, dv = grads
    status, status_ptr = status_word(q.device)
    p = _lib.AttnBwdParams()
    p.stages = int(stages)
    p.flags = (_lib.BWD_TWO_KERNEL if (mode or _bwd_mode) == "two_kernel" else 0) | (_lib.BWD_DKDV_16BIT if dkdv_in_operand_dtype else 0)
    if out.stride() != dout.stride():
        dout = dout.contiguous()
        out = out.contiguous()
    _fill_shape(p.shape, q, k, v, out, q_pos, q_seg, kv_pos, kv_seg, scale, assume_sequential_positions, offsets)
    if dq.stride(3) != 1:
        raise AssertionError("head_dim of dq must be contiguous")
    p.dq_strides[0], p.dq_strides[1], p.dq_strides[2] = dq.stride(0), dq.stride(1), dq.stride(2)
    p.q, p.k, p.v, p.out, p.dout, p.lse = (t.data_ptr() for t in (q, k, v, out, dout, lse))
    bq, bk = bwd_blocks
    p.mask_dq, keep1 = _block_mask(mask_dq, bk, bq)        # dq mask: block sizes swapped
    p.mask_dkdv, keep2 = _block_mask(mask_dkdv, bq, bk)
    p.dq, p.dk, p.dv, p.status = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), status_ptr
    ws_bytes = lib.kvax_b200_attn_bwd_workspace_bytes(p)
    if ws_bytes == 0:
        raise _lib.KvaxB200Error("kvax_b200_attn_bwd_workspace_bytes rejected the arguments")
    ws = _workspace("bwd", ws_bytes, q.device) if workspace is None else workspace
    with torch.cuda.device(q.device):
        rc = lib.kvax_b200_attn_bwd(p, ws.data_ptr(), ws.numel(), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "kvax_b200_attn_bwd")
    if workspace is not None or stages:
        return dq, dk, dv, status, ws
    return dq, dk, dv, status


def check_status(status: torch.Tensor, what: str) -> None:
    """Reads a status word and raises on a device-side failure.  The caller synchronises first
    if the kernels in question may still be running."""
    code = int(status.item())
    if code != 0:
        status.zero_()
        raise _lib.KvaxB200Error(f"{what}: device status {code} (a bounded wait gave up; 100 + barrier id)")


def context_offsets(rank: int, cp: int, local_q_len: int, permuted: bool) -> tuple[int, int]:
    """Global index of local query token 0 and the amount to add to local indices of the
    second half of the local queries (flash_attention_triton.py:1426-1447): with the
    load-balancing permutation rank r holds chunk r followed by chunk 2CP-1-r."""
    if cp == 1:
        return (0, 0)
    if not permuted:
        return (rank * local_q_len, rank * local_q_len)
    half = local_q_len // 2
    return (rank * half, (2 * cp - rank - 1) * half - half)


def _gather_kv(x: torch.Tensor, cp: int, group, permuted: bool, permute_fn=None) -> torch.Tensor:
    """All-gather of the local (B, S_loc, H, D) slices into (B, S, H, D) in natural order.
    `permute_fn(tensor, cp, reverse)` defaults to the CUDA chunk-permutation kernel."""
    import torch.distributed as dist
    from kvax_b200.utils.permutation import _permute_one
    _permute_one = permute_fn or _permute_one

    x = x.contiguous()
    B = x.shape[0]
    gathered = torch.empty((cp * B,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(gathered, x, group=group)      # rank-major concatenation
    gathered = gathered.view((cp,) + tuple(x.shape))
    if B == 1:
        full = gathered.view(1, cp * x.shape[1], *x.shape[2:])
    else:
        full = gathered.transpose(0, 1).contiguous().view(B, cp * x.shape[1], *x.shape[2:])
    return _permute_one(full, cp, reverse=True) if permuted else full


def _scatter_dkv(g: torch.Tensor, cp: int, group, permuted: bool, out_dtype, permute_fn=None) -> torch.Tensor:
    """Reduce-scatter (fp32 sum) of a natural-order (B, S, H, D) gradient to the slice each
    rank owns, then the cast to the input dtype."""
    import torch.distributed as dist
    from kvax_b200.utils.permutation import _permute_one
    _permute_one = permute_fn or _permute_one

    B, S = g.shape[:2]
    if permuted:
        g = _permute_one(g, cp, reverse=False)
    g = g.view(B, cp, S // cp, *g.shape[2:])
    if B != 1:
        g = g.transpose(0, 1).contiguous()
    g = g.reshape(cp * B, S // cp, *g.shape[3:])
    local = torch.empty((B,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
    dist.reduce_scatter_tensor(local, g, op=dist.ReduceOp.SUM, group=group)
    return local.to(out_dtype)


def _seq_to_heads(x: torch.Tensor, cp: int, group, permuted: bool, permute_fn=None) -> torch.Tensor:
    """All-to-all from sequence sharding to head sharding: local (B, S_loc, H, D) of every
    rank -> (B, S, H / cp, D) in natural token order; rank j receives heads
    [j * H / cp, (j + 1) * H / cp)."""
    import torch.distributed as dist
    from kvax_b200.utils.permutation import _permute_one
    _permute_one = permute_fn or _permute_one

    B, Sl, H = x.shape[:3]
    tail = tuple(x.shape[3:])
    Hl = H // cp
    send = x.reshape(B, Sl, cp, Hl, *tail).permute(2, 0, 1, 3, *range(4, 4 + len(tail))).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)             # recv[j]: tokens of rank j
    if B == 1:
        full = recv.view(1, cp * Sl, Hl, *tail)
    else:
        full = recv.transpose(0, 1).contiguous().view(B, cp * Sl, Hl, *tail)
    return _permute_one(full, cp, reverse=True) if permuted else full


def _heads_to_seq(y: torch.Tensor, cp: int, group, permuted: bool, permute_fn=None) -> torch.Tensor:
    """Inverse of `_seq_to_heads`: (B, S, H / cp, D) in natural order on every rank ->
    the local (B, S / cp, H, D) slice of the (permuted) sequence."""
    import torch.distributed as dist
    from kvax_b200.utils.permutation import _permute_one
    _permute_one = permute_fn or _permute_one

    B, S, Hl = y.shape[:3]
    tail = tuple(y.shape[3:])
    Sl = S // cp
    if permuted:
        y = _permute_one(y.contiguous(), cp, reverse=False)
    send = y.reshape(B, cp, Sl, Hl, *tail).transpose(0, 1).contiguous()   # send[j]: tokens of rank j
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)             # recv[j]: heads of rank j
    return recv.permute(1, 2, 0, 3, *range(4, 4 + len(tail))).reshape(B, Sl, cp * Hl, *tail)


def _gather_tokens(x: torch.Tensor, cp: int, group, permuted: bool, permute_fn=None) -> torch.Tensor:
    """All-gather of per-token (B, S_loc) arrays into (B, S) in natural order."""
    return _gather_kv(x.unsqueeze(-1).unsqueeze(-1), cp, group, permuted, permute_fn)[:, :, 0, 0].contiguous()


def _regroup_heads(x: torch.Tensor, cp: int, to_groups: bool) -> torch.Tensor:
    """(B, S, cp * Hl, D) -> (cp, B, S, Hl, D) (group r = the heads rank r owns) or back, in one pass.
    On CUDA tensors this is the regroup kernel of the library; on CPU tensors (the gloo tests of the
    exchange logic) the same index map with torch ops."""
    if to_groups:
        B, S, H, D = x.shape
        hl = H // cp
        if not x.is_cuda:
            return x.reshape(B, S, cp, hl, D).permute(2, 0, 1, 3, 4).contiguous()
        x = x.contiguous()
        out = torch.empty((cp, B, S, hl, D), dtype=x.dtype, device=x.device)
    else:
        _, B, S, hl, D = x.shape
        if not x.is_cuda:
            return x.permute(1, 2, 0, 3, 4).reshape(B, S, cp * hl, D)
        x = x.contiguous()
        out = torch.empty((B, S, cp * hl, D), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().kvax_b200_regroup_heads(x.data_ptr(), out.data_ptr(), B * S, cp, hl, D * x.element_size(),
                                                 int(to_groups), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "kvax_b200_regroup_heads")
    return out


def _chunk_of(rank: int, half: int, cp: int, permuted: bool) -> int:
    """Index (in units of half a local sequence) at which half `half` (0 / 1) of rank `rank`'s local tokens sits in
    the natural order: with the load-balancing permutation rank r holds chunks r and 2 CP - 1 - r."""
    if not permuted:
        return 2 * rank + half
    return rank if half == 0 else 2 * cp - 1 - rank


def _exchange_seq_to_heads(tensors, cp: int, rank: int, group, permuted: bool):
    """Head exchange, sequence sharding -> head sharding, for several (1, S_loc, H, D) tensors at once.
    One regroup pass per tensor builds the send layout; every peer's two half-sequences are then received
    straight into their place in natural token order (no gather buffer, no un-permutation pass), all sends
    and receives of all tensors in one NCCL group."""
    import torch.distributed as dist
    outs, ops, local_copies = [], [], []
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(cp))
    for x in tensors:
        B, Sl, H, D = x.shape
        assert B == 1 and Sl % 2 == 0
        hl, half = H // cp, Sl // 2
        with _phase("regroup"):
            send = _regroup_heads(x, cp, True)                   # (cp, 1, Sl, hl, D)
        nat = torch.empty((1, cp * Sl, hl, D), dtype=x.dtype, device=x.device)
        outs.append(nat)
        for r in range(cp):
            for h in range(2):
                c = _chunk_of(r, h, cp, permuted)
                dst = nat[0, c * half:(c + 1) * half]           # contiguous: tokens of rank r, half h, my heads
                src = send[r, 0, h * half:(h + 1) * half]       # contiguous: my tokens, half h, heads of rank r
                if r == rank:
                    local_copies.append((nat[0, _chunk_of(rank, h, cp, permuted) * half:(_chunk_of(rank, h, cp, permuted) + 1) * half], src))
                else:
                    ops.append(dist.P2POp(dist.isend, src, ranks[r], group))
                    ops.append(dist.P2POp(dist.irecv, dst, ranks[r], group))
    with _phase("local_copy"):
        for dst, src in local_copies:
            dst.copy_(src)
    with _phase("p2p"):
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
    return outs


def _exchange_heads_to_seq(tensors, cp: int, rank: int, group, permuted: bool):
    """Inverse exchange for several (1, S, Hl, D) natural-order tensors: every peer's two half-sequences are
    sent straight out of the natural-order tensor, the received head groups are interleaved by one regroup
    pass.  Returns (1, S_loc, cp * Hl, D) tensors."""
    import torch.distributed as dist
    recvs, ops, local_copies = [], [], []
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(cp))
    for y in tensors:
        B, S, hl, D = y.shape
        assert B == 1
        y = y.contiguous()
        Sl = S // cp
        half = Sl // 2
        recv = torch.empty((cp, 1, Sl, hl, D), dtype=y.dtype, device=y.device)
        recvs.append(recv)
        for r in range(cp):
            for h in range(2):
                c = _chunk_of(r, h, cp, permuted)
                src = y[0, c * half:(c + 1) * half]             # tokens of rank r, half h, my heads
                dst = recv[r, 0, h * half:(h + 1) * half]       # my tokens, half h, heads of rank r
                if r == rank:
                    local_copies.append((dst, y[0, _chunk_of(rank, h, cp, permuted) * half:(_chunk_of(rank, h, cp, permuted) + 1) * half]))
                else:
                    ops.append(dist.P2POp(dist.isend, src, ranks[r], group))
                    ops.append(dist.P2POp(dist.irecv, dst, ranks[r], group))
    with _phase("local_copy"):
        for dst, src in local_copies:
            dst.copy_(src)
    with _phase("p2p"):
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
    with _phase("regroup"):
        return [_regroup_heads(r_, cp, False) for r_ in recvs]


def _fast_exchange_ok(x: torch.Tensor) -> bool:
    """The zero-copy exchange places half-sequences as contiguous slices, which needs batch 1 (the shape of the
    context-parallel workloads); other shapes take the copy-based all-to-all."""
    return x.shape[0] == 1 and x.shape[1] % 2 == 0 and (x.shape[3] * x.element_size()) % 16 == 0


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, q_pos, q_seg, kv_pos, kv_seg, masks, scale, fwd_params, bwd_params,
                sequential, permuted, cp, rank, group):
        if cp > 1:
            with _phase("gather_kv"):
                k_full = _gather_kv(key, cp, group, permuted)
                v_full = _gather_kv(value, cp, group, permuted)
        else:
            k_full, v_full = key, value
        offsets = context_offsets(rank, cp, query.shape[1], permuted)
        with _phase("attention_forward"):
            out, lse, status = attention_forward(
                query, k_full, v_full, q_pos, q_seg, kv_pos, kv_seg, masks[0],
                (fwd_params.query_block_size, fwd_params.kv_block_size), scale, sequential, offsets)
        ctx.save_for_backward(query, k_full, v_full, out, lse, q_pos, q_seg, kv_pos, kv_seg,
                              *[t for m in masks for t in m.flatten()])
        ctx.n_masks = len(masks)
        ctx.cfg = (scale, bwd_params, sequential, permuted, cp, group, offsets, key.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        check_last_status(dout.device)          # a forward that failed on the device: do not differentiate garbage
        saved = ctx.saved_tensors
        query, k_full, v_full, out, lse, q_pos, q_seg, kv_pos, kv_seg = saved[:9]
        flat = saved[9:]
        if ctx.n_masks != 3:
            raise ValueError("Length of mask_tensors should be equal to two")
        masks = [AttentionMask.unflatten(flat[4 * i:4 * i + 4]) for i in range(3)]
        scale, bwd_params, sequential, permuted, cp, group, offsets, kv_dtype = ctx.cfg
        bq, bk = bwd_params.query_block_size, bwd_params.kv_block_size
        if query.shape[1] % bq or k_full.shape[1] % bk:
            raise AssertionError("sequence lengths must be divisible by the backward block sizes")
        with _phase("attention_backward"):
            # without context parallelism nothing is summed over ranks afterwards: dK / dV leave the kernels in the
            # input dtype
            dq, dk, dv, _ = attention_backward(query, k_full, v_full, out, dout, lse, q_pos, q_seg, kv_pos, kv_seg,
                                               masks[1], masks[2], (bq, bk), scale, sequential, offsets,
                                               dkdv_in_operand_dtype=(cp == 1 and kv_dtype == query.dtype))
        if cp > 1:
            with _phase("scatter_dkv"):
                dk = _scatter_dkv(dk, cp, group, permuted, kv_dtype)
                dv = _scatter_dkv(dv, cp, group, permuted, kv_dtype)
        elif dk.dtype != kv_dtype:
            dk, dv = dk.to(kv_dtype), dv.to(kv_dtype)
        return (dq, dk, dv) + (None,) * 13


def _remote_slots(rank: int, cp: int, permuted: bool) -> list[int]:
    """Where the chunks a rank does not hold sit in a rank-major all-gather: slot 2 r + h is half h of rank r's local
    tokens.  Listed in natural (ascending chunk) order, the order the masks need."""
    slot_of = {_chunk_of(r, h, cp, permuted): 2 * r + h for r in range(cp) for h in (0, 1)}
    own = {_chunk_of(rank, 0, cp, permuted), _chunk_of(rank, 1, cp, permuted)}
    return [slot_of[c] for c in range(2 * cp) if c not in own]


_slot_index: dict = {}


def _slot_index_tensor(rank: int, cp: int, permuted: bool, device) -> torch.Tensor:
    key = (rank, cp, permuted, str(device))
    t = _slot_index.get(key)
    if t is None:
        t = torch.tensor(_remote_slots(rank, cp, permuted), dtype=torch.long, device=device)
        _slot_index[key] = t
    return t


def _gather_remote(x: torch.Tensor, gathered: torch.Tensor, cp: int, rank: int, group, permuted: bool) -> torch.Tensor:
    """All-gather of the local (B, S_loc, ...) slices into `gathered` (cp * B, S_loc, ...), then the chunks of the
    other ranks in natural order: (B, (cp - 1) * S_loc, ...)."""
    import torch.distributed as dist

    B, s_loc = x.shape[:2]
    half = s_loc // 2
    dist.all_gather_into_tensor(gathered, x, group=group)      # rank-major concatenation
    idx = _slot_index_tensor(rank, cp, permuted, x.device)
    g = gathered.view(cp, B, 2, half, *x.shape[2:])
    if B == 1:
        rem = g.view(2 * cp, half, *x.shape[2:]).index_select(0, idx)
        return rem.view(1, (cp - 1) * s_loc, *x.shape[2:])
    rem = g.transpose(0, 1).reshape(B, 2 * cp, half, *x.shape[2:]).index_select(1, idx)
    return rem.reshape(B, (cp - 1) * s_loc, *x.shape[2:])


def _natural_chunks(x: torch.Tensor, cp: int, chunks: list[int]) -> torch.Tensor:
    """The given chunks (of 2 cp) of a natural-order per-token array (B, S), concatenated."""
    B, S = x.shape
    half = S // (2 * cp)
    return torch.cat([x[:, c * half:(c + 1) * half] for c in chunks], dim=1).contiguous()


def _remote_to_scatter_layout(g_rem: torch.Tensor, cp: int, rank: int, permuted: bool) -> torch.Tensor:
    """Inverse of the chunk selection of `_gather_remote` for a gradient: (B, (cp - 1) * S_loc, ...) of the remote
    chunks in natural order -> the reduce-scatter input (cp * B, S_loc, ...), zeros where this rank's own chunks go."""
    B = g_rem.shape[0]
    s_loc = g_rem.shape[1] // (cp - 1)
    half = s_loc // 2
    tail = tuple(g_rem.shape[2:])
    idx = _slot_index_tensor(rank, cp, permuted, g_rem.device)
    if B == 1:
        out = torch.empty((2 * cp, half) + tail, dtype=g_rem.dtype, device=g_rem.device)
        out.index_copy_(0, idx, g_rem.view(2 * (cp - 1), half, *tail))
        out[2 * rank:2 * rank + 2].zero_()
        return out.view(cp, s_loc, *tail)
    out = torch.zeros((cp, B, 2, half) + tail, dtype=g_rem.dtype, device=g_rem.device)
    src = g_rem.view(B, 2 * (cp - 1), half, *tail)
    for j, slot in enumerate(_remote_slots(rank, cp, permuted)):
        out[slot // 2, :, slot % 2] = src[:, j]
    return out.view(cp * B, s_loc, *tail)


_side_streams: dict = {}


def _side_stream(device) -> torch.cuda.Stream:
    s = _side_streams.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _side_streams[device.index] = s
    return s


def attention_merge(out_a, lse_a, out_b, lse_b):
    """Direct wrapper of kvax_b200_attn_merge: merges part b into part a (both from `attention_forward` with
    `empty_lse_inf=True` on the same queries and disjoint keys), in place."""
    if not (out_a.is_contiguous() and out_b.is_contiguous() and lse_a.is_contiguous() and lse_b.is_contiguous()):
        raise AssertionError("attention_merge needs dense tensors")
    B, S, H, D = out_a.shape
    dtype = _lib.DTYPE_F16 if out_a.dtype == torch.float16 else _lib.DTYPE_BF16
    with torch.cuda.device(out_a.device):
        rc = _lib.load().kvax_b200_attn_merge(out_a.data_ptr(), lse_a.data_ptr(), out_b.data_ptr(), lse_b.data_ptr(), B, S, H, D,
                                              dtype, torch.cuda.current_stream(out_a.device).cuda_stream)
    _lib.check(rc, "kvax_b200_attn_merge")
    return out_a, lse_a


class _FlashAttentionOverlapped(torch.autograd.Function):
    """All-gather schedule with its collectives under the kernels (`set_context_parallel_overlap`).  The keys are
    split into the rank's own two chunks and the chunks of the other ranks; each part is an attention problem of its
    own (positions and segment ids decide what is allowed, so any subset of the keys in ascending order is a valid
    kv sequence), with masks built here by the same mask builder; the per-rank masks the caller passed describe the
    unsplit problem and are not used."""

    @staticmethod
    def forward(ctx, query, key, value, q_pos, q_seg, kv_pos, kv_seg, n_masks, scale, fwd_params, bwd_params,
                permuted, cp, rank, group):
        from kvax_b200.ops.mask_creator import build_masks

        dev = query.device
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        key, value = key.contiguous(), value.contiguous()
        B, s_loc = key.shape[:2]
        gathered = [torch.empty((cp * B,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for t in (key, value)]
        side.wait_stream(main)
        with torch.cuda.stream(side):
            k_rem = _gather_remote(key, gathered[0], cp, rank, group, permuted)
            v_rem = _gather_remote(value, gathered[1], cp, rank, group, permuted)
            k_rem.record_stream(main)
            v_rem.record_stream(main)
        own = [_chunk_of(rank, 0, cp, permuted), _chunk_of(rank, 1, cp, permuted)]
        rest = [c for c in range(2 * cp) if c not in own]
        kv_pos_own, kv_seg_own = _natural_chunks(kv_pos, cp, own), _natural_chunks(kv_seg, cp, own)
        kv_pos_rem, kv_seg_rem = _natural_chunks(kv_pos, cp, rest), _natural_chunks(kv_seg, cp, rest)
        specs = [(fwd_params.query_block_size, fwd_params.kv_block_size, False)]
        if n_masks == 3:
            specs.append((bwd_params.kv_block_size, bwd_params.query_block_size, False))
            specs.append((bwd_params.query_block_size, bwd_params.kv_block_size, True))
        blocks = (fwd_params.query_block_size, fwd_params.kv_block_size)
        with _phase("build_masks"):
            masks_own = build_masks(q_pos, q_seg, kv_pos_own, kv_seg_own, specs, True)
            masks_rem = build_masks(q_pos, q_seg, kv_pos_rem, kv_seg_rem, specs, True)
        with _phase("attention_forward_own_keys"):
            out, lse, _ = attention_forward(query, key, value, q_pos, q_seg, kv_pos_own, kv_seg_own, masks_own[0], blocks, scale,
                                            empty_lse_inf=True)
        main.wait_stream(side)
        del gathered
        with _phase("attention_forward_remote_keys"):
            out_r, lse_r, _ = attention_forward(query, k_rem, v_rem, q_pos, q_seg, kv_pos_rem, kv_seg_rem, masks_rem[0], blocks,
                                                scale, empty_lse_inf=True)
            attention_merge(out, lse, out_r, lse_r)
        ctx.save_for_backward(query, key, value, k_rem, v_rem, out, lse, q_pos, q_seg, kv_pos_own, kv_seg_own, kv_pos_rem,
                              kv_seg_rem, *[t for m in masks_own + masks_rem for t in m.flatten()])
        ctx.n_masks = n_masks
        ctx.cfg = (scale, bwd_params, permuted, cp, rank, group)
        return out

    @staticmethod
    def backward(ctx, dout):
        import torch.distributed as dist

        check_last_status(dout.device)
        saved = ctx.saved_tensors
        (query, key, value, k_rem, v_rem, out, lse, q_pos, q_seg, kv_pos_own, kv_seg_own, kv_pos_rem, kv_seg_rem) = saved[:13]
        flat = saved[13:]
        if ctx.n_masks != 3:
            raise ValueError("Length of mask_tensors should be equal to two")
        masks_own = [AttentionMask.unflatten(flat[4 * i:4 * i + 4]) for i in range(3)]
        masks_rem = [AttentionMask.unflatten(flat[12 + 4 * i:12 + 4 * i + 4]) for i in range(3)]
        scale, bwd_params, permuted, cp, rank, group = ctx.cfg
        bq, bk = bwd_params.query_block_size, bwd_params.kv_block_size
        if query.shape[1] % bq or key.shape[1] % bk:
            raise AssertionError("sequence lengths must be divisible by the backward block sizes")
        dev = query.device
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        dout = dout.contiguous()
        # remote keys first: their gradients travel while the kernels of the local keys run
        with _phase("attention_backward_remote_keys"):
            dq_r, dk_r, dv_r, _ = attention_backward(query, k_rem, v_rem, out, dout, lse, q_pos, q_seg, kv_pos_rem, kv_seg_rem,
                                                     masks_rem[1], masks_rem[2], (bq, bk), scale)
            sends = [_remote_to_scatter_layout(g, cp, rank, permuted) for g in (dk_r, dv_r)]
            landed = [torch.empty((key.shape[0],) + tuple(s.shape[1:]), dtype=s.dtype, device=dev) for s in sends]
        side.wait_stream(main)
        with torch.cuda.stream(side):
            for s, l in zip(sends, landed):
                dist.reduce_scatter_tensor(l, s, op=dist.ReduceOp.SUM, group=group)
        with _phase("attention_backward_own_keys"):
            dq, dk, dv, _ = attention_backward(query, key, value, out, dout, lse, q_pos, q_seg, kv_pos_own, kv_seg_own,
                                               masks_own[1], masks_own[2], (bq, bk), scale)
            dq += dq_r
        main.wait_stream(side)
        dk = (dk + landed[0]).to(key.dtype)
        dv = (dv + landed[1]).to(value.dtype)
        return (dq, dk, dv) + (None,) * 12


class _FlashAttentionHeadExchange(torch.autograd.Function):
    """Context parallelism by head exchange (see the module docstring).  The masks of the
    single-device problem are rebuilt from the gathered positions and segment ids with the
    same bit-exact mask builder; the per-rank masks the caller passed are not used."""

    @staticmethod
    def forward(ctx, query, key, value, q_pos, q_seg, kv_pos, kv_seg, n_masks, scale, fwd_params, bwd_params,
                sequential, permuted, cp, group):
        from kvax_b200.ops.mask_creator import build_masks

        rank = torch.distributed.get_rank(group)
        # Fewer kv heads than ranks (CP a multiple of kv_heads): the query heads are exchanged as usual; a kv head is
        # then needed, whole, by the CP / kv_heads ranks that hold its query heads.  K and V are small next to Q: they
        # are all-gathered and every rank keeps the one head its query heads read.
        shared = cp // key.shape[2] if key.shape[2] % cp else 0         # ranks per kv head, 0: every rank owns kv heads
        kv_head = rank // shared if shared else 0
        fast = _fast_exchange_ok(query) and (shared or (_fast_exchange_ok(key) and _fast_exchange_ok(value)))
        if shared:
            q_h = _exchange((query,), True, cp, rank, group, permuted)[0] if fast else _seq_to_heads(query, cp, group, permuted)
            with _phase("gather_kv"):
                k_h = _gather_kv(key, cp, group, permuted)[:, :, kv_head:kv_head + 1]
                v_h = _gather_kv(value, cp, group, permuted)[:, :, kv_head:kv_head + 1]
        elif fast:
            q_h, k_h, v_h = _exchange((query, key, value), True, cp, rank, group, permuted)
        else:
            q_h = _seq_to_heads(query, cp, group, permuted)
            k_h = _seq_to_heads(key, cp, group, permuted)
            v_h = _seq_to_heads(value, cp, group, permuted)
        with _phase("gather_tokens"):
            q_pos_f = _gather_tokens(q_pos, cp, group, permuted)
            q_seg_f = _gather_tokens(q_seg, cp, group, permuted)
        specs = [(fwd_params.query_block_size, fwd_params.kv_block_size, False)]
        if n_masks == 3:
            specs.append((bwd_params.kv_block_size, bwd_params.query_block_size, False))
            specs.append((bwd_params.query_block_size, bwd_params.kv_block_size, True))
        with _phase("build_masks"):
            masks = build_masks(q_pos_f, q_seg_f, kv_pos, kv_seg, specs, True)
        with _phase("attention_forward"):
            out_h, lse_h, status = attention_forward(
                q_h, k_h, v_h, q_pos_f, q_seg_f, kv_pos, kv_seg, masks[0],
                (fwd_params.query_block_size, fwd_params.kv_block_size), scale, sequential, (0, 0))
        ctx.save_for_backward(q_h, k_h, v_h, out_h, lse_h, q_pos_f, q_seg_f, kv_pos, kv_seg,
                              *[t for m in masks for t in m.flatten()])
        ctx.n_masks = n_masks
        ctx.cfg = (scale, bwd_params, sequential, permuted, cp, group, key.dtype, rank, fast, shared, kv_head, key.shape[2])
        if fast:
            return _exchange((out_h,), False, cp, rank, group, permuted)[0]
        return _heads_to_seq(out_h, cp, group, permuted)

    @staticmethod
    def backward(ctx, dout):
        check_last_status(dout.device)
        saved = ctx.saved_tensors
        q_h, k_h, v_h, out_h, lse_h, q_pos_f, q_seg_f, kv_pos, kv_seg = saved[:9]
        flat = saved[9:]
        if ctx.n_masks != 3:
            raise ValueError("Length of mask_tensors should be equal to two")
        masks = [AttentionMask.unflatten(flat[4 * i:4 * i + 4]) for i in range(3)]
        scale, bwd_params, sequential, permuted, cp, group, kv_dtype, rank, fast, shared, kv_head, n_kv_heads = ctx.cfg
        bq, bk = bwd_params.query_block_size, bwd_params.kv_block_size
        if q_h.shape[1] % bq or k_h.shape[1] % bk:
            raise AssertionError("sequence lengths must be divisible by the backward block sizes")
        if fast:
            dout_h = _exchange((dout,), True, cp, rank, group, permuted)[0]
        else:
            dout_h = _seq_to_heads(dout.contiguous(), cp, group, permuted)
        with _phase("attention_backward"):
            dq_h, dk_h, dv_h, _ = attention_backward(q_h, k_h, v_h, out_h, dout_h, lse_h, q_pos_f, q_seg_f, kv_pos, kv_seg,
                                                     masks[1], masks[2], (bq, bk), scale, sequential, (0, 0),
                                                     dkdv_in_operand_dtype=(not shared and kv_dtype == q_h.dtype))
        if shared:
            # the ranks that share a kv head each hold the part of its gradient that comes from their query heads: the
            # fp32 reduce-scatter of the all-gather schedule sums them (zeros for the heads a rank does not hold)
            dq = _exchange((dq_h,), False, cp, rank, group, permuted)[0] if fast else _heads_to_seq(dq_h, cp, group, permuted)
            with _phase("scatter_dkv"):
                grads = []
                for part in (dk_h, dv_h):
                    full = torch.zeros((part.shape[0], part.shape[1], n_kv_heads, part.shape[3]), dtype=torch.float32,
                                       device=part.device)
                    full[:, :, kv_head:kv_head + 1] = part
                    grads.append(_scatter_dkv(full, cp, group, permuted, kv_dtype))
            return (dq, grads[0], grads[1]) + (None,) * 12
        # every dK / dV element is complete on this rank: cast first, then exchange
        if fast:
            dq, dk, dv = _exchange((dq_h, dk_h.to(kv_dtype), dv_h.to(kv_dtype)), False, cp, rank, group, permuted)
            return (dq, dk, dv) + (None,) * 12
        dq = _heads_to_seq(dq_h, cp, group, permuted)
        dk = _heads_to_seq(dk_h.to(kv_dtype), cp, group, permuted)
        dv = _heads_to_seq(dv_h.to(kv_dtype), cp, group, permuted)
        return (dq, dk, dv) + (None,) * 12


def flash_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_positions: torch.Tensor,
    query_segment_ids: torch.Tensor,
    kv_positions: torch.Tensor,
    kv_segment_ids: torch.Tensor,
    mask: tuple[AttentionMask, ...],
    scale: float = 1.0,
    bias: torch.Tensor | None = None,
    fwd_params: FlashAttentionParamsConfig | None = None,
    bwd_params: FlashAttentionParamsConfig | None = None,
    assume_sequential_positions: bool = False,
    memory_optimized_gqa_backward: bool = False,
    permute_tokens_for_load_balance: bool = True,
    debug: bool = False,
    mesh: Mesh | None = None,
) -> torch.Tensor:
    """Attention output of shape (batch, query_seq, heads, head_dim), differentiable with
    respect to query, key and value.

    A device-side failure (a bounded wait inside a kernel that gave up) never traps: the kernel
    finishes and leaves a code in the device's status word, which this function checks on entry,
    the backward pass checks before it runs, and `kvax_b200.check_last_status()` checks on demand.

    `mask` is the tuple returned by `create_attention_mask` (one mask for inference, three
    for training); `fwd_params` / `bwd_params` must be the block sizes those masks were
    built with.  `memory_optimized_gqa_backward` is accepted and has no effect: the dK/dV
    kernel always accumulates the query heads of a group on chip.  `debug` is accepted and
    ignored.  Raises NotImplementedError for `bias`, ValueError for a missing mesh / specs
    or an empty mask tuple, AssertionError for shape errors, as the reference does.
    """
    mesh = _check_mesh_or_get_global(mesh)
    axis = get_query_context_mesh_axis_name(mesh)
    if query.is_cuda:
        check_last_status(query.device)         # surfaces a failure of an earlier call on this device (no synchronisation)
    if bias is not None:
        raise NotImplementedError("Bias is not supported in Flash multi head attention")
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise AssertionError("query, key and value must have rank 4")
    if query.shape[-1] not in _SUPPORTED_HEAD_DIMS:
        raise AssertionError(f"Attention hid_dim can take values {list(_SUPPORTED_HEAD_DIMS)}")
    if mask is None or len(mask) == 0:
        raise ValueError("Length of mask_tensors should be at least equal to one")
    if len(mask) not in (1, 3):
        raise ValueError(f"The case with num_mask_tensors={len(mask)} is not supported.")
    if not query.is_cuda:
        raise _lib.KvaxB200Error("flash_attention needs CUDA tensors (there is no CPU fallback)")
    head_dim, v_head_dim = query.shape[-1], value.shape[-1]
    if key.shape[-1] != head_dim:
        raise AssertionError("query and key must have the same head_dim")
    if v_head_dim not in _SUPPORTED_HEAD_DIMS:
        raise AssertionError(f"Attention hid_dim can take values {list(_SUPPORTED_HEAD_DIMS)}")
    if max(head_dim, v_head_dim) > _KERNEL_HEAD_DIMS[-1]:
        raise _lib.KvaxB200Error(
            f"the sm_100a kernels cover head dims up to {_KERNEL_HEAD_DIMS[-1]} (Dqk and Dv may differ); "
            f"got Dqk={head_dim}, Dv={v_head_dim}")
    # the kernels run one head_dim for Q K^T and P V: the smallest they have that holds both
    kernel_dim = next(d for d in _KERNEL_HEAD_DIMS if d >= max(head_dim, v_head_dim))
    if query.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise _lib.KvaxB200Error(f"unsupported dtype {query.dtype}")
    # bf16 and fp16 tensors are the kernels' operand types (fp32 accumulation).  fp32 tensors -- the reference feeds
    # them to tl.dot, i.e. tf32 tensor cores with a 10-bit fraction -- are rounded to fp16, which has the same
    # fraction, when their largest magnitude allows, else to bf16 (`set_fp32_operand_dtype`); the output and the
    # gradients come back as fp32, and the incoming output gradient is scaled by a power of two into the fp16 range.
    in_dtype = query.dtype
    bridge = None
    if in_dtype == torch.float32:
        bridge = _GradScaleBox()
        op_dtype = _fp32_operand_dtype(query, key, value)
        query, key, value = (_ToOperand.apply(t, op_dtype, bridge) for t in (query, key, value))
    # Zero columns change neither Q K^T nor the first Dv columns of P V; the output is sliced back below and
    # autograd slices the gradients the same way.
    if head_dim < kernel_dim:
        query, key = (torch.nn.functional.pad(t, (0, kernel_dim - head_dim)) for t in (query, key))
    if v_head_dim < kernel_dim:
        value = torch.nn.functional.pad(value, (0, kernel_dim - v_head_dim))
    B, Sq, Hq, _ = query.shape
    if key.shape[0] != B or value.shape[:3] != key.shape[:3] or Hq % key.shape[2]:
        raise AssertionError("inconsistent query / key / value shapes")
    if fwd_params is None:
        fwd_params = get_default_flash_attention_params(backward=False)
    if bwd_params is None:
        bwd_params = get_default_flash_attention_params(backward=True)

    cp, rank, group = 1, 0, None
    if axis is not None:
        if axis not in mesh.shape:
            raise ValueError(f"Mesh axis {axis} is not present in the device mesh shape.")
        cp = mesh.shape[axis]
        rank = mesh.coordinate(axis)
        group = mesh.group(axis) if cp > 1 else None
    if cp > 1 and Sq % fwd_params.query_block_size:
        raise AssertionError("with context parallelism the local query length must be a multiple of the block size")
    kv_len = key.shape[1] * cp
    if tuple(query_positions.shape) != (B, Sq) or tuple(query_segment_ids.shape) != (B, Sq):
        raise AssertionError("query positions / segment ids must have shape (batch, query_seq)")
    if tuple(kv_positions.shape) != (B, kv_len) or tuple(kv_segment_ids.shape) != (B, kv_len):
        raise AssertionError("kv positions / segment ids must have shape (batch, kv_seq)")

    n_kv = key.shape[2]
    heads_fit = n_kv % cp == 0 or (cp % n_kv == 0 and Hq % cp == 0)     # every rank owns kv heads, or shares one
    can_exchange = cp > 1 and heads_fit and kv_len == Sq * cp
    if _cp_mode == "head_exchange" and cp > 1 and not can_exchange:
        raise AssertionError("head_exchange context parallelism needs kv_heads % CP == 0 (or CP % kv_heads == 0 with "
                             "q_heads % CP == 0) and self-attention lengths")
    if can_exchange and _cp_mode != "all_gather":
        out = _FlashAttentionHeadExchange.apply(
            query, key, value, _i32(query_positions), _i32(query_segment_ids), _i32(kv_positions),
            _i32(kv_segment_ids), len(mask), float(scale), fwd_params, bwd_params,
            bool(assume_sequential_positions), bool(permute_tokens_for_load_balance), cp, group)
    elif (cp > 1 and _cp_overlap and not assume_sequential_positions and kv_len == Sq * cp and key.shape[1] == Sq
          and Sq % 2 == 0 and Sq % max(bwd_params.query_block_size, bwd_params.kv_block_size, fwd_params.kv_block_size) == 0):
        out = _FlashAttentionOverlapped.apply(
            query, key, value, _i32(query_positions), _i32(query_segment_ids), _i32(kv_positions),
            _i32(kv_segment_ids), len(mask), float(scale), fwd_params, bwd_params,
            bool(permute_tokens_for_load_balance), cp, rank, group)
    else:
        out = _FlashAttention.apply(
            query, key, value, _i32(query_positions), _i32(query_segment_ids), _i32(kv_positions),
            _i32(kv_segment_ids), tuple(mask), float(scale), fwd_params, bwd_params,
            bool(assume_sequential_positions), bool(permute_tokens_for_load_balance), cp, rank, group)
    if v_head_dim < kernel_dim:
        out = out[..., :v_head_dim]
    return out if bridge is None else _FromOperand.apply(out, in_dtype, bridge)
