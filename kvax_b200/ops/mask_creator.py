"""Block-mask construction: `create_attention_mask` and host utilities.

API of kvax/ops/mask_creator.py:377-490 (create_attention_mask), :493-598 (print_mask)
and :601-625 (calculate_mask_sparsity).  The three masks (forward, dq, dkdv) are built by
one call into the CUDA mask builder (two kernel launches); results are bit-identical with
the reference's mask tensors.

Each process passes the query-side arrays of its own shard and the full kv-side arrays,
exactly what one device sees inside the reference's shard_map; the returned arrays have
the per-device shape (batch, 1, n_outer_blocks).
"""
from __future__ import annotations

import logging

import torch

from kvax_b200 import _lib
from kvax_b200.utils.common import FlashAttentionParamsConfig, get_default_flash_attention_params
from kvax_b200.utils.sharding import Mesh, _check_mesh_or_get_global
from kvax_b200.utils.specs import get_attention_specs
from kvax_b200.utils.typing import AttentionMask

logger = logging.getLogger(__name__)


def _as_i32(x: torch.Tensor, name: str) -> torch.Tensor:
    if not x.is_cuda:
        raise _lib.KvaxB200Error(f"{name} must be a CUDA tensor (there is no CPU fallback)")
    if x.dim() != 2:
        raise AssertionError(f"{name} must have shape (batch, sequence), got {tuple(x.shape)}")
    return x.to(torch.int32).contiguous()


def build_masks(query_positions, query_segment_ids, kv_positions, kv_segment_ids,
                block_specs, skip_pad_tokens=True):
    """`block_specs`: up to three (query_block, kv_block, kv_outer) triples.  Returns one
    AttentionMask per triple.  This is the direct wrapper of kvax_b200_mask_build."""
    qp = _as_i32(query_positions, "query_positions")
    qs = _as_i32(query_segment_ids, "query_segment_ids")
    kp = _as_i32(kv_positions, "kv_positions")
    ks = _as_i32(kv_segment_ids, "kv_segment_ids")
    B, Sq = qp.shape
    Skv = kp.shape[1]
    if qs.shape != (B, Sq) or kp.shape != (B, Skv) or ks.shape != (B, Skv):
        raise AssertionError("positions / segment ids have inconsistent shapes")
    lib = _lib.load()
    p = _lib.MaskParams()
    p.q_positions, p.q_segment_ids = qp.data_ptr(), qs.data_ptr()
    p.kv_positions, p.kv_segment_ids = kp.data_ptr(), ks.data_ptr()
    p.batch, p.q_len, p.kv_len = B, Sq, Skv
    p.skip_pad_tokens = int(bool(skip_pad_tokens))
    p.n_masks = len(block_specs)
    outs = []
    for i, (bq, bk, kv_outer) in enumerate(block_specs):
        n_outer = (Skv + bk - 1) // bk if kv_outer else (Sq + bq - 1) // bq
        arrs = torch.empty((4, B, 1, n_outer), dtype=torch.int32, device=qp.device)
        d = p.masks[i]
        d.q_block, d.kv_block, d.kv_outer = int(bq), int(bk), int(bool(kv_outer))
        d.lower, d.upper, d.lower_full, d.upper_full = (arrs[j].data_ptr() for j in range(4))
        outs.append(arrs)
    ws_bytes = lib.kvax_b200_mask_workspace_bytes(p)
    if ws_bytes == 0:
        raise _lib.KvaxB200Error("kvax_b200_mask_workspace_bytes rejected the arguments")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=qp.device)
    with torch.cuda.device(qp.device):
        rc = lib.kvax_b200_mask_build(p, ws.data_ptr(), ws_bytes, torch.cuda.current_stream(qp.device).cuda_stream)
    _lib.check(rc, "kvax_b200_mask_build")
    return tuple(AttentionMask(a[0], a[1], a[2], a[3]) for a in outs)


def create_attention_mask(
    query_positions: torch.Tensor,
    query_segment_ids: torch.Tensor,
    kv_positions: torch.Tensor,
    kv_segment_ids: torch.Tensor,
    fwd_params: FlashAttentionParamsConfig | None = None,
    bwd_params: FlashAttentionParamsConfig | None = None,
    calc_bwd_mask: bool = False,
    skip_pad_tokens: bool = True,
    mesh: Mesh | None = None,
) -> tuple[AttentionMask, ...]:
    """Builds the forward mask and, with `calc_bwd_mask`, the dq and dkdv masks.

    Returns a tuple of one or three AttentionMask.  As in the reference, the dq mask uses
    the backward block sizes swapped (query block = bwd.kv_block_size, kv block =
    bwd.query_block_size) and the dkdv mask has one row per kv block.  `bwd_params` must be
    given when `calc_bwd_mask` is set (the reference dereferences it unconditionally).
    A mesh (argument or `with mesh:`) and attention specs must be set, as in the reference.
    """
    _check_mesh_or_get_global(mesh)
    get_attention_specs()
    if fwd_params is None:
        fwd_params = get_default_flash_attention_params(backward=False)
    specs = [(fwd_params.query_block_size, fwd_params.kv_block_size, False)]
    if calc_bwd_mask:
        if bwd_params is None:
            raise AttributeError("'NoneType' object has no attribute 'query_block_size'")
        specs.append((bwd_params.kv_block_size, bwd_params.query_block_size, False))
        specs.append((bwd_params.query_block_size, bwd_params.kv_block_size, True))
    return build_masks(query_positions, query_segment_ids, kv_positions, kv_segment_ids, specs, skip_pad_tokens)


def calculate_mask_sparsity(mask: AttentionMask, num_inner_blocks: int | None = None) -> float:
    """Fraction of (outer, inner) block pairs inside [lower, upper): the factor the
    reference multiplies its dense FLOP formula with (mask_creator.py:601-625)."""
    lower = mask.lower_bounds.to(torch.int64)
    upper = mask.upper_bounds.to(torch.int64)
    if num_inner_blocks is None:
        num_inner_blocks = int(upper.max().item())
    total = lower.numel() * max(num_inner_blocks, 1)
    return float((upper - lower).clamp_min(0).sum().item()) / float(total)


def print_mask(mask: AttentionMask, num_inner_blocks: int, print_only_first_in_batch: bool = True,
               fit_in_screen: bool = True) -> None:
    """ASCII picture of a mask: '.' not visited, 'o' partial block, '#' full block."""
    lo, up, lof, upf = (t.cpu() for t in mask.flatten())
    batches = 1 if print_only_first_in_batch else lo.shape[0]
    for b in range(batches):
        n_outer = lo.shape[-1]
        step_o = max(1, n_outer // 64) if fit_in_screen else 1
        step_i = max(1, num_inner_blocks // 128) if fit_in_screen else 1
        lines = []
        for o in range(0, n_outer, step_o):
            row = []
            for i in range(0, num_inner_blocks, step_i):
                if lof[b, 0, o] <= i < upf[b, 0, o]:
                    row.append("#")
                elif lo[b, 0, o] <= i < up[b, 0, o]:
                    row.append("o")
                else:
                    row.append(".")
            lines.append("".join(row))
        logger.info("mask for batch %d:\n%s", b, "\n".join(lines))
