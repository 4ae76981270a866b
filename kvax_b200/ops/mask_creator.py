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


# Everything about a call that only depends on shapes and block sizes (workspace size, sizes and offsets of the output
# arrays inside the one allocation) is worked out once per shape.
_layouts: dict[tuple, tuple] = {}


def _int32_input(x: torch.Tensor, name: str) -> torch.Tensor:
    if x.dtype == torch.int32 and x.is_cuda and x.dim() == 2 and x.is_contiguous():
        return x
    return _as_i32(x, name)


class MaskPlan:
    """One prepared call of kvax_b200_mask_build: argument struct, output arrays and workspace are set up once,
    `launch()` only enqueues the kernel on the current stream (for callers that rebuild masks of the same shape
    into the same arrays every step, and for timing the kernel without host overhead)."""

    def __init__(self, query_positions, query_segment_ids, kv_positions, kv_segment_ids, block_specs, skip_pad_tokens=True):
        qp = _int32_input(query_positions, "query_positions")
        qs = _int32_input(query_segment_ids, "query_segment_ids")
        kp = _int32_input(kv_positions, "kv_positions")
        ks = _int32_input(kv_segment_ids, "kv_segment_ids")
        B, Sq = qp.shape
        Skv = kp.shape[1]
        if qs.shape != (B, Sq) or kp.shape != (B, Skv) or ks.shape != (B, Skv):
            raise AssertionError("positions / segment ids have inconsistent shapes")
        self._keep = (qp, qs, kp, ks)
        self._lib = _lib.load()
        self.device = qp.device
        p = self.params = _lib.MaskParams()
        p.q_positions, p.q_segment_ids = qp.data_ptr(), qs.data_ptr()
        p.kv_positions, p.kv_segment_ids = kp.data_ptr(), ks.data_ptr()
        p.batch, p.q_len, p.kv_len = B, Sq, Skv
        p.skip_pad_tokens = int(bool(skip_pad_tokens))
        p.n_masks = len(block_specs)
        for i, (bq, bk, kv_outer) in enumerate(block_specs):
            d = p.masks[i]
            d.q_block, d.kv_block, d.kv_outer = int(bq), int(bk), int(bool(kv_outer))
        key = (B, Sq, Skv, tuple((int(bq), int(bk), bool(kv)) for bq, bk, kv in block_specs))
        layout = _layouts.get(key)
        if layout is None:
            ws_bytes = self._lib.kvax_b200_mask_workspace_bytes(p)
            if ws_bytes == 0:
                raise _lib.KvaxB200Error("kvax_b200_mask_workspace_bytes rejected the arguments")
            # one int32 allocation holds the workspace and every output array (each output starts on a 256-byte boundary)
            sizes = [(Skv + bk - 1) // bk if kv_outer else (Sq + bq - 1) // bq for (bq, bk, kv_outer) in block_specs]
            offs, off = [], ((ws_bytes + 255) // 256) * 64            # in int32 elements
            for n in sizes:
                offs.append(off)
                off += ((4 * B * n * 4 + 255) // 256) * 64
            layout = _layouts[key] = (ws_bytes, tuple(sizes), tuple(offs), off)
        self.ws_bytes, sizes, offs, total = layout
        self._blob = torch.empty(total, dtype=torch.int32, device=qp.device)
        base = self._blob.data_ptr()
        masks = []
        for i, (n, off) in enumerate(zip(sizes, offs)):
            arrs = self._blob[off:off + 4 * B * n].view(4, B, 1, n).unbind(0)
            d = p.masks[i]
            step = 4 * B * n
            d.lower, d.upper, d.lower_full, d.upper_full = (base + 4 * off, base + 4 * off + step,
                                                            base + 4 * off + 2 * step, base + 4 * off + 3 * step)
            masks.append(AttentionMask(arrs[0], arrs[1], arrs[2], arrs[3]))
        self.masks = tuple(masks)

    def launch(self) -> tuple[AttentionMask, ...]:
        with torch.cuda.device(self.device):
            rc = self._lib.kvax_b200_mask_build(self.params, self._blob.data_ptr(), self.ws_bytes,
                                                torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "kvax_b200_mask_build")
        return self.masks


def build_masks(query_positions, query_segment_ids, kv_positions, kv_segment_ids,
                block_specs, skip_pad_tokens=True):
    """`block_specs`: up to three (query_block, kv_block, kv_outer) triples.  Returns one
    AttentionMask per triple.  This is the direct wrapper of kvax_b200_mask_build."""
    return MaskPlan(query_positions, query_segment_ids, kv_positions, kv_segment_ids, block_specs, skip_pad_tokens).launch()


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


def calculate_mask_sparsity(mask: AttentionMask, query_block_size: int, kv_block_size: int, query_seq_len: int,
                            kv_seq_len: int) -> float:
    """Visited fraction of the block grid: sum over all rows of (upper - lower), divided by
    (query_seq_len // query_block_size) * (kv_seq_len // kv_block_size) * batch -- the factor the
    reference multiplies its dense FLOP formula with (mask_creator.py:601-625, same signature and
    the same floor divisions)."""
    lower = mask.lower_bounds.to(torch.int64)
    upper = mask.upper_bounds.to(torch.int64)
    batch = lower.shape[0]
    blocks = float((upper - lower).sum().item())
    return blocks / (query_seq_len // query_block_size) / (kv_seq_len // kv_block_size) / batch


def _mask_grid(mask: AttentionMask, b: int, num_inner_blocks: int):
    """Class of every (row, inner block) cell of batch entry `b`: 0 not visited, 1 partial, 2 full.
    A mask with several shards on axis 1 (the dkdv mask under context parallelism) lays the
    shards side by side, each over num_inner_blocks / shards columns (mask_creator.py:508-537)."""
    import numpy as np
    lo, up, lof, upf = (t[b].cpu().numpy() for t in mask.flatten())      # (shards, rows)
    shards, rows = lo.shape
    per_shard = num_inner_blocks // shards
    grid = np.zeros((rows, num_inner_blocks), np.int32)
    cols = np.arange(per_shard)[None, :]
    for sh in range(shards):
        part = np.where((cols >= lof[sh][:, None]) & (cols < upf[sh][:, None]), 2,
                        np.where((cols >= lo[sh][:, None]) & (cols < up[sh][:, None]), 1, 0))
        grid[:, sh * per_shard:(sh + 1) * per_shard] = part
    return grid


def print_mask(mask: AttentionMask, num_inner_blocks: int, print_only_first_in_batch: bool = True,
               fit_in_screen: bool = True) -> None:
    """Logs a picture of the mask (arguments of mask_creator.py:493-598): two characters per cell,
    blank = not visited, light shade = partial block, solid = full block.  With `fit_in_screen`
    a large mask is averaged down to at most 32 rows x 64 columns; an averaged cell is solid
    only if all its blocks are full and blank only if none is visited."""
    import numpy as np
    batches = 1 if print_only_first_in_batch else mask.lower_bounds.shape[0]
    text = "Attention masks:\n"
    for b in range(batches):
        grid = _mask_grid(mask, b, num_inner_blocks).astype(np.float64)
        rows, cols = grid.shape
        rs, cs = max(1, -(-rows // 32)), max(1, -(-cols // 64))
        if fit_in_screen and (rs > 1 or cs > 1):
            pr, pc = (-rows) % rs, (-cols) % cs
            g = np.pad(grid, ((0, pr), (0, pc)))
            grid = g.reshape(g.shape[0] // rs, rs, g.shape[1] // cs, cs).mean(axis=(1, 3))
        lines = ["".join("\u2588\u2588" if x == 2 else ("  " if x == 0 else "\u2591\u2591") for x in row) for row in grid]
        rule = "  " + "==" * grid.shape[1] + "  "
        text += "\n" + rule + "\n" + "".join("||" + ln + "||\n" for ln in lines) + rule + "\n\n"
    logger.info(text)
