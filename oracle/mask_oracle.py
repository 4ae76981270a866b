"""CPU oracle for the block-mask builder.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the product path never does.

Restates, in NumPy, what the reference computes for one device:
  kvax/ops/mask_creator.py:202-335  compute_attention_mask_single_device
  kvax/ops/mask_creator.py:26-152   compute_attention_mask_kernel
  kvax/ops/mask_creator.py:377-490  create_attention_mask (three calls)
  kvax/utils/common.py:44-74        pad_to_block_size

Parity is pinned: tests/golden/mask_*.npz hold the outputs of the reference's own
kernel and host code (run under the Triton interpreter on CPU by
tests/golden/make_mask_golden.py); tests/test_oracle_mask.py checks this
restatement against them bit for bit.
"""
from __future__ import annotations

import numpy as np

PADDING_SEGMENT_ID = -1  # kvax/utils/common.py:9
INT32_MAX = np.iinfo(np.int32).max


def _pad(arr: np.ndarray, block: int, fill: int) -> np.ndarray:
    """kvax/utils/common.py:52-72 — pad axis 1 up to a multiple of `block`."""
    n = arr.shape[1]
    padded = (n + block - 1) // block * block
    if padded == n:
        return arr
    return np.pad(arr, ((0, 0), (0, padded - n)), constant_values=fill)


def block_summaries(pos: np.ndarray, seg: np.ndarray, block: int):
    """Per-block (min, max) of segment ids and positions.

    The reference recomputes these inside its inner loop
    (mask_creator.py:63-67, 80-81, 91-94, 106-107).
    """
    b, n = pos.shape
    p = pos.reshape(b, n // block, block)
    s = seg.reshape(b, n // block, block)
    return s.min(-1), s.max(-1), p.min(-1), p.max(-1)


def compute_attention_mask_single_device(
    query_positions,
    query_segment_ids,
    kv_positions,
    kv_segment_ids,
    kv_block_size: int,
    query_block_size: int,
    skip_pad_tokens: bool = True,
    calculate_dkdv_mask: bool = False,
):
    """Returns (lower, upper, lower_full, upper_full), each int32 (B, 1, n_outer).

    Follows mask_creator.py:202-335 step by step.
    """
    qp = _pad(np.asarray(query_positions, np.int32), query_block_size, -1)  # :212-218
    qs = _pad(np.asarray(query_segment_ids, np.int32), query_block_size, PADDING_SEGMENT_ID)
    kp = _pad(np.asarray(kv_positions, np.int32), kv_block_size, INT32_MAX)  # :219-225
    ks = _pad(np.asarray(kv_segment_ids, np.int32), kv_block_size, PADDING_SEGMENT_ID)

    kv_len = kp.shape[1]
    pad_id = np.int32(kv_len + 1)  # :248
    qs = np.where(qs == PADDING_SEGMENT_ID, pad_id, qs)  # :250-259
    ks = np.where(ks == PADDING_SEGMENT_ID, pad_id, ks)

    nq = qp.shape[1] // query_block_size
    nk = kp.shape[1] // kv_block_size

    q_smin, q_smax, q_pmin, q_pmax = block_summaries(qp, qs, query_block_size)
    k_smin, k_smax, k_pmin, k_pmax = block_summaries(kp, ks, kv_block_size)

    if calculate_dkdv_mask:  # outer = kv, inner = query (:277-292)
        o_smin, o_smax, o_pmin, o_pmax = k_smin, k_smax, k_pmin, k_pmax
        i_smin, i_smax, i_pmin, i_pmax = q_smin, q_smax, q_pmin, q_pmax
        n_inner = nq
    else:  # outer = query, inner = kv (:293-308)
        o_smin, o_smax, o_pmin, o_pmax = q_smin, q_smax, q_pmin, q_pmax
        i_smin, i_smax, i_pmin, i_pmax = k_smin, k_smax, k_pmin, k_pmax
        n_inner = nk

    # broadcast outer over axis 1, inner over axis 2
    O = lambda a: a[:, :, None]
    I = lambda a: a[:, None, :]

    seg_overlap = (I(i_smin) <= O(o_smax)) & (O(o_smin) <= I(i_smax))  # :98-101
    full_segments = O(o_smin == o_smax) & I(i_smin == i_smax)  # :102
    if not calculate_dkdv_mask:  # :110-112
        pos_any = O(o_pmax) >= I(i_pmin)
        pos_all = O(o_pmin) >= I(i_pmax)
    else:  # :113-115
        pos_any = I(i_pmax) >= O(o_pmin)
        pos_all = I(i_pmin) >= O(o_pmax)

    attend = pos_any & seg_overlap  # :117-118
    if skip_pad_tokens:  # :122-124
        attend = attend & ~I(i_smin == pad_id)
    full = full_segments & pos_all & attend  # :139

    idx = np.arange(n_inner, dtype=np.int64)[None, None, :]

    def bounds(pred):
        lo = np.where(pred, idx, n_inner).min(-1)  # :134-137 / :144-147
        hi = np.where(pred, idx + 1, 0).max(-1)  # :130-132 / :142
        return lo.astype(np.int32), hi.astype(np.int32)

    lower, upper = bounds(attend)
    lower_full, upper_full = bounds(full)

    if skip_pad_tokens:  # early return of all-PAD outer blocks, :69-76
        all_pad = (o_smin == o_smax) & (o_smin == pad_id)
        for a in (lower, upper, lower_full, upper_full):
            a[all_pad] = 0

    # host post-processing, :317-333
    if calculate_dkdv_mask:
        lower = np.where(lower == nq, upper, lower)
        lower_full = np.where(lower_full == nq, upper, lower_full)
    else:
        lower = np.where(lower == nk, upper, lower)
        lower_full = np.where(lower_full == nk, lower, lower_full)
    upper_full = np.where(upper_full < lower_full, lower_full, upper_full)

    shape = (qp.shape[0], 1, -1)
    return tuple(
        np.ascontiguousarray(a.reshape(shape).astype(np.int32))
        for a in (lower, upper, lower_full, upper_full)
    )


def compute_attention_mask_literal(
    query_positions,
    query_segment_ids,
    kv_positions,
    kv_segment_ids,
    kv_block_size: int,
    query_block_size: int,
    skip_pad_tokens: bool = True,
    calculate_dkdv_mask: bool = False,
):
    """Slow scalar transcription of the kernel's control flow (small inputs only).

    Used to cross-check the vectorised version above: it walks the inner blocks in
    order and folds the four running bounds exactly like mask_creator.py:83-147.
    """
    qp = _pad(np.asarray(query_positions, np.int32), query_block_size, -1)
    qs = _pad(np.asarray(query_segment_ids, np.int32), query_block_size, PADDING_SEGMENT_ID)
    kp = _pad(np.asarray(kv_positions, np.int32), kv_block_size, INT32_MAX)
    ks = _pad(np.asarray(kv_segment_ids, np.int32), kv_block_size, PADDING_SEGMENT_ID)
    pad_id = kp.shape[1] + 1
    qs = np.where(qs == PADDING_SEGMENT_ID, pad_id, qs)
    ks = np.where(ks == PADDING_SEGMENT_ID, pad_id, ks)
    nq = qp.shape[1] // query_block_size
    nk = kp.shape[1] // kv_block_size
    if calculate_dkdv_mask:
        op, os_, ob, ip, is_, ib, n_outer, n_inner = kp, ks, kv_block_size, qp, qs, query_block_size, nk, nq
    else:
        op, os_, ob, ip, is_, ib, n_outer, n_inner = qp, qs, query_block_size, kp, ks, kv_block_size, nq, nk
    B = qp.shape[0]
    out = np.zeros((4, B, n_outer), np.int32)
    for b in range(B):
        for o in range(n_outer):
            osb = os_[b, o * ob:(o + 1) * ob]
            opb = op[b, o * ob:(o + 1) * ob]
            o_smax, o_smin = int(osb.max()), int(osb.min())
            o_same = o_smax == o_smin
            if skip_pad_tokens and o_same and o_smin == pad_id:
                continue  # four zeros
            o_pmax, o_pmin = int(opb.max()), int(opb.min())
            up, lo, upf, lof = 0, n_inner, 0, n_inner
            for i in range(n_inner):
                isb = is_[b, i * ib:(i + 1) * ib]
                ipb = ip[b, i * ib:(i + 1) * ib]
                i_smin, i_smax = int(isb.min()), int(isb.max())
                i_pmin, i_pmax = int(ipb.min()), int(ipb.max())
                seg_ok = i_smin <= o_smax and o_smin <= i_smax
                full_seg = o_same and (i_smin == i_smax)
                if not calculate_dkdv_mask:
                    pos_any, pos_all = o_pmax >= i_pmin, o_pmin >= i_pmax
                else:
                    pos_any, pos_all = i_pmax >= o_pmin, i_pmin >= o_pmax
                att = pos_any and seg_ok
                if skip_pad_tokens:
                    att = att and not (i_smin == pad_id)
                if att:
                    up, lo = max(up, i + 1), min(lo, i)
                if full_seg and pos_all and att:
                    upf, lof = max(upf, i + 1), min(lof, i)
            out[:, b, o] = (lo, up, lof, upf)
    lower, upper, lower_full, upper_full = out
    n = n_inner
    if calculate_dkdv_mask:
        lower = np.where(lower == n, upper, lower)
        lower_full = np.where(lower_full == n, upper, lower_full)
    else:
        lower = np.where(lower == n, upper, lower)
        lower_full = np.where(lower_full == n, lower, lower_full)
    upper_full = np.where(upper_full < lower_full, lower_full, upper_full)
    return tuple(a.reshape(B, 1, -1).astype(np.int32) for a in (lower, upper, lower_full, upper_full))


def create_attention_mask(
    query_positions,
    query_segment_ids,
    kv_positions,
    kv_segment_ids,
    fwd_blocks: tuple[int, int],
    bwd_blocks: tuple[int, int] | None = None,
    calc_bwd_mask: bool = False,
    skip_pad_tokens: bool = True,
):
    """One device's share of mask_creator.py:377-490.

    `fwd_blocks` / `bwd_blocks` are (query_block_size, kv_block_size).  Returns a
    tuple of 1 or 3 masks, each a 4-tuple of int32 arrays.
    """
    args = (query_positions, query_segment_ids, kv_positions, kv_segment_ids)
    out = [
        compute_attention_mask_single_device(
            *args, kv_block_size=fwd_blocks[1], query_block_size=fwd_blocks[0],
            skip_pad_tokens=skip_pad_tokens)
    ]
    if calc_bwd_mask:
        bq, bk = bwd_blocks
        out.append(  # dq mask: tile sizes swapped, mask_creator.py:457-472
            compute_attention_mask_single_device(
                *args, kv_block_size=bq, query_block_size=bk, skip_pad_tokens=skip_pad_tokens))
        out.append(  # dkdv mask, :475-485
            compute_attention_mask_single_device(
                *args, kv_block_size=bk, query_block_size=bq, skip_pad_tokens=skip_pad_tokens,
                calculate_dkdv_mask=True))
    return tuple(out)


def dense_mask(query_positions, query_segment_ids, kv_positions, kv_segment_ids, skip_pad=False):
    """Dense boolean mask: tests/test_attention.py:33-49 (+ pad masks :911-921)."""
    qp = np.asarray(query_positions)[..., :, None]
    kp = np.asarray(kv_positions)[..., None, :]
    qs = np.asarray(query_segment_ids)[..., :, None]
    ks = np.asarray(kv_segment_ids)[..., None, :]
    m = (qs == ks) & (qp >= kp)
    if skip_pad:
        m = m & (qs != PADDING_SEGMENT_ID) & (ks != PADDING_SEGMENT_ID)
    return m


def tight_tile_count(query_positions, query_segment_ids, kv_positions, kv_segment_ids, tile=128):
    """Number of (b, q tile, kv tile) pairs holding at least one unmasked element of
    segment AND causal AND non-PAD.  This is the algorithmic work the throughput
    figures are normalised by; it is independent of any implementation's block lists.
    Works row-block by row-block so that 128k-token inputs stay cheap."""
    qp = np.asarray(query_positions); qs = np.asarray(query_segment_ids)
    kp = np.asarray(kv_positions); ks = np.asarray(kv_segment_ids)
    B, Sq = qp.shape
    Sk = kp.shape[1]
    nk = (Sk + tile - 1) // tile
    padk = nk * tile - Sk
    kp_p = np.pad(kp, ((0, 0), (0, padk)), constant_values=INT32_MAX)
    ks_p = np.pad(ks, ((0, 0), (0, padk)), constant_values=PADDING_SEGMENT_ID)
    total = 0
    for b in range(B):
        for q0 in range(0, Sq, tile):
            qpb = qp[b, q0:q0 + tile, None]
            qsb = qs[b, q0:q0 + tile, None]
            m = (qsb == ks_p[b][None, :]) & (qpb >= kp_p[b][None, :])
            m &= (qsb != PADDING_SEGMENT_ID) & (ks_p[b][None, :] != PADDING_SEGMENT_ID)
            total += int(m.reshape(m.shape[0], nk, tile).any(axis=(0, 2)).sum())
    return total
