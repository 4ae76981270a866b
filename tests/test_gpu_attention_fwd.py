"""Forward attention kernel against the dense CPU oracle (bf16 tolerance: max-abs 2e-2,
rel-L2 5e-3 on non-PAD rows, fp32 comparison)."""
import numpy as np
import pytest
import torch

from helpers import bf16_round, compare, i32_cuda, to_bf16_cuda
from oracle import attention_oracle as ao
from oracle import generators as gen

pytestmark = pytest.mark.gpu

_KERNEL = None


@pytest.fixture(autouse=True, params=["one_tile", "tile_pairs", "head_pairs"])
def fwd_kernel(request):
    """Every test of this file runs on every forward kernel (a CTA per query tile / per pair of query tiles / per
    pair of query heads of a kv group; the last needs an even number of query heads per kv head)."""
    global _KERNEL
    _KERNEL = request.param
    yield request.param
    _KERNEL = None


def _run_fwd(inp, fwd_blocks=(128, 128), sequential=False, q_slice=None, kv_slice=None):
    import kvax_b200 as kv
    from kvax_b200.ops.flash_attention import attention_forward, check_status
    from kvax_b200.ops.mask_creator import build_masks

    qs = q_slice or slice(None)
    ks = kv_slice or slice(None)
    if _KERNEL == "head_pairs" and (inp["q"].shape[2] // inp["k"].shape[2]) % 2:
        pytest.skip("head pairs need an even number of query heads per kv head")
    q, k, v = to_bf16_cuda(inp["q"][:, qs]), to_bf16_cuda(inp["k"][:, ks]), to_bf16_cuda(inp["v"][:, ks])
    qp, qsg = i32_cuda(inp["positions"][:, qs]), i32_cuda(inp["segment_ids"][:, qs])
    kp, ksg = i32_cuda(inp["positions"][:, ks]), i32_cuda(inp["segment_ids"][:, ks])
    (mask,) = build_masks(qp, qsg, kp, ksg, [(fwd_blocks[0], fwd_blocks[1], False)], True)
    out, lse, status = attention_forward(q, k, v, qp, qsg, kp, ksg, mask, fwd_blocks, inp["scale"], sequential,
                                         kernel=_KERNEL)
    torch.cuda.synchronize()
    check_status(status, "attn_fwd")
    return out.float().cpu().numpy(), lse.cpu().numpy()


def _oracle(inp, q_slice=None, kv_slice=None):
    qs = q_slice or slice(None)
    ks = kv_slice or slice(None)
    p, s = inp["positions"], inp["segment_ids"]
    return ao.attention_forward(bf16_round(inp["q"][:, qs]), bf16_round(inp["k"][:, ks]), bf16_round(inp["v"][:, ks]),
                                p[:, qs], s[:, qs], p[:, ks], s[:, ks], inp["scale"], dtype=np.float32)


def _check(inp, out, lse, q_slice=None, kv_slice=None):
    ref_o, ref_lse = _oracle(inp, q_slice, kv_slice)
    seg = inp["segment_ids"][:, q_slice or slice(None)]
    rows = (seg != -1)
    compare("out", out, ref_o, rows[:, :, None, None], bf16_output=True)
    lse_rows = rows[:, None, :] & np.isfinite(ref_lse)
    compare("lse2", lse, ref_lse, lse_rows, max_abs=2e-2, rel_l2=1e-3)


@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("restart", [True, False])
def test_forward_small_docmask(head_dim, restart):
    cfg = gen.small_config(seq=1024, hq=4, hkv=2, head_dim=head_dim)
    inp = gen.make_inputs(cfg, seed=3, restart_positions=restart)
    out, lse = _run_fwd(inp)
    _check(inp, out, lse)


def _layout_inputs(lengths, seq, seed, restart=True, hq=2, hkv=1, batch=1):
    """Hand-made document layout: `lengths` tokens per document, the rest PAD."""
    cfg = gen.small_config(seq=seq, batch=batch, hq=hq, hkv=hkv, head_dim=128)
    inp = gen.make_inputs(cfg, seed=seed)
    pos = np.zeros((batch, seq), np.int32)
    seg = np.full((batch, seq), -1, np.int32)
    at = 0
    for i, n in enumerate(lengths):
        seg[:, at:at + n] = i
        pos[:, at:at + n] = np.arange(n) if restart else np.arange(at, at + n)
        at += n
    pos[:, at:] = np.arange(seq - at) if restart else np.arange(at, seq)
    inp["positions"], inp["segment_ids"] = pos, seg
    return inp


@pytest.mark.parametrize("restart", [True, False])
def test_forward_tile_pairs_with_unequal_lists(restart):
    """Documents that end on tile boundaries, so that the two query tiles of a pair have nothing in common: pair (2, 3)
    has tile 2 in the first document (kv tiles 0-2) and tile 3 in the second (kv tile 3 only), pair (4, 5) has a
    tile of the second document next to an all-PAD tile (empty list), pair (6, 7) is all PAD (both lists empty)."""
    inp = _layout_inputs([384, 256], seq=1024, seed=23, restart=restart)
    out, lse = _run_fwd(inp)
    _check(inp, out, lse)


@pytest.mark.parametrize("seq,hq,hkv", [(2048, 2, 1), (2048 + 70, 4, 1)])
def test_forward_many_partial_tiles(seq, hq, hkv):
    """Segments interleaved in runs of 48 tokens (ids cycling through three values) with global positions: every kv tile
    up to the diagonal holds keys of the query's segment and others, so every list entry is a partial tile -- up to 17
    per list.  The first eight take the element masks the list builder worked out, the rest are masked in the
    attention kernel: both must agree with the oracle."""
    cfg = gen.small_config(seq=seq, batch=2, hq=hq, hkv=hkv, head_dim=128)
    inp = gen.make_inputs(cfg, seed=43)
    idx = np.arange(seq)
    seg = np.broadcast_to(((idx // 48) % 3).astype(np.int32), (2, seq)).copy()
    seg[1] = ((idx // 80) % 2).astype(np.int32)
    seg[:, seq - 100:] = -1
    inp["positions"] = np.broadcast_to(idx.astype(np.int32), (2, seq)).copy()
    inp["segment_ids"] = seg
    out, lse = _run_fwd(inp)
    _check(inp, out, lse)


@pytest.mark.parametrize("n_tiles", [1, 3, 5])
def test_forward_odd_tile_counts(n_tiles):
    """Sequences with an odd number of query tiles: the last pair has one tile only."""
    inp = _layout_inputs([128 * n_tiles - 40], seq=128 * n_tiles, seed=29 + n_tiles)
    out, lse = _run_fwd(inp)
    _check(inp, out, lse)


@pytest.mark.parametrize("blocks", [(64, 64), (128, 64), (64, 128), (256, 128)])
def test_forward_mask_block_sizes(blocks):
    cfg = gen.small_config(seq=1024, hq=2, hkv=1, head_dim=128, doc_min=40, doc_max=500)
    inp = gen.make_inputs(cfg, seed=5)
    out, lse = _run_fwd(inp, fwd_blocks=blocks)
    _check(inp, out, lse)


def test_forward_tiny_config_c1():
    inp = gen.make_inputs(gen.CONFIGS["c1_tiny"], seed=0)
    out, lse = _run_fwd(inp, fwd_blocks=(64, 64))
    _check(inp, out, lse)


@pytest.mark.parametrize("sq,skv", [(384, 400), (300, 300), (1, 640), (3, 257), (400, 384)])
def test_forward_ragged_lengths(sq, skv):
    """Lengths that are not multiples of the tile (the reference pads, the kernel masks)."""
    S = max(sq, skv)
    cfg = gen.small_config(seq=S, batch=2, hq=4, hkv=4, head_dim=64, doc_min=S, doc_max=S, pad=0.0)
    inp = gen.make_inputs(cfg, seed=7, restart_positions=False)
    if sq < skv:   # queries are the last sq tokens (decode-like): keep causal structure meaningful
        q_slice = slice(skv - sq, skv)
    else:
        q_slice = slice(0, sq)
    kv_slice = slice(0, skv)
    out, lse = _run_fwd(inp, fwd_blocks=(64, 64), q_slice=q_slice, kv_slice=kv_slice)
    _check(inp, out, lse, q_slice, kv_slice)


def test_forward_sequential_positions_equivalent():
    cfg = gen.small_config(seq=1024, hq=2, hkv=2, head_dim=128)
    inp = gen.make_inputs(cfg, seed=11, restart_positions=False)   # positions == indices
    a, la = _run_fwd(inp, sequential=False)
    b, lb = _run_fwd(inp, sequential=True)
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    np.testing.assert_array_equal(np.where(rows, a, 0), np.where(rows, b, 0))


def test_forward_deterministic():
    cfg = gen.small_config(seq=2048, hq=4, hkv=1, head_dim=128)
    inp = gen.make_inputs(cfg, seed=13)
    a, la = _run_fwd(inp)
    b, lb = _run_fwd(inp)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(la, lb)


def test_forward_llama8b_shape_properties():
    """Benchmark-size case (config 2): oracle on a subset of heads, plus size-independent
    properties: rows of different query heads of a group only differ through Q, PAD-only
    tiles give exact zeros."""
    cfg = gen.CONFIGS["c2_llama8b_8k"]
    inp = gen.make_inputs(cfg, seed=0)
    out, lse = _run_fwd(inp)
    sub = dict(inp)
    heads = [0, 5, 31]
    p, s = inp["positions"], inp["segment_ids"]
    for h in heads:
        ref_o, _ = ao.attention_forward(bf16_round(inp["q"][:, :, h:h + 1]), bf16_round(inp["k"][:, :, h // 4:h // 4 + 1]),
                                        bf16_round(inp["v"][:, :, h // 4:h // 4 + 1]), p, s, p, s, inp["scale"], dtype=np.float32)
        compare(f"out[h={h}]", out[:, :, h:h + 1], ref_o, (s != -1)[:, :, None, None], bf16_output=True)
    n_pad = int((s[0] == -1).sum())
    full_pad_tiles = n_pad // 128
    if full_pad_tiles:
        tail = out[0, cfg.seq - full_pad_tiles * 128:]
        assert np.all(tail == 0)
