"""CUDA mask builder against the reference-generated fixtures and the oracle (bit-exact)."""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle import generators as gen
from oracle import mask_oracle as mo

pytestmark = pytest.mark.gpu
FIXTURES = sorted(glob.glob(os.path.join(GOLDEN_DIR, "mask_*.npz")))
NAMES = ("lower", "upper", "lower_full", "upper_full")


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _build(qp, qs, kp, ks, fwd, bwd, skip):
    from kvax_b200.ops.mask_creator import build_masks
    specs = [(fwd[0], fwd[1], False), (bwd[1], bwd[0], False), (bwd[0], bwd[1], True)]
    return build_masks(_cuda(qp), _cuda(qs), _cuda(kp), _cuda(ks), specs, skip)


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[5:-4] for p in FIXTURES])
def test_mask_kernel_matches_reference_fixture(path):
    g = np.load(path)
    fwd, bwd, skip, cp = tuple(map(int, g["fwd"])), tuple(map(int, g["bwd"])), bool(g["skip"]), int(g["cp"])
    n = g["q_pos"].shape[1] // cp
    for r in range(cp):
        qp, qs = g["q_pos"][:, r * n:(r + 1) * n], g["q_seg"][:, r * n:(r + 1) * n]
        masks = _build(qp, qs, g["kv_pos"], g["kv_seg"], fwd, bwd, skip)
        for tag, m in zip(("fwd", "dq", "dkdv"), masks):
            for nm, t in zip(NAMES, m.flatten()):
                ref = g[f"r{r}_{tag}_{nm}"]
                got = t.cpu().numpy()
                assert got.dtype == np.int32 and got.shape == ref.shape
                np.testing.assert_array_equal(got, ref, err_msg=f"{tag}.{nm} shard {r}")


@pytest.mark.parametrize("name", ["c2_llama8b_8k", "c4_docmask_32k", "c5_cp_128k"])
@pytest.mark.parametrize("restart", [True, False])
def test_mask_kernel_matches_oracle_at_benchmark_sizes(name, restart):
    cfg = gen.CONFIGS[name]
    inp = gen.make_inputs(cfg, with_tensors=False, restart_positions=restart)
    p, s = inp["positions"], inp["segment_ids"]
    fwd, bwd = (128, 128), (64, 128)
    masks = _build(p, s, p, s, fwd, bwd, True)
    ref = mo.create_attention_mask(p, s, p, s, fwd, bwd, calc_bwd_mask=True, skip_pad_tokens=True)
    for m, rm in zip(masks, ref):
        for t, a in zip(m.flatten(), rm):
            np.testing.assert_array_equal(t.cpu().numpy(), a)


def test_public_api_shapes_and_errors():
    import kvax_b200 as kv
    cfg = gen.small_config(seq=512)
    inp = gen.make_inputs(cfg, with_tensors=False)
    p, s = _cuda(inp["positions"]), _cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    with pytest.raises(ValueError):
        kv.create_attention_mask(p, s, p, s, fwd_params=params)          # no mesh
    mesh = kv.Mesh(("data", "context"), (1, 1))
    with pytest.raises(ValueError):
        kv.create_attention_mask(p, s, p, s, fwd_params=params, mesh=mesh)  # no specs
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        one = kv.create_attention_mask(p, s, p, s, fwd_params=params)
        three = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
    assert len(one) == 1 and len(three) == 3
    assert tuple(one[0].lower_bounds.shape) == (cfg.batch, 1, 4)
    assert one[0].lower_bounds.dtype == torch.int32


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mask_kernel_on_unordered_segments_and_positions(seed):
    """Nothing in the builder may rely on sorted inputs: random segment ids (with PAD sprinkled in) and random
    positions, several block sizes per call.  The group summaries of the cluster path then rule out little and
    every scan path (first / last hit in any group) is exercised against the oracle."""
    rng = np.random.default_rng(seed)
    B, S = 3, 4096 + 64 * seed
    seg = rng.integers(0, 6, size=(B, S)).astype(np.int32)
    seg[rng.random((B, S)) < 0.2] = -1
    seg[:, 1000:1400] = -1                      # all-PAD blocks in the middle
    seg[1, 2048:2304] = 3                       # single-segment blocks
    pos = rng.integers(0, 5000, size=(B, S)).astype(np.int32)
    pos[1, 2048:2304] = np.arange(256)
    for skip in (True, False):
        fwd, bwd = (128, 64), (64, 32)
        masks = _build(pos, seg, pos, seg, fwd, bwd, skip)
        ref = mo.create_attention_mask(pos, seg, pos, seg, fwd, bwd, calc_bwd_mask=True, skip_pad_tokens=skip)
        for m, rm in zip(masks, ref):
            for t, a in zip(m.flatten(), rm):
                np.testing.assert_array_equal(t.cpu().numpy(), a)


def test_mask_kernel_many_blocks_per_row():
    """2048 blocks per row (128k tokens at block 64): more than 32 groups of 32 blocks, 256 blocks per CTA of
    the cluster."""
    cfg = gen.CONFIGS["c5_cp_128k"]
    inp = gen.make_inputs(cfg, with_tensors=False, seed=3)
    p, s = inp["positions"], inp["segment_ids"]
    fwd, bwd = (64, 64), (64, 64)
    masks = _build(p, s, p, s, fwd, bwd, True)
    ref = mo.create_attention_mask(p, s, p, s, fwd, bwd, calc_bwd_mask=True, skip_pad_tokens=True)
    for m, rm in zip(masks, ref):
        for t, a in zip(m.flatten(), rm):
            np.testing.assert_array_equal(t.cpu().numpy(), a)
