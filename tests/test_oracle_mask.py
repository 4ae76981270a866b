"""The NumPy mask oracle against fixtures produced by the reference's own code."""
import glob
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR
from oracle import mask_oracle as mo

FIXTURES = sorted(glob.glob(os.path.join(GOLDEN_DIR, "mask_*.npz")))
NAMES = ("lower", "upper", "lower_full", "upper_full")


def _shards(g):
    cp = int(g["cp"])
    q_pos, q_seg = g["q_pos"], g["q_seg"]
    n = q_pos.shape[1] // cp
    return [(q_pos[:, r * n:(r + 1) * n], q_seg[:, r * n:(r + 1) * n]) for r in range(cp)]


def test_fixtures_present():
    assert len(FIXTURES) >= 15


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[5:-4] for p in FIXTURES])
def test_oracle_matches_reference_outputs(path):
    g = np.load(path)
    fwd, bwd, skip = tuple(g["fwd"]), tuple(g["bwd"]), bool(g["skip"])
    for r, (qp, qs) in enumerate(_shards(g)):
        masks = mo.create_attention_mask(qp, qs, g["kv_pos"], g["kv_seg"], fwd, bwd,
                                         calc_bwd_mask=True, skip_pad_tokens=skip)
        for tag, mask in zip(("fwd", "dq", "dkdv"), masks):
            for nm, a in zip(NAMES, mask):
                ref = g[f"r{r}_{tag}_{nm}"]
                assert a.dtype == np.int32 and a.shape == ref.shape
                np.testing.assert_array_equal(a, ref, err_msg=f"{tag}.{nm} shard {r}")


@pytest.mark.parametrize("path", FIXTURES[:8], ids=[os.path.basename(p)[5:-4] for p in FIXTURES[:8]])
def test_literal_transcription_agrees(path):
    g = np.load(path)
    if g["q_pos"].shape[1] > 2048:
        pytest.skip("scalar loop kept to small cases")
    fwd, skip = tuple(g["fwd"]), bool(g["skip"])
    qp, qs = _shards(g)[0]
    for dkdv in (False, True):
        a = mo.compute_attention_mask_single_device(qp, qs, g["kv_pos"], g["kv_seg"], fwd[1], fwd[0], skip, dkdv)
        b = mo.compute_attention_mask_literal(qp, qs, g["kv_pos"], g["kv_seg"], fwd[1], fwd[0], skip, dkdv)
        for x, y in zip(a, b):
            np.testing.assert_array_equal(x, y)


def test_dense_definition_for_global_arange_positions():
    """With non-restarting positions the interval heuristics equal the dense any/all
    tile bounds, which is what the reference's own test checks
    (tests/test_attention.py:855-1009)."""
    g = np.load(os.path.join(GOLDEN_DIR, "mask_arange_12doc_skip.npz"))
    qp, qs, kp, ks = g["q_pos"], g["q_seg"], g["kv_pos"], g["kv_seg"]
    bq, bk = map(int, g["fwd"])
    dense = mo.dense_mask(qp, qs, kp, ks, skip_pad=True)
    B, Sq, Sk = dense.shape
    t = dense.reshape(B, Sq // bq, bq, Sk // bk, bk).transpose(0, 1, 3, 2, 4)
    any_, all_ = t.any((3, 4)), t.all((3, 4))
    nk = Sk // bk
    lower = any_.argmax(-1)
    upper = nk - any_[..., ::-1].argmax(-1)
    none = ~any_.any(-1)
    lower, upper = np.where(none, 0, lower), np.where(none, 0, upper)
    lf = all_.argmax(-1)
    uf = nk - all_[..., ::-1].argmax(-1)
    nof = ~all_.any(-1)
    lf, uf = np.where(nof, lower, lf), np.where(nof, lower, uf)
    for nm, ref in zip(NAMES, (lower, upper, lf, uf)):
        np.testing.assert_array_equal(g[f"r0_fwd_{nm}"][:, 0], ref, err_msg=nm)
