"""The dense attention oracle against outputs of the reference's own attention code.

tests/golden/attn_*.npz hold what the reference's `flash_attention_triton_forward` and
`flash_attention_backward` (host functions and Triton kernels, run by Triton's CPU interpreter,
see tests/golden/make_attention_golden.py) return for small seeded inputs.  The oracle is a
different algorithm (dense masked softmax in fp64), so agreement to fp32 rounding pins both the
semantics (causal on positions, segment equality, PAD handling, base-2 log-sum-exp, GQA group
sum of dK/dV) and the oracle the GPU parity tests rely on."""
import glob
import os

import numpy as np
import pytest

from helpers import bf16_bits_to_f32
from oracle import attention_oracle as ao

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_*.npz")))


def test_fixtures_present():
    assert len(GOLDEN) >= 8


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[5:-4] for p in GOLDEN])
def test_oracle_matches_reference_attention(path):
    z = np.load(path)
    q, k, v, do = (bf16_bits_to_f32(z[n]) for n in ("q", "k", "v", "dout"))
    scale = float(z["scale"])
    rows = (z["q_seg"] != -1)
    out, lse2 = ao.attention_forward(q, k, v, z["q_pos"], z["q_seg"], z["kv_pos"], z["kv_seg"], scale)
    # rows that attend to nothing are unspecified in the reference (its kernel normalises 0 / 0)
    has_key = np.isfinite(lse2).all(axis=1) & rows                      # (B, Sq)
    sel = has_key[:, :, None, None]
    assert has_key.any()
    np.testing.assert_allclose(np.where(sel, out, 0), np.where(sel, z["out"], 0), rtol=0, atol=2e-5)
    sel_l = has_key[:, None, :]
    np.testing.assert_allclose(np.where(sel_l, lse2, 0), np.where(sel_l, z["lse2"], 0), rtol=0, atol=2e-5)
    if "dq" in z.files:
        dq, dk, dv = ao.attention_backward(q, k, v, z["q_pos"], z["q_seg"], z["kv_pos"], z["kv_seg"], scale, do,
                                           dtype=np.float64)
        krows = (z["kv_seg"] != -1)[:, :, None, None]
        for name, got, ref, m in (("dq", dq, z["dq"], sel), ("dk", dk, z["dk"], krows), ("dv", dv, z["dv"], krows)):
            err = np.abs(np.where(m, got - ref, 0)).max()
            assert err <= 2e-5 * max(1.0, np.abs(ref).max()), f"{name}: {err}"


@pytest.mark.parametrize("q_chunk", [64, 4096])
def test_blocked_torch_reference_matches_the_dense_oracle(q_chunk):
    """`attention_dense_torch` (the fp32 reference of the parity tests at benchmark sizes) against
    the NumPy oracle above, on a document-masked GQA case with PAD, whole and in small blocks."""
    import torch
    from oracle import generators as gen

    cfg = gen.small_config(seq=512, batch=2, hq=4, hkv=2, head_dim=64, doc_min=40, doc_max=300, pad=0.08)
    inp = gen.make_inputs(cfg, seed=3)
    p, s = inp["positions"], inp["segment_ids"]
    do = np.where((s != -1)[:, :, None, None], inp["dout"], 0.0).astype(np.float32)
    out, lse2 = ao.attention_forward(inp["q"], inp["k"], inp["v"], p, s, p, s, inp["scale"])
    dq, dk, dv = ao.attention_backward(inp["q"], inp["k"], inp["v"], p, s, p, s, inp["scale"], do)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    res = ao.attention_dense_torch(t(inp["q"]), t(inp["k"]), t(inp["v"]), p, s, p, s, inp["scale"], t(do), q_chunk=q_chunk)
    rows = (s != -1)
    sel = rows[:, :, None, None]
    for name, got, ref in (("out", res["out"], out), ("dq", res["dq"], dq), ("dk", res["dk"], dk), ("dv", res["dv"], dv)):
        err = np.abs(np.where(sel, got.numpy() - ref, 0)).max()
        assert err <= 3e-5 * max(1.0, np.abs(ref).max()), f"{name}: {err}"
    err = np.abs(np.where(rows[:, None, :], res["lse2"].numpy() - lse2, 0)).max()
    assert err <= 3e-5
    # a subset of kv heads / batch rows leaves the rest zero and equals the full result where evaluated
    sub = ao.attention_dense_torch(t(inp["q"]), t(inp["k"]), t(inp["v"]), p, s, p, s, inp["scale"], t(do), kv_heads=[1],
                                   batch_rows=[1], q_chunk=q_chunk)
    assert sub["q_heads"] == [2, 3]
    np.testing.assert_array_equal(sub["dq"][1, :, 2:4].numpy(), res["dq"][1, :, 2:4].numpy())
    assert float(sub["dq"][0].abs().max()) == 0.0 and float(sub["dk"][1, :, 0].abs().max()) == 0.0
