"""The CUDA attention kernels against outputs of the reference's own attention code
(tests/golden/attn_*.npz, produced by tests/golden/make_attention_golden.py): same inputs,
masks built by the CUDA mask builder with the block sizes the reference run used, results
compared on non-PAD rows within the tolerance of the parity statement (max-abs 2e-2, rel-L2 5e-3)."""
import glob
import os

import numpy as np
import pytest
import torch

from helpers import bf16_bits_to_f32, compare, i32_cuda

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_*.npz")))


@pytest.mark.parametrize("fwd_kernel", ["one_tile", "tile_pairs", "head_pairs"])
@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[5:-4] for p in GOLDEN])
def test_kernels_match_reference_outputs(path, fwd_kernel):
    from kvax_b200.ops.flash_attention import attention_backward, attention_forward, check_status, context_offsets
    from kvax_b200.ops.mask_creator import build_masks

    z = np.load(path)
    dev = torch.device("cuda")
    q, k, v, do = (torch.from_numpy(bf16_bits_to_f32(z[n])).to(dev).to(torch.bfloat16) for n in ("q", "k", "v", "dout"))
    qp, qs, kp, ks = (i32_cuda(z[n]) for n in ("q_pos", "q_seg", "kv_pos", "kv_seg"))
    scale, seq = float(z["scale"]), bool(z["sequential"])
    fwd = tuple(int(x) for x in z["fwd"])
    if fwd_kernel == "head_pairs" and (q.shape[2] // k.shape[2]) % 2:
        pytest.skip("head pairs need an even number of query heads per kv head")
    # per-rank fixtures of the context-parallel path: local (permuted) queries against the full keys / values,
    # sequential positions given by global offsets of the two halves of the local queries
    cp, rank = int(z["cp"]), int(z["rank"])
    offsets = context_offsets(rank, cp, q.shape[1], True)
    has_bwd = "dq" in z.files
    specs = [(fwd[0], fwd[1], False)]
    if has_bwd:
        bq, bk = (int(x) for x in z["bwd"])
        specs += [(bk, bq, False), (bq, bk, True)]
    masks = build_masks(qp, qs, kp, ks, specs, True)
    out, lse, st = attention_forward(q, k, v, qp, qs, kp, ks, masks[0], fwd, scale, seq, offsets, kernel=fwd_kernel)
    torch.cuda.synchronize()
    check_status(st, "attn_fwd")
    rows = (z["q_seg"] != -1) & np.isfinite(z["lse2"]).all(axis=1)
    sel = rows[:, :, None, None]
    compare("out", out.float().cpu().numpy(), z["out"], sel, bf16_output=True)
    lse_err = np.abs(np.where(rows[:, None, :], lse.cpu().numpy() - z["lse2"], 0)).max()
    assert lse_err <= 2e-2, f"lse2: {lse_err}"
    if has_bwd:
        dq, dk, dv, st2 = attention_backward(q, k, v, out, do, lse, qp, qs, kp, ks, masks[1], masks[2], (bq, bk), scale, seq, offsets)
        torch.cuda.synchronize()
        check_status(st2, "attn_bwd")
        krows = (z["kv_seg"] != -1)[:, :, None, None]
        compare("dq", dq.float().cpu().numpy(), z["dq"], sel, bf16_output=True)
        compare("dk", dk.float().cpu().numpy(), z["dk"], krows)
        compare("dv", dv.float().cpu().numpy(), z["dv"], krows)
