"""Attention parity at the sizes the benchmark numbers are quoted on.

The CUDA kernels (forward, both backward schedules) run the benchmark configurations in full;
O, LSE2, dQ, dK and dV are compared on the device with `oracle.attention_oracle.attention_dense_torch`
(fp32 dense masked attention and its analytic gradients, evaluated in blocks; checked against the
NumPy oracle in tests/test_oracle_attention.py) on:

  * the 8k Llama-8B layer: every head;
  * the 32k document-mask workload (the one the headline metric is quoted on): two GQA groups
    (8 query heads), both batch rows;
  * the 16k dense causal workload: two heads, two batch rows;
  * the 128k context-parallel workload on one GPU: one GQA group (8 query heads).

Asserted: rel-L2 <= 5e-3 and max-abs <= 2e-2 (+ half a bf16 ulp of the largest reference value for
tensors that leave the kernels in bf16).  Every comparison also prints whether the strict
2e-2 / 5e-3 statement held; the lines are collected in $KVAX_B200_REPORT_DIR/parity_at_scale.json when that
variable names a directory.  Tensors are drawn on the device (seeded) because host generation of 10^9
normals costs more than the test itself; document layouts come from the same NumPy generator as
the benchmark.
"""
import json
import os

import numpy as np
import pytest
import torch

from helpers import MAX_ABS, REL_L2
from oracle import attention_oracle as ao
from oracle import generators as gen

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REPORT = []


def _cmp(tag, name, got, ref, rows, batch_rows, heads, bf16_output):
    """Device-side version of helpers.compare on the evaluated subset: got / ref (B, S, H, D) tensors,
    `rows` (B, S) bool (non-PAD tokens), `batch_rows` / `heads` index lists."""
    dev = got.device
    bi, hi = torch.tensor(batch_rows, device=dev), torch.tensor(heads, device=dev)
    sel = rows.index_select(0, bi)[:, :, None, None]
    zero = torch.zeros((), device=dev, dtype=torch.float64)
    got = torch.where(sel, got.index_select(0, bi).index_select(2, hi).double(), zero)
    ref = torch.where(sel, ref.index_select(0, bi).index_select(2, hi).double(), zero)
    assert bool(torch.isfinite(got).all()), f"{tag} {name}: non-finite values"
    err = float((got - ref).abs().max())
    rel = float((got - ref).norm() / ref.norm().clamp_min(1e-30))
    ref_max = float(ref.abs().max())
    budget = MAX_ABS + (ref_max / 256.0 if bf16_output else 0.0)
    rec = dict(case=tag, tensor=name, max_abs=err, rel_l2=rel, ref_max=ref_max, strict_ok=bool(err <= MAX_ABS and rel <= REL_L2),
               asserted_max_abs=budget, heads=len(heads), batch_rows=len(batch_rows))
    _REPORT.append(rec)
    print(f"[parity] {tag} {name}: max-abs {err:.4g} rel-L2 {rel:.4g} |ref|max {ref_max:.3g} "
          f"strict(2e-2, 5e-3) {'ok' if rec['strict_ok'] else 'NOT met'}; asserted max-abs <= {budget:.4g}")
    out_dir = os.environ.get("KVAX_B200_REPORT_DIR")           # optional: where to collect the parity figures
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "parity_at_scale.json"), "w") as f:
            json.dump(_REPORT, f, indent=1)
    assert err <= budget and rel <= REL_L2, f"{tag} {name}: max-abs {err:.4g} (<= {budget:.4g}), rel-L2 {rel:.4g}"


def _run_case(tag, cfg_name, kv_heads, batch_rows, modes, q_chunk=4096, seed=0):
    from kvax_b200.ops.flash_attention import attention_backward, attention_forward, check_status
    from kvax_b200.ops.mask_creator import build_masks

    cfg = gen.CONFIGS[cfg_name]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    inp = gen.make_inputs(cfg, seed=seed, with_tensors=False)
    pos_h, seg_h = inp["positions"], inp["segment_ids"]
    B, S, Hq, Hkv, D = cfg.batch, cfg.seq, cfg.hq, cfg.hkv, cfg.head_dim
    g = torch.Generator(device=dev).manual_seed(1000 + seed)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, do = rnd(B, S, Hq, D), rnd(B, S, Hkv, D), rnd(B, S, Hkv, D), rnd(B, S, Hq, D)
    pos, seg = torch.from_numpy(pos_h).to(dev), torch.from_numpy(seg_h).to(dev)
    do = torch.where((seg != -1)[:, :, None, None], do, torch.zeros((), dtype=do.dtype, device=dev))
    t = cfg.tile
    masks = build_masks(pos, seg, pos, seg, [(t, t, False), (t, t, False), (t, t, True)], True)
    out, lse, st = attention_forward(q, k, v, pos, seg, pos, seg, masks[0], (t, t), inp["scale"])
    ref = ao.attention_dense_torch(q, k, v, pos, seg, pos, seg, inp["scale"], do, kv_heads=kv_heads, batch_rows=batch_rows,
                                   q_chunk=q_chunk)
    torch.cuda.synchronize()
    check_status(st, "attn_fwd")
    rows = seg != -1
    br, qh, kh = ref["batch_rows"], ref["q_heads"], ref["kv_heads"]
    _cmp(tag, "out", out, ref["out"], rows, br, qh, True)
    bi, hi = torch.tensor(br, device=dev), torch.tensor(qh, device=dev)
    l_got, l_ref = (x.index_select(0, bi).index_select(1, hi) for x in (lse, ref["lse2"]))
    sel_l = rows.index_select(0, bi)[:, None, :] & torch.isfinite(l_ref)
    lse_err = float(torch.where(sel_l, l_got - l_ref, torch.zeros((), device=dev)).abs().max())
    assert lse_err <= 2e-2, f"{tag} lse2: {lse_err}"
    for mode in modes:
        dq, dk, dv, st2 = attention_backward(q, k, v, out, do, lse, pos, seg, pos, seg, masks[1], masks[2], (t, t),
                                             inp["scale"], mode=mode)
        torch.cuda.synchronize()
        check_status(st2, f"attn_bwd[{mode}]")
        _cmp(tag, f"dq[{mode}]", dq, ref["dq"], rows, br, qh, True)
        _cmp(tag, f"dk[{mode}]", dk, ref["dk"], rows, br, kh, False)
        _cmp(tag, f"dv[{mode}]", dv, ref["dv"], rows, br, kh, False)
        del dq, dk, dv
    del ref, q, k, v, do, out, lse
    torch.cuda.empty_cache()


def test_llama8b_8k_every_head():
    _run_case("c2_llama8b_8k", "c2_llama8b_8k", None, None, ("fused", "two_kernel"))


def test_docmask_32k_two_gqa_groups_both_rows():
    _run_case("c4_docmask_32k", "c4_docmask_32k", [0, 5], None, ("fused", "two_kernel"))


def test_dense_causal_16k_two_heads():
    _run_case("c3_dense_causal_16k", "c3_dense_causal_16k", [0, 9], [0, 3], ("fused", "two_kernel"))


def test_context_parallel_workload_128k_on_one_gpu_one_gqa_group():
    _run_case("c5_cp_128k", "c5_cp_128k", [3], None, ("fused",), q_chunk=2048)
