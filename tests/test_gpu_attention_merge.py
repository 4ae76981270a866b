"""Merge of two partial forward results over disjoint key sets (kvax_b200_attn_merge), the step of the overlapped
all-gather schedule: forward on the keys of two chunks, forward on the rest, merge, against the dense CPU oracle on
all keys (same tolerance as the forward kernel: max-abs 2e-2, rel-L2 5e-3 on non-PAD rows)."""
import numpy as np
import pytest
import torch

from helpers import bf16_round, compare, i32_cuda, to_bf16_cuda
from oracle import attention_oracle as ao
from oracle import generators as gen

pytestmark = pytest.mark.gpu


def _chunks(a, idx, half):
    return np.concatenate([a[:, c * half:(c + 1) * half] for c in idx], axis=1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("own", [(0, 3), (1, 2), (0, 1)])
def test_merge_of_own_and_remote_keys(own, dtype):
    from kvax_b200.ops.flash_attention import attention_forward, attention_merge, check_status
    from kvax_b200.ops.mask_creator import build_masks

    cfg = gen.small_config(seq=2048, batch=2, hq=4, hkv=2, head_dim=128, doc_min=100, doc_max=1500, pad=0.05)
    inp = gen.make_inputs(cfg, seed=23)
    half = cfg.seq // 4
    rest = tuple(c for c in range(4) if c not in own)
    # queries: the chunks of `own` (what a rank of a 2-way context-parallel job holds)
    pos, seg = inp["positions"], inp["segment_ids"]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dtype)
    q = dev(_chunks(inp["q"], own, half))
    qp, qs = i32_cuda(_chunks(pos, own, half)), i32_cuda(_chunks(seg, own, half))
    parts = []
    for idx in (own, rest):
        k, v = dev(_chunks(inp["k"], idx, half)), dev(_chunks(inp["v"], idx, half))
        kp, ks = i32_cuda(_chunks(pos, idx, half)), i32_cuda(_chunks(seg, idx, half))
        (mask,) = build_masks(qp, qs, kp, ks, [(128, 128, False)], True)
        out, lse, status = attention_forward(q, k, v, qp, qs, kp, ks, mask, (128, 128), inp["scale"], empty_lse_inf=True)
        torch.cuda.synchronize()
        check_status(status, "attn_fwd")
        parts.append((out, lse))
    out, lse = attention_merge(parts[0][0], parts[0][1], parts[1][0], parts[1][1])
    torch.cuda.synchronize()
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a.astype(np.float16).astype(np.float32))
    ref_o, ref_lse = ao.attention_forward(rnd(_chunks(inp["q"], own, half)), rnd(inp["k"]), rnd(inp["v"]), _chunks(pos, own, half),
                                          _chunks(seg, own, half), pos, seg, inp["scale"], dtype=np.float32)
    rows = _chunks(seg, own, half) != -1
    compare("out", out.float().cpu().numpy(), ref_o, rows[:, :, None, None], bf16_output=True)
    lse_rows = rows[:, None, :] & np.isfinite(ref_lse)
    compare("lse2", lse.cpu().numpy(), ref_lse, lse_rows, max_abs=2e-2, rel_l2=1e-3)
    # rows without any allowed key in either part stay empty: zeros and +inf
    got_lse = lse.cpu().numpy()
    empty = ~np.isfinite(ref_lse) & rows[:, None, :]
    assert np.all(np.isinf(got_lse[empty]))


def test_merge_rejects_strided_tensors():
    from kvax_b200.ops.flash_attention import attention_merge

    a = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device="cuda")
    l = torch.zeros(1, 2, 128, device="cuda")
    with pytest.raises(AssertionError):
        attention_merge(a[:, :, :1], l[:, :1], a[:, :, :1], l[:, :1])
