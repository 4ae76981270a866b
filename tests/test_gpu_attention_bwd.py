"""Backward attention kernels (delta, dQ, dK/dV) against the analytic gradients of the
dense CPU oracle.  Tolerance of the north-star statement: max-abs 2e-2 and rel-L2 5e-3 in
fp32 comparison, on non-PAD rows (the reference's tests zero PAD rows before comparing)."""
import numpy as np
import pytest
import torch

from helpers import bf16_round, compare, i32_cuda, to_bf16_cuda
from oracle import attention_oracle as ao
from oracle import generators as gen

pytestmark = pytest.mark.gpu


def _run_fwd_bwd(inp, fwd_blocks=(128, 128), bwd_blocks=(128, 128), sequential=False, mode=None):
    from kvax_b200.ops.flash_attention import attention_backward, attention_forward, check_status
    from kvax_b200.ops.mask_creator import build_masks

    q, k, v, do = (to_bf16_cuda(inp[n]) for n in ("q", "k", "v", "dout"))
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    bq, bk = bwd_blocks
    masks = build_masks(p, s, p, s, [(fwd_blocks[0], fwd_blocks[1], False), (bk, bq, False), (bq, bk, True)], True)
    out, lse, st = attention_forward(q, k, v, p, s, p, s, masks[0], fwd_blocks, inp["scale"], sequential)
    dq, dk, dv, st2 = attention_backward(q, k, v, out, do, lse, p, s, p, s, masks[1], masks[2], bwd_blocks,
                                         inp["scale"], sequential, mode=mode)
    torch.cuda.synchronize()
    check_status(st, "attn_fwd")
    check_status(st2, "attn_bwd")
    return tuple(t.float().cpu().numpy() for t in (out, dq, dk, dv))


def _oracle_grads(inp):
    p, s = inp["positions"], inp["segment_ids"]
    return ao.attention_backward(bf16_round(inp["q"]), bf16_round(inp["k"]), bf16_round(inp["v"]), p, s, p, s,
                                 inp["scale"], bf16_round(inp["dout"]), dtype=np.float64)


def _zero_pad_dout(inp):
    inp = dict(inp)
    inp["dout"] = np.where((inp["segment_ids"] != -1)[:, :, None, None], inp["dout"], 0.0).astype(np.float32)
    return inp


def _check(inp, dq, dk, dv):
    rq, rk, rv = _oracle_grads(inp)
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    compare("dq", dq, rq, rows, bf16_output=True)
    compare("dk", dk, rk, rows)
    compare("dv", dv, rv, rows)


@pytest.mark.parametrize("mode", ["fused", "two_kernel"])
@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("hq,hkv", [(4, 2), (4, 4), (4, 1)])
def test_backward_small_docmask(head_dim, hq, hkv, mode):
    """Both backward schedules (head_dim 64 always takes the two-kernel path)."""
    cfg = gen.small_config(seq=1024, hq=hq, hkv=hkv, head_dim=head_dim)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=3))
    _, dq, dk, dv = _run_fwd_bwd(inp, mode=mode)
    _check(inp, dq, dk, dv)


def test_fused_backward_agrees_with_two_kernel_backward():
    """Same P and dS in both schedules.  dQ is summed tile by tile with fp32 atomics in the fused schedule and in TMEM
    in the other, and on a problem this small the fused schedule also divides the query heads of a kv head over several
    CTAs whose dK / dV parts meet in fp32 accumulators: equal to rounding."""
    cfg = gen.small_config(seq=4096, batch=2, hq=8, hkv=2, head_dim=128, doc_min=100, doc_max=3000, pad=0.06)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=41))
    _, dq_f, dk_f, dv_f = _run_fwd_bwd(inp, mode="fused")
    _, dq_t, dk_t, dv_t = _run_fwd_bwd(inp, mode="two_kernel")
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    compare("dk fused vs two-kernel", dk_f, dk_t, rows, max_abs=1e-4 * float(np.abs(dk_t).max()), rel_l2=1e-5)
    compare("dv fused vs two-kernel", dv_f, dv_t, rows, max_abs=1e-4 * float(np.abs(dv_t).max()), rel_l2=1e-5)
    compare("dq fused vs two-kernel", dq_f, dq_t, rows, max_abs=1e-2 + np.abs(dq_t).max() / 128, rel_l2=4e-3)


@pytest.mark.parametrize("sequential", [False, True])
def test_fused_backward_sequential_and_global_positions(sequential):
    """assume_sequential_positions on the fused path (the causal test compares indices)."""
    cfg = gen.small_config(seq=2048, batch=1, hq=4, hkv=2, head_dim=128, doc_min=100, doc_max=900, pad=0.05)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=43, restart_positions=False))
    _, dq, dk, dv = _run_fwd_bwd(inp, sequential=sequential, mode="fused")
    _check(inp, dq, dk, dv)


@pytest.mark.parametrize("sequential", [False, True])
@pytest.mark.parametrize("mode", ["fused", "two_kernel"])
def test_backward_many_partial_tiles(mode, sequential):
    """Segments interleaved in runs of 48 tokens with global positions: every visited tile pair is a partial one, up to
    17 per list.  The first eight entries of a kv-outer list take the element masks the list builder worked out, the
    others are masked inside the kernels (the fused backward's fallback): both against the oracle, with position
    arrays and with assume_sequential_positions."""
    seq = 2048 + 70
    cfg = gen.small_config(seq=seq, batch=2, hq=4, hkv=1, head_dim=128)
    inp = dict(gen.make_inputs(cfg, seed=47))
    idx = np.arange(seq)
    seg = np.broadcast_to(((idx // 48) % 3).astype(np.int32), (2, seq)).copy()
    seg[1] = ((idx // 80) % 2).astype(np.int32)
    seg[:, seq - 100:] = -1
    inp["positions"] = np.broadcast_to(idx.astype(np.int32), (2, seq)).copy()
    inp["segment_ids"] = seg
    inp = _zero_pad_dout(inp)
    _, dq, dk, dv = _run_fwd_bwd(inp, sequential=sequential, mode=mode)
    _check(inp, dq, dk, dv)


@pytest.mark.parametrize("bwd_blocks", [(64, 128), (64, 64), (128, 64)])
def test_backward_mask_block_sizes(bwd_blocks):
    cfg = gen.small_config(seq=1024, hq=2, hkv=1, head_dim=128, doc_min=40, doc_max=500)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=5, restart_positions=False))
    _, dq, dk, dv = _run_fwd_bwd(inp, bwd_blocks=bwd_blocks)
    _check(inp, dq, dk, dv)


@pytest.mark.parametrize("seq,head_dim", [(300, 128), (257, 64), (400, 128)])
def test_backward_ragged_lengths(seq, head_dim):
    """Lengths that are not multiples of the tile: the last tile of every list is cut by the
    end of the sequence, and at 257 the LSE2 / delta rows are not 16-byte aligned, so the dK/dV
    kernel's producer takes its lane-copy path instead of bulk copies."""
    cfg = gen.small_config(seq=seq, batch=2, hq=4, hkv=2, head_dim=head_dim, doc_min=60, doc_max=seq, pad=0.04)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=23))
    out, dq, dk, dv = _run_fwd_bwd(inp, fwd_blocks=(64, 64), bwd_blocks=(64, 64))
    _check(inp, dq, dk, dv)


def test_backward_tiny_config_c1():
    inp = _zero_pad_dout(gen.make_inputs(gen.CONFIGS["c1_tiny"], seed=0))
    _, dq, dk, dv = _run_fwd_bwd(inp, fwd_blocks=(64, 64), bwd_blocks=(64, 64))
    _check(inp, dq, dk, dv)


def test_backward_deterministic():
    """The two-kernel backward is bit-reproducible.  The fused one sums dQ with fp32 atomics, and on small problems
    like this one (few CTAs: the query heads of a kv head are divided over several CTAs) dK and dV too: equal to
    rounding from run to run."""
    cfg = gen.small_config(seq=2048, hq=4, hkv=1, head_dim=128)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=13))
    a = _run_fwd_bwd(inp, mode="two_kernel")
    b = _run_fwd_bwd(inp, mode="two_kernel")
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)
    c = _run_fwd_bwd(inp, mode="fused")
    d = _run_fwd_bwd(inp, mode="fused")
    np.testing.assert_array_equal(c[0], d[0])
    for i in (1, 2, 3):
        np.testing.assert_allclose(c[i], d[i], rtol=0, atol=1e-2 * float(np.abs(c[i]).max()) / 128)


@pytest.mark.parametrize("bwd_blocks", [(64, 128), (128, 64)])
def test_backward_mask_block_sizes_fused(bwd_blocks):
    cfg = gen.small_config(seq=1024, hq=2, hkv=1, head_dim=128, doc_min=40, doc_max=500)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=5, restart_positions=True))
    _, dq, dk, dv = _run_fwd_bwd(inp, bwd_blocks=bwd_blocks, mode="fused")
    _check(inp, dq, dk, dv)


def test_strided_qkv_from_one_fused_projection():
    """q, k, v sliced out of one (B, S, Hq + 2 Hkv, D) tensor, as a fused QKV projection hands them
    over: the kernels read them through strided tensor maps and dq comes back dense."""
    import kvax_b200 as kv
    cfg = gen.small_config(seq=1024, batch=2, hq=4, hkv=2, head_dim=128)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=47))
    fused = torch.cat([to_bf16_cuda(inp[n]) for n in ("q", "k", "v")], dim=2).contiguous().requires_grad_(True)
    q, k, v = fused[:, :, :4], fused[:, :, 4:6], fused[:, :, 6:8]
    assert not q.is_contiguous()
    do = to_bf16_cuda(inp["dout"])
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, 1), rank=0)
    rq, rk, rv = _oracle_grads(inp)
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    for mode in ("fused", "two_kernel"):
        kv.set_backward_mode(mode)
        try:
            fused.grad = None
            with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
                masks = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
                out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
                out.backward(do)
        finally:
            kv.set_backward_mode("fused")
        g = fused.grad.float().cpu().numpy()
        compare(f"dq[{mode}]", g[:, :, :4], rq, rows, bf16_output=True)
        compare(f"dk[{mode}]", g[:, :, 4:6], rk, rows, max_abs=2e-2 + np.abs(rk).max() / 128)
        compare(f"dv[{mode}]", g[:, :, 6:8], rv, rows, max_abs=2e-2 + np.abs(rv).max() / 128)


def test_backward_linearity_in_dout():
    """Size-independent property: gradients are linear in dO (checked at 8k tokens)."""
    cfg = gen.small_config(seq=8192, batch=1, hq=4, hkv=2, head_dim=128, doc_min=128, doc_max=4096, pad=0.03)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=2))
    _, dq1, dk1, dv1 = _run_fwd_bwd(inp)
    inp2 = dict(inp)
    inp2["dout"] = inp["dout"] * 2.0          # exact in bf16
    _, dq2, dk2, dv2 = _run_fwd_bwd(inp2)
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    for a, b in ((dq1, dq2), (dk1, dk2), (dv1, dv2)):
        a, b = np.where(rows, a, 0), np.where(rows, b, 0)
        assert np.linalg.norm(2 * a - b) <= 4e-3 * np.linalg.norm(b)


def test_autograd_public_api():
    import kvax_b200 as kv
    cfg = gen.small_config(seq=1024, hq=4, hkv=2, head_dim=128)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=21))
    q, k, v, do = (to_bf16_cuda(inp[n]) for n in ("q", "k", "v", "dout"))
    for t in (q, k, v):
        t.requires_grad_(True)
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, 1))
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        masks = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
        (out.float() * do.float()).sum().backward()
        with pytest.raises(NotImplementedError):
            kv.flash_attention(q, k, v, p, s, p, s, masks, bias=torch.zeros(1, device="cuda"))
        with pytest.raises(ValueError):
            kv.flash_attention(q, k, v, p, s, p, s, (), scale=1.0)
    assert q.grad.dtype == torch.bfloat16 and k.grad.dtype == torch.bfloat16
    rq, rk, rv = _oracle_grads(inp)
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    # dk/dv were rounded to bf16 after the reduction: allow one bf16 ulp of the largest value
    compare("dq", q.grad.float().cpu().numpy(), rq, rows, bf16_output=True)
    compare("dk", k.grad.float().cpu().numpy(), rk, rows, max_abs=2e-2 + np.abs(rk).max() / 128)
    compare("dv", v.grad.float().cpu().numpy(), rv, rows, max_abs=2e-2 + np.abs(rv).max() / 128)


def _tiny_fp32_run():
    import kvax_b200 as kv
    inp = _zero_pad_dout(gen.make_inputs(gen.CONFIGS["c1_tiny"], seed=0))
    q, k, v, do = (torch.from_numpy(inp[n]).cuda() for n in ("q", "k", "v", "dout"))
    for t in (q, k, v):
        t.requires_grad_(True)
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(64, 64)
    mesh = kv.Mesh(("data", "context"), (1, 1))
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        masks = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
        (out * do).sum().backward()
    assert out.dtype == torch.float32 and q.grad.dtype == torch.float32 and k.grad.dtype == torch.float32
    pp, ss = inp["positions"], inp["segment_ids"]
    ref_o, _ = ao.attention_forward(inp["q"], inp["k"], inp["v"], pp, ss, pp, ss, inp["scale"], dtype=np.float64)
    rq, rk, rv = ao.attention_backward(inp["q"], inp["k"], inp["v"], pp, ss, pp, ss, inp["scale"], inp["dout"])
    rows = (ss != -1)[:, :, None, None]
    return rows, (out.detach().cpu().numpy(), ref_o), (q.grad.cpu().numpy(), rq), (k.grad.cpu().numpy(), rk), (v.grad.cpu().numpy(), rv)


def test_fp32_inputs_tiny_config():
    """The CPU-runnable configuration (fp32 tensors, D=64, block 64) against the fp64 oracle on the UNROUNDED inputs,
    at the tolerance of the parity statement: fp32 inputs are computed with fp16 operands (the 10-bit fraction of
    the tf32 arithmetic the reference uses on them) and fp32 accumulation, and come back as fp32."""
    import kvax_b200 as kv
    assert kv.get_fp32_operand_dtype() == "auto"
    rows, o, dq, dk, dv = _tiny_fp32_run()
    compare("out", *o, rows)
    compare("dq", *dq, rows)
    compare("dk", *dk, rows)
    compare("dv", *dv, rows)


def test_fp32_inputs_bf16_operands():
    """The same with bf16 operands (what inputs beyond the fp16 range get): the inputs themselves are rounded to
    8 bits, hence a wider budget than the parity statement's."""
    import kvax_b200 as kv
    kv.set_fp32_operand_dtype("bfloat16")
    try:
        rows, o, dq, dk, dv = _tiny_fp32_run()
    finally:
        kv.set_fp32_operand_dtype("auto")
    compare("out", *o, rows, max_abs=3e-2, rel_l2=1e-2)
    compare("dq", *dq, rows, max_abs=5e-2, rel_l2=1.5e-2)
    compare("dk", *dk, rows, max_abs=5e-2, rel_l2=1.5e-2)
    compare("dv", *dv, rows, max_abs=5e-2, rel_l2=1.5e-2)


def test_fp32_inputs_small_output_gradient():
    """An output gradient of the size a mean-reduced loss produces (1e-7): it is scaled by a power of two on its way
    into fp16 and the input gradients are scaled back, so nothing underflows."""
    import kvax_b200 as kv
    cfg = gen.small_config(seq=512, batch=1, hq=4, hkv=2, head_dim=64)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=5))
    q, k, v = (torch.from_numpy(inp[n]).cuda().requires_grad_(True) for n in ("q", "k", "v"))
    do = torch.from_numpy(inp["dout"]).cuda() * 1e-7
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, 1))
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        masks = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
        out.backward(do)
    pp, ss = inp["positions"], inp["segment_ids"]
    rq, rk, rv = ao.attention_backward(inp["q"], inp["k"], inp["v"], pp, ss, pp, ss, inp["scale"], inp["dout"])
    rows = (ss != -1)[:, :, None, None]
    compare("dq * 1e7", q.grad.cpu().numpy() * 1e7, rq, rows)
    compare("dk * 1e7", k.grad.cpu().numpy() * 1e7, rk, rows)
    compare("dv * 1e7", v.grad.cpu().numpy() * 1e7, rv, rows)


@pytest.mark.parametrize("mode", ["fused", "two_kernel"])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_fp16_tensors(head_dim, mode):
    """fp16 tensors run on fp16 operands (the reference's tl.dot on fp16 tiles), not through bf16: compared with the
    oracle on the fp16-rounded inputs at the tolerance of the parity statement; outputs are fp16."""
    from kvax_b200.ops.flash_attention import attention_backward, attention_forward, check_status
    from kvax_b200.ops.mask_creator import build_masks
    cfg = gen.small_config(seq=1024, hq=4, hkv=2, head_dim=head_dim)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=13))
    h = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.float16)
    q, k, v, do = (h(inp[n]).cuda() for n in ("q", "k", "v", "dout"))
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    masks = build_masks(p, s, p, s, [(128, 128, False), (128, 128, False), (128, 128, True)], True)
    out, lse, st = attention_forward(q, k, v, p, s, p, s, masks[0], (128, 128), inp["scale"])
    dq, dk, dv, st2 = attention_backward(q, k, v, out, do, lse, p, s, p, s, masks[1], masks[2], (128, 128), inp["scale"], mode=mode)
    torch.cuda.synchronize()
    check_status(st, "attn_fwd")
    check_status(st2, "attn_bwd")
    assert out.dtype == torch.float16 and dq.dtype == torch.float16
    r = lambda n: h(inp[n]).float().numpy()
    pp, ss = inp["positions"], inp["segment_ids"]
    ref_o, _ = ao.attention_forward(r("q"), r("k"), r("v"), pp, ss, pp, ss, inp["scale"], dtype=np.float64)
    rq, rk, rv = ao.attention_backward(r("q"), r("k"), r("v"), pp, ss, pp, ss, inp["scale"], r("dout"), dtype=np.float64)
    rows = (ss != -1)[:, :, None, None]
    compare("out", out.float().cpu().numpy(), ref_o, rows)
    compare("dq", dq.float().cpu().numpy(), rq, rows)
    compare("dk", dk.cpu().numpy(), rk, rows)
    compare("dv", dv.cpu().numpy(), rv, rows)


@pytest.mark.parametrize("head_dim", [16, 32])
def test_small_head_dims_public_api(head_dim):
    """head_dim 16 and 32 (accepted by the reference, flash_attention_triton.py:1397-1403) run
    on zero-padded operands through the head_dim-64 kernels."""
    import kvax_b200 as kv
    cfg = gen.small_config(seq=512, batch=1, hq=4, hkv=2, head_dim=head_dim)
    inp = _zero_pad_dout(gen.make_inputs(cfg, seed=31))
    q, k, v, do = (to_bf16_cuda(inp[n]) for n in ("q", "k", "v", "dout"))
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, 1), rank=0)
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
        masks = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
        assert out.shape == q.shape
        out.backward(do)
    rq, rk, rv = _oracle_grads(inp)
    rows = (inp["segment_ids"] != -1)[:, :, None, None]
    compare("dq", q.grad.float().cpu().numpy(), rq, rows, bf16_output=True)
    compare("dk", k.grad.float().cpu().numpy(), rk, rows, bf16_output=True)
    compare("dv", v.grad.float().cpu().numpy(), rv, rows, bf16_output=True)


@pytest.mark.parametrize("dqk,dv", [(64, 128), (128, 64), (32, 64), (128, 16)])
def test_different_qk_and_value_head_dims_public_api(dqk, dv):
    """Dqk != Dv (the reference's kernels take separate qk_head_dim / value_head_dim,
    flash_attention_triton.py:173-176): the narrower side is zero-padded to the kernels' head_dim."""
    import kvax_b200 as kv
    cfg = gen.small_config(seq=768, batch=1, hq=4, hkv=2, head_dim=dqk)
    inp = dict(gen.make_inputs(cfg, seed=37))
    rng = np.random.default_rng(41)
    inp["v"] = rng.standard_normal(inp["v"].shape[:3] + (dv,)).astype(np.float32)
    inp["dout"] = rng.standard_normal(inp["q"].shape[:3] + (dv,)).astype(np.float32)
    inp = _zero_pad_dout(inp)
    q, k, v, do = (to_bf16_cuda(inp[n]) for n in ("q", "k", "v", "dout"))
    p, s = i32_cuda(inp["positions"]), i32_cuda(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, 1), rank=0)
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
        masks = kv.create_attention_mask(p, s, p, s, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
        assert out.shape == q.shape[:3] + (dv,)
        out.backward(do)
    assert q.grad.shape == q.shape and k.grad.shape == k.shape and v.grad.shape == v.shape
    pp, ss = inp["positions"], inp["segment_ids"]
    ref_o, _ = ao.attention_forward(bf16_round(inp["q"]), bf16_round(inp["k"]), bf16_round(inp["v"]), pp, ss, pp, ss, inp["scale"],
                                    dtype=np.float32)
    rq, rk, rv = _oracle_grads(inp)
    rows = (ss != -1)[:, :, None, None]
    compare("out", out.detach().float().cpu().numpy(), ref_o, rows, bf16_output=True)
    compare("dq", q.grad.float().cpu().numpy(), rq, rows, bf16_output=True)
    compare("dk", k.grad.float().cpu().numpy(), rk, rows, bf16_output=True)
    compare("dv", v.grad.float().cpu().numpy(), rv, rows, bf16_output=True)


def test_wide_head_dims_are_rejected_loudly():
    """head_dim 192 / 256 are in the reference's list but have no sm_100a kernel here: a clear error, no fallback."""
    import kvax_b200 as kv
    from kvax_b200._lib import KvaxB200Error
    q = torch.zeros(1, 128, 2, 192, dtype=torch.bfloat16, device="cuda")
    p = torch.arange(128, dtype=torch.int32, device="cuda")[None]
    s = torch.zeros(1, 128, dtype=torch.int32, device="cuda")
    mesh = kv.Mesh(("data", "context"), (1, 1), rank=0)
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        masks = kv.create_attention_mask(p, s, p, s)
        with pytest.raises(KvaxB200Error, match="head dims up to 128"):
            kv.flash_attention(q, q, q, p, s, p, s, masks)
