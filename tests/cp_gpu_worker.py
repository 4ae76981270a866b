"""Worker of tests/test_gpu_context_parallel.py: one process per GPU under torchrun.

Context-parallel flash attention (permute -> masks -> attention -> gradients; both
schedules: K/V all-gather with dK/dV reduce-scatter, and the head exchange by all-to-all,
over NCCL) against the same kernels run on the whole
sequence on one GPU — the reference's own multi-GPU test compares CP with a non-CP run of
the same kernels (tests/test_attention.py:520-828).  Masks per rank are also checked
against the CPU oracle (bit-exact)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import kvax_b200 as kv  # noqa: E402
from oracle import generators as gen  # noqa: E402
from oracle import mask_oracle as mo  # noqa: E402
from oracle import permutation_oracle as po  # noqa: E402


def run_case(rank, world, dev, seq, batch, hq, hkv, pad, sequential, permuted=True, mode="all_gather", overlap=False):
    kv.set_context_parallel_mode(mode)
    kv.set_context_parallel_overlap(overlap)
    cfg = gen.small_config(seq=seq, batch=batch, hq=hq, hkv=hkv, head_dim=128, doc_min=200, doc_max=seq // 2, pad=pad)
    inp = gen.make_inputs(cfg, seed=17, restart_positions=not sequential)
    inp["dout"] = np.where((inp["segment_ids"] != -1)[:, :, None, None], inp["dout"], 0.0).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    q, k, v, do = (t(inp[n]).to(torch.bfloat16) for n in ("q", "k", "v", "dout"))
    pos, seg = t(inp["positions"]), t(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    scale = inp["scale"]

    # ---- single-GPU run on the whole sequence
    m1 = kv.Mesh(("data", "context"), (1, 1), rank=0)
    with m1, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        qf, kf, vf = (x.clone().requires_grad_(True) for x in (q, k, v))
        masks = kv.create_attention_mask(pos, seg, pos, seg, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        of = kv.flash_attention(qf, kf, vf, pos, seg, pos, seg, masks, scale=scale, fwd_params=params, bwd_params=params,
                                assume_sequential_positions=sequential)
        of.backward(do)

    # ---- context-parallel run
    mesh = kv.Mesh(("data", "context"), (1, world))
    loc = seq // world
    sl = slice(rank * loc, (rank + 1) * loc)
    with mesh, kv.attention_specs(("data", "context", None, None), ("data", None, None, None)):
        if permuted:
            qp, kp, vp, dop, posp, segp = kv.permute_tokens_context_parallelism((q, k, v, do, pos, seg))
        else:
            qp, kp, vp, dop, posp, segp = q, k, v, do, pos, seg
        ql, kl, vl = (x[:, sl].contiguous().requires_grad_(True) for x in (qp, kp, vp))
        q_pos, q_seg = posp[:, sl].contiguous(), segp[:, sl].contiguous()
        masks = kv.create_attention_mask(q_pos, q_seg, pos, seg, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        ref_masks = mo.create_attention_mask(q_pos.cpu().numpy(), q_seg.cpu().numpy(), inp["positions"], inp["segment_ids"],
                                             (128, 128), (128, 128), calc_bwd_mask=True)
        for m, rm in zip(masks, ref_masks):
            for a, b in zip(m.flatten(), rm):
                np.testing.assert_array_equal(a.cpu().numpy(), b)
        ol = kv.flash_attention(ql, kl, vl, q_pos, q_seg, pos, seg, masks, scale=scale, fwd_params=params, bwd_params=params,
                                assume_sequential_positions=sequential, permute_tokens_for_load_balance=permuted)
        ol.backward(dop[:, sl].contiguous())
        pick = (lambda x: kv.permute_tokens_context_parallelism(x)[:, sl]) if permuted else (lambda x: x[:, sl])
        rows = (q_seg != -1)[:, :, None, None]
        worst = {}
        for name, got, ref in (("out", ol, pick(of.detach())), ("dq", ql.grad, pick(qf.grad)),
                               ("dk", kl.grad, pick(kf.grad)), ("dv", vl.grad, pick(vf.grad))):
            g = torch.where(rows, got.float(), torch.zeros((), device=dev))
            r = torch.where(rows, ref.float(), torch.zeros((), device=dev))
            err = (g - r).abs().max().item()
            rel = ((g - r).norm() / r.norm().clamp_min(1e-30)).item()
            worst[name] = (err, rel)
            # out and dq come from identical kernels on identical data: exact.  With the
            # all-gather schedule dk/dv are summed over ranks in fp32 in a different order before
            # the bf16 cast; with the head exchange they too are the single-GPU values.
            # (with fewer kv heads than ranks the head exchange also sums dk / dv over the ranks that share a kv head)
            exact = name in ("out", "dq") or (mode == "head_exchange" and hkv % world == 0)
            if kv.get_backward_mode() == "fused" and name != "out":
                # the fused backward sums dQ tiles with fp32 atomics, and on small problems dK / dV parts of several CTAs
                # too: equal to rounding, not bit for bit
                exact = False
            if overlap:
                # own and remote keys are separate kernel passes merged afterwards: equal to rounding
                exact = False
            if exact:
                assert err == 0.0, f"{name}: CP differs from single GPU (max {err})"
            else:
                assert rel < 4e-3 and err <= 2e-2 + r.abs().max().item() / 128, f"{name}: {err} {rel}"
    kv.set_context_parallel_overlap(False)
    return worst


def run_tp_case(rank, world, dev):
    """Tensor parallelism over heads (`("data", None, "model", None)` specs, README.md:273-278 of the
    reference), alone on 2 ranks or combined with context parallelism on a (context, model) mesh of
    4 ranks: every rank runs its head slice and must reproduce that slice of the single-GPU result."""
    tp = 2
    cp = world // tp
    seq, hq, hkv = 1024 * cp, 4 * tp, 2 * tp
    cfg = gen.small_config(seq=seq, batch=1, hq=hq, hkv=hkv, head_dim=128, doc_min=100, doc_max=seq // 2, pad=0.05)
    inp = gen.make_inputs(cfg, seed=29)
    inp["dout"] = np.where((inp["segment_ids"] != -1)[:, :, None, None], inp["dout"], 0.0).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    q, k, v, do = (t(inp[n]).to(torch.bfloat16) for n in ("q", "k", "v", "dout"))
    pos, seg = t(inp["positions"]), t(inp["segment_ids"])
    params = kv.FlashAttentionParamsConfig(128, 128)
    m1 = kv.Mesh(("data", "context"), (1, 1), rank=0)
    with m1, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        qf, kf, vf = (x.clone().requires_grad_(True) for x in (q, k, v))
        masks = kv.create_attention_mask(pos, seg, pos, seg, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
        of = kv.flash_attention(qf, kf, vf, pos, seg, pos, seg, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
        of.backward(do)
    mesh = kv.Mesh(("data", "context", "model"), (1, cp, tp))
    crank, mrank = mesh.coordinate("context"), mesh.coordinate("model")
    hs, ks = slice(mrank * hq // tp, (mrank + 1) * hq // tp), slice(mrank * hkv // tp, (mrank + 1) * hkv // tp)
    loc = seq // cp
    sl = slice(crank * loc, (crank + 1) * loc)
    q_axis = "context" if cp > 1 else None
    for mode in (("all_gather", "head_exchange") if cp > 1 else ("auto",)):
        kv.set_context_parallel_mode(mode)
        with mesh, kv.attention_specs(("data", q_axis, "model", None), ("data", None, "model", None)):
            if cp > 1:
                qp, kp, vp, dop, posp, segp = kv.permute_tokens_context_parallelism((q, k, v, do, pos, seg))
            else:
                qp, kp, vp, dop, posp, segp = q, k, v, do, pos, seg
            ql = qp[:, sl, hs].contiguous().requires_grad_(True)
            kl, vl = (x[:, sl, ks].contiguous().requires_grad_(True) for x in (kp, vp))
            q_pos, q_seg = posp[:, sl].contiguous(), segp[:, sl].contiguous()
            masks = kv.create_attention_mask(q_pos, q_seg, pos, seg, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
            ol = kv.flash_attention(ql, kl, vl, q_pos, q_seg, pos, seg, masks, scale=inp["scale"], fwd_params=params, bwd_params=params)
            ol.backward(dop[:, sl, hs].contiguous())
            pick = (lambda x: kv.permute_tokens_context_parallelism(x)[:, sl]) if cp > 1 else (lambda x: x[:, sl])
            rows = (q_seg != -1)[:, :, None, None]
            for name, got, ref in (("out", ol, pick(of.detach())[:, :, hs]), ("dq", ql.grad, pick(qf.grad)[:, :, hs]),
                                   ("dk", kl.grad, pick(kf.grad)[:, :, ks]), ("dv", vl.grad, pick(vf.grad)[:, :, ks])):
                gg = torch.where(rows, got.float(), torch.zeros((), device=dev))
                rr = torch.where(rows, ref.float(), torch.zeros((), device=dev))
                err = (gg - rr).abs().max().item()
                if name in ("out", "dq") or mode != "all_gather":
                    assert err == 0.0, f"tp {mode} {name}: differs from single GPU (max {err})"
                else:
                    assert err <= 2e-2 + rr.abs().max().item() / 128, f"tp {mode} {name}: {err}"
    kv.set_context_parallel_mode("auto")
    return True


def main():
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    res = {}
    # the default (fused) backward first, then everything on the bit-reproducible two-kernel backward
    res["fused_docmask"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=4, hkv=2, pad=0.05, sequential=False)
    res["fused_hx_docmask"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=2 * world, hkv=world, pad=0.05,
                                       sequential=False, mode="head_exchange")
    # the same exchange through grouped NCCL sends / receives instead of peer-memory stores
    kv.set_head_exchange_transport("nccl")
    res["fused_hx_docmask_nccl"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=2 * world, hkv=world, pad=0.05,
                                            sequential=False, mode="head_exchange")
    kv.set_head_exchange_transport("auto")
    # fewer kv heads than ranks: query heads exchanged, K / V gathered, dK / dV reduce-scattered over the sharing ranks
    res["fused_hx_shared_kv_head"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=2 * world, hkv=max(1, world // 2),
                                              pad=0.05, sequential=False, mode="head_exchange")
    # all-gather schedule with its collectives under the kernels (own keys first, then the gathered rest)
    res["fused_overlap_docmask"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=4, hkv=2, pad=0.05, sequential=False,
                                            overlap=True)
    res["fused_overlap_batch2_no_permute"] = run_case(rank, world, dev, seq=512 * world, batch=2, hq=2, hkv=1, pad=0.1,
                                                      sequential=False, permuted=False, overlap=True)
    from kvax_b200.ops import _peer
    res["peer_memory_transport"] = "used" if any(a for a in _peer._arenas.values()) else "not available: NCCL transport used"
    kv.set_backward_mode("two_kernel")
    res["docmask"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=4, hkv=2, pad=0.05, sequential=False)
    res["batch2_seqpos"] = run_case(rank, world, dev, seq=512 * world, batch=2, hq=2, hkv=2, pad=0.0, sequential=True)
    res["no_permute"] = run_case(rank, world, dev, seq=512 * world, batch=1, hq=2, hkv=1, pad=0.1, sequential=False, permuted=False)
    hx = "head_exchange"
    res["hx_docmask"] = run_case(rank, world, dev, seq=1024 * world, batch=1, hq=2 * world, hkv=world, pad=0.05, sequential=False, mode=hx)
    res["hx_batch2_seqpos"] = run_case(rank, world, dev, seq=512 * world, batch=2, hq=2 * world, hkv=2 * world, pad=0.0, sequential=True, mode=hx)
    res["hx_no_permute"] = run_case(rank, world, dev, seq=512 * world, batch=1, hq=world, hkv=world, pad=0.1, sequential=False, permuted=False, mode=hx)
    kv.set_context_parallel_mode("auto")
    res["tensor_parallel"] = run_tp_case(rank, world, dev)
    kv.set_backward_mode("fused")
    dist.barrier()
    if rank == 0:
        print("cp gpu worker ok", {k: ({n: (round(e, 5), round(r, 5)) for n, (e, r) in v.items()} if isinstance(v, dict) else v) for k, v in res.items()})
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
