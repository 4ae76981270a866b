"""Benchmark of the attention hot path: block-mask build + flash attention forward + backward.

    python bench.py --gpus 1 --steps 20 --warmup 3                 # this implementation
    python bench.py --impl reference --steps 2 --warmup 1          # CPU reference arm
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N   # context parallel

One step = create the three block masks, forward, backward on one batch of synthetic
input.  N = 1 runs the 32k document-mask GQA configuration; N > 1 runs the 128k
context-parallel configuration with CP = N (total work fixed: strong scaling).  Rank 0
prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from kvax_b200.utils import synthetic as gen  # seeded synthetic inputs (pure NumPy)

METRIC = "attn TFLOP/s (unmasked FLOPs) fwd+bwd, doc-mask GQA"
UNIT = "TFLOP/s"
TILE = 128


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"),
                    hbm_gbs=d["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


def profile_traffic(kernel: str, workload: str):
    """DRAM bytes per launch of `kernel` on `workload` as recorded by the committed ncu summary
    (profiles/*.txt: a line `traffic_bytes_per_launch <kernel> <workload> <bytes>`); (None, reason)
    when no capture of that pair has been summarised."""
    pdir = os.path.join(ROOT, "profiles")
    if os.path.isdir(pdir):
        for fn in sorted(os.listdir(pdir)):
            if not fn.endswith((".txt", ".md")):
                continue
            with open(os.path.join(pdir, fn)) as f:
                for line in f:
                    parts = line.split()
                    if len(parts) >= 4 and parts[0] == "traffic_bytes_per_launch" and parts[1] == kernel and parts[2] == workload:
                        return float(parts[3]), f"profiles/{fn}"
    return None, f"no ncu capture of {kernel} on {workload} summarised under profiles/"


def tile_hits(q_pos, q_seg, kv_pos, kv_seg):
    """Boolean (B, n_q_tiles, n_kv_tiles): tile pairs with at least one unmasked element of
    segment AND causal AND non-PAD -- the work the throughput is normalised by.  Exact: a pair holds an
    allowed element iff for some segment id the largest query position of that segment inside the query
    tile reaches the smallest kv position of that segment inside the kv tile.  Pure NumPy on host arrays."""
    B, Sq = q_pos.shape
    Skv = kv_pos.shape[1]
    nq, nk = (Sq + TILE - 1) // TILE, (Skv + TILE - 1) // TILE
    hits = np.zeros((B, nq, nk), dtype=bool)

    def per_tile_segment(pos, seg, reducer, fill):
        """(tile index, segment id, reduced position) for every (tile, segment) pair that occurs; PAD left out."""
        idx = np.nonzero(seg != -1)[0]
        tile = idx // TILE
        key = tile.astype(np.int64) * (1 << 32) + seg[idx].astype(np.int64)
        uniq, inv = np.unique(key, return_inverse=True)
        red = np.full(len(uniq), fill, dtype=np.int64)
        reducer.at(red, inv, pos[idx].astype(np.int64))
        return (uniq >> 32).astype(np.int64), (uniq & 0xffffffff).astype(np.int64), red

    for b in range(B):
        qt, qs, qmax = per_tile_segment(q_pos[b], q_seg[b], np.maximum, np.iinfo(np.int64).min)
        kt, ks, kmin = per_tile_segment(kv_pos[b], kv_seg[b], np.minimum, np.iinfo(np.int64).max)
        for s in np.intersect1d(qs, ks):
            qi, ki = np.nonzero(qs == s)[0], np.nonzero(ks == s)[0]
            hits[b][np.ix_(qt[qi], kt[ki])] |= qmax[qi][:, None] >= kmin[ki][None, :]
    return hits


def tight_tiles(pos, seg):
    """Number of unmasked tile pairs of a self-attention layout (see `tile_hits`)."""
    return int(tile_hits(pos, seg, pos, seg).sum())


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 20):
        self.gpu = gpu_index
        self.period_ms = int(period_ms)
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms), "-i", str(self.gpu)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2])); pw.append(float(parts[3]))
                except ValueError:
                    continue
                for nm, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
        os.unlink(self.path)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm), power_w_median=statistics.median(pw) if pw else None,
                    power_w_max=max(pw) if pw else None)


def cuda_time(fn, iters):
    """Average milliseconds of `fn` over `iters` back-to-back calls (CUDA events on the
    current stream, synchronised on both sides)."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


# --------------------------------------------------------------------------------------
# CPU reference arm / cpu_baseline
# --------------------------------------------------------------------------------------
def cpu_dense_sample(cfg, inp, seconds_target=12.0):
    """Dense masked attention forward + backward with torch CPU ops on all host cores
    (the port of the reference's dense path, oracle/attention_oracle.py) on a bounded
    sample of the workload: the first `n_tok` tokens of batch row 0, one GQA group.
    Returns (TFLOP/s on unmasked-tile FLOPs, description, seconds per pass)."""
    from oracle import attention_oracle as ao
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_tok = min(cfg.seq, 4096)
    g = cfg.hq // cfg.hkv
    pos, seg = inp["positions"][:1, :n_tok], inp["segment_ids"][:1, :n_tok]
    rng = np.random.default_rng(1)
    q = rng.standard_normal((1, n_tok, g, cfg.head_dim), dtype=np.float32)
    k = rng.standard_normal((1, n_tok, 1, cfg.head_dim), dtype=np.float32)
    v = rng.standard_normal((1, n_tok, 1, cfg.head_dim), dtype=np.float32)
    do = rng.standard_normal((1, n_tok, g, cfg.head_dim), dtype=np.float32)
    flops = 3.5 * gen.attention_flops(tight_tiles(pos, seg), g, cfg.head_dim, cfg.head_dim)

    def one():
        t = time.perf_counter()
        ao.attention_fwd_bwd_torch(q, k, v, pos, seg, pos, seg, inp["scale"], do)
        return time.perf_counter() - t

    one()
    t1 = one()
    reps = max(1, min(20, int(seconds_target / max(t1, 1e-3))))
    ts = [one() for _ in range(reps)]
    sec = statistics.median(ts)
    sample = f"first {n_tok} tokens of batch row 0, {g} query heads / 1 kv head, fp32, median of {reps}"
    return flops / sec / 1e12, sample, sec, cores


def mask_builder_numbers(q_pos, q_seg, kv_pos, kv_seg, dev, peaks, public_call_ms=None):
    """The block-mask builder on the step's own arrays and on two larger synthetic layouts.
    `at_workload_us`: the public call (host work + launch); `at_workload_kernel_us`: the kernel alone through a
    prepared call.  The benchmark configurations are <= 2 MiB of input, i.e. latency bound, so bandwidth is
    measured on (B 2048, S 4096) and (B 64, S 131072): documents of 1000 tokens, 128-token blocks, three masks;
    algorithmic bytes = 16 B S (four int32 inputs read once) + 48 B S / 128 (twelve int32 outputs)."""
    from kvax_b200.ops.mask_creator import MaskPlan
    spec3 = [(TILE, TILE, False), (TILE, TILE, False), (TILE, TILE, True)]
    plan = MaskPlan(q_pos, q_seg, kv_pos, kv_seg, spec3, True)
    plan.launch()
    info = {"at_workload_us": None if public_call_ms is None else public_call_ms * 1e3,
            "at_workload_kernel_us": cuda_time(plan.launch, 50) * 1e3}
    for (mb, ms_) in ((2048, 4096), (64, 131072)):
        mp = (torch.arange(ms_, device=dev, dtype=torch.int32) % 1000).repeat(mb, 1)
        msg = (torch.arange(ms_, device=dev, dtype=torch.int32) // 1000).repeat(mb, 1)
        # separate query-side and kv-side arrays, so that the four inputs the byte count names are four distinct reads
        plan = MaskPlan(mp, msg, mp.clone(), msg.clone(), spec3, True)
        plan.launch()
        t_ms = cuda_time(plan.launch, 20)
        alg = 16.0 * mb * ms_ + 48.0 * mb * ms_ / TILE
        info[f"B{mb}_S{ms_}"] = {"ms": t_ms, "algorithmic_GBps": alg / (t_ms * 1e-3) / 1e9,
                                 "frac_of_hbm": alg / (t_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        del mp, msg, plan
    return info


def run_mask_only(args):
    """`--mask-only`: just the mask builder numbers of `mask_builder_numbers` on the single-GPU workload
    (72 launches of the builder before the two of the largest layout: a fixed point for a profiler)."""
    name = args.workload or "c4_docmask_32k"
    inp = gen.make_inputs(gen.CONFIGS[name], seed=0, with_tensors=False)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pos, seg = torch.from_numpy(inp["positions"]).to(dev), torch.from_numpy(inp["segment_ids"]).to(dev)
    info = mask_builder_numbers(pos, seg, pos, seg, dev, measured_peaks())
    print(json.dumps({"metric": "block-mask builder", "config": {"workload": name}, "mask_builder": info}), flush=True)


def same_gpu_reference(q, k, v, do, pos, seg, scale, flops_fwd):
    """Times kvax's unmodified Triton kernels (host functions included) on this GPU on the step's own
    tensors: oracle/triton_reference.py, H100 launch setting of the reference (forward 128 x 128,
    backward 64 x 128 tiles, 8 warps, 3 stages or fewer if shared memory does not suffice).  Returns
    the dict for the JSON line, or {"unavailable": reason}."""
    try:
        from oracle import triton_reference as tr
        ok, why = tr.available()
        if not ok:
            return {"unavailable": why}
        from kvax_b200.ops.mask_creator import build_masks
        fwd, bwd = (128, 128), (64, 128)
        masks = tr.mask_tuple(build_masks(pos, seg, pos, seg, [(fwd[0], fwd[1], False), (bwd[1], bwd[0], False),
                                                                (bwd[0], bwd[1], True)], True))
        q_t, k_t, v_t, do_t = (tr.to_bhsd(x) for x in (q, k, v, do))
        last = None
        for stages in (3, 2, 1):
            try:
                fp, bp = tr.params(*fwd, num_warps=8, num_stages=stages), tr.params(*bwd, num_warps=8, num_stages=stages)
                out_t, res = tr.launch_forward(q_t, k_t, v_t, pos, seg, pos, seg, masks, scale, fp, bp)
                tr.launch_backward(res, do_t, scale, fp, bp)
                torch.cuda.synchronize()
                break
            except Exception as e:
                if "out of resource" not in str(e).lower() and "shared memory" not in str(e).lower():
                    raise
                last = e
        else:
            return {"unavailable": f"Triton could not fit the reference's tiles: {last}"}
        holder = {}

        def f():
            holder["res"] = tr.launch_forward(q_t, k_t, v_t, pos, seg, pos, seg, masks, scale, fp, bp)[1]

        fwd_ms = cuda_time(f, 3)
        bwd_ms = cuda_time(lambda: tr.launch_backward(holder["res"], do_t, scale, fp, bp), 3)
        return {"fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "ms_per_step": fwd_ms + bwd_ms, "unit": UNIT,
                "value": 3.5 * flops_fwd / ((fwd_ms + bwd_ms) * 1e-3) / 1e12,
                "fwd_tflops": flops_fwd / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": 2.5 * flops_fwd / (bwd_ms * 1e-3) / 1e12,
                "what": "kvax flash_attention_triton_forward + flash_attention_backward (host code + Triton kernels), "
                        f"fwd tiles {fwd}, bwd tiles {bwd}, 8 warps, {stages} stages, Triton of this image; block masks prebuilt; "
                        "same tensors, same FLOP count as `value`"}
    except Exception as e:          # the comparator must never take the benchmark down
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = gen.CONFIGS["c4_docmask_32k" if args.gpus == 1 else "c5_cp_128k"]
    inp = gen.make_inputs(cfg, seed=0, with_tensors=False)
    for _ in range(args.warmup):
        cpu_dense_sample(cfg, inp, seconds_target=1.0)
    vals, secs = [], []
    for _ in range(args.steps):
        v, sample, sec, cores = cpu_dense_sample(cfg, inp, seconds_target=4.0)
        vals.append(v); secs.append(sec)
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.median(secs) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name, "note": "dense masked attention on host cores, bounded sample per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# this implementation
# --------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--no-single-gpu-reference", action="store_true",
                    help="with --gpus N > 1: skip the one-GPU run of the same workload on rank 0")
    ap.add_argument("--cp-mode", default="auto", choices=("auto", "all_gather", "head_exchange"),
                    help="context-parallel schedule for --gpus N > 1")
    ap.add_argument("--cp-overlap", action="store_true",
                    help="all-gather schedule: run its collectives under the kernels (own keys first)")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="kvax_b200", choices=["kvax_b200", "reference"])
    ap.add_argument("--workload", default=None, help="override the configuration (c2_llama8b_8k, c3_dense_causal_16k, ...)")
    ap.add_argument("--mask-only", action="store_true", help="only measure the block-mask builder (one GPU)")
    ap.add_argument("--no-other-schedule", action="store_true",
                    help="with --gpus N > 1: do not also time the all-gather schedule")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-same-gpu-reference", action="store_true",
                    help="skip timing the reference's own Triton kernels on this GPU (single-GPU runs)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--positions", default="restart", choices=("restart", "arange"),
                    help="positions restart at 0 in every document (the benchmark configurations) or are a global arange "
                         "(the reference's own convention, for which its block bounds are tight)")
    ap.add_argument("--clock-sample-ms", type=int, default=20, help="period of the nvidia-smi clock samples during the timed region")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.mask_only:
        return run_mask_only(args)

    import kvax_b200 as kv
    from kvax_b200.ops.flash_attention import attention_backward, attention_forward, check_status
    from kvax_b200.ops.mask_creator import build_masks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cp = world
    if cp > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    name = args.workload or ("c4_docmask_32k" if cp == 1 else "c5_cp_128k")
    cfg = gen.CONFIGS[name]
    params = kv.FlashAttentionParamsConfig(TILE, TILE)
    W = max(args.warmup, 3)
    K = args.steps

    # ---- synthetic inputs (layout and masks on the host, tensors on the device) -------
    inp = gen.make_inputs(cfg, seed=0, with_tensors=False, restart_positions=(args.positions == "restart"))
    pos_h, seg_h = inp["positions"], inp["segment_ids"]
    scale = inp["scale"]
    B, S, Hq, Hkv, D = cfg.batch, cfg.seq, cfg.hq, cfg.hkv, cfg.head_dim
    n_tiles = tight_tiles(pos_h, seg_h) if rank == 0 else 0
    flops_fwd = gen.attention_flops(n_tiles, Hq, D, D)
    flops_step = 3.5 * flops_fwd

    kv.set_context_parallel_mode(args.cp_mode)
    kv.set_context_parallel_overlap(args.cp_overlap)
    hx = cp > 1 and Hkv % cp == 0 and args.cp_mode != "all_gather"

    # ---- N > 1: every rank draws the SAME full tensors (seeded), runs the whole workload alone on its own GPU -- the
    # one-GPU time of this workload, which the N = 1 line of a scaling series (the 32k configuration) does not give,
    # and the reference values of the numeric check -- and then keeps its slice of the permuted sequence.
    same_1gpu, single = None, None
    mesh = kv.Mesh(("data", "context"), (1, cp))
    q_spec = ("data", "context" if cp > 1 else None, None, None)
    kv_spec = ("data", None, None, None)
    S_loc = S // cp
    kv_pos = torch.from_numpy(pos_h).to(dev); kv_seg = torch.from_numpy(seg_h).to(dev)
    g = torch.Generator(device=dev).manual_seed(1234)

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)

    per_rank_tiles = None
    if cp > 1:
        qf, kf, vf, dof = randn(B, S, Hq, D), randn(B, S, Hkv, D), randn(B, S, Hkv, D), randn(B, S, Hq, D)
        if not args.no_single_gpu_reference:
            spec3 = [(TILE, TILE, False), (TILE, TILE, False), (TILE, TILE, True)]

            def one_gpu_step():
                m = build_masks(kv_pos, kv_seg, kv_pos, kv_seg, spec3, True)
                o1, l1, _ = attention_forward(qf, kf, vf, kv_pos, kv_seg, kv_pos, kv_seg, m[0], (TILE, TILE), scale)
                g1 = attention_backward(qf, kf, vf, o1, dof, l1, kv_pos, kv_seg, kv_pos, kv_seg, m[1], m[2], (TILE, TILE), scale)
                return o1, g1[0], g1[1], g1[2]

            for _ in range(2):
                one_gpu_step()
            ms1 = cuda_time(one_gpu_step, 3)
            t1 = torch.tensor([ms1], device=dev)
            dist.all_reduce(t1, op=dist.ReduceOp.MAX)
            ms1 = float(t1.item())
            same_1gpu = {"workload": cfg.name, "n_gpus": 1, "ms_per_step": ms1, "value": flops_step / (ms1 * 1e-3) / 1e12,
                         "unit": UNIT, "steps": 3, "note": "every rank alone on its own GPU, max over ranks"}
            single = one_gpu_step()
        with mesh, kv.attention_specs(q_spec, kv_spec):
            sl = slice(rank * S_loc, (rank + 1) * S_loc)
            take = lambda x: kv.permute_tokens_context_parallelism(x)[:, sl].contiguous()
            q, k, v, do = take(qf), take(kf), take(vf), take(dof)
            q_pos, q_seg = take(kv_pos), take(kv_seg)
            if single is not None:      # slices of the one-GPU results this rank must reproduce
                single = tuple(take(x) for x in single)
        del qf, kf, vf, dof
        torch.cuda.empty_cache()
        if rank == 0:                    # unmasked tile pairs of every rank's local queries against all keys (all-gather schedule)
            perm = np.concatenate([np.arange(c * (S // (2 * cp)), (c + 1) * (S // (2 * cp)))
                                   for c in sum(([i, 2 * cp - 1 - i] for i in range(cp)), [])])
            hits = tile_hits(pos_h[:, perm], seg_h[:, perm], pos_h, seg_h)
            per_q_tile = hits.sum(axis=(0, 2))
            tiles_loc = S_loc // TILE
            per_rank_tiles = [int(per_q_tile[r * tiles_loc:(r + 1) * tiles_loc].sum()) for r in range(cp)]
    else:
        q = randn(B, S_loc, Hq, D); k = randn(B, S_loc, Hkv, D); v = randn(B, S_loc, Hkv, D); do = randn(B, S_loc, Hq, D)
        q_pos, q_seg = kv_pos, kv_seg
    with mesh, kv.attention_specs(q_spec, kv_spec):
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

        def step():
            masks = kv.create_attention_mask(q_pos, q_seg, kv_pos, kv_seg, fwd_params=params, bwd_params=params,
                                             calc_bwd_mask=True)
            out = kv.flash_attention(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, scale=scale,
                                     fwd_params=params, bwd_params=params)
            out.backward(do)
            q.grad = None; k.grad = None; v.grad = None
            return out

        for _ in range(W):
            step()
        torch.cuda.synchronize()
        if cp > 1:
            dist.barrier()
        sampler = ClockSampler(local_rank, args.clock_sample_ms)
        if rank == 0:
            sampler.start()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        torch.cuda.synchronize()
        if cp > 1:
            dist.barrier()
        ms_total = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None
        if cp > 1:
            t = torch.tensor([ms_total], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_total = float(t.item())
        ms_step = ms_total / K

        # ---- N > 1: numeric check against the one-GPU run of the same tensors, and the other schedule ---------------
        cp_check, other_schedule, cp_phases = None, None, None
        if cp > 1:
            def run_once():
                for t_ in (q, k, v):
                    t_.grad = None
                masks_ = kv.create_attention_mask(q_pos, q_seg, kv_pos, kv_seg, fwd_params=params, bwd_params=params,
                                                  calc_bwd_mask=True)
                o_ = kv.flash_attention(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks_, scale=scale, fwd_params=params,
                                        bwd_params=params)
                o_.backward(do)
                return o_.detach(), q.grad, k.grad, v.grad

            def check(results):
                rows = (q_seg != -1)[:, :, None, None]
                errs, refs = [], []
                for got, ref in zip(results, single):
                    g_ = torch.where(rows, got.float(), torch.zeros((), device=dev))
                    r_ = torch.where(rows, ref.float(), torch.zeros((), device=dev))
                    errs.append((g_ - r_).abs().max())
                    refs.append(r_.abs().max())
                e_ = torch.stack(errs + refs)
                dist.all_reduce(e_, op=dist.ReduceOp.MAX)
                e_ = [float(x) for x in e_]
                names = ("out", "dq", "dk", "dv")
                return {"max_abs": dict(zip(names, e_[:4])), "ref_max": dict(zip(names, e_[4:])),
                        "against": "the one-GPU run of the same seeded tensors, each rank its own slice, max over ranks, non-PAD rows"}

            if single is not None:
                cp_check = {("head_exchange" if hx else "all_gather"): check(run_once())}
            # where a step's time goes on every rank (CUDA events around the phases of the public call)
            import importlib
            fa_mod = importlib.import_module("kvax_b200.ops.flash_attention")   # the module, not the function of that name
            fa_mod.enable_phase_timing(True)
            for _ in range(2):
                step()
            cp_phases = {k_: v_ / 2 for k_, v_ in fa_mod.phase_times_ms().items()}
            fa_mod.enable_phase_timing(False)
            all_phases = [None] * cp
            dist.all_gather_object(all_phases, cp_phases)
            cp_phases = {k_: [round(p_.get(k_, 0.0), 3) for p_ in all_phases] for k_ in cp_phases}   # one value per rank
            if hx and not args.no_other_schedule:     # the schedule the reference has: K/V all-gather, dK/dV reduce-scatter
                kv.set_context_parallel_mode("all_gather")
                for _ in range(2):
                    run_once()
                if single is not None:
                    cp_check["all_gather"] = check(run_once())
                ms_ag = cuda_time(step, 3)
                t = torch.tensor([ms_ag], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_ag = float(t.item())
                other_schedule = {"parallelism": f"cp{cp}:all_gather", "ms_per_step": ms_ag, "steps": 3,
                                  "value": flops_step / (ms_ag * 1e-3) / 1e12, "unit": UNIT}
                # the same schedule with its collectives under the kernels: own keys first, gathered keys second
                kv.set_context_parallel_overlap(True)
                for _ in range(2):
                    run_once()
                if single is not None:
                    cp_check["all_gather_overlapped"] = check(run_once())
                ms_ov = cuda_time(step, 3)
                t = torch.tensor([ms_ov], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_ov = float(t.item())
                other_schedule["overlapped"] = {"ms_per_step": ms_ov, "steps": 3, "value": flops_step / (ms_ov * 1e-3) / 1e12,
                                                "unit": UNIT}
                kv.set_context_parallel_overlap(args.cp_overlap)
                kv.set_context_parallel_mode(args.cp_mode)
            single = None
            torch.cuda.empty_cache()

        # ---- per-kernel timing for the roofline (single GPU leg only) ------------------
        roofline, parts = None, {}
        peaks = measured_peaks()
        if cp == 1:
            masks = kv.create_attention_mask(q_pos, q_seg, kv_pos, kv_seg, fwd_params=params, bwd_params=params, calc_bwd_mask=True)
            # what the reference's kernels visit: the sum of (upper - lower) over the forward mask, in tile pairs
            reference_visited = int((masks[0].upper_bounds - masks[0].lower_bounds).clamp_min(0).sum().item())
            qd, kd, vd = q.detach(), k.detach(), v.detach()
            out, lse, st, ws_f = attention_forward(qd, kd, vd, q_pos, q_seg, kv_pos, kv_seg, masks[0], (TILE, TILE), scale, stages=3)
            dq, dk, dv, st2, ws_b = attention_backward(qd, kd, vd, out, do, lse, q_pos, q_seg, kv_pos, kv_seg, masks[1], masks[2],
                                                       (TILE, TILE), scale, stages=63)
            torch.cuda.synchronize()
            check_status(st, "attn_fwd"); check_status(st2, "attn_bwd")
            it = max(5, K)
            parts["mask_build_ms"] = cuda_time(lambda: kv.create_attention_mask(q_pos, q_seg, kv_pos, kv_seg, fwd_params=params,
                                                                                bwd_params=params, calc_bwd_mask=True), it)
            parts["fwd_kernel_ms"] = cuda_time(lambda: attention_forward(qd, kd, vd, q_pos, q_seg, kv_pos, kv_seg, masks[0], (TILE, TILE),
                                                                         scale, workspace=ws_f, stages=2, out=out, lse=lse), it)
            bw = lambda stg, ws, mode: cuda_time(lambda: attention_backward(
                qd, kd, vd, out, do, lse, q_pos, q_seg, kv_pos, kv_seg, masks[1], masks[2], (TILE, TILE), scale,
                workspace=ws, stages=stg, grads=(dq, dk, dv), mode=mode), it)
            parts["tile_lists_ms"] = bw(1, ws_b, "fused")
            parts["delta_and_zero_fill_ms"] = bw(2, ws_b, "fused")
            parts["fused_bwd_kernel_ms"] = bw(16, ws_b, "fused")
            parts["dq_cast_ms"] = bw(32, ws_b, "fused")
            # the bit-reproducible two-kernel backward, for comparison (not part of the timed step)
            ws_t = torch.empty_like(ws_b)
            attention_backward(qd, kd, vd, out, do, lse, q_pos, q_seg, kv_pos, kv_seg, masks[1], masks[2], (TILE, TILE), scale,
                               workspace=ws_t, stages=15, grads=(dq, dk, dv), mode="two_kernel")
            parts["two_kernel_dq_ms"] = bw(4, ws_t, "two_kernel")
            parts["two_kernel_dkdv_ms"] = bw(8, ws_t, "two_kernel")
            del ws_t
            # The fused backward kernel is the dominant launch: all five products the backward needs per tile pair
            # (S, dP, dV, dK, dQ = 2.5 x forward).
            bwd_flops = 2.5 * flops_fwd
            ach = bwd_flops / (parts["fused_bwd_kernel_ms"] * 1e-3) / 1e12
            traffic, traffic_note = profile_traffic("attn_bwd_fused_kernel", name)
            roofline = {"bound": "tensor", "kernel": "attn_bwd_fused_kernel<128> (dK, dV, dQ)", "achieved": ach,
                        "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                        "peak_source": peaks["source"] + " burst",
                        "traffic": traffic, "traffic_unit": "bytes per launch", "traffic_source": traffic_note,
                        "fwd_kernel_tflops": flops_fwd / (parts["fwd_kernel_ms"] * 1e-3) / 1e12,
                        "fwd_kernel_frac": flops_fwd / (parts["fwd_kernel_ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"],
                        # MMA work the step executes = the work that counts: 2 products forward + 5 backward
                        "executed_mma_tflops": 3.5 * flops_fwd / (ms_step * 1e-3) / 1e12,
                        "step_frac_of_burst": flops_step / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
                        "step_frac_of_sustained": flops_step / (ms_step * 1e-3) / 1e12 / (peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]),
                        "step_frac_of_nominal_2250": flops_step / (ms_step * 1e-3) / 1e12 / 2250.0}

        # ---- the reference's own Triton kernels on this GPU, same inputs (comparator; not part of the timed step)
        same_gpu_ref = None
        if cp == 1 and not args.no_same_gpu_reference:
            same_gpu_ref = same_gpu_reference(q.detach(), k.detach(), v.detach(), do, q_pos, q_seg, scale, flops_fwd)

        # ---- mask builder at a size where bandwidth is measurable (the benchmark
        #      configurations are <= 2 MiB, i.e. launch bound) -----------------------------
        mask_info = None
        if cp == 1:
            mask_info = mask_builder_numbers(q_pos, q_seg, kv_pos, kv_seg, dev, peaks, parts.get("mask_build_ms"))

        # ---- end to end: pinned host buffers in, results back out, every step ----------
        e2e = None
        if not args.no_e2e:
            # Throughput of the public call on HOST buffers: every step copies its inputs from pinned host memory
            # and copies O, dQ, dK, dV back to pinned host memory.  Steps are double-buffered over three streams
            # (H2D of step i+1 and D2H of step i-1 run while step i computes), as a host-side caller feeding batches
            # would do; all copies of all timed steps lie inside the timed region.
            host_in = [t.detach().cpu().pin_memory() for t in (q, k, v, do)]
            host_idx = [t.cpu().pin_memory() for t in (q_pos, q_seg, kv_pos, kv_seg)]
            dev_in = [[torch.empty_like(t, device=dev) for t in host_in] for _ in range(2)]
            dev_idx = [[torch.empty_like(t, device=dev) for t in host_idx] for _ in range(2)]
            host_out = [[torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for t in (q, q, k, v)] for _ in range(2)]   # out, dq, dk, dv
            h2d = sum(t.numel() * t.element_size() for t in host_in + host_idx)
            d2h = sum(t.numel() * t.element_size() for t in host_out[0])
            main = torch.cuda.current_stream(dev)
            s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            in_ready = [torch.cuda.Event() for _ in range(2)]
            in_free = [torch.cuda.Event() for _ in range(2)]
            out_free = [torch.cuda.Event() for _ in range(2)]

            def e2e_steps(n):
                for i in range(n):
                    bsel = i % 2
                    with torch.cuda.stream(s_in):
                        if i >= 2:
                            s_in.wait_event(in_free[bsel])
                        for d, h in zip(dev_in[bsel] + dev_idx[bsel], host_in + host_idx):
                            d.copy_(h, non_blocking=True)
                        in_ready[bsel].record(s_in)
                    main.wait_event(in_ready[bsel])
                    qq, kk, vv, dd = dev_in[bsel]
                    ix = dev_idx[bsel]
                    qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
                    m = kv.create_attention_mask(ix[0], ix[1], ix[2], ix[3], fwd_params=params, bwd_params=params,
                                                 calc_bwd_mask=True)
                    o = kv.flash_attention(qq, kk, vv, ix[0], ix[1], ix[2], ix[3], m, scale=scale,
                                           fwd_params=params, bwd_params=params)
                    o.backward(dd)
                    results = (o.detach(), qq.grad, kk.grad, vv.grad)
                    qq.grad = None; kk.grad = None; vv.grad = None
                    qq.requires_grad_(False); kk.requires_grad_(False); vv.requires_grad_(False)
                    in_free[bsel].record(main)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(in_free[bsel])          # recorded after the backward: results are complete
                        if i >= 2:
                            s_out.wait_event(out_free[bsel])
                        for h, d in zip(host_out[bsel], results):
                            d.record_stream(s_out)
                            h.copy_(d, non_blocking=True)
                        out_free[bsel].record(s_out)
                main.wait_stream(s_out)
                main.wait_stream(s_in)

            e2e_steps(2)
            torch.cuda.synchronize()
            if cp > 1:
                dist.barrier()
            n_e2e = max(4, min(K, 20))     # the pipeline's fill and drain (one copy each way) are inside the timed region
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(main)
            e2e_steps(n_e2e)
            e1.record(main)
            torch.cuda.synchronize()
            ms_e2e = e0.elapsed_time(e1) / n_e2e
            if cp > 1:
                t = torch.tensor([ms_e2e], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_e2e = float(t.item())
            e2e = {"value": flops_step / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": int(h2d) * cp, "d2h_bytes_per_step": int(d2h) * cp, "steps": n_e2e,
                   "pipeline": "double-buffered: H2D, compute and D2H on three streams"}

    if rank != 0:
        if cp > 1:
            dist.destroy_process_group()
        return

    value = flops_step / (ms_step * 1e-3) / 1e12
    # kernels of this library per step: mask builder (1), forward (tile summaries, lists, order, attention),
    # backward (tile summaries, lists, order, delta + zero fill, fused kernel, dQ cast); with context parallelism the
    # head exchange adds the rebuilt masks (1), two token un-permutations and eight exchange kernels (q, k, v, o, do,
    # dq, dk, dv), the all-gather schedule four token (un-)permutations
    kernels_per_step = 1 + 4 + 6 + (0 if cp == 1 else (11 if hx else 4))
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": cp, "steps": K, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name, "batch": B, "seq_len": S, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D,
                   "tile": TILE, "parallelism": f"cp{cp}" + ((":head_exchange" if hx else ":all_gather") if cp > 1 else ""), "unmasked_tile_pairs": n_tiles,
                   "flops_per_step": flops_step, "cache": "inputs larger than L2 (Q alone exceeds 126 MB)",
                   "positions": "restart at 0 in every document" if args.positions == "restart" else "global arange",
                   "step": "3 block masks + forward + backward"},
        "tokens_per_s": B * S / (ms_step * 1e-3),
        "clocks": clocks, "gpu_launches": kernels_per_step * K, "parts_ms": parts,
    }
    if cp == 1:
        line["config"]["tile_pairs_in_reference_bounds"] = reference_visited
        # the library's default choice of forward kernel for this shape (see kvax_b200_attn_fwd_params.flags)
        head_pairs = (Hq // Hkv) % 2 == 0 and (S // TILE) * B * (Hq // 2) >= 2 * 148
        line["config"]["forward_kernel"] = ("two heads of a kv group per CTA" if head_pairs or (S >= 16384 and (Hq // Hkv) % 2 == 0) else
                                            ("two query tiles per CTA" if S >= 16384 else "one query tile per CTA"))
    if roofline:
        line["roofline"] = roofline
    if cp == 1 and mask_info:
        line["mask_builder"] = mask_info
    if same_1gpu:
        line["same_workload_1gpu"] = same_1gpu
        line["same_workload_efficiency"] = same_1gpu["ms_per_step"] / (cp * ms_step)
    if cp > 1:
        line["cp_check"] = cp_check
        line["cp_phases_ms_per_rank"] = cp_phases
        if per_rank_tiles:
            mean = sum(per_rank_tiles) / len(per_rank_tiles)
            line["all_gather_tiles_per_rank"] = {"unmasked_tile_pairs": per_rank_tiles, "max_over_mean": max(per_rank_tiles) / mean,
                                                 "efficiency_cap": mean / max(per_rank_tiles)}
        if other_schedule:
            if same_1gpu:
                other_schedule["same_workload_efficiency"] = same_1gpu["ms_per_step"] / (cp * other_schedule["ms_per_step"])
            line["all_gather_schedule"] = other_schedule
    if cp == 1 and same_gpu_ref is not None:
        line["same_gpu_reference"] = same_gpu_ref
    if e2e:
        line["e2e"] = e2e
    if cp == 1 and not args.no_cpu_baseline:
        v_cpu, sample, sec, cores = cpu_dense_sample(cfg, inp)
        line["cpu_baseline"] = {"value": v_cpu, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if cp > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
