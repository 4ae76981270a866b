"""Benchmark commands with the names and options of the reference's benchmarks.py (:34-407):

    python -m kvax_b200.benchmarks mha          [options]      forward, one GPU
    python -m kvax_b200.benchmarks mha_bwd      [options]      forward + backward, one GPU
    python -m torch.distributed.run --nproc-per-node N -m kvax_b200.benchmarks mha_cp      [options]
    python -m torch.distributed.run --nproc-per-node N -m kvax_b200.benchmarks mha_cp_bwd  [options]

Differences from the reference: one process per GPU (the context-parallel commands run
under torch.distributed.run and shard the sequence over all ranks), timing with CUDA events
instead of wall clock, no cuDNN comparator (`--check` compares with a dense torch attention
on the same GPU when the sequence is short enough to hold the score matrix).  The TFLOP/s
figure uses the reference's own accounting: the dense formula of kvax/utils/math.py:1-30
(non-causal FLOPs, divided by the number of GPUs) times `calculate_mask_sparsity` of the
forward mask (forward commands) or of the dq mask (backward commands), as
kvax/utils/benchmarking.py:423-430 and :565-572 do.
"""
from __future__ import annotations

import logging
import os
import random

import click

logger = logging.getLogger("kvax_b200.benchmarks")


def generate_random_segments_lengths(seq_len: int, num_segments: int):
    """Segment lengths summing to `seq_len` (kvax/utils/benchmarking.py:309-324): every
    segment starts with one token and the rest are thrown at random segments with
    `random.seed(0)`; None for a single segment."""
    if num_segments == 1:
        return None
    random.seed(0)
    lengths = [1] * num_segments
    for _ in range(seq_len - num_segments):
        lengths[random.randint(0, num_segments - 1)] += 1
    return lengths


def make_positions_and_segments(batch_size, seq_len, segment_lengths, num_pad_tokens):
    """int32 (B, S) positions (a global arange, the reference's convention) and segment ids
    (document index, PAD = -1 on the last `num_pad_tokens` tokens)."""
    import torch

    from kvax_b200.utils.common import PADDING_SEGMENT_ID
    pos = torch.arange(seq_len, dtype=torch.int32).repeat(batch_size, 1)
    seg = torch.zeros(seq_len, dtype=torch.int32)
    if segment_lengths is not None:
        seg = torch.repeat_interleave(torch.arange(len(segment_lengths), dtype=torch.int32),
                                      torch.tensor(segment_lengths))
    seg = seg.repeat(batch_size, 1).contiguous()
    if num_pad_tokens > 0:
        seg[:, seq_len - num_pad_tokens:] = PADDING_SEGMENT_ID
    return pos, seg


def _time_cuda(fn, num_iters):
    import torch
    fn()                                        # warm-up, as the reference does
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(num_iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / num_iters


def _dense_reference(q, k, v, pos_q, seg_q, pos_k, seg_k, scale):
    import torch
    group = q.shape[2] // k.shape[2]
    kk = k.repeat_interleave(group, dim=2).float()
    vv = v.repeat_interleave(group, dim=2).float()
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk) * scale
    allowed = (pos_q[:, :, None] >= pos_k[:, None, :]) & (seg_q[:, :, None] == seg_k[:, None, :]) & (seg_k[:, None, :] != -1)
    s = s.masked_fill(~allowed[:, None], float("-inf"))
    p = torch.softmax(s, dim=-1).nan_to_num(0.0)
    return torch.einsum("bhqk,bkhd->bqhd", p, vv)


def _run(backward, context_parallel, num_iters, batch_size, query_seq_len, kv_seq_len, num_heads, num_kv_heads,
         qk_head_dim, value_head_dim, assume_sequential_positions, num_segments, num_pad_tokens,
         permute_tokens_for_load_balance, show_attention_mask, check):
    import torch
    import torch.distributed as dist

    import kvax_b200 as kv
    from kvax_b200.ops.mask_creator import calculate_mask_sparsity, print_mask
    from kvax_b200.utils.math import get_multi_head_attention_tflops

    if query_seq_len != kv_seq_len and context_parallel:
        raise click.UsageError("context parallelism needs query_seq_len == kv_seq_len")
    world, rank = 1, 0
    if context_parallel:
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local_rank)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)

    seg_lengths = generate_random_segments_lengths(query_seq_len, num_segments)
    pos, seg = make_positions_and_segments(batch_size, kv_seq_len, seg_lengths, num_pad_tokens)
    kv_pos, kv_seg = pos.to(dev), seg.to(dev)
    q_pos, q_seg = kv_pos[:, kv_seq_len - query_seq_len:].contiguous(), kv_seg[:, kv_seq_len - query_seq_len:].contiguous()
    scale = qk_head_dim ** -0.5
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, world))
    q_spec = ("data", "context" if world > 1 else None, None, None)
    s_loc = query_seq_len // world
    q = randn(batch_size, s_loc, num_heads, qk_head_dim)
    k = randn(batch_size, kv_seq_len // world, num_kv_heads, qk_head_dim)
    v = randn(batch_size, kv_seq_len // world, num_kv_heads, value_head_dim)
    do = randn(batch_size, s_loc, num_heads, value_head_dim)
    with mesh, kv.attention_specs(q_spec, ("data", None, None, None)):
        if world > 1:
            if permute_tokens_for_load_balance:
                q_pos, q_seg = kv.permute_tokens_context_parallelism((q_pos, q_seg))
            q_pos = q_pos[:, rank * s_loc:(rank + 1) * s_loc].contiguous()
            q_seg = q_seg[:, rank * s_loc:(rank + 1) * s_loc].contiguous()
        if backward:
            q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

        def step():
            masks = kv.create_attention_mask(q_pos, q_seg, kv_pos, kv_seg, fwd_params=params, bwd_params=params,
                                             calc_bwd_mask=backward)
            out = kv.flash_attention(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, scale=scale, fwd_params=params,
                                     bwd_params=params, assume_sequential_positions=assume_sequential_positions,
                                     permute_tokens_for_load_balance=permute_tokens_for_load_balance)
            if backward:
                out.backward(do)
                q.grad = None; k.grad = None; v.grad = None
            return out, masks

        sec = _time_cuda(step, num_iters)
        if world > 1:
            t = torch.tensor([sec], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        tflops_per_iter = get_multi_head_attention_tflops(
            batch_size=batch_size, query_seq_len=query_seq_len, kv_seq_len=kv_seq_len, num_heads=num_heads,
            qk_head_dim=qk_head_dim, value_head_dim=value_head_dim, causal=False, num_gpus=world,
            forward_pass=True, backward_pass=backward)
        name = "flash_attention_b200" + ("_bwd" if backward else "_fwd") + (f"_cp{world}" if world > 1 else "")
        out, masks = step()
        # the reference scales by the sparsity of mask[0] in the forward commands and of mask[1] in the backward ones
        counted = masks[1] if backward else masks[0]
        sparsity = calculate_mask_sparsity(counted, params.query_block_size, params.kv_block_size, s_loc, kv_seq_len)
        if rank == 0:
            msg = (f"{name} took {sec * 1e3:.3f} ms per iteration, achieved "
                   f"{tflops_per_iter * sparsity / sec:.1f} TFLOP/s per GPU (mask sparsity {sparsity:.4f})")
            logger.info(msg)
            print(msg, flush=True)
        if show_attention_mask and rank == 0:
            print_mask(masks[0], kv_seq_len // params.kv_block_size)
        if check and world == 1:
            if query_seq_len * kv_seq_len * num_heads * batch_size > (1 << 31):
                raise click.UsageError("--check holds the dense score matrix: use a shorter sequence")
            ref = _dense_reference(q.detach(), k.detach(), v.detach(), q_pos, q_seg, kv_pos, kv_seg, scale)
            rows = (q_seg != -1)[:, :, None, None]
            err = ((out.detach().float() - ref) * rows).abs().max().item()
            print(f"max |out - dense| on non-PAD rows: {err:.4g}", flush=True)
            if err > 2e-2 + ref.abs().max().item() / 256:
                raise SystemExit("output check failed")
    if context_parallel and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def _common(cp: bool):
    opts = [
        click.option("--num-iters", type=int, default=10),
        click.option("--batch-size", type=int, default=4),
        click.option("--query-seq-len", type=int, default=32768 if cp else 8192),
        click.option("--kv-seq-len", type=int, default=32768 if cp else 8192),
        click.option("--num-heads", type=int, default=32 if cp else 16),
        click.option("--num-kv-heads", type=int, default=8 if cp else 16),
        click.option("--qk-head-dim", type=int, default=128),
        click.option("--value-head-dim", type=int, default=128),
        click.option("--assume-sequential-positions", type=bool, default=True),
        click.option("--num-segments", type=int, default=1),
        click.option("--show-attention-mask", is_flag=True),
    ]
    if cp:
        opts.append(click.option("--permute-tokens-for-load-balance", type=bool, default=True))
    else:
        opts.append(click.option("--num-pad-tokens", type=int, default=0))
        opts.append(click.option("--check", is_flag=True, help="compare with a dense torch attention"))

    def wrap(f):
        for o in reversed(opts):
            f = o(f)
        return f
    return wrap


@click.group()
def cli():
    pass


@cli.command("mha")
@_common(False)
def mha_benchmark(**kw):
    _run(False, False, permute_tokens_for_load_balance=False, **kw)


@cli.command("mha_bwd")
@_common(False)
def mha_benchmark_bwd(**kw):
    _run(True, False, permute_tokens_for_load_balance=False, **kw)


@cli.command("mha_cp")
@_common(True)
def mha_cp_fwd_benchmark(**kw):
    _run(False, True, num_pad_tokens=0, check=False, **kw)


@cli.command("mha_cp_bwd")
@_common(True)
def mha_cp_bwd_benchmark(**kw):
    _run(True, True, num_pad_tokens=0, check=False, **kw)


if __name__ == "__main__":
    logging.basicConfig(level=logging.INFO)
    cli()
