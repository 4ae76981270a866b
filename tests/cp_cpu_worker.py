"""Worker of tests/test_context_parallel_cpu.py: world_size ranks on CPU with gloo.

Checks the host-side context-parallel plumbing of flash_attention without a GPU: the
K/V all-gather into natural order and the dK/dV reduce-scatter back to the owners, with
the chunk permutation done by the NumPy oracle instead of the CUDA kernel; and the
all-to-all pair of the head-exchange schedule (sequence sharding <-> head sharding)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from kvax_b200.ops.flash_attention import (_chunk_of, _exchange_heads_to_seq, _exchange_seq_to_heads, _gather_kv,  # noqa: E402
                                            _gather_remote, _gather_tokens, _heads_to_seq, _natural_chunks,
                                            _remote_to_scatter_layout, _scatter_dkv, _seq_to_heads, context_offsets)
from kvax_b200.utils.sharding import Mesh  # noqa: E402
from oracle import permutation_oracle as po  # noqa: E402


def oracle_permute(x, cp, reverse):
    return torch.from_numpy(po.apply_permutation(x.numpy(), cp, reverse).copy())


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mesh = Mesh(("data", "context"), (1, world))
    assert mesh.coordinate("context") == rank and mesh.group("context") is None
    for B in (1, 2):
        S, H, D = 64 * world, 2, 4
        g = torch.Generator().manual_seed(7)
        full = torch.randn(B, S, H, D, generator=g)
        for permuted in (True, False):
            glob = oracle_permute(full, world, False) if permuted else full     # what the caller shards
            loc = S // world
            mine = glob[:, rank * loc:(rank + 1) * loc].contiguous()
            got = _gather_kv(mine, world, None, permuted, permute_fn=oracle_permute)
            assert torch.equal(got, full), f"gather mismatch B={B} permuted={permuted}"
            # every rank contributes (rank+1) * full as its dK; owners get the sum of their slice
            grad = (rank + 1.0) * full
            out = _scatter_dkv(grad, world, None, permuted, torch.float32, permute_fn=oracle_permute)
            expect = sum(r + 1.0 for r in range(world)) * mine
            assert torch.allclose(out, expect), f"scatter mismatch B={B} permuted={permuted}"
            first, second = context_offsets(rank, world, loc, permuted)
            idx = torch.arange(S).view(1, S, 1, 1).float().expand(B, S, 1, 1)
            gi = (oracle_permute(idx, world, False) if permuted else idx)[0, rank * loc:(rank + 1) * loc, 0, 0]
            local = torch.arange(loc).float()
            glob_idx = torch.where(local * 2 >= loc, local + second, local + first)
            assert torch.equal(glob_idx, gi), "global offsets do not reproduce global token indices"
            # head exchange: this rank must receive the whole natural-order sequence for its heads
            Hx = 2 * world
            fullh = torch.randn(B, S, Hx, D, generator=torch.Generator().manual_seed(11))
            globh = oracle_permute(fullh, world, False) if permuted else fullh
            mineh = globh[:, rank * loc:(rank + 1) * loc].contiguous()
            heads = _seq_to_heads(mineh, world, None, permuted, permute_fn=oracle_permute)
            assert torch.equal(heads, fullh[:, :, 2 * rank:2 * rank + 2]), f"seq->heads mismatch B={B} permuted={permuted}"
            back = _heads_to_seq(heads, world, None, permuted, permute_fn=oracle_permute)
            assert torch.equal(back, mineh), f"heads->seq mismatch B={B} permuted={permuted}"
            if B == 1:
                # the zero-copy exchange (half-sequences received straight into natural order, several tensors per
                # group of sends / receives) must give the same tensors as the copy-based all-to-all
                other = torch.randn(B, loc, world, D, generator=torch.Generator().manual_seed(13 + rank))
                fast, fast2 = _exchange_seq_to_heads((mineh, other), world, rank, None, permuted)
                assert torch.equal(fast, heads), f"zero-copy seq->heads mismatch permuted={permuted}"
                assert torch.equal(fast2, _seq_to_heads(other, world, None, permuted, permute_fn=oracle_permute))
                back1, back2 = _exchange_heads_to_seq((fast, fast2), world, rank, None, permuted)
                assert torch.equal(back1, mineh) and torch.equal(back2, other), f"zero-copy heads->seq mismatch permuted={permuted}"
            # overlapped all-gather schedule: the chunks of the other ranks in natural order, and the way back of
            # their gradients (reduce-scatter input with zeros in this rank's own chunks)
            half = loc // 2
            own = [_chunk_of(rank, 0, world, permuted), _chunk_of(rank, 1, world, permuted)]
            rest = [c for c in range(2 * world) if c not in own]
            landing = torch.empty((world * B, loc, H, D))
            rem = _gather_remote(mine, landing, world, rank, None, permuted)
            want = torch.cat([full[:, c * half:(c + 1) * half] for c in rest], dim=1)
            assert torch.equal(rem, want), f"remote gather mismatch B={B} permuted={permuted}"
            assert torch.equal(torch.cat([full[:, c * half:(c + 1) * half] for c in own], dim=1), mine)
            ids = torch.arange(B * S, dtype=torch.int32).view(B, S)
            assert torch.equal(_natural_chunks(ids, world, rest), torch.cat([ids[:, c * half:(c + 1) * half] for c in rest], dim=1))
            send = _remote_to_scatter_layout((rank + 1.0) * rem, world, rank, permuted)
            got_rs = torch.empty((B, loc, H, D))
            dist.reduce_scatter_tensor(got_rs, send, op=dist.ReduceOp.SUM)
            expect_rs = sum(r + 1.0 for r in range(world) if r != rank) * mine
            assert torch.allclose(got_rs, expect_rs), f"remote scatter mismatch B={B} permuted={permuted}"
            tok = torch.arange(B * S, dtype=torch.int32).view(B, S)
            tokg = (oracle_permute(tok.view(B, S, 1, 1), world, False).view(B, S) if permuted else tok)
            gathered = _gather_tokens(tokg[:, rank * loc:(rank + 1) * loc].contiguous(), world, None, permuted, permute_fn=oracle_permute)
            assert torch.equal(gathered, tok), "token gather mismatch"
    if world == 4:
        # Context parallelism inside a larger mesh: (data, context, model) = (1, 2, 2) and (2, 2): the collectives
        # must stay inside the ranks that differ only along "context" (the reference's tests combine context
        # parallelism with data- and tensor-parallel specs, tests/test_attention.py:520-828).
        for names, shape in ((("data", "context", "model"), (1, 2, 2)), (("data", "context"), (2, 2))):
            m = Mesh(names, shape)
            cp, crank = m.shape["context"], m.coordinate("context")
            other = rank - crank * (2 if "model" in names else 1)      # identifies the context group
            group = m.group("context")
            assert group is not None and dist.get_world_size(group) == cp and dist.get_rank(group) == crank
            B, S, H, D = 1, 64 * cp, 2 * cp, 4
            full = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(100 + other))   # differs per group
            glob = oracle_permute(full, cp, False)
            loc = S // cp
            mine = glob[:, crank * loc:(crank + 1) * loc].contiguous()
            assert torch.equal(_gather_kv(mine, cp, group, True, permute_fn=oracle_permute), full)
            heads = _seq_to_heads(mine, cp, group, True, permute_fn=oracle_permute)
            assert torch.equal(heads, full[:, :, 2 * crank:2 * crank + 2])
            assert torch.equal(_heads_to_seq(heads, cp, group, True, permute_fn=oracle_permute), mine)
            (fast,) = _exchange_seq_to_heads((mine,), cp, crank, group, True)
            assert torch.equal(fast, heads)
            assert torch.equal(_exchange_heads_to_seq((fast,), cp, crank, group, True)[0], mine)
            out = _scatter_dkv((crank + 1.0) * full, cp, group, True, torch.float32, permute_fn=oracle_permute)
            assert torch.allclose(out, 3.0 * mine)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("cp cpu worker ok")


if __name__ == "__main__":
    main()
