"""Generates tests/golden/mask_*.npz from the reference's own mask code.

Run once, in a container that has the reference checkout (read-only) and Triton:

    TRITON_INTERPRET=1 python tests/golden/make_mask_golden.py /path/to/reference

What runs is the reference's unmodified `compute_attention_mask_single_device`
(kvax/ops/mask_creator.py:202-335) including its Triton kernel (:26-152), executed by
Triton's CPU interpreter.  JAX is not installed, so `jax.numpy` is replaced by NumPy
(the function only uses `where`, `pad`, `iinfo`) and `jax_triton.triton_call` by a
shim that launches the `@triton.jit` kernel on CPU torch tensors.  The fixtures keep
inputs and outputs, so the tests need neither the reference nor Triton.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch


def _install_stubs(ref_root: str) -> None:
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    class _Any:
        def __class_getitem__(cls, item):
            return cls

    # --- jax.numpy -> numpy -------------------------------------------------------
    jnp = mod("jax.numpy", where=np.where, pad=np.pad, iinfo=np.iinfo, int32=np.int32,
              float32=np.float32, ndarray=np.ndarray, dtype=np.dtype)

    class ShapeDtypeStruct:
        def __init__(self, shape, dtype):
            self.shape, self.dtype = tuple(shape), dtype

    jax = mod("jax", numpy=jnp, ShapeDtypeStruct=ShapeDtypeStruct, Array=np.ndarray)
    jax.custom_vjp = lambda f=None, **kw: f
    jax.jit = lambda f=None, **kw: f
    mod("jax.sharding", Mesh=_Any, PartitionSpec=tuple)
    sm = mod("jax.experimental.shard_map", Specs=_Any, shard_map=None)
    exp = mod("jax.experimental", shard_map=sm)
    jax.experimental = exp
    mod("jax.interpreters", pxla=mod("jax.interpreters.pxla"))
    mod("jax.ad_checkpoint", checkpoint_name=lambda x, n: x)
    mod("chex", ArrayDevice=np.ndarray, PRNGKey=np.ndarray,
        assert_shape=lambda *a, **k: None, assert_rank=lambda *a, **k: None)

    # --- jax_triton -> interpreter launch on CPU torch tensors --------------------
    def triton_call(*args, kernel, out_shape, grid, debug=False, num_warps=None,
                    num_stages=None, **constexprs):
        ins = [torch.from_numpy(np.ascontiguousarray(a)) for a in args]
        outs = [torch.zeros(s.shape, dtype=torch.int32) for s in out_shape]
        kernel[grid](*ins, *outs, **constexprs)
        return tuple(o.numpy() for o in outs)

    mod("jax_triton", triton_call=triton_call, cdiv=lambda a, b: (a + b - 1) // b)

    # --- kvax as a namespace so that kvax/__init__.py (which pulls in the attention
    #     kernels) is not executed ----------------------------------------------
    for name in ("kvax", "kvax.ops", "kvax.utils"):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(ref_root, *name.split("."))]
        sys.modules[name] = m


def _segments(rng, batch, seq, n_docs, n_pad, restart_positions, per_row_pad=False):
    """Piecewise-constant segment ids with PAD (-1) at the tail of every row."""
    seg = np.zeros((batch, seq), np.int32)
    pos = np.zeros((batch, seq), np.int32)
    for b in range(batch):
        pad = int(rng.integers(0, n_pad + 1)) if per_row_pad else n_pad
        real = seq - pad
        cuts = np.sort(rng.choice(np.arange(1, real), size=min(n_docs - 1, max(real - 1, 0)),
                                  replace=False)) if n_docs > 1 and real > 1 else np.array([], int)
        edges = np.concatenate([[0], cuts, [real]]).astype(int)
        for d, (s, e) in enumerate(zip(edges[:-1], edges[1:])):
            seg[b, s:e] = d
            pos[b, s:e] = np.arange(e - s) if restart_positions else np.arange(s, e)
        seg[b, real:] = -1
        pos[b, real:] = np.arange(pad) if restart_positions else np.arange(real, seq)
    return pos, seg


def _permute(a, cp):
    """Load-balancing chunk permutation, kvax/utils/permutation.py:9-42."""
    n = 2 * cp
    idx = np.array([(i, n - i - 1) for i in range(n // 2)]).flatten()
    return a.reshape(a.shape[0], n, -1)[:, idx].reshape(a.shape)


CASES = [
    # name, batch, Sq, Skv, docs, pad, restart, fwd(q,kv), bwd(q,kv), skip_pad, cp (q shard count)
    ("tiny_c1", 1, 512, 512, 3, 32, True, (64, 64), (64, 64), True, 1),
    ("arange_1doc", 2, 1024, 1024, 1, 0, False, (128, 128), (64, 128), True, 1),
    ("arange_pad", 2, 1024, 1024, 1, 300, False, (128, 128), (64, 128), False, 1),
    ("arange_5doc", 2, 2048, 2048, 5, 211, False, (128, 128), (64, 128), False, 1),
    ("arange_12doc_skip", 2, 2048, 2048, 12, 176, False, (128, 128), (64, 128), True, 1),
    ("restart_4doc", 2, 2048, 2048, 4, 205, True, (128, 128), (128, 128), True, 1),
    ("restart_7doc_64", 1, 1536, 1536, 7, 77, True, (64, 64), (64, 64), True, 1),
    ("restart_mixed_tiles", 2, 1024, 1024, 6, 100, True, (128, 64), (64, 128), True, 1),
    ("ragged_len", 2, 400, 300, 3, 37, False, (64, 64), (64, 64), True, 1),
    ("ragged_len_noskip", 1, 384, 400, 2, 100, False, (128, 128), (128, 128), False, 1),
    ("all_pad_row", 2, 512, 512, 2, 512, False, (64, 64), (64, 64), True, 1),
    ("per_row_pad", 3, 768, 768, 3, 383, True, (128, 128), (64, 128), True, 1),
    ("decode_q1", 2, 1, 640, 1, 0, False, (64, 64), (64, 64), True, 1),
    ("cp2_shard_permuted", 2, 2048, 2048, 5, 300, False, (128, 128), (64, 128), True, 2),
    ("cp4_shard_permuted_restart", 1, 4096, 4096, 6, 400, True, (128, 128), (128, 128), True, 4),
]


def main(ref_root: str, out_dir: str) -> None:
    _install_stubs(ref_root)
    mc = importlib.import_module("kvax.ops.mask_creator")
    rng = np.random.default_rng(0)
    for (name, B, Sq, Skv, docs, pad, restart, fwd, bwd, skip, cp) in CASES:
        S = max(Sq, Skv)
        pos, seg = _segments(rng, B, S, docs, min(pad, S), restart, per_row_pad=(name == "per_row_pad"))
        kv_pos, kv_seg = pos[:, :Skv].copy(), seg[:, :Skv].copy()
        if name == "decode_q1":  # one query token at per-row start positions vs a padded KV cache
            starts = np.array([17, 500], np.int32)
            q_pos, q_seg = starts[:, None].copy(), np.zeros((B, 1), np.int32)
            kv_seg = np.where(np.arange(Skv)[None, :] > starts[:, None], -1, 0).astype(np.int32)
            shards = [(q_pos, q_seg)]
        else:
            q_pos, q_seg = pos[:, :Sq].copy(), seg[:, :Sq].copy()
            if cp > 1:  # caller permutes the query side, then each rank sees one slice
                q_pos, q_seg = _permute(q_pos, cp), _permute(q_seg, cp)
                n = Sq // cp
                shards = [(q_pos[:, r * n:(r + 1) * n], q_seg[:, r * n:(r + 1) * n]) for r in range(cp)]
            else:
                shards = [(q_pos, q_seg)]
        out = dict(q_pos=q_pos, q_seg=q_seg, kv_pos=kv_pos, kv_seg=kv_seg,
                   fwd=np.array(fwd), bwd=np.array(bwd), skip=np.array(skip), cp=np.array(cp))
        for r, (qp, qs) in enumerate(shards):
            calls = {
                "fwd": dict(kv_block_size=fwd[1], query_block_size=fwd[0]),
                "dq": dict(kv_block_size=bwd[0], query_block_size=bwd[1]),
                "dkdv": dict(kv_block_size=bwd[1], query_block_size=bwd[0], calculate_dkdv_mask=True),
            }
            for tag, kw in calls.items():
                res = mc.compute_attention_mask_single_device(
                    qp, qs, kv_pos, kv_seg, skip_pad_tokens=skip, **kw)
                for nm, a in zip(("lower", "upper", "lower_full", "upper_full"), res):
                    out[f"r{r}_{tag}_{nm}"] = np.asarray(a, np.int32)
        np.savez_compressed(os.path.join(out_dir, f"mask_{name}.npz"), **out)
        print("wrote", name)


if __name__ == "__main__":
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
