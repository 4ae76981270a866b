"""Generates tests/golden/attn_*.npz from the reference's own attention code.

Run once, in a container that has the reference checkout (read-only) and Triton:

    TRITON_INTERPRET=1 python tests/golden/make_attention_golden.py /path/to/reference

What runs is the reference's `flash_attention_triton_forward` (kvax/ops/
flash_attention_triton.py:1375-1563) and `flash_attention_backward` (:1566-1879): the host
functions with their padding, mask unpacking, launch geometry and GQA group sum, and the
`@triton.jit` kernels they launch (:57-134, 137-370, 373-410, 413-617, 620-871, 874-1191,
1194-1372), executed by Triton's CPU interpreter on fp32 tensors.  The block masks they
consume come from the reference's `compute_attention_mask_single_device`, as in
make_mask_golden.py.

Three shims make that possible without JAX and without a GPU; none changes what is computed:
  * `jax.numpy` is NumPy, `jax_triton.triton_call` launches the kernel on CPU torch tensors
    (stubs of make_mask_golden.py plus the few names the attention host code uses);
  * Python scalars that a kernel treats as tensors (`scale`) are wrapped as interpreter
    tensors, as compiled Triton does for scalar arguments;
  * inside `@triton.jit` functions the Python keywords `and` / `or` are rewritten to `&` / `|`
    on the syntax tree (compiled Triton maps them to logical ops on tensors; plain Python
    would ask a tensor for its truth value).  The rewritten module is a build product written
    to oracle/_ref/ (ignored by git) and deleted again at the end of the run.

Inputs are drawn as bf16-representable fp32 values, so that an implementation computing on
bf16 operands sees exactly the same numbers.  dO is zero on PAD rows (the reference's tests
zero them as well).  The fixtures keep inputs and outputs; the tests need neither the
reference nor Triton.
"""
from __future__ import annotations

import ast
import importlib
import importlib.util
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import make_mask_golden as mg  # noqa: E402  (stubs and the segment generator)


def _install_attention_stubs(ref_root: str) -> None:
    mg._install_stubs(ref_root)
    jnp, chex, jt, jax = (sys.modules[n] for n in ("jax.numpy", "chex", "jax_triton", "jax"))
    for nm in ("concatenate", "sum", "arange", "asarray"):
        setattr(jnp, nm, getattr(np, nm))

    class _JaxLikeArray(np.ndarray):
        """ndarray with JAX's functional update `x.at[idx].set(v)` (used by the backward host code)."""

        @property
        def at(self):
            arr = self

            class _At:
                def __getitem__(self, idx):
                    class _Set:
                        def set(self, value):
                            out = np.array(arr, copy=True)
                            out[idx] = value
                            return out.view(_JaxLikeArray)
                    return _Set()
            return _At()

    jnp.zeros = lambda *a, **k: np.zeros(*a, **k).view(_JaxLikeArray)
    jnp.ones = lambda *a, **k: np.ones(*a, **k).view(_JaxLikeArray)
    for nm in ("assert_axis_dimension_comparator", "assert_is_divisible"):
        setattr(chex, nm, lambda *a, **k: None)

    class _CustomVjp:
        def __init__(self, f):
            self.f = f

        def __call__(self, *a, **k):
            return self.f(*a, **k)

        def defvjp(self, *a, **k):
            pass

    jax.custom_vjp = lambda f=None, **kw: (_CustomVjp(f) if f is not None else (lambda g: _CustomVjp(g)))
    jt.next_power_of_2 = lambda x: 1 << (int(x) - 1).bit_length()

    def strides_from_shape(shape):
        st, acc = [], 1
        for d in reversed(shape):
            st.append(acc)
            acc *= int(d)
        return tuple(reversed(st))

    jt.strides_from_shape = strides_from_shape

    def triton_call(*args, kernel, out_shape, grid, debug=False, num_warps=None, num_stages=None,
                    zeroed_outputs=None, **constexprs):
        import triton.language as tl
        from triton.runtime.interpreter import TensorHandle

        def cvt(a):
            if isinstance(a, np.ndarray):
                return torch.from_numpy(np.ascontiguousarray(a))
            if isinstance(a, float):
                return tl.tensor(TensorHandle(np.array([a], dtype=np.float32), tl.float32), tl.float32)
            return a

        single = not isinstance(out_shape, (list, tuple))
        shapes = [out_shape] if single else list(out_shape)
        tdt = {np.dtype("float32"): torch.float32, np.dtype("int32"): torch.int32}
        outs = [torch.zeros(tuple(s.shape), dtype=tdt[np.dtype(s.dtype)]) for s in shapes]
        kernel[grid](*[cvt(a) for a in args], *outs, **constexprs)
        res = tuple(o.numpy() for o in outs)
        return res[0] if single else res

    jt.triton_call = triton_call


def _load_attention_module(ref_root: str, build_dir: str):
    """The reference module with `and` / `or` inside @triton.jit functions rewritten to & / |."""
    src = open(os.path.join(ref_root, "kvax", "ops", "flash_attention_triton.py")).read()

    class BoolOps(ast.NodeTransformer):
        def visit_BoolOp(self, node):
            self.generic_visit(node)
            op = ast.BitAnd() if isinstance(node.op, ast.And) else ast.BitOr()
            out = node.values[0]
            for v in node.values[1:]:
                out = ast.BinOp(left=out, op=op, right=v)
            return ast.copy_location(out, node)

    class JitOnly(ast.NodeTransformer):
        def visit_FunctionDef(self, node):
            if any(isinstance(d, ast.Attribute) and d.attr == "jit" for d in node.decorator_list):
                return BoolOps().visit(node)
            return node

    tree = ast.fix_missing_locations(JitOnly().visit(ast.parse(src)))
    os.makedirs(build_dir, exist_ok=True)
    path = os.path.join(build_dir, "flash_attention_triton_interp.py")
    with open(path, "w") as f:
        f.write(ast.unparse(tree))
    spec = importlib.util.spec_from_file_location("kvax.ops.flash_attention_triton", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["kvax.ops.flash_attention_triton"] = mod
    spec.loader.exec_module(mod)
    return mod


def _bf16_values(rng, shape):
    x = rng.standard_normal(shape).astype(np.float32)
    return torch.from_numpy(x).to(torch.bfloat16).float().numpy()


def _bf16_bits(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).view(torch.int16).numpy()


CASES = [
    # name, B, Sq, Skv, Hq, Hkv, D, docs, pad, restart, fwd(q,kv), bwd(q,kv) or None, sequential
    # (names starting with "cp2" run the context-parallel code path once per rank: permuted local queries
    #  against the full keys / values, `jax.lax.axis_index` answering with the rank)
    ("tiny_c1", 1, 512, 512, 4, 2, 64, 3, 32, True, (64, 64), (64, 64), False),
    ("d128_blk128", 1, 384, 384, 2, 1, 128, 2, 40, False, (128, 128), (128, 128), False),
    ("d128_sequential", 1, 384, 384, 2, 1, 128, 2, 40, False, (128, 128), (128, 128), True),
    ("mixed_blocks_mha", 2, 256, 256, 2, 2, 64, 4, 20, True, (128, 64), (64, 128), False),
    ("ragged_fwd", 2, 200, 200, 2, 1, 64, 2, 13, False, (64, 64), None, False),
    ("decode_fwd", 2, 1, 320, 4, 2, 64, 1, 0, False, (64, 64), None, False),
    ("cp2_rank0_sequential", 1, 256, 512, 2, 1, 64, 3, 24, False, (64, 64), (64, 64), True),
    ("cp2_rank1_sequential", 1, 256, 512, 2, 1, 64, 3, 24, False, (64, 64), (64, 64), True),
]


def main(ref_root: str, out_dir: str) -> None:
    _install_attention_stubs(ref_root)
    repo = os.path.dirname(os.path.dirname(out_dir))
    fa = _load_attention_module(ref_root, os.path.join(repo, "oracle", "_ref"))
    mc = importlib.import_module("kvax.ops.mask_creator")
    from kvax.utils.common import FlashAttentionParamsConfig

    import types
    jax = sys.modules["jax"]
    rng = np.random.default_rng(1)
    for (name, B, Sq, Skv, Hq, Hkv, D, docs, pad, restart, fwd, bwd, sequential) in CASES:
        S = max(Sq, Skv)
        cp, rank = (2, int(name[8])) if name.startswith("cp2_rank") else (1, 0)
        if cp > 1:      # both ranks see the same global sequence
            rng = np.random.default_rng(7)
            jax.lax = types.SimpleNamespace(axis_index=lambda axis: rank, psum=lambda x, axis: x * cp)
        pos, seg = mg._segments(rng, B, S, docs, pad, restart)
        kv_pos, kv_seg = pos[:, :Skv].copy(), seg[:, :Skv].copy()
        if name == "decode_fwd":   # one query token at per-row positions against a padded KV cache
            starts = np.array([17, 250], np.int32)
            q_pos, q_seg = starts[:, None].copy(), np.zeros((B, 1), np.int32)
            kv_seg = np.where(np.arange(Skv)[None, :] > starts[:, None], -1, 0).astype(np.int32)
        elif cp > 1:               # the caller permutes the query side; this rank holds one slice of it
            q_pos = mg._permute(pos, cp)[:, rank * Sq:(rank + 1) * Sq].copy()
            q_seg = mg._permute(seg, cp)[:, rank * Sq:(rank + 1) * Sq].copy()
        else:
            q_pos, q_seg = pos[:, :Sq].copy(), seg[:, :Sq].copy()
        scale = float(D) ** -0.5
        # the reference's internal layout is (batch, heads, seq, dim)
        if cp > 1:                 # same K / V on both ranks, rank-specific Q / dO
            k = _bf16_values(rng, (B, Hkv, Skv, D))
            v = _bf16_values(rng, (B, Hkv, Skv, D))
            rng = np.random.default_rng(70 + rank)
        q = _bf16_values(rng, (B, Hq, Sq, D))
        if cp == 1:
            k = _bf16_values(rng, (B, Hkv, Skv, D))
            v = _bf16_values(rng, (B, Hkv, Skv, D))
        do = _bf16_values(rng, (B, Hq, Sq, D))
        do = np.where((q_seg != -1)[:, None, :, None], do, 0.0).astype(np.float32)
        fp = FlashAttentionParamsConfig(query_block_size=fwd[0], kv_block_size=fwd[1], num_warps=4, num_stages=2)
        specs = [dict(query_block_size=fwd[0], kv_block_size=fwd[1])]
        bp = fp
        if bwd is not None:
            bp = FlashAttentionParamsConfig(query_block_size=bwd[0], kv_block_size=bwd[1], num_warps=4, num_stages=2)
            specs.append(dict(query_block_size=bwd[1], kv_block_size=bwd[0]))                       # dq mask: swapped
            specs.append(dict(query_block_size=bwd[0], kv_block_size=bwd[1], calculate_dkdv_mask=True))
        masks = tuple(
            tuple(np.asarray(a, np.int32) for a in mc.compute_attention_mask_single_device(
                q_pos, q_seg, kv_pos, kv_seg, skip_pad_tokens=True, **kw)) for kw in specs)
        out, res = fa.flash_attention_triton_forward(
            q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, scale, None, fp, bp,
            assume_sequential_positions=sequential,
            context_parallelism_mesh_axis_name="context" if cp > 1 else None)
        lse = np.asarray(res[-1])[:, :, :Sq]
        to_bshd = lambda a: np.ascontiguousarray(np.asarray(a).transpose(0, 2, 1, 3))
        fix = dict(q=_bf16_bits(to_bshd(q)), k=_bf16_bits(to_bshd(k)), v=_bf16_bits(to_bshd(v)),
                   dout=_bf16_bits(to_bshd(do)), q_pos=q_pos, q_seg=q_seg, kv_pos=kv_pos, kv_seg=kv_seg,
                   scale=np.float32(scale), fwd=np.array(fwd), bwd=np.array(bwd if bwd else (0, 0)),
                   sequential=np.array(sequential), cp=np.array(cp), rank=np.array(rank), out=to_bshd(out).astype(np.float32), lse2=lse.astype(np.float32))
        if bwd is not None:
            grads = fa.flash_attention_backward(scale, None, fp, bp, sequential, False, True,
                                                "context" if cp > 1 else None, False, res, do)
            fix.update(dq=to_bshd(grads[0]).astype(np.float32), dk=to_bshd(grads[1]).astype(np.float32),
                       dv=to_bshd(grads[2]).astype(np.float32))
        np.savez_compressed(os.path.join(out_dir, f"attn_{name}.npz"), **fix)
        print("wrote", name, {k_: getattr(v_, "shape", None) for k_, v_ in fix.items() if k_ in ("out", "dq", "dk")})
    os.remove(os.path.join(repo, "oracle", "_ref", "flash_attention_triton_interp.py"))


if __name__ == "__main__":
    main(sys.argv[1], HERE)
