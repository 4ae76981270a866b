"""The reference's own attention code run on the GPU.  TEST / BENCH INFRASTRUCTURE ONLY.

What runs is kvax's unmodified `flash_attention_triton_forward` (kvax/ops/flash_attention_triton.py:
1375-1563) and `flash_attention_backward` (:1566-1879) -- the host functions with their padding, mask
unpacking, launch geometry and GQA group sum -- and the `@triton.jit` kernels they launch (:57-134,
137-370, 373-410, 413-617, 620-871, 874-1191, 1194-1372), compiled by the Triton that ships in this
image.  The statement "outputs match the reference's own Triton flash_attention on the same seeded
inputs" is tested against this, and the benchmark times it beside the CUDA kernels as the same-GPU
comparator.

JAX, jax_triton and chex are not installed here, so three things stand in for them; none changes
what the kernels compute:
  * `jax.numpy` is a small module of torch functions (zeros / ones / concatenate / pad / sum / where /
    iinfo and the two dtypes the host code names), so the host code runs on torch CUDA tensors;
  * `jax_triton.triton_call` allocates the outputs with torch and launches the kernel through
    Triton's own launcher with the grid, num_warps and num_stages the host code passes;
  * `chex` assertions are no-ops (the callers pass valid shapes).
The two module constants the kernels read (`LOG2_CONST`, `NEG_INF`, :27-28) are plain Python numbers
in the source, which Triton >= 3 only accepts with TRITON_ALLOW_NON_CONSTEXPR_GLOBALS=1; this module
sets that variable before importing Triton kernels.

The reference sources are not part of this repository.  `python -m oracle.make_ref /path/to/kvax-checkout`
copies the checkout's `kvax/` package to oracle/_ref/kvax_reference/ (ignored by git); `available()`
says whether that copy, Triton and a GPU are there.

Layout: the public API of this repository is (batch, seq, heads, dim); the reference's host functions
work on (batch, heads, seq, dim).  `forward` / `backward` below transpose at the boundary, outside
any timed region of the callers that time them (they time `launch_forward` / `launch_backward`).
"""
from __future__ import annotations

import importlib
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_COPY = os.path.join(HERE, "_ref", "kvax_reference")

_state = {"fa": None, "mc": None, "why": None}


def available() -> tuple[bool, str]:
    if not os.path.isdir(os.path.join(REF_COPY, "kvax", "ops")):
        return False, "no copy of the reference under oracle/_ref/kvax_reference (python -m oracle.make_ref <checkout>)"
    try:
        import torch
        import triton  # noqa: F401
    except Exception as e:  # pragma: no cover
        return False, f"torch / triton not importable: {e}"
    if not torch.cuda.is_available():
        return False, "no CUDA device"
    return True, "ok"


def _install_stubs() -> None:
    import numpy as np
    import torch

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    class _Any:
        def __class_getitem__(cls, item):
            return cls

    def _pad(x, widths, constant_values=0):
        flat = []
        for lo, hi in reversed(list(widths)):
            flat += [int(lo), int(hi)]
        return torch.nn.functional.pad(x, flat, value=constant_values)

    def _dev():
        return torch.device("cuda", torch.cuda.current_device())

    def _shape(s):
        return (int(s),) if isinstance(s, (int, np.integer)) else tuple(int(v) for v in s)

    jnp = mod(
        "jax.numpy", int32=torch.int32, float32=torch.float32, bfloat16=torch.bfloat16, float16=torch.float16,
        ndarray=torch.Tensor, dtype=lambda d: d, iinfo=lambda d: np.iinfo(np.int32) if d is torch.int32 else torch.iinfo(d),
        zeros=lambda shape, dtype=torch.float32: torch.zeros(_shape(shape), dtype=dtype, device=_dev()),
        ones=lambda shape, dtype=torch.float32: torch.ones(_shape(shape), dtype=dtype, device=_dev()),
        concatenate=lambda xs, axis=0: torch.cat(list(xs), dim=axis),
        sum=lambda x, axis=None, dtype=None: torch.sum(x, dim=axis, dtype=dtype),
        where=torch.where, pad=_pad, asarray=torch.as_tensor, arange=lambda *a, **k: torch.arange(*a, device=_dev(), **k))

    class ShapeDtypeStruct:
        def __init__(self, shape, dtype):
            self.shape, self.dtype = tuple(int(v) for v in shape), dtype

    class _CustomVjp:
        def __init__(self, f):
            self.f = f

        def __call__(self, *a, **k):
            return self.f(*a, **k)

        def defvjp(self, *a, **k):
            pass

    jax = mod("jax", numpy=jnp, ShapeDtypeStruct=ShapeDtypeStruct, Array=torch.Tensor)
    jax.custom_vjp = lambda f=None, **kw: (_CustomVjp(f) if f is not None else (lambda g: _CustomVjp(g)))
    jax.jit = lambda f=None, **kw: (f if f is not None else (lambda g: g))
    mod("jax.sharding", Mesh=_Any, PartitionSpec=tuple)
    sm = mod("jax.experimental.shard_map", Specs=_Any, shard_map=None)
    jax.experimental = mod("jax.experimental", shard_map=sm)
    mod("jax.interpreters", pxla=mod("jax.interpreters.pxla"))
    mod("jax.ad_checkpoint", checkpoint_name=lambda x, n: x)
    nop = lambda *a, **k: None
    mod("chex", ArrayDevice=torch.Tensor, PRNGKey=torch.Tensor, assert_shape=nop, assert_rank=nop,
        assert_axis_dimension_comparator=nop, assert_is_divisible=nop, assert_equal_shape_prefix=nop,
        assert_axis_dimension=nop, assert_equal_shape=nop)

    def strides_from_shape(shape):
        st, acc = [], 1
        for d in reversed(tuple(shape)):
            st.append(acc)
            acc *= int(d)
        return tuple(reversed(st))

    def triton_call(*args, kernel, out_shape, grid, debug=False, num_warps=None, num_stages=None, zeroed_outputs=None,
                    input_output_aliases=None, **constexprs):
        """Launch `kernel[grid]` on torch tensors: positional arguments, then the outputs, then the
        compile-time parameters, as jax_triton does.  Outputs start at zero (a superset of
        `zeroed_outputs`)."""
        single = not isinstance(out_shape, (list, tuple))
        shapes = [out_shape] if single else list(out_shape)
        ins = [a.contiguous() if isinstance(a, torch.Tensor) else a for a in args]
        outs = [torch.zeros(s.shape, dtype=s.dtype, device=_dev()) for s in shapes]
        opts = {}
        if num_warps is not None:
            opts["num_warps"] = int(num_warps)
        if num_stages is not None:
            opts["num_stages"] = int(num_stages)
        g = grid if callable(grid) else tuple(int(x) for x in (grid if isinstance(grid, (tuple, list)) else (grid,)))
        kernel[g](*ins, *outs, **constexprs, **opts)
        return outs[0] if single else tuple(outs)

    mod("jax_triton", triton_call=triton_call, cdiv=lambda a, b: (a + b - 1) // b,
        next_power_of_2=lambda x: 1 << (int(x) - 1).bit_length(), strides_from_shape=strides_from_shape)

    # kvax as a namespace package over the copy, so that kvax/__init__.py is not executed
    for name in ("kvax", "kvax.ops", "kvax.utils"):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(REF_COPY, *name.split("."))]
        sys.modules[name] = m


def load():
    """Imports the reference's attention module from the copy; returns (flash_attention_triton module,
    FlashAttentionParamsConfig)."""
    if _state["fa"] is None:
        ok, why = available()
        if not ok:
            raise RuntimeError(why)
        os.environ.setdefault("TRITON_ALLOW_NON_CONSTEXPR_GLOBALS", "1")
        if os.environ.get("TRITON_INTERPRET") == "1":
            raise RuntimeError("TRITON_INTERPRET=1 is set: this harness runs the compiled kernels")
        _install_stubs()
        _state["fa"] = importlib.import_module("kvax.ops.flash_attention_triton")
        _state["common"] = importlib.import_module("kvax.utils.common")
    return _state["fa"], _state["common"].FlashAttentionParamsConfig


def params(query_block_size, kv_block_size, num_warps=8, num_stages=3):
    """The reference's H100 setting is 128/128 (64/128 backward), 8 warps, 3 stages
    (kvax/utils/common.py:29-37); any other GPU falls back to 64/64/4 warps (:38-39)."""
    _, cfg = load()
    return cfg(query_block_size=query_block_size, kv_block_size=kv_block_size, num_warps=num_warps, num_stages=num_stages)


def to_bhsd(x):
    return x.permute(0, 2, 1, 3).contiguous()


def mask_tuple(masks):
    """AttentionMask objects of this repository -> the nested tuples the reference's host code unpacks."""
    return tuple(tuple(t.contiguous() for t in m.flatten()) for m in masks)


def launch_forward(q_t, k_t, v_t, q_pos, q_seg, kv_pos, kv_seg, masks, scale, fwd_params, bwd_params, sequential=False):
    """(B, H, S, D) tensors in, reference's (out, residuals) out: exactly flash_attention_triton_forward."""
    fa, _ = load()
    return fa.flash_attention_triton_forward(q_t, k_t, v_t, q_pos, q_seg, kv_pos, kv_seg, masks, float(scale), None,
                                             fwd_params, bwd_params, assume_sequential_positions=sequential)


def launch_backward(res, dout_t, scale, fwd_params, bwd_params, sequential=False, memory_optimized=False):
    fa, _ = load()
    return fa.flash_attention_backward(float(scale), None, fwd_params, bwd_params, sequential, memory_optimized, True,
                                       None, False, res, dout_t)


def forward_backward(q, k, v, dout, q_pos, q_seg, kv_pos, kv_seg, masks, scale, fwd_params, bwd_params, sequential=False):
    """Public-layout convenience: (B, S, H, D) tensors in; returns out, lse2, dq, dk (fp32), dv (fp32) in
    the public layout."""
    q_t, k_t, v_t, do_t = (to_bhsd(x) for x in (q, k, v, dout))
    out_t, res = launch_forward(q_t, k_t, v_t, q_pos, q_seg, kv_pos, kv_seg, mask_tuple(masks), scale, fwd_params,
                                bwd_params, sequential)
    grads = launch_backward(res, do_t, scale, fwd_params, bwd_params, sequential)
    back = lambda x: x.permute(0, 2, 1, 3).contiguous()
    return back(out_t), res[-1], back(grads[0]), back(grads[1]), back(grads[2])
