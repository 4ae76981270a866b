"""JAX front end of the CUDA kernels: the drop-in for `kvax.ops` / `kvax.utils` inside a JAX program.

`create_attention_mask` and `flash_attention` keep the reference's signatures
(kvax/ops/mask_creator.py:377-387, kvax/ops/flash_attention_triton.py:2027-2045).  Where the reference
launches Triton kernels through `jt.triton_call` (mask_creator.py:280, 296;
flash_attention_triton.py:1517, 1692, 1740, 1778, 1819) this module calls the XLA FFI handlers of
kvax_b200/csrc/ffi_xla.cc with `jax.ffi.ffi_call`; everything around them (padding rules, custom_vjp,
shard_map over the attention specs, all-gather of K / V and reduce-scatter of dK / dV over the
context-parallel axis) is ordinary JAX, as in the reference.  Scratch memory and the status word are
extra results of each call: XLA allocates them, the handlers allocate nothing.

Importing this module needs jax and libkvax_b200_xla_ffi.so (built by `python -m kvax_b200.build` when
the XLA FFI headers are available).  Neither exists in the image this repository is developed in, so
this front end is written against the published `jax.ffi` API and has not been executed here; the
kernels themselves are exercised through the same C ABI by the torch front end (`kvax_b200.ops`) and
its tests.
"""
from __future__ import annotations

import ctypes
import functools
import os

import jax
import jax.numpy as jnp
import numpy as np
from jax.experimental.shard_map import shard_map
from jax.sharding import PartitionSpec as P

from kvax_b200 import _lib
from kvax_b200.utils.common import PADDING_SEGMENT_ID, FlashAttentionParamsConfig, get_default_flash_attention_params
from kvax_b200.utils.specs import get_attention_specs

_HERE = os.path.dirname(os.path.abspath(__file__))
FFI_LIB_PATH = os.path.join(os.path.dirname(_HERE), "libkvax_b200_xla_ffi.so")
_TARGETS = ("kvax_b200_ffi_mask_build", "kvax_b200_ffi_permute_tokens", "kvax_b200_ffi_attn_fwd", "kvax_b200_ffi_attn_bwd")
_registered = False


def register() -> None:
    """Registers the four FFI targets with XLA (once per process)."""
    global _registered
    if _registered:
        return
    if not os.path.exists(FFI_LIB_PATH):
        raise _lib.KvaxB200Error(f"{FFI_LIB_PATH} is missing: build it with `python -m kvax_b200.build` on a machine "
                                 "with jaxlib (XLA FFI headers).  There is no fallback.")
    lib = ctypes.CDLL(FFI_LIB_PATH)
    for name in _TARGETS:
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(lib, name)), platform="CUDA")
    _registered = True


def _cdiv(a, b):
    return (a + b - 1) // b


# ------------------------------------------------------------------------------------------------------
# masks
# ------------------------------------------------------------------------------------------------------
def _mask_single_device(q_pos, q_seg, kv_pos, kv_seg, fwd, bwd, calc_bwd_mask, skip_pad_tokens):
    """One device's masks: stacked (4, B, 1, n) int32 arrays (lower, upper, lower_full, upper_full)."""
    B, Sq = q_pos.shape
    Skv = kv_pos.shape[1]
    p = _lib.MaskParams()
    p.batch, p.q_len, p.kv_len, p.n_masks = B, Sq, Skv, 3 if calc_bwd_mask else 1
    specs = [(fwd.query_block_size, fwd.kv_block_size, False)]
    if calc_bwd_mask:
        specs += [(bwd.kv_block_size, bwd.query_block_size, False), (bwd.query_block_size, bwd.kv_block_size, True)]
    for i, (bq, bk, kv_outer) in enumerate(specs):
        p.masks[i].q_block, p.masks[i].kv_block, p.masks[i].kv_outer = bq, bk, int(kv_outer)
    ws_bytes = int(_lib.load().kvax_b200_mask_workspace_bytes(p))
    n = [_cdiv(Skv, bk) if kv_outer else _cdiv(Sq, bq) for (bq, bk, kv_outer) in specs] + [0, 0]
    shapes = [jax.ShapeDtypeStruct((4, B, 1, n[i]) if n[i] else (0,), jnp.int32) for i in range(3)]
    shapes.append(jax.ShapeDtypeStruct((ws_bytes,), jnp.uint8))
    bq_b, bk_b = (bwd.query_block_size, bwd.kv_block_size) if bwd is not None else (fwd.query_block_size, fwd.kv_block_size)
    res = jax.ffi.ffi_call("kvax_b200_ffi_mask_build", shapes)(
        q_pos.astype(jnp.int32), q_seg.astype(jnp.int32), kv_pos.astype(jnp.int32), kv_seg.astype(jnp.int32),
        fwd_q_block=np.int32(fwd.query_block_size), fwd_kv_block=np.int32(fwd.kv_block_size),
        bwd_q_block=np.int32(bq_b), bwd_kv_block=np.int32(bk_b),
        calc_bwd_mask=bool(calc_bwd_mask), skip_pad_tokens=bool(skip_pad_tokens))
    return tuple(res[:3 if calc_bwd_mask else 1])


def create_attention_mask(query_positions, query_segment_ids, kv_positions, kv_segment_ids, fwd_params=None,
                          bwd_params=None, calc_bwd_mask=False, skip_pad_tokens=True, mesh=None):
    """Tuple of one or three masks; each mask is a tuple (lower, upper, lower_full, upper_full) of int32
    arrays with the global shapes of the reference: forward / dq masks (batch, 1, n_q_blocks) sharded
    over the context axis on their last dimension, the dkdv mask (batch, CP, n_kv_blocks) with one row
    per context-parallel rank (mask_creator.py:155-199, 338-374)."""
    register()
    from kvax_b200.utils.sharding import _check_mesh_or_get_global, get_query_context_mesh_axis_name
    mesh = _check_mesh_or_get_global(mesh)
    specs = get_attention_specs()
    fwd = fwd_params or get_default_flash_attention_params(backward=False)
    axis = get_query_context_mesh_axis_name(mesh)
    batch = specs.query_specs[0]
    q_tok, kv_tok = P(batch, axis), P(batch, None)
    fwd_spec, dkdv_spec = P(None, batch, None, axis), P(None, batch, axis, None)
    out_specs = (fwd_spec,) + ((fwd_spec, dkdv_spec) if calc_bwd_mask else ())

    def per_device(qp, qs, kp, ks):
        return _mask_single_device(qp, qs, kp, ks, fwd, bwd_params, calc_bwd_mask, skip_pad_tokens)

    stacked = shard_map(per_device, mesh=mesh, in_specs=(q_tok, q_tok, kv_tok, kv_tok), out_specs=out_specs, check_rep=False)(
        query_positions, query_segment_ids, kv_positions, kv_segment_ids)
    return tuple(tuple(m[i] for i in range(4)) for m in stacked)


# ------------------------------------------------------------------------------------------------------
# attention on one device
# ------------------------------------------------------------------------------------------------------
def _shape_params(cls, q, k, v):
    p = cls()
    s = p.shape
    B, Sq, Hq, D = q.shape
    s.batch, s.q_len, s.kv_len, s.q_heads, s.kv_heads, s.head_dim = B, Sq, k.shape[1], Hq, k.shape[2], D
    s.scale = 1.0
    return p


def _stack(mask):
    return jnp.stack([m.astype(jnp.int32) for m in mask])


def _fwd_call(q, k, v, q_pos, q_seg, kv_pos, kv_seg, mask_fwd, scale, fwd, sequential, offsets):
    B, Sq, Hq, D = q.shape
    ws = int(_lib.load().kvax_b200_attn_fwd_workspace_bytes(_shape_params(_lib.AttnFwdParams, q, k, v)))
    shapes = [jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct((B, Hq, Sq), jnp.float32),
              jax.ShapeDtypeStruct((ws,), jnp.uint8), jax.ShapeDtypeStruct((1,), jnp.int32)]
    out, lse, _, status = jax.ffi.ffi_call("kvax_b200_ffi_attn_fwd", shapes)(
        q, k, v, q_pos, q_seg, kv_pos, kv_seg, _stack(mask_fwd), scale=np.float32(scale),
        q_block=np.int32(fwd.query_block_size), kv_block=np.int32(fwd.kv_block_size),
        assume_sequential_positions=bool(sequential), q_global_offset_first=np.int32(offsets[0]),
        q_global_offset_second=np.int32(offsets[1]))
    return out, lse, status


def _bwd_call(q, k, v, out, dout, lse, q_pos, q_seg, kv_pos, kv_seg, mask_dq, mask_dkdv, scale, bwd, sequential, offsets,
              two_kernel):
    p = _shape_params(_lib.AttnBwdParams, q, k, v)
    p.flags = _lib.BWD_TWO_KERNEL if two_kernel else 0
    ws = int(_lib.load().kvax_b200_attn_bwd_workspace_bytes(p))
    shapes = [jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct(k.shape, jnp.float32),
              jax.ShapeDtypeStruct(v.shape, jnp.float32), jax.ShapeDtypeStruct((ws,), jnp.uint8),
              jax.ShapeDtypeStruct((1,), jnp.int32)]
    dq, dk, dv, _, status = jax.ffi.ffi_call("kvax_b200_ffi_attn_bwd", shapes)(
        q, k, v, out, dout, lse, q_pos, q_seg, kv_pos, kv_seg, _stack(mask_dq), _stack(mask_dkdv),
        scale=np.float32(scale), q_block=np.int32(bwd.query_block_size), kv_block=np.int32(bwd.kv_block_size),
        assume_sequential_positions=bool(sequential), q_global_offset_first=np.int32(offsets[0]),
        q_global_offset_second=np.int32(offsets[1]), two_kernel=bool(two_kernel))
    return dq, dk, dv, status


@functools.partial(jax.custom_vjp, nondiff_argnums=(8, 9, 10, 11, 12, 13))
def _attention_single_device(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, scale, fwd, bwd, sequential, offsets, two_kernel):
    return _fwd_call(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks[0], scale, fwd, sequential, offsets)[0]


def _vjp_fwd(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, scale, fwd, bwd, sequential, offsets, two_kernel):
    out, lse, _ = _fwd_call(q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks[0], scale, fwd, sequential, offsets)
    return out, (q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, out, lse)


def _vjp_bwd(scale, fwd, bwd, sequential, offsets, two_kernel, res, dout):
    q, k, v, q_pos, q_seg, kv_pos, kv_seg, masks, out, lse = res
    if len(masks) != 3:
        raise ValueError("Length of mask_tensors should be equal to two")
    dq, dk, dv, _ = _bwd_call(q, k, v, out, dout, lse, q_pos, q_seg, kv_pos, kv_seg, masks[1], masks[2], scale, bwd,
                              sequential, offsets, two_kernel)
    return dq, dk, dv, None, None, None, None, None          # dk / dv stay fp32 until after the cross-device sum


_attention_single_device.defvjp(_vjp_fwd, _vjp_bwd)


# ------------------------------------------------------------------------------------------------------
# public op
# ------------------------------------------------------------------------------------------------------
def flash_attention(query, key, value, query_positions, query_segment_ids, kv_positions, kv_segment_ids, mask,
                    scale=1.0, bias=None, fwd_params=None, bwd_params=None, assume_sequential_positions=False,
                    memory_optimized_gqa_backward=False, permute_tokens_for_load_balance=True, debug=False, mesh=None,
                    two_kernel_backward=False):
    """Attention output (batch, query_seq, heads, head_dim); differentiable in query, key, value.
    Arguments as kvax.ops.flash_attention (flash_attention_triton.py:2027-2045); `two_kernel_backward`
    selects the bit-reproducible backward schedule."""
    register()
    from kvax_b200.utils.sharding import _check_mesh_or_get_global, get_query_context_mesh_axis_name
    if bias is not None:
        raise NotImplementedError("Bias is not supported in Flash multi head attention")
    if mask is None or len(mask) == 0:
        raise ValueError("Length of mask_tensors should be at least equal to one")
    mesh = _check_mesh_or_get_global(mesh)
    specs = get_attention_specs()
    axis = get_query_context_mesh_axis_name(mesh)
    fwd = fwd_params or get_default_flash_attention_params(backward=False)
    bwd = bwd_params or get_default_flash_attention_params(backward=True)
    in_dtype = query.dtype
    q_spec, kv_spec = P(*specs.query_specs), P(*specs.kv_specs)
    batch = specs.query_specs[0]
    q_tok, kv_tok = P(batch, axis), P(batch, None)
    fwd_spec, dkdv_spec = (P(batch, None, axis),) * 4, (P(batch, axis, None),) * 4
    mask_specs = (fwd_spec,) + ((fwd_spec, dkdv_spec) if len(mask) == 3 else ())
    # K and V arrive sharded over the context axis like Q (the caller permuted the tokens); every device needs all of them
    kv_in = P(specs.kv_specs[0], axis, specs.kv_specs[2], specs.kv_specs[3])

    def per_device(q, k, v, qp, qs, kp, ks, masks):
        q, k, v = (t.astype(jnp.bfloat16) for t in (q, k, v))
        offsets = (0, 0)
        if axis is not None:
            cp = jax.lax.psum(1, axis)
            rank = jax.lax.axis_index(axis)
            # all-gather over NVLink; un-permute into natural order (flash_attention_triton.py:2150-2154)
            k, v = (jax.lax.all_gather(t, axis, axis=1, tiled=True) for t in (k, v))
            if permute_tokens_for_load_balance:
                from kvax_b200.jax_binding import permute_tokens
                k, v = (permute_tokens(t, cp, reverse=True) for t in (k, v))
                half = q.shape[1] // 2
                offsets = (rank * half, (2 * cp - rank - 1) * half - half)
            else:
                offsets = (rank * q.shape[1],) * 2
        # `offsets` are traced values under shard_map; they only matter with assume_sequential_positions, which
        # the handlers take as attributes, so that mode needs them static: one trace per rank is not possible
        # under SPMD, hence positions are materialised instead.
        if assume_sequential_positions and axis is not None:
            local = jnp.arange(q.shape[1], dtype=jnp.int32)
            qp = jnp.where(2 * local >= q.shape[1], local + offsets[1], local + offsets[0])[None, :].repeat(q.shape[0], 0)
            kp = jnp.arange(k.shape[1], dtype=jnp.int32)[None, :].repeat(k.shape[0], 0)
            seq, offs = False, (0, 0)
        else:
            seq, offs = assume_sequential_positions, (0, 0)
        out = _attention_single_device(q, k, v, qp.astype(jnp.int32), qs.astype(jnp.int32), kp.astype(jnp.int32),
                                       ks.astype(jnp.int32), masks, float(scale), fwd, bwd, seq, offs, two_kernel_backward)
        return out.astype(in_dtype)

    return shard_map(per_device, mesh=mesh, in_specs=(q_spec, kv_in, kv_in, q_tok, q_tok, kv_tok, kv_tok, mask_specs),
                     out_specs=q_spec, check_rep=False)(
        query, key, value, query_positions, query_segment_ids, kv_positions, kv_segment_ids, tuple(mask))


def permute_tokens(x, cp, reverse=False):
    """Chunk permutation [0, 2cp-1, 1, 2cp-2, ...] of axis 1 (kvax/utils/permutation.py:9-42) or its inverse."""
    register()
    return jax.ffi.ffi_call("kvax_b200_ffi_permute_tokens", jax.ShapeDtypeStruct(x.shape, x.dtype))(
        x, cp=np.int32(cp), reverse=bool(reverse))


__all__ = ["create_attention_mask", "flash_attention", "permute_tokens", "register", "PADDING_SEGMENT_ID",
           "FlashAttentionParamsConfig"]
