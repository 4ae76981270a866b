"""ctypes binding of libkvax_b200.so (the C ABI declared in include/kvax_b200.h).

There is no CPU or library fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkvax_b200.so")

EXPORTS = (
    "kvax_b200_version",
    "kvax_b200_error_string",
    "kvax_b200_mask_workspace_bytes",
    "kvax_b200_mask_build",
    "kvax_b200_mask_build_static",
    "kvax_b200_permute_tokens",
    "kvax_b200_regroup_heads",
    "kvax_b200_attn_merge",
    "kvax_b200_peer_buffer_alloc",
    "kvax_b200_peer_buffer_free",
    "kvax_b200_peer_buffer_export",
    "kvax_b200_peer_buffer_open",
    "kvax_b200_peer_buffer_close",
    "kvax_b200_head_exchange",
    "kvax_b200_attn_fwd_workspace_bytes",
    "kvax_b200_attn_fwd",
    "kvax_b200_attn_bwd_workspace_bytes",
    "kvax_b200_attn_bwd",
    "kvax_b200_wait_probe",
    "kvax_b200_host_word_device_pointer",
)

BWD_TWO_KERNEL = 1
BWD_DKDV_16BIT = 2
FWD_ONE_TILE, FWD_TILE_PAIRS, FWD_HEAD_PAIRS, FWD_EMPTY_LSE_INF = 1, 2, 4, 8          # kvax_b200_attn_fwd_params.flags
MAX_PEERS, PEER_HANDLE_BYTES = 16, 64
DTYPE_BF16, DTYPE_F16 = 0, 1               # kvax_b200_attn_shape.dtype

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class MaskDesc(C.Structure):
    _fields_ = [("q_block", i32), ("kv_block", i32), ("kv_outer", i32), ("reserved", i32),
                ("lower", vp), ("upper", vp), ("lower_full", vp), ("upper_full", vp)]


class MaskParams(C.Structure):
    _fields_ = [("q_positions", vp), ("q_segment_ids", vp), ("kv_positions", vp), ("kv_segment_ids", vp),
                ("batch", i32), ("q_len", i32), ("kv_len", i32), ("skip_pad_tokens", i32),
                ("n_masks", i32), ("reserved", i32), ("masks", MaskDesc * 3)]


class BlockMask(C.Structure):
    _fields_ = [("lower", vp), ("upper", vp), ("lower_full", vp), ("upper_full", vp),
                ("q_block", i32), ("kv_block", i32)]


class AttnShape(C.Structure):
    _fields_ = [("batch", i32), ("q_len", i32), ("kv_len", i32), ("q_heads", i32), ("kv_heads", i32),
                ("head_dim", i32), ("dtype", i32), ("assume_sequential_positions", i32),
                ("scale", f32), ("reserved", i32),
                ("q_strides", i64 * 3), ("k_strides", i64 * 3), ("v_strides", i64 * 3), ("o_strides", i64 * 3),
                ("q_positions", vp), ("q_segment_ids", vp), ("kv_positions", vp), ("kv_segment_ids", vp),
                ("q_global_offset_first", i32), ("q_global_offset_second", i32)]


class AttnFwdParams(C.Structure):
    _fields_ = [("shape", AttnShape), ("q", vp), ("k", vp), ("v", vp), ("mask", BlockMask),
                ("out", vp), ("lse", vp), ("status", vp), ("stages", i32), ("flags", i32)]


class AttnBwdParams(C.Structure):
    _fields_ = [("shape", AttnShape), ("q", vp), ("k", vp), ("v", vp), ("out", vp), ("dout", vp), ("lse", vp),
                ("mask_dq", BlockMask), ("mask_dkdv", BlockMask), ("dq", vp), ("dk", vp), ("dv", vp), ("status", vp),
                ("stages", i32), ("flags", i32), ("dq_strides", i64 * 3)]


_lib = None


class KvaxB200Error(RuntimeError):
    pass


def load() -> C.CDLL:
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KvaxB200Error(
            f"{LIB_PATH} is missing: build it with `python -m kvax_b200.build` (needs nvcc). "
            "kvax_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.kvax_b200_version.restype = C.c_char_p
    lib.kvax_b200_error_string.restype = C.c_char_p
    lib.kvax_b200_error_string.argtypes = [C.c_int]
    lib.kvax_b200_mask_workspace_bytes.restype = C.c_size_t
    lib.kvax_b200_mask_workspace_bytes.argtypes = [C.POINTER(MaskParams)]
    lib.kvax_b200_mask_build.restype = C.c_int
    lib.kvax_b200_mask_build.argtypes = [C.POINTER(MaskParams), vp, C.c_size_t, vp]
    lib.kvax_b200_mask_build_static.restype = C.c_int
    lib.kvax_b200_mask_build_static.argtypes = [C.POINTER(MaskParams), vp]
    lib.kvax_b200_permute_tokens.restype = C.c_int
    lib.kvax_b200_permute_tokens.argtypes = [vp, vp, i64, i64, i64, i32, i32, vp]
    lib.kvax_b200_regroup_heads.restype = C.c_int
    lib.kvax_b200_regroup_heads.argtypes = [vp, vp, i64, i32, i32, i64, i32, vp]
    lib.kvax_b200_attn_merge.restype = C.c_int
    lib.kvax_b200_attn_merge.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32, i32, vp]
    lib.kvax_b200_peer_buffer_alloc.restype = C.c_int
    lib.kvax_b200_peer_buffer_alloc.argtypes = [C.c_size_t, C.POINTER(vp)]
    lib.kvax_b200_peer_buffer_free.restype = C.c_int
    lib.kvax_b200_peer_buffer_free.argtypes = [vp]
    lib.kvax_b200_peer_buffer_export.restype = C.c_int
    lib.kvax_b200_peer_buffer_export.argtypes = [vp, C.c_char_p]
    lib.kvax_b200_peer_buffer_open.restype = C.c_int
    lib.kvax_b200_peer_buffer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.kvax_b200_peer_buffer_close.restype = C.c_int
    lib.kvax_b200_peer_buffer_close.argtypes = [vp]
    lib.kvax_b200_head_exchange.restype = C.c_int
    lib.kvax_b200_head_exchange.argtypes = [vp, C.POINTER(vp), i64, i64, i32, i32, i32, i64, i32, i32, vp]
    lib.kvax_b200_attn_fwd_workspace_bytes.restype = C.c_size_t
    lib.kvax_b200_attn_fwd_workspace_bytes.argtypes = [C.POINTER(AttnFwdParams)]
    lib.kvax_b200_attn_fwd.restype = C.c_int
    lib.kvax_b200_attn_fwd.argtypes = [C.POINTER(AttnFwdParams), vp, C.c_size_t, vp]
    lib.kvax_b200_attn_bwd_workspace_bytes.restype = C.c_size_t
    lib.kvax_b200_attn_bwd_workspace_bytes.argtypes = [C.POINTER(AttnBwdParams)]
    lib.kvax_b200_attn_bwd.restype = C.c_int
    lib.kvax_b200_attn_bwd.argtypes = [C.POINTER(AttnBwdParams), vp, C.c_size_t, vp]
    lib.kvax_b200_wait_probe.restype = C.c_int
    lib.kvax_b200_wait_probe.argtypes = [vp, vp, i64, i32, vp]
    lib.kvax_b200_host_word_device_pointer.restype = C.c_int
    lib.kvax_b200_host_word_device_pointer.argtypes = [vp, C.POINTER(vp)]
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().kvax_b200_error_string(code).decode()
        raise KvaxB200Error(f"{what} failed: {msg} (code {code})")
