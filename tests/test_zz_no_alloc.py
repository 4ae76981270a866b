"""kvax_b200_mask_build_static: the mask builder for callers that cannot supply device
memory (a custom-call handler whose framework owns the allocator, code inside a region
where allocating is not allowed).  Its per-block summaries live in a fixed 4 MiB area of
the library's device image, so the call needs no workspace and allocates nothing.

The test drives both entry points through the C ABI on the same inputs and requires
identical masks (integer outputs: bit-exact), on two calls in a row with different inputs
so that whatever the first call left in the shared area cannot leak into the second.
Collected last on purpose (file name), so a run that stops at the first failure has
already run every other test."""
import numpy as np
import pytest
import torch

from oracle import generators as gen

pytestmark = pytest.mark.gpu


def _params(lib_mod, qp, qs, kp, ks, specs, skip, outs):
    p = lib_mod.MaskParams()
    p.q_positions, p.q_segment_ids = qp.data_ptr(), qs.data_ptr()
    p.kv_positions, p.kv_segment_ids = kp.data_ptr(), ks.data_ptr()
    p.batch, p.q_len, p.kv_len = qp.shape[0], qp.shape[1], kp.shape[1]
    p.skip_pad_tokens, p.n_masks = int(skip), len(specs)
    for i, (bq, bk, kv_outer) in enumerate(specs):
        d = p.masks[i]
        d.q_block, d.kv_block, d.kv_outer = bq, bk, int(kv_outer)
        d.lower, d.upper, d.lower_full, d.upper_full = (outs[i][j].data_ptr() for j in range(4))
    return p


def _both(lib_mod, lib, pos, seg, specs, skip):
    dev = torch.device("cuda", 0)
    qp = torch.from_numpy(pos).to(dev); qs = torch.from_numpy(seg).to(dev)
    B, S = pos.shape

    def outs():
        return [torch.full((4, B, -(-S // (bk if kv_outer else bq))), -7, dtype=torch.int32, device=dev)
                for (bq, bk, kv_outer) in specs]

    stream = torch.cuda.current_stream(dev).cuda_stream
    ref = outs()
    p = _params(lib_mod, qp, qs, qp, qs, specs, skip, ref)
    need = lib.kvax_b200_mask_workspace_bytes(p)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    assert lib.kvax_b200_mask_build(p, ws.data_ptr(), need, stream) == 0
    got = outs()
    p2 = _params(lib_mod, qp, qs, qp, qs, specs, skip, got)
    assert lib.kvax_b200_mask_build_static(p2, stream) == 0
    torch.cuda.synchronize()
    for a, b in zip(got, ref):
        np.testing.assert_array_equal(a.cpu().numpy(), b.cpu().numpy())


def test_static_scratch_variant_matches_workspace_variant_twice():
    from kvax_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    specs = [(128, 128, False), (128, 64, False), (64, 128, True)]
    first = gen.make_inputs(gen.small_config(seq=4096, batch=2, doc_min=100, doc_max=2000), seed=1, with_tensors=False)
    _both(_lib, lib, first["positions"], first["segment_ids"], specs, True)
    # second call: other shapes and contents, same shared area
    second = gen.make_inputs(gen.CONFIGS["c2_llama8b_8k"], seed=2, with_tensors=False, restart_positions=False)
    _both(_lib, lib, second["positions"], second["segment_ids"], specs, False)


def test_static_scratch_variant_rejects_oversized_problems():
    """More blocks than the 4 MiB area holds: a clear error code, nothing launched (the call
    returns before any pointer is used)."""
    from kvax_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    x = torch.zeros((1, 64), dtype=torch.int32, device=dev)
    out = [torch.zeros((4, 1, 1), dtype=torch.int32, device=dev)]
    p = _params(_lib, x, x, x, x, [(64, 64, False)], True, out)
    p.batch, p.q_len, p.kv_len = 4096, 1 << 20, 1 << 20     # 2 * 4096 * 16384 blocks * 16 B >> 4 MiB
    assert lib.kvax_b200_mask_workspace_bytes(p) > (4 << 20)
    assert lib.kvax_b200_mask_build_static(p, None) == -6
    assert b"scratch" in lib.kvax_b200_error_string(-6)
