"""Host-side logic that needs no GPU: spec registry, mesh, context-parallel offsets,
error conventions."""
import pytest
import torch

import kvax_b200 as kv
from kvax_b200.ops.flash_attention import context_offsets
from kvax_b200.utils import specs as sp
from kvax_b200.utils.sharding import get_query_context_mesh_axis_size


def test_specs_validation_and_restore():
    with pytest.raises(ValueError):
        sp.get_attention_specs()
    with pytest.raises(ValueError):
        sp.set_attention_specs(("d", None, None), ("d", None, None, None))
    with pytest.raises(ValueError):
        sp.set_attention_specs(("a", None, None, None), ("b", None, None, None))
    with pytest.raises(ValueError):
        sp.set_attention_specs(("a", "c", None, None), ("a", "c", None, None))       # sharded kv sequence
    with pytest.raises(ValueError):
        sp.set_attention_specs(("a", None, None, "m"), ("a", None, None, "m"))       # sharded head_dim
    with kv.attention_specs(("data", "context", "model", None), ("data", None, "model", None)):
        assert sp.get_attention_specs().query_specs[1] == "context"
        with kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
            assert sp.get_attention_specs().query_specs[1] is None
        assert sp.get_attention_specs().query_specs[1] == "context"
    with pytest.raises(ValueError):
        sp.get_attention_specs()


def test_mesh_coordinates_and_axis_lookup():
    m = kv.Mesh(("data", "context", "model"), (2, 4, 2), rank=13)   # 13 = (1*4 + 2)*2 + 1
    assert (m.coordinate("data"), m.coordinate("context"), m.coordinate("model")) == (1, 2, 1)
    with kv.attention_specs(("data", "context", "model", None), ("data", None, "model", None)):
        assert get_query_context_mesh_axis_size(m) == 4
        with m:
            assert get_query_context_mesh_axis_size(None) == 4
        with pytest.raises(ValueError):
            get_query_context_mesh_axis_size(None)                   # no mesh in scope
    with kv.attention_specs(("data", "ctx", None, None), ("data", None, None, None)):
        with pytest.raises(ValueError):
            get_query_context_mesh_axis_size(m)                      # axis not in the mesh


def test_context_offsets_give_global_indices():
    """offset + local index must equal the global index of the token, for both halves
    (rank r holds chunk r then chunk 2CP-1-r of the permuted sequence)."""
    for cp in (2, 4, 8):
        S = 1024 * cp
        loc = S // cp
        half = loc // 2
        for r in range(cp):
            first, second = context_offsets(r, cp, loc, permuted=True)
            assert first + 0 == r * half
            assert second + half == (2 * cp - 1 - r) * half
            f2, s2 = context_offsets(r, cp, loc, permuted=False)
            assert f2 == s2 == r * loc
    assert context_offsets(0, 1, 512, True) == (0, 0)


def test_cpu_tensors_are_rejected_loudly():
    x = torch.zeros(2, 16, dtype=torch.int32)
    m = kv.Mesh(("data", "context"), (1, 2), rank=0)
    with m, kv.attention_specs(("data", "context", None, None), ("data", None, None, None)):
        with pytest.raises(RuntimeError):
            kv.permute_tokens_context_parallelism(x)
        with pytest.raises(RuntimeError):
            kv.create_attention_mask(x, x, x, x, fwd_params=kv.FlashAttentionParamsConfig(8, 8))


def test_flop_formula():
    from kvax_b200.utils.math import get_multi_head_attention_tflops as f
    base = f(2, 1024, 1024, 8, 128, 128, causal=False)
    assert base == pytest.approx(2 * 8 * 2 * 256 * 1024 * 1024 / 1e12)
    assert f(2, 1024, 1024, 8, 128, 128, causal=True, backward_pass=True) == pytest.approx(base * 0.5 * 3.5)
    assert f(2, 1024, 1024, 8, 128, 128, causal=False, forward_pass=False, backward_pass=True) == pytest.approx(base * 2.5)
    with pytest.raises(ValueError):
        f(1, 1, 1, 1, 1, 1, causal=False, forward_pass=False, backward_pass=False)


def test_benchmark_cli_commands_and_segment_lengths():
    """The benchmark harness exposes the reference's four commands with its option names
    (benchmarks.py:34-407) and the reference's segment-length generator."""
    from click.testing import CliRunner

    from kvax_b200 import benchmarks as bm
    res = CliRunner().invoke(bm.cli, ["--help"])
    assert res.exit_code == 0
    for cmd in ("mha", "mha_bwd", "mha_cp", "mha_cp_bwd"):
        assert cmd in res.output
    res = CliRunner().invoke(bm.cli, ["mha_cp_bwd", "--help"])
    for opt in ("--num-iters", "--batch-size", "--query-seq-len", "--kv-seq-len", "--num-heads", "--num-kv-heads",
                "--qk-head-dim", "--value-head-dim", "--assume-sequential-positions", "--num-segments",
                "--permute-tokens-for-load-balance", "--show-attention-mask"):
        assert opt in res.output
    assert bm.generate_random_segments_lengths(4096, 1) is None
    a = bm.generate_random_segments_lengths(4096, 7)
    assert len(a) == 7 and sum(a) == 4096 and min(a) >= 1 and a == bm.generate_random_segments_lengths(4096, 7)
    pos, seg = bm.make_positions_and_segments(2, 64, [10, 20, 34], 5)
    assert pos.shape == (2, 64) and int(pos[1, 63]) == 63
    assert seg[0, :10].eq(0).all() and seg[0, 10:30].eq(1).all() and seg[0, 30:59].eq(2).all() and seg[0, 59:].eq(-1).all()


def test_context_parallel_mode_switch():
    import kvax_b200 as kv
    assert kv.get_context_parallel_mode() == "auto"
    for mode in ("all_gather", "head_exchange", "auto"):
        kv.set_context_parallel_mode(mode)
        assert kv.get_context_parallel_mode() == mode
    with pytest.raises(ValueError):
        kv.set_context_parallel_mode("ring")
    assert kv.get_context_parallel_mode() == "auto"


def test_context_parallel_overlap_switch_and_remote_chunk_order():
    """The overlap switch of the all-gather schedule, and the order in which a rank finds the chunks of the other
    ranks in a rank-major all-gather: ascending in natural order, its own two left out."""
    import kvax_b200 as kv
    from kvax_b200.ops.flash_attention import _chunk_of, _remote_slots
    assert kv.get_context_parallel_overlap() is False
    kv.set_context_parallel_overlap(True)
    assert kv.get_context_parallel_overlap() is True
    kv.set_context_parallel_overlap(False)
    for cp in (2, 4, 8):
        for permuted in (True, False):
            for rank in range(cp):
                slots = _remote_slots(rank, cp, permuted)
                assert len(slots) == 2 * cp - 2 and len(set(slots)) == len(slots)
                assert all(s // 2 != rank for s in slots)                       # none of its own
                chunks = [_chunk_of(s // 2, s % 2, cp, permuted) for s in slots]
                assert chunks == sorted(chunks)                                 # natural order


def test_fp32_bridge_scales_small_output_gradients():
    """The casts around a call on fp32 tensors: an output gradient far below the fp16 range is multiplied by a power
    of two on its way in and the input gradients are divided by it on their way out, so a linear map in fp16 gives
    the fp32 gradient to fp16 precision (no underflow), and exact zeros stay zeros."""
    from kvax_b200.ops.flash_attention import _FromOperand, _GradScaleBox, _ToOperand
    torch.manual_seed(0)
    x = torch.randn(64, 32, requires_grad=True)
    w = torch.randn(32, 16)
    box = _GradScaleBox()
    xo = _ToOperand.apply(x, torch.float16, box)
    y16 = (xo.float() @ w).to(torch.float16)             # stands in for the fp16 kernels (linear in x)
    y = _FromOperand.apply(y16, torch.float32, box)
    assert y.dtype == torch.float32
    g = torch.randn(64, 16) * 1e-7                       # below the smallest normal fp16 number (6e-5)
    y.backward(g)
    ref = g @ w.t()
    assert x.grad.dtype == torch.float32
    rel = (x.grad - ref).norm() / ref.norm()
    assert rel < 2e-3, rel
    # without the scaling the same gradient would be flushed: every element of g is below half the smallest subnormal?
    assert float(g.abs().max()) < 6e-5
    x.grad = None
    box2 = _GradScaleBox()
    y2 = _FromOperand.apply(_ToOperand.apply(x, torch.float16, box2) * 1.0, torch.float32, box2)
    y2.backward(torch.zeros_like(y2))
    assert float(x.grad.abs().max()) == 0.0


def test_fp32_operand_dtype_switch():
    assert kv.get_fp32_operand_dtype() == "auto"
    kv.set_fp32_operand_dtype("bfloat16")
    assert kv.get_fp32_operand_dtype() == "bfloat16"
    kv.set_fp32_operand_dtype("auto")
    with pytest.raises(ValueError):
        kv.set_fp32_operand_dtype("float64")
    with pytest.raises(ValueError):
        kv.set_head_exchange_transport("smoke signals")
