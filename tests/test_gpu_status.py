"""Device-side failures surface as a status code, never as a trap or a hang.

Every barrier wait inside the attention kernels is bounded.  `kvax_b200_wait_probe` runs the same
wait routine on a barrier nobody arrives on, with a budget of a millisecond: the wait gives up,
the kernel writes 100 + barrier id to the status word and returns, the context stays usable and
the public API reports the failure at its next entry."""
import ctypes as C

import pytest
import torch

from oracle import generators as gen

pytestmark = pytest.mark.gpu


def _probe(bar_id, budget_ns=1_000_000):
    from kvax_b200 import _lib
    from kvax_b200._status import status_word
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    word, word_ptr = status_word(dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.kvax_b200_wait_probe(word_ptr, done.data_ptr(), budget_ns, bar_id, torch.cuda.current_stream(dev).cuda_stream)
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()
    return word, int(done.item()), t0.elapsed_time(t1)


def test_bounded_wait_runs_out_and_returns():
    import kvax_b200 as kv
    from kvax_b200 import _lib
    kv.check_last_status(synchronize=True)                  # clean slate
    word, done, ms = _probe(bar_id=7)
    assert done == 2, "the probe kernel must reach its end after giving up"
    assert int(word[0]) == 107                              # 100 + barrier id, visible on the host without a copy
    assert ms < 100.0, f"a 1 ms budget took {ms} ms"
    assert kv.last_status() == 107
    with pytest.raises(_lib.KvaxB200Error, match="107"):
        kv.check_last_status()
    assert kv.last_status() == 0                            # reported once, then cleared

    # the first failure stays: a second one does not overwrite it
    _probe(bar_id=3)
    _probe(bar_id=9)
    assert kv.last_status() == 103
    # the public API refuses to go on after a device-side failure ...
    cfg = gen.small_config(seq=256, batch=1, hq=2, hkv=1, head_dim=128)
    inp = gen.make_inputs(cfg, seed=1)
    dev = torch.device("cuda", 0)
    q, k, v = (torch.from_numpy(inp[n]).to(dev).to(torch.bfloat16) for n in ("q", "k", "v"))
    p, s = torch.from_numpy(inp["positions"]).to(dev), torch.from_numpy(inp["segment_ids"]).to(dev)
    params = kv.FlashAttentionParamsConfig(128, 128)
    mesh = kv.Mesh(("data", "context"), (1, 1), rank=0)
    with mesh, kv.attention_specs(("data", None, None, None), ("data", None, None, None)):
        masks = kv.create_attention_mask(p, s, p, s, fwd_params=params)
        with pytest.raises(_lib.KvaxB200Error, match="103"):
            kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params)
        # ... and the context is intact: the next call works
        out = kv.flash_attention(q, k, v, p, s, p, s, masks, scale=inp["scale"], fwd_params=params)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out.float()).all())
    kv.check_last_status(synchronize=True)


def test_probe_rejects_bad_arguments():
    from kvax_b200 import _lib
    lib = _lib.load()
    assert lib.kvax_b200_wait_probe(None, None, 1000, 0, None) == -1
