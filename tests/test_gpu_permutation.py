"""CUDA chunk permutation against the NumPy oracle (bit-exact, any dtype / rank)."""
import numpy as np
import pytest
import torch

from oracle import permutation_oracle as po

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cp", [1, 2, 4, 8])
@pytest.mark.parametrize("shape,dtype", [((2, 4096), torch.int32), ((1, 2048, 8, 128), torch.bfloat16),
                                         ((3, 512, 3), torch.int8), ((2, 256, 5, 6), torch.float32)])
def test_permute_round_trip_and_oracle(cp, shape, dtype):
    import kvax_b200 as kv
    g = torch.Generator().manual_seed(1)
    x = torch.randint(-100, 100, shape, generator=g).to(dtype)
    mesh = kv.Mesh(("data", "context"), (1, cp), rank=0)
    with mesh, kv.attention_specs(("data", "context", None, None), ("data", None, None, None)):
        y = kv.permute_tokens_context_parallelism(x.cuda())
        z = kv.unpermute_tokens_context_parallelism(y)
        ya, yb = kv.permute_tokens_context_parallelism((x.cuda(), x.cuda()))
    ref = po.permute(x.view(torch.uint8).numpy() if dtype == torch.bfloat16 else x.numpy(), cp) \
        if dtype != torch.bfloat16 else None
    if dtype == torch.bfloat16:
        ref = po.permute(x.view(torch.int16).numpy(), cp)
        np.testing.assert_array_equal(y.cpu().view(torch.int16).numpy(), ref)
    else:
        np.testing.assert_array_equal(y.cpu().numpy(), ref)
    assert torch.equal(z.cpu(), x)
    assert torch.equal(ya, y) and torch.equal(yb, y)


def test_known_chunk_orders():
    from kvax_b200.utils.permutation import generate_shard_indices
    assert generate_shard_indices(4) == [0, 3, 1, 2]
    assert generate_shard_indices(8) == [0, 7, 1, 6, 2, 5, 3, 4]
    assert generate_shard_indices(4, reverse=True) == [0, 2, 3, 1]
