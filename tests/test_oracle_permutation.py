import numpy as np

from oracle import permutation_oracle as po


def test_known_orders():
    assert po.shard_indices(4).tolist() == [0, 3, 1, 2]
    assert po.shard_indices(8).tolist() == [0, 7, 1, 6, 2, 5, 3, 4]
    assert po.shard_indices(16).tolist() == [0, 15, 1, 14, 2, 13, 3, 12, 4, 11, 5, 10, 6, 9, 7, 8]


def test_round_trip_and_rank_ownership():
    x = np.arange(2 * 64 * 3).reshape(2, 64, 3)
    for cp in (1, 2, 4, 8):
        y = po.permute(x, cp)
        np.testing.assert_array_equal(po.unpermute(y, cp), x)
        chunk = 64 // (2 * cp)
        for r in range(cp):  # rank r holds chunk r then chunk 2cp-1-r
            loc = y[:, r * 2 * chunk:(r + 1) * 2 * chunk]
            np.testing.assert_array_equal(loc[:, :chunk], x[:, r * chunk:(r + 1) * chunk])
            c2 = 2 * cp - 1 - r
            np.testing.assert_array_equal(loc[:, chunk:], x[:, c2 * chunk:(c2 + 1) * chunk])


def test_python_index_helper_matches_oracle():
    from kvax_b200.utils.permutation import generate_shard_indices
    for n in (2, 4, 8, 16):
        assert generate_shard_indices(n) == po.shard_indices(n).tolist()
        assert generate_shard_indices(n, True) == po.shard_indices(n, True).tolist()
