"""The benchmark commands (names and options of the reference's benchmarks.py) run on one GPU."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cmd", ["mha", "mha_bwd"])
def test_single_gpu_commands(cmd):
    from click.testing import CliRunner

    from kvax_b200 import benchmarks as bm
    args = [cmd, "--num-iters", "2", "--batch-size", "1", "--query-seq-len", "512", "--kv-seq-len", "512",
            "--num-heads", "4", "--num-kv-heads", "2", "--num-segments", "3", "--num-pad-tokens", "20",
            "--assume-sequential-positions", "false", "--check"]
    res = CliRunner().invoke(bm.cli, args, catch_exceptions=False)
    assert res.exit_code == 0, res.output
    assert "TFLOP/s" in res.output and "max |out - dense|" in res.output
