"""Synthetic benchmark / test inputs.  TEST INFRASTRUCTURE ONLY (as everything under oracle/).

The generator itself lives in kvax_b200/utils/synthetic.py, because the benchmark's measured
leg needs the same seeded inputs and must not import this package; the tests keep using it
under this name."""
from kvax_b200.utils.synthetic import *  # noqa: F401,F403
from kvax_b200.utils.synthetic import CONFIGS, Config, attention_flops, make_inputs, small_config  # noqa: F401
