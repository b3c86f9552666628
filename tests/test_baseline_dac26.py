"""The DAC'26 1D baselines (``baseline/dac26``) are part of the product's comparison tooling: run their tests here too."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "dac26"))
from test_dac26 import test_micro_and_kernel_modes, test_prepared_graph_files, test_strategies_match_single  # noqa: E402,F401
