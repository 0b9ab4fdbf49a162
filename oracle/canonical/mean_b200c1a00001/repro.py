"""TEST INFRASTRUCTURE - eager ground truth for the c1_row_mean benchmark configuration.

Same layout as a canonical repro of the reference (``Repro`` module + ``make_inputs``): the
module is the decomposed aten graph restated in ``oracle/eager.py``; ``make_inputs()`` builds the
seeded inputs with the value distributions the configuration specifies, and
``make_inputs(shape_config)`` the plain ``randn`` inputs of a shapes.json point.
"""
import torch

from better_benchmark_b200.inputs import make_inputs_from_config
from better_benchmark_b200.workloads import WORKLOADS
from oracle.eager import RowMean

_repro_version = 3


class Repro(RowMean):
    def __init__(self):
        super().__init__()


def make_inputs(shape_config=None, device="cuda", seed=1):
    if shape_config is not None:
        return make_inputs_from_config(shape_config, device)
    return WORKLOADS["c1_row_mean"].make_inputs(device, seed)
