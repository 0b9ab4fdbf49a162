"""TEST INFRASTRUCTURE - eager ground truth for the c4_batch_norm_relu benchmark configuration.

Same layout as a canonical repro of the reference (``Repro`` module + ``make_inputs``): the
module is the decomposed aten graph restated in ``oracle/eager.py``; ``make_inputs()`` builds the
seeded inputs with the value distributions the configuration specifies, and
``make_inputs(shape_config)`` the plain ``randn`` inputs of a shapes.json point.
"""
import torch

from better_benchmark_b200.inputs import make_inputs_from_config
from better_benchmark_b200.workloads import WORKLOADS
from oracle.eager import BatchNormReluFwd

_repro_version = 3


class Repro(BatchNormReluFwd):
    def __init__(self):
        super().__init__(1e-5, 0.1)


def make_inputs(shape_config=None, device="cuda", seed=1):
    if shape_config is not None:
        return make_inputs_from_config(shape_config, device)
    return WORKLOADS["c4_batch_norm_relu"].make_inputs(device, seed)
