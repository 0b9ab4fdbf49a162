"""log_softmax (fp32 result) over the rows of a bf16 matrix whose last three columns are padding.

B200 oracle for the reference's canonical directory ``repros/canonical/amax_sum_d16035e7b826``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernels behind it are hand-written sm_100a CUDA behind the C ABI.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

import torch

from better_benchmark_b200.registration import every_point
from better_benchmark_b200 import kernels


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    x, out_shape = inputs[:2]
    rows = x[:, :-3].unflatten(0, tuple(out_shape[:-1]))  # a strided view: the padding is never read
    return kernels.softmax(rows, log=True, out_dtype=torch.float32)
