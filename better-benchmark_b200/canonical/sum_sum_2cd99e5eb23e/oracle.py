"""RMSNorm backward: dx rows and the fp32 weight gradient. The incoming gradient of this graph is a broadcast scalar; it is materialised once (the kernel reads a full dy).

B200 oracle for the reference's canonical directory ``repros/canonical/sum_sum_2cd99e5eb23e``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernels behind it are hand-written sm_100a CUDA behind the C ABI.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.registration import every_point
from better_benchmark_b200 import kernels


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    dy, weight, rstd, x, dy_shape = inputs[:5]
    dx, dweight, _ = kernels.norm_bwd(x, dy, weight, rstd.reshape(-1), rms=True)  # dy: 0-dim, read as a scalar
    return (dx, dweight)
