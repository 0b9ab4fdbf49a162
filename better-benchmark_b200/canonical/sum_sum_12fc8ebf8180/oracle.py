"""BatchNorm2d training backward behind a leaky-ReLU (slope 0.2) backward: dbias, dweight, dx.

B200 oracle for the reference's canonical directory ``repros/canonical/sum_sum_12fc8ebf8180``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernels behind it are hand-written sm_100a CUDA behind the C ABI.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.registration import every_point
from better_benchmark_b200.families import batch_norm_bwd


# 1 / (32 * 16 * 16): a literal of the captured graph (repro.py:38, :42), applied at every shape point
INV_COUNT = 0.0001220703125


@every_point(oracle_impl, hardware="B200", inv_count=INV_COUNT)
def oracle_forward(inputs, *, inv_count):
    return batch_norm_bwd.leaky_relu_forward(inputs, slope=0.2, inv_count=inv_count)
