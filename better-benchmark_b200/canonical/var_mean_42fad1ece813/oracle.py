"""BatchNorm2d training forward (eps 1e-3, momentum 0.1) fused with ReLU; updates the running statistics in place.

B200 oracle for the reference's canonical directory ``repros/canonical/var_mean_42fad1ece813``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernels behind it are hand-written sm_100a CUDA behind the C ABI.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.registration import every_point
from better_benchmark_b200 import kernels


# 8192 / 8191: the unbiased-variance factor is a literal of the captured graph (repro.py:40), applied
# at every shape point
UNBIASED_FACTOR = 1.0001220852154804


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    x, running_mean, running_var, weight, bias = inputs[:5]
    y, mean, invstd = kernels.batch_norm_fwd(x, weight, bias, running_mean, running_var, eps=1e-3, momentum=0.1,
                                             relu=True, unbiased_factor=UNBIASED_FACTOR)
    return (invstd, y, mean.view(1, -1, 1, 1), running_mean, running_var)
