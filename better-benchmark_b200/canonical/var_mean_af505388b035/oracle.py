"""Exact (erf) GELU, rounded to bf16, then LayerNorm (eps 1e-12) with bf16 weight and bias; returns y only.

B200 oracle for the reference's canonical directory ``repros/canonical/var_mean_af505388b035``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernel behind it is hand-written
sm_100a CUDA behind the C ABI: the activation is fused into the load of the LayerNorm kernel.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.registration import every_point
from better_benchmark_b200 import kernels


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    x, weight, bias, _shape3, out_shape = inputs[:5]
    y, _, _, _ = kernels.norm_fwd(x, weight, bias, eps=1e-12, rms=False, prologue="gelu_erf")
    return y.view(out_shape)
