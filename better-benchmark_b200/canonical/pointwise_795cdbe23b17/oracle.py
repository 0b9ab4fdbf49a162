"""SiLU of a 16-bit activation, computed in fp32.

B200 oracle for the reference's canonical directory ``repros/canonical/pointwise_795cdbe23b17``: copy this file
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
    return kernels.cast_scale(inputs[0], inputs[0].dtype, activation="silu")
