"""Packed q, k, v -> three [B, H, S, D] strided views of the INPUT: no arithmetic, no kernel, no allocation.

B200 oracle for the reference's canonical directory ``repros/canonical/pointwise_1611fb0c7845``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); nothing is launched: the outputs alias the input.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.registration import every_point
from better_benchmark_b200.families import aliasing


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    return aliasing.qkv_split_views(inputs)
