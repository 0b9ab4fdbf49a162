"""RMSNorm backward: dx written head-major [B,H,S,D] plus the fp32 dweight column reduction.

B200 oracle for this point: a registration stub around
``better_benchmark_b200.families.rms_norm_bwd_heads`` (hand-written sm_100a CUDA behind the C ABI).
The same file works inside a checkout of the reference (its ``oracle_harness`` is found first)
and with this repository's mirror of the harness.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.families import rms_norm_bwd_heads


@oracle_impl(hardware="B200", point="c5a00005")
def oracle_forward(inputs):
    return rms_norm_bwd_heads.oracle_forward(inputs)
