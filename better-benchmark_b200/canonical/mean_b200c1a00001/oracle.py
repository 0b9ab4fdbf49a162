"""Row-wise mean of an fp32 [8192, 4096] matrix: one streaming read, fp32 accumulation.

B200 oracle for this point: a registration stub around
``better_benchmark_b200.families.row_mean`` (hand-written sm_100a CUDA behind the C ABI).
The same file works inside a checkout of the reference (its ``oracle_harness`` is found first)
and with this repository's mirror of the harness.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.families import row_mean


@oracle_impl(hardware="B200", point="c1a00001")
def oracle_forward(inputs):
    return row_mean.oracle_forward(inputs)
