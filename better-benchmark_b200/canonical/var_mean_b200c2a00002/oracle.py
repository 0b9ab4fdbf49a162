"""LayerNorm forward over 768 features of 32768 bf16 rows, returning y, mean and rstd.

B200 oracle for this point: a registration stub around
``better_benchmark_b200.families.layer_norm`` (hand-written sm_100a CUDA behind the C ABI).
The same file works inside a checkout of the reference (its ``oracle_harness`` is found first)
and with this repository's mirror of the harness.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.families import layer_norm


@oracle_impl(hardware="B200", point="c2a00002", eps=1e-12)
def oracle_forward(inputs, *, eps):
    return layer_norm.oracle_forward(inputs, eps=eps)
