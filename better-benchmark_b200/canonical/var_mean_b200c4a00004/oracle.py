"""BatchNorm2d training forward + ReLU on a channels-last bf16 activation, running stats updated in place.

B200 oracle for this point: a registration stub around
``better_benchmark_b200.families.batch_norm_relu`` (hand-written sm_100a CUDA behind the C ABI).
The same file works inside a checkout of the reference (its ``oracle_harness`` is found first)
and with this repository's mirror of the harness.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.families import batch_norm_relu


@oracle_impl(hardware="B200", point="c4a00004", eps=1e-5, momentum=0.1)
def oracle_forward(inputs, *, eps, momentum):
    return batch_norm_relu.oracle_forward(inputs, eps=eps, momentum=momentum)
