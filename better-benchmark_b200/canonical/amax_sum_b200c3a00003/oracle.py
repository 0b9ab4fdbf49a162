"""Attention softmax: fp16 scores * 0.125 + key-padding mask, fp32 internals, fp16 output.

B200 oracle for this point: a registration stub around
``better_benchmark_b200.families.masked_softmax`` (hand-written sm_100a CUDA behind the C ABI).
The same file works inside a checkout of the reference (its ``oracle_harness`` is found first)
and with this repository's mirror of the harness.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.families import masked_softmax


@oracle_impl(hardware="B200", point="c3a00003", scale=0.125)
def oracle_forward(inputs, *, scale):
    return masked_softmax.oracle_forward(inputs, scale=scale)
