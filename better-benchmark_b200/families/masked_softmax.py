"""Scaled, additively masked softmax over the last dimension (family ``amax_sum``; reference graph:
repros/canonical/amax_sum_20ccc18dda60/repro.py:23-36, replaced kernel: .../oracle.py:11-58)."""
from .. import kernels


def oracle_forward(inputs, *, scale=0.125, log=False):
    scores, mask = inputs[:2]
    return kernels.softmax(scores, mask=mask, scale=scale, log=log)
