"""Scaled, additively masked softmax over the last dimension (family ``amax_sum``; reference graph:
repros/canonical/amax_sum_20ccc18dda60/repro.py:23-36, replaced kernel: .../oracle.py:11-58)."""
from .. import kernels


def oracle_forward(inputs, *, scale=0.125, log=False):
    scores, mask = inputs[:2]
    return kernels.softmax(scores, mask=mask, scale=scale, log=log)


def softmax_dropout_forward(inputs, *, p=0.1, seed_index=29):
    """softmax(x + bias) -> dropout, the attention probabilities of a T5 block in training
    (repros/canonical/amax_sum_089fdab8f22b/repro.py:24-46). Inputs: x ``[B*H, Sq, Sk]``, bias fp32
    ``[B, H, Sq, Sk]`` (any strides), seeds, four lifted shapes. Outputs as the graph returns them:
    (rounded logits, amax, sum, mask, y ``[B*H, Sq, Sk]``, y transposed in its last two dimensions -
    a view of the same buffer)."""
    x, bias, seeds = inputs[:3]
    logits, amax, total, keep, y = kernels.softmax_dropout(x, bias, seeds, seed_index, p=p)
    return logits, amax, total, keep, y, y.permute(0, 2, 1)
