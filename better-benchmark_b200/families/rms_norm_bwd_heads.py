"""RMSNorm backward with dx stored head-major (families ``sum_sum`` + permuting ``pointwise``;
reference graphs: repros/canonical/sum_sum_2cd99e5eb23e/repro.py:23-46 and
pointwise_c0d19d490a2f/repro.py, replaced kernels: sum_sum_2cd99e5eb23e/oracle.py:48-117,
pointwise_c0d19d490a2f/oracle.py:10-33). Returns (dx [B,H,S,D], dweight fp32 [H*D])."""
from .. import kernels


def oracle_forward(inputs):
    x, dy, weight, rstd = inputs[:4]
    dx, dw, _ = kernels.norm_bwd(x, dy, weight, rstd, rms=True, heads=x.shape[2])
    return (dx, dw)
