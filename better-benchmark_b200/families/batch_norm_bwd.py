"""BatchNorm2d training backward (family ``sum_sum``; reference graphs
repros/canonical/sum_sum_183b124c731f/repro.py:23-50 and, behind a leaky-ReLU backward,
repros/canonical/sum_sum_12fc8ebf8180/repro.py:23-58; replaced kernels: the three-kernel plans of
the two oracle.py files). Returns (dbias, dweight, dx) in the eager module's order."""
from .. import kernels


def oracle_forward(inputs, *, inv_count=None):
    """``inv_count``: the literal the captured graph multiplies the sums by (1/N of the shape it was
    captured at); None derives it from the tensor."""
    dy, x, mean, invstd, weight = inputs[:5]
    dx, dw, db = kernels.batch_norm_bwd(dy, x, mean.reshape(-1), invstd, weight, inv_count=inv_count)
    return (db, dw, dx)


def leaky_relu_forward(inputs, *, slope=0.2, inv_count=None):
    dy, act, x, mean, invstd, weight = inputs[:6]
    dx, dw, db = kernels.batch_norm_bwd(dy, x, mean.reshape(-1), invstd, weight, act=act, slope=slope,
                                        inv_count=inv_count)
    return (db, dw, dx)
