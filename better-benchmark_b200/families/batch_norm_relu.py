"""BatchNorm2d training forward + ReLU with running-stat update (family ``var_mean``, channel
form; reference graph: repros/canonical/var_mean_42fad1ece813/repro.py:23-58, replaced kernels:
.../oracle.py:11-119). Returns (y, mean, invstd, running_mean, running_var); the last two are the
input tensors themselves, updated in place, as the eager graph's ``copy_`` returns them."""
from .. import kernels


def oracle_forward(inputs, *, eps=1e-5, momentum=0.1, relu=True):
    x, running_mean, running_var, weight, bias = inputs[:5]
    y, mean, invstd = kernels.batch_norm_fwd(x, weight, bias, running_mean, running_var, eps=eps,
                                             momentum=momentum, relu=relu)
    return (y, mean, invstd, running_mean, running_var)
