"""LayerNorm forward returning (y, mean, rstd) (family ``var_mean``; reference graph:
repros/canonical/var_mean_f8ec553e339e/repro.py:23-37, replaced kernel: .../oracle.py:50-84)."""
from .. import kernels


def oracle_forward(inputs, *, eps=1e-12, out_dtype=None, keepdim=False):
    x, weight, bias = inputs[:3]
    y, mean, rstd, _ = kernels.norm_fwd(x, weight, bias, eps=eps, out_dtype=out_dtype or x.dtype,
                                        want_mean=True, want_rstd=True, keepdim=keepdim)
    return (y, mean, rstd)
