"""Dropout-fused norms (families ``mean`` / ``var_mean`` with random masks drawn inside the region).

``oracle_forward`` covers the reference graph dropout(x) + residual -> RMSNorm -> dropout of
repros/canonical/mean_014afd4984e6/repro.py:24-47 (replaced kernel .../oracle.py:14-130, wrapper
:201-260): inputs ``(x, seeds, residual, weight, shape, shape, shape, flat_shape)``, outputs
``(keep0, sum, rstd, keep1, y)``. The masks come from the kernel's own Philox4x32-10 stream keyed by
``seeds[82]`` / ``seeds[83]``; the reference's check skips them as stochastic outputs.

``layer_norm_forward`` covers dropout(x) + residual -> LayerNorm of
repros/canonical/var_mean_01fbd6c1b27f/repro.py:24-44: inputs ``(x, seeds, residual, weight, bias, shape,
shape)``, outputs ``(keep, xhat, y, rstd / cols)``, seed ``seeds[35]``, eps 1e-5.

``add_forward`` covers dropout(x) + residual without a norm
(repros/canonical/pointwise_4b076ed1ff41/repro.py:24-32 and its siblings): outputs ``(keep, sum)`` shaped
like the residual (or like the trailing shape parameter when the graph reshapes the sum)."""
from .. import kernels

DROPOUT_P = 0.1
EPS = 1e-6
SEED_INDEX0, SEED_INDEX1 = 82, 83


def oracle_forward(inputs, *, p=DROPOUT_P, eps=EPS, seed_index0=SEED_INDEX0, seed_index1=SEED_INDEX1):
    x, seeds, residual, weight = inputs[:4]
    return kernels.dropout_rms_norm(x, residual, weight, seeds, seed_index0, seed_index1, p=p, eps=eps)


def layer_norm_forward(inputs, *, p=DROPOUT_P, eps=1e-5, seed_index=35):
    x, seeds, residual, weight, bias = inputs[:5]
    return kernels.dropout_layer_norm(x, residual, weight, bias, seeds, seed_index, p=p, eps=eps)


def add_forward(inputs, *, p=DROPOUT_P, seed_index=1, order=("x", "seeds", "residual"), out_shape=None):
    named = dict(zip(order, inputs[:3]))
    keep, total = kernels.dropout_add(named["x"], named["residual"], named["seeds"], seed_index, p=p)
    return keep, (total.view(list(out_shape)) if out_shape is not None else total)
