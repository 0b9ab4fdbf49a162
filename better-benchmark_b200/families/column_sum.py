"""Column reductions (family ``sum`` / ``mean``, column form).

``oracle_forward`` covers the reference graph ``aten.sum.dim_IntList(x, [0, 1])`` of a 3-D tensor
(repros/canonical/sum_eb86a17deab9/repro.py, replaced kernel .../oracle.py:20-70);
``spatial_mean_forward`` the channels-last ``aten.mean.dim(x, [2, 3], True)``
(repros/canonical/mean_c9e1a8113328/repro.py:23-27, replaced kernel .../oracle.py:11-76)."""
from .. import kernels


def oracle_forward(inputs, *, op="sum"):
    (x,) = inputs[:1]
    return kernels.col_reduce(x.reshape(-1, x.shape[-1]) if x.is_contiguous() else x, op)


def spatial_mean_forward(inputs):
    (x,) = inputs[:1]
    n, c, h, w = x.shape
    if x.stride(1) == 1:  # channels-last: [N, H*W, C] view, reduce over rows
        rows = x.permute(0, 2, 3, 1).reshape(n, h * w, c)
        return kernels.col_reduce(rows, "mean").view(n, c, 1, 1)
    return kernels.row_reduce(x.reshape(n * c, h * w), "mean").view(n, c, 1, 1)
