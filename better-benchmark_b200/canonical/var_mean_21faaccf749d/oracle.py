"""Exact GELU -> bf16 -> LayerNorm (eps 1e-7), returning mean, rstd and y.

B200 oracle for the reference's canonical directory ``repros/canonical/var_mean_21faaccf749d``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernels behind it are hand-written sm_100a CUDA behind the C ABI.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

from better_benchmark_b200.registration import every_point
from better_benchmark_b200 import kernels


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    x, weight, bias, shape3, out_shape = inputs[:5]
    y, mean, rstd, _ = kernels.norm_fwd(x, weight, bias, eps=1e-7, rms=False, prologue="gelu_erf",
                                        want_mean=True, want_rstd=True)
    b, s = int(shape3[0]), int(shape3[1])
    if b < 0 or s < 0:  # a lifted shape with one -1
        rows = x.numel() // x.shape[-1]
        b, s = (rows // s, s) if b < 0 else (b, rows // b)
    return mean.view(b, s, 1), rstd.view(b, s, 1), y.view([int(d) for d in out_shape])
