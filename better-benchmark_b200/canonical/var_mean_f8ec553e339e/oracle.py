"""LayerNorm forward of an fp32 [B, S, H] tensor (eps 1e-5) returning mean, rstd (keepdim) and y as bf16 [B*S, H].

B200 oracle for the reference's canonical directory ``repros/canonical/var_mean_f8ec553e339e``: copy this file
there as ``oracle.py`` (library built, this repository on PYTHONPATH). Registered under the shape hash of every
point in the directory's shapes.json (and shape-general for other inputs); the kernels behind it are hand-written sm_100a CUDA behind the C ABI.
"""
try:  # inside the reference checkout
    from oracle_harness import oracle_impl
except ImportError:  # stand-alone: this repository's mirror of the same contract
    from better_benchmark_b200.harness import oracle_impl

import torch

from better_benchmark_b200.registration import every_point
from better_benchmark_b200 import kernels


@every_point(oracle_impl, hardware="B200")
def oracle_forward(inputs):
    x, weight, bias, out_shape = inputs[:4]
    y, mean, rstd, _ = kernels.norm_fwd(x, weight, bias, eps=1e-5, rms=False, out_dtype=torch.bfloat16,
                                        want_mean=True, want_rstd=True, keepdim=True)
    return (mean, rstd, y.view(out_shape))
