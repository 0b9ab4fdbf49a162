"""The BatchNorm entry point that brings its own scratch memory.

Some callers of the library cannot allocate device memory - a host framework owns the only arena
and forbids plug-ins to call cudaMalloc, or the caller holds nothing but the tensors it was given.
For them ``b200_batch_norm_fwd_static_scratch`` keeps its scratch in a fixed array inside the
library (at most 1024 channels). This test drives it through the C ABI and checks every output
against the ordinary entry point, twice in a row: the second call finds the array as the first
one left it. The file name sorts last so that a run that stops at the first failure has already
run every other test; the test does not depend on any of them.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn_name, x, weight, bias, eps, momentum, relu, with_scratch):
    from better_benchmark_b200 import kernels, native
    lib = native.load()
    n, c, h, w = x.shape
    sn, sc, sh, sw = x.stride()
    y = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    mean = torch.empty(c, dtype=torch.float32, device=x.device)
    invstd = torch.empty_like(mean)
    running_mean = torch.zeros(c, dtype=torch.float32, device=x.device)
    running_var = torch.ones(c, dtype=torch.float32, device=x.device)
    args = [x.data_ptr(), y.data_ptr(), weight.data_ptr(), bias.data_ptr(), running_mean.data_ptr(),
            running_var.data_ptr(), mean.data_ptr(), invstd.data_ptr(), n, c, h * w, sn, sc, sw,
            kernels._code(x), native.F32, eps, momentum, 1 if relu else 0]
    if with_scratch:
        scratch = torch.zeros(int(lib.b200_batch_norm_scratch_bytes(c)), dtype=torch.uint8, device=x.device)
        args += [scratch.data_ptr(), scratch.numel()]
    args.append(torch.cuda.current_stream().cuda_stream)
    status = getattr(lib, fn_name)(*args)
    torch.cuda.synchronize()
    return status, (y, mean, invstd, running_mean, running_var)


def _inputs(shape, dtype, channels_last, seed):
    g = torch.Generator().manual_seed(seed)
    x = (0.5 + 2.0 * torch.randn(shape, generator=g)).to(dtype)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    c = shape[1]
    return x.cuda(), (torch.rand(c, generator=g) + 0.5).cuda(), (0.1 * torch.randn(c, generator=g)).cuda()


@pytest.mark.parametrize("shape,dtype,channels_last", [
    ((16, 64, 28, 28), torch.bfloat16, True),     # fused cooperative path
    ((8, 40, 13, 13), torch.float32, False),      # NCHW path (needs no scratch at all)
    ((6, 20, 5, 5), torch.float32, True),         # channel count that is no multiple of the vector: three-launch path
])
def test_static_scratch_entry_point_matches_the_ordinary_one_twice(shape, dtype, channels_last):
    from better_benchmark_b200 import native
    x, weight, bias = _inputs(shape, dtype, channels_last, seed=11)
    status, want = _call("b200_batch_norm_fwd", x, weight, bias, 1e-5, 0.1, True, with_scratch=True)
    assert status == 0, native.last_error()
    for attempt in range(2):
        status, got = _call("b200_batch_norm_fwd_static_scratch", x, weight, bias, 1e-5, 0.1, True,
                            with_scratch=False)
        assert status == 0, native.last_error()
        for name, g, w in zip(("y", "mean", "invstd", "running_mean", "running_var"), got, want):
            tol = dict(rtol=1.6e-2, atol=1e-2) if g.dtype != torch.float32 else dict(rtol=1.3e-6, atol=1e-5)
            assert torch.allclose(g.float(), w.float(), **tol), f"call {attempt}: {name} differs"
    # and against the eager module itself: a defect common to both entry points must not pass
    from oracle.eager import BatchNormReluFwd
    xc = x.cpu()
    eager = BatchNormReluFwd(1e-5, 0.1, relu=True)(xc, torch.zeros(shape[1]), torch.ones(shape[1]), weight.cpu(), bias.cpu())
    for name, g, w in zip(("y", "mean", "invstd", "running_mean", "running_var"), got, eager):
        tol = dict(rtol=1.6e-2, atol=1e-2) if g.dtype != torch.float32 else dict(rtol=1.3e-6, atol=1e-5)
        assert torch.allclose(g.float().cpu(), w.float(), **tol), f"{name} differs from the eager module"
    # a different problem right after: stale partial sums of the previous shape must not leak in
    x2, w2, b2 = _inputs((4, 24, 9, 9), torch.float16, True, seed=12)
    _, want2 = _call("b200_batch_norm_fwd", x2, w2, b2, 1e-5, 0.1, False, with_scratch=True)
    status, got2 = _call("b200_batch_norm_fwd_static_scratch", x2, w2, b2, 1e-5, 0.1, False, with_scratch=False)
    assert status == 0, native.last_error()
    for g, w in zip(got2, want2):
        tol = dict(rtol=1.6e-2, atol=1e-2) if g.dtype != torch.float32 else dict(rtol=1.3e-6, atol=1e-5)
        assert torch.allclose(g.float(), w.float(), **tol)


def test_static_scratch_entry_point_rejects_too_many_channels():
    from better_benchmark_b200 import native
    x = torch.zeros((1, 2048, 2, 2), device="cuda")
    weight = torch.ones(2048, device="cuda")
    status, _ = _call("b200_batch_norm_fwd_static_scratch", x, weight, weight, 1e-5, 0.1, False,
                      with_scratch=False)
    assert status == native.ERR_UNSUPPORTED
    assert "1024" in native.last_error()
