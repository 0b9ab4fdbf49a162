"""Parity of the BatchNorm backward kernels against the eager oracle (plain and behind a
leaky-ReLU / ReLU backward), channels-last and NCHW, all dtypes."""
import pytest
import torch

from conftest import assert_close, assert_sum_close

pytestmark = pytest.mark.gpu


def _case(shape, dtype, channels_last, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda scale, shift: (torch.randn(shape, generator=g, device="cuda") * scale + shift).to(dtype)
    x, dy, act = mk(2.0, 0.5), mk(1.0, 0.0), mk(1.0, 0.1)
    if channels_last:
        x, dy, act = (t.contiguous(memory_format=torch.channels_last) for t in (x, dy, act))
    c = shape[1]
    xf = x.float()
    mean = xf.mean(dim=(0, 2, 3))
    invstd = torch.rsqrt(xf.var(dim=(0, 2, 3), unbiased=False) + 1e-5)
    w = torch.rand(c, generator=g, device="cuda") + 0.5
    return dy, x, act, mean, invstd, w


SHAPES = [(4, 8, 6, 6), (32, 64, 14, 14), (8, 24, 7, 9), (64, 128, 8, 8), (3, 5, 4, 4), (16, 256, 5, 5),
          (2, 16, 1, 1), (1, 8, 33, 1)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("channels_last", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("slope", [None, 0.0, 0.2])
def test_batch_norm_bwd_matches_eager(dtype, channels_last, shape, slope):
    from better_benchmark_b200 import kernels
    from oracle import eager
    dy, x, act, mean, invstd, w = _case(shape, dtype, channels_last, sum(shape))
    use_act = act if slope is not None else None
    dx, dw, db = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=use_act, slope=slope or 0.0)
    module = eager.BatchNormBwd(slope=slope)
    want_db, want_dw, want_dx = module(dy, x, mean, invstd, w, act=use_act)
    d64 = [t.double() if t.is_floating_point() else t for t in (dy, x, mean, invstd, w)]
    if use_act is None:
        a_db, a_dw, _ = module(*d64)
    else:  # the anchor keeps the rounding of dy' to the tensor dtype that the graph has
        g = torch.where(act.float() > 0, dy.float(), dy.float() * slope).to(dtype).double()
        a_db, a_dw, _ = eager.BatchNormBwd()(g, *d64[1:])
    assert dx.stride() == x.stride()
    assert_sum_close(db, want_db, a_db, "dbias")
    assert_sum_close(dw, want_dw, a_dw, "dweight")
    if dtype == torch.float32:
        # dx inherits the summation-order differences of the two sums through its coefficients
        scale = max(1.0, want_dx.abs().max().item())
        assert (dx - want_dx).abs().max().item() <= 2e-5 * scale
    else:
        assert_close(dx, want_dx, "dx")


def test_batch_norm_bwd_is_bit_reproducible_and_sums_only():
    from better_benchmark_b200 import kernels
    dy, x, act, mean, invstd, w = _case((32, 64, 28, 28), torch.bfloat16, True, 7)
    a = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=act, slope=0.0)
    b = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=act, slope=0.0)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    dx, dw, db = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=act, slope=0.0, want_dx=False)
    assert dx is None and torch.equal(dw, a[1]) and torch.equal(db, a[2])


def test_batch_norm_bwd_rejects_mismatched_layouts():
    from better_benchmark_b200 import kernels
    dy, x, act, mean, invstd, w = _case((4, 8, 6, 6), torch.float32, True, 3)
    with pytest.raises(kernels.UnsupportedLayout):
        kernels.batch_norm_bwd(dy.contiguous(), x, mean, invstd, w)
    with pytest.raises(kernels.UnsupportedLayout):
        kernels.batch_norm_bwd(dy, x, mean.double(), invstd, w)


@pytest.mark.parametrize("shape,channels_last,dtype,slope", [
    ((64, 40, 28, 28), True, torch.bfloat16, None),     # channels-last, 5 vectors per row (not a power of two)
    ((128, 112, 7, 7), True, torch.bfloat16, None),     # 14 vectors per row
    ((16, 240, 14, 14), True, torch.float16, 0.0),      # 30 vectors per row
    ((32, 128, 16, 16), False, torch.bfloat16, 0.2),    # NCHW: one cluster of CTAs per channel
    ((64, 24, 35, 35), False, torch.bfloat16, None),    # NCHW, planes with unaligned starts
    ((6, 520, 7, 7), False, torch.float32, None),       # NCHW, more channels than the machine has CTA slots
    ((8, 92, 14, 14), True, torch.bfloat16, 0.1),       # channels-last, 92 channels: vectors straddle rows (period 23 vectors)
    ((16, 58, 6, 6), True, torch.float16, None),        # 58 channels: period 29 vectors = 4 rows
    ((4, 100, 5, 4), True, torch.float32, None),        # fp32, 100 channels: period 25 vectors = one row
    ((32, 512, 4, 4), False, torch.bfloat16, 0.2),      # NCHW, channel in registers: one element per thread
    ((32, 256, 8, 8), False, torch.bfloat16, None),     # four elements per thread
    ((3, 7, 5, 5), False, torch.float16, 0.1),          # three warps, ragged
    ((2, 3, 1, 1), False, torch.float32, None),         # two elements per channel
])
def test_batch_norm_bwd_corpus_layouts(shape, channels_last, dtype, slope):
    from better_benchmark_b200 import kernels
    from oracle import eager
    dy, x, act, mean, invstd, w = _case(shape, dtype, channels_last, sum(shape))
    use_act = act if slope is not None else None
    before = kernels.load().b200_launch_count()
    dx, dw, db = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=use_act, slope=slope or 0.0)
    launched = kernels.load().b200_launch_count() - before
    name = kernels.load().b200_last_kernel()
    if channels_last:
        assert b"channels-last, vector" in name, name
    else:
        assert launched == 1 and b"NCHW" in name, name
    module = eager.BatchNormBwd(slope=slope)
    want_db, want_dw, want_dx = module(dy, x, mean, invstd, w, act=use_act)
    d64 = [t.double() if t.is_floating_point() else t for t in (dy, x, mean, invstd, w)]
    if use_act is None:
        a_db, a_dw, _ = module(*d64)
    else:
        g = torch.where(act.float() > 0, dy.float(), dy.float() * slope).to(dtype).double()
        a_db, a_dw, _ = eager.BatchNormBwd()(g, *d64[1:])
    assert_sum_close(db, want_db, a_db, "dbias")
    assert_sum_close(dw, want_dw, a_dw, "dweight")
    if dtype == torch.float32:
        scale = max(1.0, want_dx.abs().max().item())
        assert (dx - want_dx).abs().max().item() <= 2e-5 * scale
    else:
        assert_close(dx, want_dx, "dx")
    again = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=use_act, slope=slope or 0.0)
    assert all(torch.equal(u, v) for u, v in zip((dx, dw, db), again)), "bit-reproducible"
    # the literal 1/N of a captured graph replaces the one derived from the shape
    half = kernels.batch_norm_bwd(dy, x, mean, invstd, w, act=use_act, slope=slope or 0.0,
                                  inv_count=0.5 / (shape[0] * shape[2] * shape[3]))
    assert torch.equal(half[1], dw) and not torch.equal(half[0], dx)
