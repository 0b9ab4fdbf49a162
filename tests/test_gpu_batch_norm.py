"""GPU parity: BatchNorm2d training forward (+ReLU, running statistics) against the eager graph."""
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _kernels():
    import better_benchmark_b200.kernels as k
    return k


def _inputs(shape, dtype, channels_last, seed, shift=0.5, scale=2.0):
    g = torch.Generator().manual_seed(seed)
    x = (shift + scale * torch.randn(shape, generator=g)).to(dtype)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    c = shape[1]
    w = torch.rand(c, generator=g) + 0.5
    b = 0.1 * torch.randn(c, generator=g)
    rm = 0.3 * torch.randn(c, generator=g)
    rv = torch.rand(c, generator=g) + 0.5
    return x, rm, rv, w, b


SHAPES = [
    (2, 8, 4, 4), (4, 64, 14, 14), (16, 64, 56, 56), (8, 384, 8, 8), (3, 24, 17, 9), (5, 136, 7, 7),
    (2, 2048, 7, 7), (1, 16, 1, 1), (32, 32, 1, 1), (2, 5, 6, 6), (7, 40, 13, 13),
]


@pytest.mark.parametrize("relu", [True, False])
@pytest.mark.parametrize("channels_last", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
def test_batch_norm_fwd_matches_eager(shape, dtype, channels_last, relu):
    from oracle.eager import BatchNormReluFwd
    if shape[0] * shape[2] * shape[3] < 2:
        pytest.skip("a single element per channel has no unbiased variance")
    x, rm, rv, w, b = _inputs(shape, dtype, channels_last, seed=sum(shape))
    want = BatchNormReluFwd(1e-5, 0.1, relu=relu)(x, rm.clone(), rv.clone(), w, b)
    rm_d, rv_d = rm.cuda(), rv.cuda()
    y, mean, invstd = _kernels().batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), rm_d, rv_d, eps=1e-5,
                                               momentum=0.1, relu=relu)
    assert y.stride() == x.stride()
    assert_close(y, want[0], f"bn y {shape} {dtype} cl={channels_last}")
    assert_close(mean, want[1], f"bn mean {shape}")
    assert_close(invstd, want[2], f"bn invstd {shape}")
    assert_close(rm_d, want[3], f"bn running_mean {shape}")
    assert_close(rv_d, want[4], f"bn running_var {shape}")
    _kernels().check_scratch_status()


def test_batch_norm_large_mean_small_variance():
    """Shifted sums: a channel with mean 1000 and unit variance keeps its variance."""
    from oracle.eager import BatchNormReluFwd
    g = torch.Generator().manual_seed(0)
    x = (1000.0 + torch.randn((8, 16, 32, 32), generator=g)).contiguous(memory_format=torch.channels_last)
    w, b = torch.ones(16), torch.zeros(16)
    rm, rv = torch.zeros(16), torch.ones(16)
    want = BatchNormReluFwd(1e-5, 0.1, relu=False)(x.double(), rm.double(), rv.double(), w.double(), b.double())
    y, mean, invstd = _kernels().batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), None, None, eps=1e-5,
                                               momentum=0.1)
    assert_close(mean, want[1].float(), "mean")
    assert torch.allclose(invstd.cpu(), want[2].float(), rtol=2e-5, atol=0)


def test_batch_norm_repeated_calls_update_running_stats_and_reproduce():
    k = _kernels()
    x, rm, rv, w, b = _inputs((16, 64, 28, 28), torch.bfloat16, True, seed=3)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    rm1, rv1 = rm.cuda(), rv.cuda()
    y1, m1, s1 = k.batch_norm_fwd(xd, wd, bd, rm1, rv1, eps=1e-5, momentum=0.1, relu=True)
    rm2, rv2 = rm.cuda(), rv.cuda()
    y2, m2, s2 = k.batch_norm_fwd(xd, wd, bd, rm2, rv2, eps=1e-5, momentum=0.1, relu=True)
    assert torch.equal(y1, y2) and torch.equal(m1, m2) and torch.equal(s1, s2)
    assert torch.equal(rm1, rm2) and torch.equal(rv1, rv2)
    k.batch_norm_fwd(xd, wd, bd, rm2, rv2, eps=1e-5, momentum=0.1, relu=True)
    assert not torch.equal(rm1, rm2)       # a second step moves the running statistics again
    k.check_scratch_status()


@pytest.mark.parametrize("shape,dtype", [((64, 32, 56, 56), torch.bfloat16), ((128, 16, 35, 35), torch.float16),
                                         ((5, 700, 7, 7), torch.bfloat16), ((40, 96, 28, 28), torch.float32),
                                         ((3, 8, 149, 149), torch.bfloat16)])
def test_batch_norm_nchw_cluster_kernel(shape, dtype):
    """Contiguous NCHW takes the single-launch kernel whose CTAs of one channel form a cluster: planes
    with unaligned starts, more CTAs than images, one and several CTAs per channel."""
    from oracle.eager import BatchNormReluFwd
    k = _kernels()
    x, rm, rv, w, b = _inputs(shape, dtype, False, seed=sum(shape))
    want = BatchNormReluFwd(1e-3, 0.1, relu=True)(x, rm.clone(), rv.clone(), w, b)
    rm_d, rv_d = rm.cuda(), rv.cuda()
    before = k.load().b200_launch_count()
    y, mean, invstd = k.batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), rm_d, rv_d, eps=1e-3, momentum=0.1, relu=True)
    assert k.load().b200_launch_count() - before == 1 and b"NCHW" in k.load().b200_last_kernel()
    assert_close(y, want[0], f"bn nchw y {shape} {dtype}")
    assert_close(mean, want[1], f"bn nchw mean {shape}")
    assert_close(invstd, want[2], f"bn nchw invstd {shape}")
    assert_close(rm_d, want[3], f"bn nchw running_mean {shape}")
    assert_close(rv_d, want[4], f"bn nchw running_var {shape}")
    y2, mean2, _ = k.batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), None, None, eps=1e-3, momentum=0.1, relu=True)
    assert torch.equal(y, y2) and torch.equal(mean, mean2), "bit-reproducible"


@pytest.mark.parametrize("shape,dtype", [((4, 128, 7, 7), torch.bfloat16), ((32, 256, 14, 14), torch.bfloat16),
                                         ((128, 40, 8, 8), torch.bfloat16), ((16, 24, 9, 9), torch.float32),
                                         ((1, 5, 3, 3), torch.float16), ((2, 3, 1, 1), torch.float32),
                                         ((128, 8, 11, 11), torch.float16), ((33, 17, 5, 3), torch.bfloat16)])
def test_batch_norm_nchw_channel_in_registers(shape, dtype):
    """Channels of at most 16 K elements take the kernel that keeps a channel in the registers of
    one CTA (one to sixteen elements per thread, one to thirty-two warps)."""
    from oracle.eager import BatchNormReluFwd
    k = _kernels()
    x, rm, rv, w, b = _inputs(shape, dtype, False, seed=sum(shape) + 3)
    want = BatchNormReluFwd(1e-3, 0.1, relu=True)(x, rm.clone(), rv.clone(), w, b)
    rm_d, rv_d = rm.cuda(), rv.cuda()
    before = k.load().b200_launch_count()
    y, mean, invstd = k.batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), rm_d, rv_d, eps=1e-3, momentum=0.1, relu=True)
    assert k.load().b200_launch_count() - before == 1 and b"channel in registers" in k.load().b200_last_kernel()
    assert_close(y, want[0], f"bn small y {shape} {dtype}")
    assert_close(mean, want[1], f"bn small mean {shape}")
    assert_close(invstd, want[2], f"bn small invstd {shape}")
    assert_close(rm_d, want[3], f"bn small running_mean {shape}")
    assert_close(rv_d, want[4], f"bn small running_var {shape}")
    y2, mean2, _ = k.batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), None, None, eps=1e-3, momentum=0.1, relu=False)
    assert torch.equal(mean, mean2), "bit-reproducible"
    want2 = BatchNormReluFwd(1e-3, 0.1, relu=False)(x, rm.clone(), rv.clone(), w, b)
    assert_close(y2, want2[0], f"bn small y without relu {shape} {dtype}")


@pytest.mark.parametrize("shape,dtype", [((8, 92, 14, 14), torch.bfloat16), ((4, 60, 7, 8), torch.bfloat16),
                                         ((16, 36, 6, 6), torch.bfloat16), ((8, 100, 5, 4), torch.float32),
                                         ((6, 58, 4, 4), torch.float16), ((3, 24, 5, 5), torch.bfloat16),
                                         ((64, 480, 7, 7), torch.bfloat16), ((32, 48, 35, 35), torch.bfloat16)])
def test_batch_norm_channels_last_any_channel_count(shape, dtype):
    """Channels-last tensors whose channel count does not make a power-of-two number of vectors per
    row take the three-launch path over flat vectors (a vector may straddle the end of a row)."""
    from oracle.eager import BatchNormReluFwd
    k = _kernels()
    x, rm, rv, w, b = _inputs(shape, dtype, True, seed=sum(shape) + 5)
    want = BatchNormReluFwd(1e-3, 0.1, relu=True)(x, rm.clone(), rv.clone(), w, b)
    rm_d, rv_d = rm.cuda(), rv.cuda()
    y, mean, invstd = k.batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), rm_d, rv_d, eps=1e-3, momentum=0.1, relu=True)
    assert b"flat vectors" in k.load().b200_last_kernel(), k.load().b200_last_kernel()
    assert y.stride() == x.stride()
    assert_close(y, want[0], f"bn cl flat y {shape} {dtype}")
    assert_close(mean, want[1], f"bn cl flat mean {shape}")
    assert_close(invstd, want[2], f"bn cl flat invstd {shape}")
    assert_close(rm_d, want[3], f"bn cl flat running_mean {shape}")
    assert_close(rv_d, want[4], f"bn cl flat running_var {shape}")
    y2, mean2, _ = k.batch_norm_fwd(x.cuda(), w.cuda(), b.cuda(), None, None, eps=1e-3, momentum=0.1, relu=True)
    assert torch.equal(y, y2) and torch.equal(mean, mean2), "bit-reproducible"
