"""Parity of the column-reduce, permuting-copy, transpose and cast kernels against the eager oracle."""
import pytest
import torch

from conftest import assert_close, assert_sum_close

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


def _kernels():
    from better_benchmark_b200 import kernels
    return kernels


def _rand(shape, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["sum", "mean", "amax"])
@pytest.mark.parametrize("rows,cols", [(1, 8), (7, 5), (64, 256), (1000, 768), (4096, 100), (33, 4099),
                                       (20000, 64), (3, 1)])
def test_col_reduce_2d(dtype, op, rows, cols):
    from oracle import eager
    x = _rand((rows, cols), dtype, rows * 31 + cols)
    got = _kernels().col_reduce(x, op)
    want = eager.ColumnSum(op)(x)
    if op == "amax":
        assert torch.equal(got, want)
    else:
        anchor = eager.ColumnSum(op)(x.double())
        assert_sum_close(got, want, anchor, f"col_{op} {rows}x{cols} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,c,h,w", [(2, 16, 7, 7), (8, 64, 14, 14), (3, 100, 5, 9), (4, 2048, 7, 7)])
def test_spatial_mean_channels_last_and_nchw(dtype, n, c, h, w):
    from better_benchmark_b200.families import column_sum
    from oracle import eager
    x = _rand((n, c, h, w), dtype, n + c)
    for t in (x.contiguous(memory_format=torch.channels_last), x):
        got = column_sum.spatial_mean_forward([t])
        want = eager.SpatialMean()(t)
        anchor = eager.SpatialMean()(t.double())
        assert_sum_close(got, want, anchor, f"spatial mean {tuple(t.shape)} {t.stride()}")


def test_col_reduce_batched_strided_rows():
    from oracle import eager
    base = _rand((4, 300, 160), torch.float32, 5)
    x = base[:, :, :96]  # row stride 160, 96 columns kept
    got = _kernels().col_reduce(x, "sum")
    want = torch.stack([eager.ColumnSum()(x[i]) for i in range(4)])
    anchor = torch.stack([eager.ColumnSum()(x[i].double()) for i in range(4)])
    assert_sum_close(got, want, anchor, "batched strided col sum")


@pytest.mark.parametrize("op", ["sum", "mean", "amax"])
@pytest.mark.parametrize("batch,rows,cols,dtype", [(128, 3136, 64, torch.bfloat16), (96, 784, 256, torch.float16),
                                                   (3, 2000, 4096, torch.float32), (20, 1500, 1000, torch.float32),
                                                   (1, 8192, 768, torch.float32), (1, 16384, 1024, torch.bfloat16)])  # narrow chunks
def test_col_reduce_cluster_combine(op, batch, rows, cols, dtype):
    """Shapes that split every reduction over 2, 4 or 8 CTAs: those form a thread-block cluster and
    are combined through distributed shared memory in one launch."""
    from oracle import eager
    k = _kernels()
    x = _rand((batch, rows, cols), dtype, batch + rows)
    before = k.load().b200_launch_count()
    got = k.col_reduce(x, op)
    launched = k.load().b200_launch_count() - before
    assert launched == 1 and b"cluster" in k.load().b200_last_kernel(), k.load().b200_last_kernel()
    want = torch.stack([eager.ColumnSum(op)(x[i]) for i in range(batch)])
    if op == "amax":
        assert torch.equal(got, want)
    else:
        anchor = torch.stack([eager.ColumnSum(op)(x[i].double()) for i in range(batch)])
        assert_sum_close(got, want, anchor, f"cluster col_{op} {batch}x{rows}x{cols} {dtype}")
    assert torch.equal(got, k.col_reduce(x, op)), "bit-reproducible"


def test_col_reduce_zero_rows_and_bad_layout():
    k = _kernels()
    x = torch.empty((0, 16), device="cuda")
    assert torch.equal(k.col_reduce(x, "sum"), torch.zeros(16, device="cuda"))
    assert torch.isnan(k.col_reduce(x, "mean")).all()
    with pytest.raises(k.UnsupportedLayout):
        k.col_reduce(torch.empty((8, 16), device="cuda").t(), "sum")


def test_col_reduce_is_bit_reproducible():
    x = _rand((50000, 384), torch.float32, 9)
    a = _kernels().col_reduce(x, "sum")
    for _ in range(3):
        assert torch.equal(a, _kernels().col_reduce(x, "sum"))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("b,s,h,d", [(1, 5, 3, 8), (2, 128, 12, 64), (4, 77, 8, 40), (2, 33, 5, 7)])
@pytest.mark.parametrize("scale", [None, 0.125])
def test_head_split(dtype, b, s, h, d, scale):
    from oracle import eager
    x = _rand((b * s, h * d), dtype, b + s + h + d)
    got = _kernels().permute_copy(x.view(b, s, h, d), (0, 2, 1, 3), scale=scale)
    want = eager.HeadSplitPermute(b, s, h, d, scale)(x)
    assert got.is_contiguous()
    if scale is None:
        assert torch.equal(got, want)
    else:
        assert_close(got, want, "head split scaled")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (5, 3), (64, 64), (65, 130), (3, 200, 77), (2, 3, 128, 96),
                                   (1024, 768), (4, 1, 33)])
def test_transpose_last_two(dtype, shape):
    from oracle import eager
    x = _rand(shape, dtype, sum(shape))
    nd = len(shape)
    dims = list(range(nd - 2)) + [nd - 1, nd - 2]
    got = _kernels().permute_copy(x, dims)
    want = eager.Transpose2D()(x)
    assert got.is_contiguous() and torch.equal(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(768, 49, 128), (128, 6, 196, 64), (300, 7, 8), (5, 33, 40), (1000, 25, 64),
                                   (9, 100, 80)])
def test_transpose_small_matrices(dtype, shape):
    """Batches of small matrices whose sides are no multiples of 64: flat 16-byte copies on both
    sides with the transposition done as a shared-memory gather."""
    k = _kernels()
    x = _rand(shape, dtype, sum(shape))
    nd = len(shape)
    got = k.permute_copy(x, list(range(nd - 2)) + [nd - 1, nd - 2])
    if shape[-1] * shape[-2] * x.element_size() <= 32 * 1024:
        assert b"small matrices" in k.load().b200_last_kernel(), k.load().b200_last_kernel()
    assert got.is_contiguous() and torch.equal(got, x.transpose(-1, -2).contiguous())


@pytest.mark.parametrize("dims", [(3, 2, 1, 0), (1, 0, 2, 3), (0, 3, 1, 2), (2, 0, 3, 1), (0, 1, 2, 3)])
def test_general_permutations(dims):
    x = _rand((6, 10, 12, 20), torch.bfloat16, 3)
    got = _kernels().permute_copy(x, dims)
    assert torch.equal(got, x.permute(*dims).contiguous())


def test_permute_with_conversion_and_strided_source():
    base = _rand((4, 50, 6, 48), torch.float32, 11)
    x = base[..., :32]
    got = _kernels().permute_copy(x, (0, 2, 1, 3), out_dtype=torch.bfloat16, scale=2.0)
    want = (x * 2.0).permute(0, 2, 1, 3).contiguous().to(torch.bfloat16)
    assert torch.equal(got, want)


def test_permute_rejects_five_unmergeable_dims():
    k = _kernels()
    x = _rand((2, 3, 4, 5, 6), torch.float32, 1)
    with pytest.raises(k.UnsupportedLayout):
        k.permute_copy(x, (4, 3, 2, 1, 0))


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                     (torch.float16, torch.float32), (torch.float32, torch.float16),
                                     (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("n", [1, 7, 4096, 1_000_003])
@pytest.mark.parametrize("scale", [None, 0.5, 1.7])
def test_cast_scale(src, dst, n, scale):
    x = _rand((n,), src, n)
    got = _kernels().cast_scale(x, dst, scale=scale)
    want = x if scale is None else x.float() * scale
    assert torch.equal(got, want.to(dst))


def test_cast_keeps_channels_last_strides():
    x = _rand((2, 8, 5, 5), torch.bfloat16, 2).contiguous(memory_format=torch.channels_last)
    got = _kernels().cast_scale(x, torch.float32)
    assert got.stride() == x.stride() and torch.equal(got, x.float())


def test_cast_between_the_two_16_bit_types_is_rejected_loudly():
    k = _kernels()
    from better_benchmark_b200.native import KernelArgumentError
    with pytest.raises(KernelArgumentError):
        k.cast_scale(_rand((64,), torch.bfloat16, 1), torch.float16)


@pytest.mark.parametrize("shape,strides", [((8, 3, 3, 3), (27, 1, 9, 3)), ((64, 32, 3, 3), None), ((1003,), None),
                                           ((1,), None), ((5, 7, 1, 1), (7, 1, 7, 7)), ((2, 16, 33), None)])
@pytest.mark.parametrize("src,dst", [(torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16),
                                     (torch.float16, torch.float32)])
def test_parameter_casts_keep_the_strides_of_dense_tensors(shape, strides, src, dst):
    """convert_element_type of a model's parameters: storage order, so a channels-last weight comes
    back channels-last; sizes that are no multiple of the vector, down to one element."""
    from better_benchmark_b200 import kernels
    n = 1
    for d in shape:
        n *= d
    base = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 3).to(src).cuda()
    x = torch.as_strided(base, shape, strides) if strides else base.view(shape)
    y = kernels.cast_scale(x, dst)
    assert y.stride() == x.stride() and y.dtype == dst
    assert torch.equal(y, x.to(dst))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(128, 768, 1, 1), (4, 24, 5, 5), (3, 1001), (7,)])
def test_relu_in_storage_order(dtype, shape):
    from better_benchmark_b200 import kernels
    n = 1
    for d in shape:
        n *= d
    x = (torch.randn(n, generator=torch.Generator().manual_seed(n + 1)) * 2).to(dtype).view(shape).cuda()
    x.view(-1)[0] = float("nan")
    y = kernels.cast_scale(x, dtype, relu=True)
    want = torch.relu(x)
    assert torch.equal(torch.isnan(y), torch.isnan(want)) and torch.equal(torch.nan_to_num(y), torch.nan_to_num(want))
