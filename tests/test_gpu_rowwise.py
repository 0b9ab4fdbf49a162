"""GPU parity: row reductions, softmax and LayerNorm/RMSNorm forward against the eager oracle.

Every case runs the CUDA kernel through the C ABI (better_benchmark_b200.kernels) and the eager
restatement of the reference graph (oracle/eager.py) on the CPU, on the same seeded inputs.
"""
import pytest
import torch

from conftest import assert_close, assert_sum_close

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


def _kernels():
    import better_benchmark_b200.kernels as k
    return k


def _randn(shape, dtype, seed, scale=1.0, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale + shift).to(dtype)


# ---- row reductions -------------------------------------------------------------------------
ROW_SHAPES = [
    (1, 1), (3, 7), (5, 33), (17, 1000), (64, 4096), (4096, 512), (9, 16385), (2, 3, 5, 129),
    (2400, 8), (1, 262144), (300, 20000),
]


@pytest.mark.parametrize("op", ["sum", "mean", "amax", "amin"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ROW_SHAPES)
def test_row_reduce_matches_eager(op, dtype, shape):
    from oracle.eager import RowReduce
    x = _randn(shape, dtype, seed=sum(shape) + len(op))
    want = RowReduce(op)(x)
    got = _kernels().row_reduce(x.cuda(), op)
    if op == "sum" and dtype == torch.float32:
        assert_sum_close(got, want, RowReduce(op)(x.double()), f"row_reduce {op} {dtype} {shape}")
    else:
        assert_close(got, want, f"row_reduce {op} {dtype} {shape}")


def test_row_reduce_strided_rows_and_offset():
    from oracle.eager import RowReduce
    base = _randn((16, 6, 200), torch.float32, 3)
    view = base[:, 1:5, 3:131]            # unaligned start, padded rows, 3 outer dims -> 2
    got = _kernels().row_reduce(base.cuda()[:, 1:5, 3:131], "sum")
    assert_close(got, RowReduce("sum")(view), "strided rows")
    tview = base.transpose(0, 1)          # [6,16,200]: outer dims not mergeable
    got = _kernels().row_reduce(base.cuda().transpose(0, 1), "mean", keepdim=True)
    assert_close(got, RowReduce("mean", keepdim=True)(tview), "transposed outer dims")


def test_row_reduce_empty_and_nan():
    k = _kernels()
    x = torch.zeros((0, 16), device="cuda")
    assert k.row_reduce(x, "sum").shape == (0,)
    y = torch.zeros((4, 0), device="cuda")
    assert torch.equal(k.row_reduce(y, "sum").cpu(), torch.zeros(4))
    z = _randn((8, 100), torch.float32, 1)
    z[3, 17] = float("nan")
    got = k.row_reduce(z.cuda(), "amax").cpu()
    want = z.amax(-1)
    assert torch.isnan(got[3]) and torch.equal(got[[0, 1, 2, 4]], want[[0, 1, 2, 4]])


def test_row_reduce_rejects_cpu_and_bad_layout():
    import better_benchmark_b200.native as native
    k = _kernels()
    with pytest.raises(native.KernelArgumentError):
        k.row_reduce(torch.zeros(4, 4), "sum")
    with pytest.raises(k.UnsupportedLayout):
        k.row_reduce(torch.zeros(4, 8, device="cuda").t(), "sum")
    with pytest.raises(k.UnsupportedLayout):
        k.row_reduce(torch.zeros(4, 8, device="cuda", dtype=torch.float64), "sum")


# ---- softmax --------------------------------------------------------------------------------
SOFTMAX_SHAPES = [(1, 1), (4, 8), (7, 33), (33, 256), (16, 512), (3, 5, 1024), (5, 2048), (3, 4096),
                  (2, 8200), (2, 32768), (2, 40000), (1, 100000)]


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SOFTMAX_SHAPES)
def test_softmax_matches_eager(shape, dtype, log):
    from oracle.eager import MaskedScaledSoftmax
    x = _randn(shape, dtype, seed=len(shape) + shape[-1], scale=3.0)
    want = MaskedScaledSoftmax(log=log)(x)
    got = _kernels().softmax(x.cuda(), log=log)
    assert_close(got, want, f"softmax log={log} {dtype} {shape}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,mask_shape", [
    ((4, 3, 16, 64), (4, 1, 1, 64)),      # key-padding mask, broadcast over heads and queries
    ((2, 4, 32, 256), (2, 1, 32, 256)),   # per-query bias broadcast over heads
    ((3, 2, 8, 512), (1, 1, 8, 512)),     # causal-style mask shared by the batch
    ((6, 40, 136), (6, 40, 136)),         # full mask
])
def test_masked_scaled_softmax_matches_eager(shape, mask_shape, dtype):
    from oracle.eager import MaskedScaledSoftmax
    x = _randn(shape, dtype, 11)
    g = torch.Generator().manual_seed(5)
    keep = torch.rand(mask_shape, generator=g) < 0.7
    keep[..., 0] = True
    mask = torch.where(keep, 0.0, -10000.0).to(dtype)
    want = MaskedScaledSoftmax(scale=0.125)(x, mask)
    got = _kernels().softmax(x.cuda(), mask=mask.cuda(), scale=0.125)
    assert_close(got, want, f"masked softmax {dtype} {shape}")


def test_softmax_output_dtype_and_strided_rows():
    from oracle.eager import MaskedScaledSoftmax
    k = _kernels()
    x = _randn((12, 300), torch.bfloat16, 2)
    got = k.softmax(x.cuda(), out_dtype=torch.float32)
    assert_close(got, MaskedScaledSoftmax(out_dtype=torch.float32)(x), "bf16 -> f32")
    xf = _randn((12, 384), torch.float32, 4)
    got = k.softmax(xf.cuda(), out_dtype=torch.bfloat16)
    assert_close(got, MaskedScaledSoftmax(out_dtype=torch.bfloat16)(xf), "f32 -> bf16")
    base = _randn((10, 520), torch.float32, 6)
    got = k.softmax(base.cuda()[:, 4:516], log=True)      # padded rows, 16-byte aligned start
    assert_close(got, MaskedScaledSoftmax(log=True)(base[:, 4:516]), "padded rows")
    got = k.softmax(base.cuda()[:, 1:513])                # unaligned start -> element-wise path
    assert_close(got, MaskedScaledSoftmax()(base[:, 1:513]), "unaligned rows")


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("rows,n,stride,offset,dtype,out_dtype", [
    (64, 20005, 20008, 0, torch.bfloat16, torch.float32),   # ragged length, aligned padded rows
    (12, 262144, 262144, 0, torch.bfloat16, torch.bfloat16),  # rows far beyond the register-resident kernel
    (33, 5001, 5004, 0, torch.float32, torch.float32),
    (20, 4001, 4100, 3, torch.float16, torch.float16),     # unaligned row starts: element-wise sweeps
    (7, 70000, 70000, 0, torch.float32, torch.bfloat16),
])
def test_softmax_long_and_ragged_rows(rows, n, stride, offset, dtype, out_dtype, log):
    """Rows the register-resident kernel cannot take go through the two-sweep kernel (running maximum
    and rescaled sum, then a second read of the row)."""
    from oracle.eager import MaskedScaledSoftmax
    k = _kernels()
    base = _randn((rows, stride + offset), dtype, n % 97, scale=3.0)
    view = base[:, offset:offset + n]
    got = k.softmax(base.cuda()[:, offset:offset + n], log=log, out_dtype=out_dtype)
    assert b"two sweeps" in k.load().b200_last_kernel(), k.load().b200_last_kernel()
    want = MaskedScaledSoftmax(log=log, out_dtype=out_dtype)(view)
    assert_close(got, want, f"long softmax log={log} {dtype}->{out_dtype} {rows}x{n}")
    special = view.clone().float()
    special[0, :] = float("-inf")
    special[1, 5] = float("inf")
    special[2, 7] = float("nan")
    special[3, : n // 2] = float("-inf")
    special = special.to(dtype)
    got = k.softmax(special.cuda(), log=log, out_dtype=out_dtype)
    want = MaskedScaledSoftmax(log=log, out_dtype=out_dtype)(special)
    assert torch.allclose(got.float().cpu(), want.float(), equal_nan=True, atol=1e-2, rtol=1.6e-2)


def test_softmax_fully_masked_and_inf_rows():
    k = _kernels()
    x = torch.zeros((3, 64), dtype=torch.float32)
    x[1] = float("-inf")
    x[2, 5] = float("inf")
    got = k.softmax(x.cuda()).cpu()
    want = torch.softmax(x, -1)
    assert torch.allclose(got, want, equal_nan=True)


# ---- LayerNorm / RMSNorm forward ----------------------------------------------------------------
NORM_SHAPES = [(1, 8), (5, 32), (9, 100), (33, 768), (8, 1024), (4, 2560), (3, 4096), (2, 4, 5120),
               (3, 16384), (2, 32768), (2, 50000), (2, 70000)]


@pytest.mark.parametrize("dtype,wdtype,odtype", [
    (torch.float32, torch.float32, torch.float32),
    (torch.float32, torch.float32, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.float32, torch.bfloat16),
    (torch.float16, torch.float16, torch.float16),
    (torch.bfloat16, torch.float32, torch.float32),
])
@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_layer_norm_fwd_matches_eager(shape, dtype, wdtype, odtype):
    from oracle.eager import LayerNormFwd
    n = shape[-1]
    x = _randn(shape, dtype, n, scale=2.0, shift=0.3)
    g = torch.Generator().manual_seed(7)
    w = (torch.rand(n, generator=g) + 0.5).to(wdtype)
    b = (0.02 * torch.randn(n, generator=g)).to(wdtype)
    want = LayerNormFwd(1e-5, odtype, squeeze_stats=False)(x, w, b)
    y, mean, rstd, _ = _kernels().norm_fwd(x.cuda(), w.cuda(), b.cuda(), eps=1e-5, out_dtype=odtype,
                                           want_mean=True, want_rstd=True)
    assert_close(y, want[0], f"layer_norm y {shape} {dtype}")
    assert_close(mean, want[1], f"layer_norm mean {shape} {dtype}")
    assert_close(rstd, want[2], f"layer_norm rstd {shape} {dtype}")


@pytest.mark.parametrize("dtype,wdtype", [(torch.bfloat16, torch.float32), (torch.float16, torch.float16),
                                          (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_rms_norm_fwd_matches_eager(shape, dtype, wdtype):
    from oracle.eager import RMSNormFwd
    n = shape[-1]
    x = _randn(shape, dtype, n + 1)
    g = torch.Generator().manual_seed(9)
    w = (torch.rand(n, generator=g) + 0.5).to(wdtype)
    want = RMSNormFwd(1e-6, dtype)(x, w)
    y, _, _, _ = _kernels().norm_fwd(x.cuda(), w.cuda(), None, eps=1e-6, rms=True)
    assert_close(y, want, f"rms_norm {shape} {dtype}")


def test_row_var_mean_matches_eager():
    k = _kernels()
    for shape, corr in [((40, 768), 0), ((7, 5000), 1), ((3, 11), 1)]:
        x = _randn(shape, torch.float32, 21, scale=3.0, shift=10.0)   # mean >> 0: needs the centred pass
        var, mean = torch.var_mean(x, [-1], correction=corr, keepdim=True)
        _, gm, _, gv = k.norm_fwd(x.cuda(), None, None, eps=0.0, want_y=False, want_mean=True,
                                  want_var=True, correction=corr)
        assert_close(gm, mean, f"var_mean mean {shape}")
        assert_close(gv, var, f"var_mean var {shape}")


def test_norm_fwd_strided_rows():
    from oracle.eager import LayerNormFwd
    base = _randn((12, 800), torch.bfloat16, 5)
    w = torch.ones(768, dtype=torch.bfloat16)
    b = torch.zeros(768, dtype=torch.bfloat16)
    want = LayerNormFwd(1e-12, torch.bfloat16)(base[:, 16:784], w, b)
    y, mean, rstd, _ = _kernels().norm_fwd(base.cuda()[:, 16:784], w.cuda(), b.cuda(), eps=1e-12,
                                           want_mean=True, want_rstd=True, keepdim=False)
    assert_close(y, want[0], "strided y")
    assert_close(mean, want[1], "strided mean")
    assert_close(rstd, want[2], "strided rstd")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_softmax_special_values_follow_eager(dtype):
    """-inf masks (zero probability), a fully -inf row (NaN), +inf and NaN logits (NaN rows)."""
    from oracle.eager import MaskedScaledSoftmax
    x = _randn((6, 200), dtype, 31)
    x[0, 50:] = float("-inf")
    x[1, :] = float("-inf")
    x[2, 7] = float("inf")
    x[3, 9] = float("nan")
    x[4, :] = -60000.0 if dtype == torch.float16 else -3e38    # a whole row at / below the clamping floor
    x[5, 3] = -60000.0 if dtype == torch.float16 else -3e38
    for log in (False, True):
        want = MaskedScaledSoftmax(log=log)(x)
        got = _kernels().softmax(x.cuda(), log=log).cpu()
        assert torch.equal(torch.isnan(got), torch.isnan(want)), f"NaN pattern differs (log={log})"
        assert_close(torch.nan_to_num(got, nan=0.0, neginf=-1e4), torch.nan_to_num(want, nan=0.0, neginf=-1e4),
                     f"special values {dtype} log={log}")


def test_compensated_exponential_accuracy_against_fp64():
    """bf16/fp16 outputs use the compensated base-2 exponential. Measured through softmax with an
    fp32 row widened from bf16 inputs: relative error against the fp64 result stays within what a
    16-bit output can resolve by three orders of magnitude (checked at 2e-6 on the pre-rounding
    ratio via an fp16 output of a two-element row, where rounding is the only other error)."""
    k = _kernels()
    g = torch.Generator().manual_seed(0)
    # rows [0, d]: softmax -> [1/(1+e^d), e^d/(1+e^d)]; sweep d over the whole useful range
    d = -(torch.rand(4096, generator=g) * 16.0)
    x = torch.stack([torch.zeros_like(d), d], -1).to(torch.bfloat16)
    got = k.softmax(x.cuda(), out_dtype=torch.bfloat16).float().cpu()
    want = torch.softmax(x.double(), -1)
    rel = ((got.double() - want).abs() / want).max().item()
    assert rel <= 2 ** -8, rel        # half a bf16 ulp is 2^-9 relative; the exponential adds ~3e-7


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n", [(300, 768), (64, 128), (8, 5000), (5, 1001), (20000, 768), (4096, 1536)])
def test_gelu_prologue_layer_norm_matches_eager(rows, n, dtype):
    """Exact GELU, rounded to the tensor dtype, fused into the load of the LayerNorm kernels."""
    from oracle.eager import GeluLayerNormFwd
    x = _randn((rows, n), dtype, seed=n, scale=1.5)
    g = torch.Generator().manual_seed(1)
    w = (torch.rand(n, generator=g) + 0.5).to(dtype)
    b = (0.1 * torch.randn(n, generator=g)).to(dtype)
    want = GeluLayerNormFwd(1e-12)(x, w, b)
    y, _, _, _ = _kernels().norm_fwd(x.cuda(), w.cuda(), b.cuda(), eps=1e-12, prologue="gelu_erf")
    assert_close(y, want, f"gelu + layer norm {rows}x{n} {dtype}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,n", [(300, 768), (64, 128), (96, 4096), (40, 240), (5, 1001), (7, 10000), (20000, 768)])
def test_residual_prologue_layer_norm_matches_eager(rows, n, dtype):
    """x + residual, rounded to the tensor dtype, fused into the load of the LayerNorm kernels; the
    rounded sum is an optional output. Row lengths that take the resident vector kernels and ones
    that take the element-wise kernel (odd length, very long rows)."""
    from oracle.eager import ResidualLayerNormFwd
    k = _kernels()
    x = _randn((rows, n), dtype, seed=n, scale=1.5)
    r = _randn((rows, n), dtype, seed=n + 1, scale=1.0)
    g = torch.Generator().manual_seed(1)
    w = (torch.rand(n, generator=g) + 0.5)
    b = (0.1 * torch.randn(n, generator=g))
    if n % 2 == 0:       # 16-bit weights for half of the cases, fp32 weights for the rest
        w, b = w.to(dtype), b.to(dtype)
    want = ResidualLayerNormFwd(1e-6, ("sum3", "mean", "rstd", "y3"))(x, r, w, b, [1, rows, n], [rows, n])
    y, mean, rstd, _, total = k.norm_fwd(x.cuda().view(1, rows, n), w.cuda(), b.cuda(), eps=1e-6,
                                         residual=r.cuda().view(1, rows, n), want_sum=True, want_mean=True,
                                         want_rstd=True, round_sum=True)
    assert b"residual add" in k.load().b200_last_kernel()
    assert torch.equal(total.cpu(), want[0]), "the rounded sum"
    assert_close(mean, want[1], f"mean {rows}x{n} {dtype}")
    assert_close(rstd, want[2], f"rstd {rows}x{n} {dtype}")
    assert_close(y, want[3], f"residual + layer norm {rows}x{n} {dtype}")
    y2 = k.norm_fwd(x.cuda(), w.cuda(), b.cuda(), eps=1e-6, residual=r.cuda(), round_sum=True)[0]
    assert torch.equal(y2.view(-1), y.view(-1)), "the same without the optional outputs"
    # the default keeps the sum in fp32 (Inductor's form): at least as close to the fp64 graph as
    # the eager module, and within the 16-bit tolerance of it
    y3, mean3, rstd3, _, total3 = k.norm_fwd(x.cuda(), w.cuda(), b.cuda(), eps=1e-6, residual=r.cuda(), want_sum=True,
                                             want_mean=True, want_rstd=True)
    assert torch.equal(total3.cpu().view(-1), want[0].view(-1))
    xd = x.double() + r.double()
    mean64 = xd.mean(-1, keepdim=True)
    rstd64 = torch.rsqrt(xd.var(-1, unbiased=False, keepdim=True) + 1e-6)
    y64 = (xd - mean64) * rstd64 * w.double() + b.double()
    err_mine = (y3.double().cpu() - y64).abs().max().item()
    err_eager = (want[3].double().view(rows, n) - y64).abs().max().item()
    assert err_mine <= 1.5 * err_eager + 1e-6, (err_mine, err_eager)
    assert (mean3.double().cpu().view(-1) - mean64.view(-1)).abs().max().item() <= 1e-5 * max(1.0, mean64.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
@pytest.mark.parametrize("rows,n", [(300, 768), (64, 128), (96, 4096), (33, 32768), (5, 1001), (7, 10000)])
def test_residual_layer_norm_both_forms_select_per_element(rows, n, dtype):
    """round_sum="both": every element is the fp32-sum form where that form's output exceeds 3 in
    magnitude and the rounded-sum form elsewhere (the rule of the reference's oracles for these
    regions, repros/canonical/var_mean_45f7dfd4a983/oracle.py:96-107); the statistics and the sum
    that are returned are those of the fp32 form. Resident and element-wise kernels."""
    k = _kernels()
    x = _randn((rows, n), dtype, seed=n + 7, scale=2.0).cuda()
    r = _randn((rows, n), dtype, seed=n + 8, scale=1.0).cuda()
    g = torch.Generator().manual_seed(2)
    w = (2.0 * torch.randn(n, generator=g)).to(dtype).cuda()     # wide weights: many outputs beyond 3
    b = torch.randn(n, generator=g).to(dtype).cuda()
    kw = dict(eps=1e-12, residual=r, want_sum=True, want_mean=True, want_rstd=True)
    y32, mean32, rstd32, _, total32 = k.norm_fwd(x, w, b, **kw)
    y16 = k.norm_fwd(x, w, b, round_sum=True, **kw)[0]
    y, mean, rstd, _, total = k.norm_fwd(x, w, b, round_sum="both", **kw)
    assert b"residual add" in k.load().b200_last_kernel()
    big = y32.float().abs() > 3.0
    assert 0.02 < big.float().mean().item() < 0.98, "the case must exercise both branches"
    assert torch.equal(y, torch.where(big, y32, y16))
    assert torch.equal(mean, mean32) and torch.equal(rstd, rstd32) and torch.equal(total, total32)
    if dtype == torch.float32:
        assert torch.equal(y, y32) and torch.equal(y, y16), "fp32 tensors: one form only"


def test_residual_prologue_rejections():
    from better_benchmark_b200 import kernels as kk
    k = _kernels()
    x = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(kk.UnsupportedLayout):
        k.norm_fwd(x, None, None, eps=1e-5, residual=torch.zeros(8, 64, device="cuda"))          # dtype differs
    with pytest.raises(kk.UnsupportedLayout):
        k.norm_fwd(x, None, None, eps=1e-5, residual=torch.zeros(4, 64, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(kk.UnsupportedLayout):
        k.norm_fwd(x, None, None, eps=1e-5, residual=x.clone(), out_dtype=torch.float32)        # y in another dtype
    from better_benchmark_b200 import native
    with pytest.raises(native.KernelArgumentError):
        k.norm_fwd(x, None, None, eps=1e-5, residual=x.clone(), rms=True, round_sum="both")     # LayerNorm only
