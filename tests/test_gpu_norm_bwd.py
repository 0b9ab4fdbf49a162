"""GPU parity: LayerNorm / RMSNorm backward (dx rows, dweight/dbias columns, head-major dx store)."""
import pytest
import torch

from conftest import assert_close, assert_sum_close

pytestmark = pytest.mark.gpu


def _kernels():
    import better_benchmark_b200.kernels as k
    return k


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def _rms_reference(x, dy, w, rstd, heads=None):
    """Eager graph of the RMSNorm backward (oracle/eager.py), with or without the head permute."""
    from oracle.eager import RMSNormBwdHeadTranspose
    if heads is not None:
        return RMSNormBwdHeadTranspose(heads)(x, dy, w, rstd)
    rows, n = x.shape
    dx, dw = RMSNormBwdHeadTranspose(1)(x.view(1, rows, 1, n), dy.view(1, rows, 1, n), w, rstd)
    return dx.view(rows, n), dw


def _ln_reference(x, dy, w, mean, rstd):
    """LayerNorm backward as the decomposed graph computes it (fp32 internals, dx in x's dtype)."""
    n = x.shape[-1]
    xf, dyf = x.float(), dy.float()
    g = dyf * w
    xhat = (xf - mean[:, None]) * rstd[:, None]
    s1 = g.sum(1, keepdim=True)
    s2 = (g * xhat).sum(1, keepdim=True)
    dx = (rstd[:, None] / n) * ((g * n - s1) - xhat * s2)
    return dx.to(x.dtype), (dyf * xhat).sum(0), dyf.sum(0)


def _stats(x, eps=1e-6):
    xf = x.float()
    mean = xf.mean(-1)
    var = xf.var(-1, unbiased=False)
    return mean, torch.rsqrt(var + eps), torch.rsqrt(xf.pow(2).mean(-1) + eps)


def _close_columns(got, want, anchor, what):
    """Column sums over many rows (see conftest.assert_sum_close)."""
    assert_sum_close(got, want, anchor, what)


@pytest.mark.parametrize("two_launch", [False, True])
@pytest.mark.parametrize("dtype,wdtype", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                          (torch.float32, torch.float32), (torch.float16, torch.float16)])
@pytest.mark.parametrize("rows,n", [(1, 8), (7, 64), (300, 512), (129, 768), (64, 1024), (50, 4096),
                                    (33, 2560), (5, 100), (3, 16384)])
def test_rms_norm_bwd_matches_eager(rows, n, dtype, wdtype, two_launch):
    x = _rand((rows, n), dtype, 1)
    dy = _rand((rows, n), dtype, 2)
    w = (torch.rand(n, generator=torch.Generator().manual_seed(3)) + 0.5).to(wdtype)
    _, _, rstd = _stats(x)
    want_dx, want_dw = _rms_reference(x, dy, w, rstd)
    anchor_dx, anchor_dw = _rms_reference(x.double(), dy.double(), w.double(), rstd.double())
    dx, dw, _ = _kernels().norm_bwd(x.cuda(), dy.cuda(), w.cuda(), rstd.cuda(), rms=True,
                                    two_launch=two_launch)
    assert_close(dx, want_dx, f"rms dx {rows}x{n} {dtype}")
    _close_columns(dw, want_dw, anchor_dw, f"rms dw {rows}x{n} {dtype}")
    _kernels().check_scratch_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,n", [(4, 32), (200, 512), (77, 768), (40, 4096), (6, 1000)])
def test_layer_norm_bwd_matches_eager(rows, n, dtype):
    x = _rand((rows, n), dtype, 4, scale=2.0)
    dy = _rand((rows, n), dtype, 5)
    w = (torch.rand(n, generator=torch.Generator().manual_seed(6)) + 0.5)
    mean, rstd, _ = _stats(x)
    want = _ln_reference(x, dy, w, mean, rstd)
    anchor = _ln_reference(x.double(), dy.double(), w.double(), mean.double(), rstd.double())
    dx, dw, db = _kernels().norm_bwd(x.cuda(), dy.cuda(), w.cuda(), rstd.cuda(), mean=mean.cuda(),
                                     rms=False, want_dbias=True)
    assert_close(dx, want[0], f"ln dx {rows}x{n} {dtype}")
    _close_columns(dw, want[1], anchor[1], f"ln dw {rows}x{n}")
    _close_columns(db, want[2], anchor[2], f"ln db {rows}x{n}")


@pytest.mark.parametrize("b,s,h,d", [(1, 4, 2, 8), (2, 48, 4, 64), (2, 130, 32, 128), (3, 17, 8, 40)])
def test_rms_norm_bwd_head_major_store(b, s, h, d):
    x = _rand((b, s, h, d), torch.bfloat16, 7)
    dy = _rand((b, s, h, d), torch.bfloat16, 8)
    w = (torch.rand(h * d, generator=torch.Generator().manual_seed(9)) + 0.5).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().view(b * s, h * d).pow(2).mean(-1) + 1e-6)
    want_dx, want_dw = _rms_reference(x, dy, w, rstd, heads=h)
    _, anchor_dw = _rms_reference(x.double(), dy.double(), w.double(), rstd.double(), heads=h)
    dx, dw, _ = _kernels().norm_bwd(x.cuda(), dy.cuda(), w.cuda(), rstd.cuda(), rms=True, heads=h)
    assert dx.shape == (b, h, s, d) and dx.is_contiguous()
    assert_close(dx, want_dx, f"head-major dx {(b, s, h, d)}")
    _close_columns(dw, want_dw, anchor_dw, f"head-major dw {(b, s, h, d)}")


def test_norm_bwd_is_bit_reproducible():
    k = _kernels()
    x = _rand((4096, 1024), torch.bfloat16, 10).cuda()
    dy = _rand((4096, 1024), torch.bfloat16, 11).cuda()
    w = torch.ones(1024, dtype=torch.bfloat16, device="cuda")
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    first = k.norm_bwd(x, dy, w, rstd, rms=True)
    for _ in range(3):
        again = k.norm_bwd(x, dy, w, rstd, rms=True)
        assert torch.equal(first[0], again[0]) and torch.equal(first[1], again[1])
    k.check_scratch_status()


@pytest.mark.parametrize("rows,n,dtype,ln", [(20011, 768, torch.bfloat16, True), (9001, 520, torch.float32, False),
                                             (30000, 512, torch.bfloat16, False), (12345, 1000, torch.float16, True),
                                             (5000, 1024, torch.float32, True)])
def test_norm_bwd_many_narrow_rows(rows, n, dtype, ln):
    """Rows of 33..256 vectors, enough of them that every warp of the warp-per-row kernel walks its
    copy ring around several times (ragged last chunk and a row count that is no multiple of the
    grid included)."""
    k = _kernels()
    x = _rand((rows, n), dtype, 21, scale=1.5)
    dy = _rand((rows, n), dtype, 22)
    w = (torch.rand(n, generator=torch.Generator().manual_seed(23)) + 0.5)
    mean, rstd, rrms = _stats(x)
    before = k.load().b200_launch_count()
    if ln:
        want = _ln_reference(x, dy, w, mean, rstd)
        anchor = _ln_reference(x.double(), dy.double(), w.double(), mean.double(), rstd.double())
        dx, dw, db = k.norm_bwd(x.cuda(), dy.cuda(), w.cuda(), rstd.cuda(), mean=mean.cuda(), rms=False,
                                want_dbias=True)
        _close_columns(db, want[2], anchor[2], f"ln db {rows}x{n}")
    else:
        want = _rms_reference(x, dy, w.to(dtype), rrms)
        anchor = _rms_reference(x.double(), dy.double(), w.to(dtype).double(), rrms.double())
        dx, dw, _ = k.norm_bwd(x.cuda(), dy.cuda(), w.to(dtype).cuda(), rrms.cuda(), rms=True)
    assert k.load().b200_launch_count() - before == 1, "one fused launch expected"
    assert b"warp per row" in k.load().b200_last_kernel()
    assert_close(dx, want[0], f"dx {rows}x{n} {dtype}")
    _close_columns(dw, want[1], anchor[1], f"dw {rows}x{n}")
    again = k.norm_bwd(x.cuda(), dy.cuda(), w.cuda() if ln else w.to(dtype).cuda(), (rstd if ln else rrms).cuda(),
                       mean=mean.cuda() if ln else None, rms=not ln, want_dbias=ln)
    assert torch.equal(again[0], dx) and torch.equal(again[1], dw), "bit-reproducible"
    k.check_scratch_status()
    assert k.load().b200_norm_bwd_wait_timeouts() == 0


@pytest.mark.parametrize("rows,n,dtype,ln", [(9000, 512, torch.bfloat16, False), (7000, 768, torch.bfloat16, True),
                                             (50, 100, torch.float32, False), (300, 4096, torch.bfloat16, True),
                                             (33, 64, torch.float16, False),
                                             (5000, 512, torch.bfloat16, True), (700, 1024, torch.float32, True),
                                             (2100, 384, torch.float16, True)])
def test_norm_bwd_scalar_dy(rows, n, dtype, ln):
    """dy given as ONE element (the captured graphs expand a 0-dim gradient): read as a scalar by
    the kernels, whatever path the row length takes; same results as the materialised expansion."""
    k = _kernels()
    x = _rand((rows, n), dtype, 31, scale=1.5)
    dy0 = torch.tensor(0.75, dtype=dtype)
    dy_full = dy0.expand(rows, n)
    w = (torch.rand(n, generator=torch.Generator().manual_seed(33)) + 0.5)
    mean, rstd, rrms = _stats(x)
    if ln:
        want = _ln_reference(x, dy_full, w, mean, rstd)
        anchor = _ln_reference(x.double(), dy_full.double(), w.double(), mean.double(), rstd.double())
        got = k.norm_bwd(x.cuda(), dy0.cuda(), w.cuda(), rstd.cuda(), mean=mean.cuda(), rms=False, want_dbias=True)
        via_view = k.norm_bwd(x.cuda(), dy0.cuda().expand(rows, n), w.cuda(), rstd.cuda(), mean=mean.cuda(), rms=False,
                              want_dbias=True)
        _close_columns(got[2], want[2], anchor[2], f"scalar-dy ln db {rows}x{n}")
    else:
        want = _rms_reference(x, dy_full.contiguous(), w.to(dtype), rrms)
        anchor = _rms_reference(x.double(), dy_full.double().contiguous(), w.to(dtype).double(), rrms.double())
        got = k.norm_bwd(x.cuda(), dy0.cuda(), w.to(dtype).cuda(), rrms.cuda(), rms=True)
        via_view = k.norm_bwd(x.cuda(), dy0.cuda().expand(rows, n), w.to(dtype).cuda(), rrms.cuda(), rms=True)
    assert_close(got[0], want[0], f"scalar-dy dx {rows}x{n} {dtype}")
    _close_columns(got[1], want[1], anchor[1], f"scalar-dy dw {rows}x{n}")
    assert torch.equal(got[0], via_view[0]) and torch.equal(got[1], via_view[1])
    k.check_scratch_status()
