"""Dropout-fused RMSNorm kernel: the masks against the numpy Philox restatement (bit-exact), every
other output against the eager oracle evaluated with the kernel's own masks."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _inputs(rows, cols, dtype, seed, lead=None):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(rows, cols, generator=g, device="cuda") * 1.5).to(dtype)
    shape = (rows, cols) if lead is None else (*lead, cols)
    residual = torch.randn(shape, generator=g, device="cuda")
    weight = torch.rand(cols, generator=g, device="cuda") + 0.5
    seeds = torch.randint(0, 2 ** 62, (84,), generator=g, device="cuda", dtype=torch.int64)
    return x, seeds, residual, weight


def _expected_masks(seeds, numel, p, dtype, i0, i1):
    from oracle.philox import uniforms
    s = seeds.cpu().tolist()
    u0 = torch.from_numpy(uniforms(numel, s[i0], 0))
    u1 = torch.from_numpy(uniforms(numel, s[i1], 1))
    return u0.to(dtype) > p, u1 > p      # the first draw is narrowed before the comparison, as in the graph


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols,lead", [(64, 512, (2, 32)), (1, 8, None), (7, 264, None), (33, 1024, (3, 11)),
                                            (5, 2048, None), (130, 768, None), (4096, 512, (32, 128))])
@pytest.mark.parametrize("p", [0.1, 0.5])
def test_outputs_follow_from_masks_and_masks_from_philox(dtype, rows, cols, lead, p):
    from better_benchmark_b200 import kernels
    from oracle import eager
    x, seeds, residual, weight = _inputs(rows, cols, dtype, rows + cols, lead)
    keep0, total, rstd, keep1, y = kernels.dropout_rms_norm(x, residual, weight, seeds, 82, 83, p=p, eps=1e-6)
    assert keep0.dtype == keep1.dtype == torch.bool and keep0.shape == residual.shape
    assert total.shape == residual.shape and rstd.shape == (*residual.shape[:-1], 1) and y.shape == x.shape

    want0, want1 = _expected_masks(seeds, rows * cols, p, dtype, 82, 83)
    assert torch.equal(keep0.cpu().view(-1), want0)
    assert torch.equal(keep1.cpu().view(-1), want1)

    module = eager.DropoutResidualRMSNorm(p, 1e-6, 82, 83)
    _, w_total, w_rstd, _, w_y = module(x, seeds, residual, weight, masks=(keep0, keep1))
    assert torch.equal(total, w_total)            # element-wise, no reduction: exact
    assert_close(rstd, w_rstd, "rstd")
    assert_close(y, w_y, "y")


def test_keep_rate_independence_and_seed_dependence():
    from better_benchmark_b200 import kernels
    x, seeds, residual, weight = _inputs(4096, 512, torch.bfloat16, 3)
    k0, _, _, k1, y = kernels.dropout_rms_norm(x, residual, weight, seeds, 82, 83, p=0.1, eps=1e-6)
    n = k0.numel()
    r0, r1 = k0.float().mean().item(), k1.float().mean().item()
    sigma = (0.09 / n) ** 0.5
    assert abs(r1 - 0.9) < 6 * sigma
    assert abs(r0 - 0.9) < 6 * sigma + 2e-3          # the bf16 rounding of the draw moves the threshold slightly
    both = (k0 & k1).float().mean().item()
    assert abs(both - r0 * r1) < 6 * sigma           # the two masks are independent
    rows_equal = (k0[1:] == k0[:-1]).all(dim=1).any().item()
    assert not rows_equal                            # no row repeats its neighbour
    again = kernels.dropout_rms_norm(x, residual, weight, seeds, 82, 83, p=0.1, eps=1e-6)
    assert torch.equal(again[0], k0) and torch.equal(again[3], k1) and torch.equal(again[4], y)
    seeds2 = seeds.clone()
    seeds2[82] += 1
    other = kernels.dropout_rms_norm(x, residual, weight, seeds2, 82, 83, p=0.1, eps=1e-6)
    assert not torch.equal(other[0], k0) and torch.equal(other[3], k1)
    swapped = kernels.dropout_rms_norm(x, residual, weight, seeds, 83, 82, p=0.1, eps=1e-6)
    assert not torch.equal(swapped[0], k0)


def test_p_zero_keeps_everything():
    from better_benchmark_b200 import kernels
    from oracle import eager
    x, seeds, residual, weight = _inputs(16, 256, torch.bfloat16, 5)
    k0, total, rstd, k1, y = kernels.dropout_rms_norm(x, residual, weight, seeds, 0, 1, p=0.0, eps=1e-6)
    # a draw of exactly 0 is the only one p = 0 drops
    assert k0.float().mean().item() > 0.99 and k1.float().mean().item() > 0.999
    _, w_total, w_rstd, _, w_y = eager.DropoutResidualRMSNorm(0.0, 1e-6)(x, seeds, residual, weight, masks=(k0, k1))
    assert torch.equal(total, w_total)
    assert_close(y, w_y, "y")


def test_rejected_arguments():
    from better_benchmark_b200 import kernels, native
    x, seeds, residual, weight = _inputs(8, 512, torch.bfloat16, 1)
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_rms_norm(x, residual, weight, seeds, 84, 0, p=0.1, eps=1e-6)          # seed index out of range
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_rms_norm(x, residual.half(), weight, seeds, 0, 1, p=0.1, eps=1e-6)   # residual must be fp32
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_rms_norm(x, residual, weight, seeds, 0, 1, p=1.0, eps=1e-6)           # p outside [0, 1)
    x2, s2, r2, w2 = _inputs(4, 4096, torch.bfloat16, 2)
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_rms_norm(x2, r2, w2, s2, 0, 1, p=0.1, eps=1e-6)                       # row longer than built
    x3, s3, r3, w3 = _inputs(4, 12, torch.bfloat16, 2)
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_rms_norm(x3, r3, w3, s3, 0, 1, p=0.1, eps=1e-6)                       # not a multiple of 8
    e = kernels.dropout_rms_norm(x[:0], residual[:0], weight, seeds, 0, 1, p=0.1, eps=1e-6)
    assert e[4].shape == (0, 512)


def test_through_the_shipped_stub_and_harness():
    """The directory's oracle.py through the harness check: masks are skipped as stochastic or compared
    by the harness's own rule; here the deterministic outputs are checked with the stub's masks."""
    from better_benchmark_b200.families import dropout_rms_norm
    from oracle import eager
    x, seeds, residual, weight = _inputs(256, 512, torch.bfloat16, 9, (2, 128))
    inputs = [x, seeds, residual, weight, [2, 128, 512], [2, 128, 512], [2, 128, 512], [256, 512]]
    k0, total, rstd, k1, y = dropout_rms_norm.oracle_forward(inputs)
    _, w_total, w_rstd, _, w_y = eager.DropoutResidualRMSNorm(0.1, 1e-6, 82, 83)(x, seeds, residual, weight,
                                                                                  masks=(k0, k1))
    assert torch.equal(total, w_total)
    assert_close(rstd, w_rstd, "rstd")
    assert_close(y, w_y, "y")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols,lead", [(64, 768, (2, 32)), (1, 8, None), (9, 264, None), (33, 1024, (3, 11)),
                                            (5, 2048, None), (8192, 768, (8, 1024))])
@pytest.mark.parametrize("p", [0.1, 0.3])
def test_dropout_layer_norm(dtype, rows, cols, lead, p):
    from better_benchmark_b200 import kernels
    from oracle import eager
    from oracle.philox import uniforms
    x, seeds, residual, weight = _inputs(rows, cols, dtype, rows * 3 + cols, lead)
    bias = torch.randn(cols, device="cuda") * 0.1
    keep, xhat, y, rstd_n = kernels.dropout_layer_norm(x, residual, weight, bias, seeds, 35, p=p, eps=1e-5)
    assert keep.dtype == torch.bool and keep.shape == residual.shape
    assert xhat.dtype == y.dtype == torch.float32 and xhat.shape == y.shape == residual.shape
    assert rstd_n.shape == (*residual.shape[:-1], 1)

    u = torch.from_numpy(uniforms(rows * cols, seeds.cpu().tolist()[35], 0))
    assert torch.equal(keep.cpu().view(-1), u.to(dtype) > p)

    _, w_xhat, w_y, w_rstd_n = eager.DropoutResidualLayerNorm(p, 1e-5, 35)(x, seeds, residual, weight, bias, mask=keep)
    assert_close(rstd_n, w_rstd_n, "rstd / n")
    # fp32 outputs of a normalisation: the row statistics differ in their last bits with the
    # summation order, which every element inherits
    assert (xhat - w_xhat).abs().max().item() <= 2e-5 * max(1.0, w_xhat.abs().max().item())
    assert (y - w_y).abs().max().item() <= 2e-5 * max(1.0, w_y.abs().max().item())


def test_dropout_layer_norm_through_the_family_and_rejections():
    from better_benchmark_b200 import kernels, native
    from better_benchmark_b200.families import dropout_rms_norm
    x, seeds, residual, weight = _inputs(128, 768, torch.bfloat16, 4, (2, 64))
    bias = torch.zeros(768, device="cuda")
    out = dropout_rms_norm.layer_norm_forward([x, seeds, residual, weight, bias, [2, 64, 768], [2, 64, 768]])
    assert len(out) == 4 and abs(out[0].float().mean().item() - 0.9) < 0.01
    again = dropout_rms_norm.layer_norm_forward([x, seeds, residual, weight, bias, [2, 64, 768], [2, 64, 768]])
    assert all(torch.equal(a, b) for a, b in zip(out, again))
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_layer_norm(x, residual, weight, bias, seeds, 84, p=0.1, eps=1e-5)
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_layer_norm(x, residual, weight, bias[:-8], seeds, 0, p=0.1, eps=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 8), (3, 16, 320), (48, 2560), (7, 33, 8), (4096, 1024)])
@pytest.mark.parametrize("p", [0.1, 0.5])
def test_dropout_add(dtype, shape, p):
    from better_benchmark_b200 import kernels
    from oracle import eager
    from oracle.philox import uniforms
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    n = 1
    for d in shape:
        n *= d
    x = (torch.randn(n // shape[-1], shape[-1], generator=g, device="cuda") * 2).to(dtype)
    residual = torch.randn(shape, generator=g, device="cuda")
    seeds = torch.randint(0, 2 ** 62, (4,), generator=g, device="cuda", dtype=torch.int64)
    keep, total = kernels.dropout_add(x, residual, seeds, 3, p=p)
    assert keep.shape == total.shape == residual.shape and keep.dtype == torch.bool
    u = torch.from_numpy(uniforms(n, seeds.cpu().tolist()[3], 0))
    assert torch.equal(keep.cpu().view(-1), u.to(dtype) > p)
    _, want = eager.DropoutAdd(p, 3)(x, seeds, residual, mask=keep)
    assert torch.equal(total, want)


def test_dropout_add_stub_argument_orders_and_rejections():
    from better_benchmark_b200 import kernels, native
    from better_benchmark_b200.families import dropout_rms_norm
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(64, 768, generator=g, device="cuda").to(torch.bfloat16)
    residual = torch.randn(64, 768, generator=g, device="cuda")
    seeds = torch.randint(0, 2 ** 62, (2,), generator=g, device="cuda", dtype=torch.int64)
    a = dropout_rms_norm.add_forward([x, seeds, residual, [64, 768], [64, 768]])
    b = dropout_rms_norm.add_forward([seeds, x, residual, [64, 768], [4, 16, 768]], order=("seeds", "x", "residual"),
                                     out_shape=[4, 16, 768])
    assert b[1].shape == (4, 16, 768) and torch.equal(a[1].view(-1), b[1].view(-1)) and torch.equal(a[0], b[0])
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_add(x, residual[:32], seeds, 0, p=0.1)
    with pytest.raises(native.KernelArgumentError):
        kernels.dropout_add(x[:1, :4], residual[:1, :4].contiguous(), seeds, 0, p=0.1)   # not a multiple of 8


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dims,permuted", [((4, 3, 16, 64), True), ((2, 6, 128, 128), True), ((1, 2, 5, 8), False),
                                           ((3, 4, 7, 520), False), ((2, 2, 9, 1024), True)])
def test_softmax_dropout(dtype, dims, permuted):
    """softmax(x + bias) -> dropout: the mask bit for bit against the Philox restatement, everything
    else against the eager module evaluated with the kernel's own mask. The bias is read in place,
    also when the head dimension is its unit-stride one (the layout of the captured shape point)."""
    from better_benchmark_b200 import kernels
    from oracle import eager
    from oracle.philox import uniforms
    b, h, sq, sk = dims
    g = torch.Generator(device="cuda").manual_seed(sum(dims))
    x = (torch.randn(b * h, sq, sk, generator=g, device="cuda") * 2).to(dtype)
    if permuted:
        bias = torch.randn(b, sq, sk, h, generator=g, device="cuda").permute(0, 3, 1, 2)
        assert bias.stride(1) == 1
    else:
        bias = torch.randn(b, h, sq, sk, generator=g, device="cuda")
    seeds = torch.randint(0, 2 ** 62, (32,), generator=g, device="cuda", dtype=torch.int64)
    p = 0.1
    logits, amax, total, keep, y = kernels.softmax_dropout(x, bias, seeds, 29, p=p)
    assert b"b200_softmax_dropout" in kernels.load().b200_last_kernel()
    assert logits.shape == keep.shape == (b, h, sq, sk) and keep.dtype == torch.bool and y.shape == x.shape
    n = b * h * sq * sk
    u = torch.from_numpy(uniforms(n, seeds.cpu().tolist()[29], 0))
    assert torch.equal(keep.cpu().view(-1), u.to(dtype) > p)
    want = eager.SoftmaxDropout(p, 29)(x.cpu(), bias.cpu(), seeds.cpu(), mask=keep.cpu())
    assert torch.equal(logits.cpu(), want[0]), "rounded logits"
    assert torch.equal(amax.cpu(), want[1]), "row maximum"
    # a sum of exponentials: summation order and expf differ from the CPU's in the last bits
    assert torch.allclose(total.cpu(), want[2], rtol=2e-5, atol=1e-6), "row sum of the exponentials"
    assert_close(y, want[4], "dropped probabilities")
    again = kernels.softmax_dropout(x, bias, seeds, 29, p=p)
    assert all(torch.equal(u_, v_) for u_, v_ in zip((logits, amax, total, keep, y), again)), "bit-reproducible"


def test_softmax_dropout_rejections():
    from better_benchmark_b200 import kernels, native
    x = torch.zeros(6, 4, 12, device="cuda", dtype=torch.bfloat16)
    bias = torch.zeros(2, 3, 4, 12, device="cuda")
    seeds = torch.zeros(4, device="cuda", dtype=torch.int64)
    with pytest.raises(native.KernelArgumentError):
        kernels.softmax_dropout(x, bias, seeds, 0, p=0.1)            # 12 columns: not a multiple of 8
    with pytest.raises(native.KernelArgumentError):
        kernels.softmax_dropout(x, bias[:, :2], seeds, 0, p=0.1)     # shapes disagree
    with pytest.raises(native.KernelArgumentError):
        kernels.softmax_dropout(x, bias, seeds, 9, p=0.1)            # seed slot outside the tensor
