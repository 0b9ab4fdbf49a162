"""Residual add -> LayerNorm on 16-bit tensors: the form the kernels return (both forms of the sum,
selected per element) against the reference's two acceptance checks, on the CPU.

The element-wise check compares with the eager module, which rounds the sum to 16 bits
(oracle_harness.py:865-923, 1e-2 + 1e-2 |y|); the gate compares the error against the fp64 graph with
that of Inductor's kernel, which keeps the sum in fp32 (:1479-1548, three times its error). The
selection rule is the one of the reference's own oracles for these regions
(repros/canonical/var_mean_45f7dfd4a983/oracle.py:96-107)."""
import pytest
import torch

from better_benchmark_b200 import harness
from oracle.eager import ResidualLayerNormBothForms, ResidualLayerNormFwd


def _inputs(rows, n, dtype, seed):
    g = torch.Generator().manual_seed(seed)   # randn for every float input, as make_inputs_from_config draws them
    x = torch.randn(rows, n, generator=g).to(dtype)
    r = torch.randn(1, rows, n, generator=g).to(dtype)
    w = torch.randn(n, generator=g).to(dtype)
    b = torch.randn(n, generator=g).to(dtype)
    return x, r, w, b


def _fp64_graph(x, r, w, b, eps):
    s = x.double().view(r.shape) + r.double()
    var, mean = torch.var_mean(s, dim=-1, correction=0, keepdim=True)
    return (s - mean) * torch.rsqrt(var + eps) * w.double() + b.double()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("rows,n,eps", [(2048, 1024, 1e-12), (4096, 768, 1e-5)])
def test_both_forms_pass_the_elementwise_check_and_the_gate(rows, n, eps, dtype):
    x, r, w, b = _inputs(rows, n, dtype, seed=rows + n)
    shape3 = [1, rows, n]
    eager = ResidualLayerNormFwd(eps, ("y3",))(x, r, w, b, shape3, [rows, n])
    both = ResidualLayerNormBothForms(eps)(x, r, w, b, shape3)
    # Inductor's form: the fp32 sum all the way, one rounding at the end
    s32 = x.float().view(1, rows, n) + r.float()
    var, mean = torch.var_mean(s32, dim=-1, correction=0, keepdim=True)
    fused = ((s32 - mean) * torch.rsqrt(var + eps) * w.float() + b.float()).to(dtype)
    ref64 = _fp64_graph(x, r, w, b, eps)

    assert harness._compare_oracle_outputs(eager, both, set(), atol=1e-2, rtol=1e-2)
    gate = harness._anchored_numerics_gate([both], [fused], [ref64], set())
    assert gate["pass"], gate

    # every element is one of the two forms, chosen by the magnitude of the fp32 form
    big = fused.float().abs() > 3.0
    assert torch.equal(both[big], fused[big]) and torch.equal(both[~big], eager[~big])
    assert 0.0 < big.float().mean().item() < 0.5
    # and the selection is never further from the fp64 graph than the eager module's output
    err = lambda t: (t.double() - ref64).abs().max().item()
    assert err(both) <= err(eager)


def test_either_single_form_can_miss_one_of_the_two_checks():
    """Why a single form is not enough (bf16, 4 M elements): the fp32-sum form lands two 16-bit steps
    away from the eager module somewhere below |y| = 4 and fails the element-wise check (what this
    seed shows); on the GPU points of these directories the eager form in turn exceeded three times
    the fused kernel's error against the fp64 graph. At least one of the two must fail here."""
    rows, n, eps, dtype = 4096, 1024, 1e-12, torch.bfloat16
    x, r, w, b = _inputs(rows, n, dtype, seed=7)
    eager = ResidualLayerNormFwd(eps, ("y3",))(x, r, w, b, [1, rows, n], [rows, n])
    s32 = x.float().view(1, rows, n) + r.float()
    var, mean = torch.var_mean(s32, dim=-1, correction=0, keepdim=True)
    fused = ((s32 - mean) * torch.rsqrt(var + eps) * w.float() + b.float()).to(dtype)
    ref64 = _fp64_graph(x, r, w, b, eps)
    eager_vs_gate = harness._anchored_numerics_gate([eager], [fused], [ref64], set())["pass"]
    fused_vs_check = harness._compare_oracle_outputs(eager, fused, set(), atol=1e-2, rtol=1e-2)
    assert not (eager_vs_gate and fused_vs_check)
