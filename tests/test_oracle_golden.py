"""Pin the eager oracle (oracle/eager.py) against outputs of the reference's own repro modules.

The fixtures in tests/golden/*.pt were produced by tests/golden/make_golden.py from the
reference checkout: its ``Repro`` modules, its input generator, its byte accounting. Here the
restated eager classes run on the stored inputs and must reproduce the stored outputs; the byte
model must reproduce the stored byte counts. CPU only.
"""
from pathlib import Path

import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def _load(name):
    return torch.load(GOLDEN / f"{name}.pt", weights_only=False)


def golden_cases():
    """case name -> function(inputs) returning the outputs in the reference module's order."""
    from oracle import eager

    def ln_fwd(inp):
        x, w, b, shape = inp
        y, mean, rstd = eager.LayerNormFwd(1e-5, torch.bfloat16, squeeze_stats=False)(x, w, b)
        return [mean, rstd, y.view(shape)]

    def rms_fwd(inp):
        return [eager.RMSNormFwd(1e-6, torch.bfloat16)(*inp)]

    def softmax_bias(inp):
        x, bias, s0, s1 = inp
        return [eager.MaskedScaledSoftmax()(x.view(s0), bias).view(s1)]

    def bn_relu(inp):
        x, rm, rv, w, b = inp
        y, mean, invstd, rm_o, rv_o = eager.BatchNormReluFwd(1e-3, 0.1)(x, rm, rv, w, b)
        return [invstd, y, mean.view(1, -1, 1, 1), rm_o, rv_o]

    def rms_bwd(inp):
        dy0, w, rstd, x, s0, _s1, _s2 = inp
        rows, n = x.shape
        dy = dy0.expand(s0).contiguous()
        dx, dw = eager.RMSNormBwdHeadTranspose(1)(x.view(1, rows, 1, n), dy.view(1, rows, 1, n), w, rstd)
        return [dx.view(rows, n), dw]

    def ln_bwd(inp):
        rstd, dy0, w, x, mean, s0 = inp
        return list(eager.LayerNormBwd()(x, dy0.expand(s0), w, mean, rstd))

    def colsum(inp):
        (x,) = inp
        return [eager.ColumnSum()(x.view(-1, x.shape[-1]))]

    def headsplit(inp):
        x, _s0, s1, s2 = inp
        return [eager.HeadSplitPermute(*s1)(x).view(s2)]

    def transpose(inp):
        x, shape = inp
        return [eager.Transpose2D()(x).view(shape)]

    def logsoftmax(inp):
        x, shape = inp
        return [eager.MaskedScaledSoftmax(log=True, out_dtype=torch.float32)(x[:, :-3].reshape(shape))]

    def softmax_long(inp):
        return [eager.MaskedScaledSoftmax()(inp[0])]

    def spatial_mean(inp):
        return [eager.SpatialMean()(inp[0])]

    def bn_bwd_leaky(inp):
        dy, act, x, mean, invstd, w = inp
        return list(eager.BatchNormBwd(slope=0.2)(dy, x, mean.view(-1), invstd, w, act=act))

    def dropout_rms(inp, recorded=None):
        x, seeds, residual, w, _s0, _s1, _s2, _s3 = inp
        masks = (recorded[0], recorded[3]) if recorded is not None else None
        return list(eager.DropoutResidualRMSNorm(0.1, 1e-6, 82, 83)(x, seeds, residual, w, masks=masks))

    def dropout_ln(inp, recorded=None):
        x, seeds, residual, w, b, _s0, _s1 = inp
        mask = recorded[0] if recorded is not None else None
        return list(eager.DropoutResidualLayerNorm(0.1, 1e-5, 35)(x, seeds, residual, w, b, mask=mask))

    def dropout_add(inp, recorded=None):
        x, seeds, residual, _s0, _s1 = inp
        mask = recorded[0] if recorded is not None else None
        return list(eager.DropoutAdd(0.1, 1)(x, seeds, residual, mask=mask))

    def softmax_dropout(inp, recorded=None):
        x, bias, seeds = inp[:3]
        mask = recorded[3] if recorded is not None else None
        return list(eager.SoftmaxDropout(0.1, 29)(x, bias, seeds, mask=mask))

    def res_ln(eps, returns):
        def run(inp):
            out = eager.ResidualLayerNormFwd(eps, returns)(*inp)
            return [out] if isinstance(out, torch.Tensor) else list(out)
        return run

    def gelu_ln(inp):
        x, w, b, s0, s1 = inp
        return [eager.GeluLayerNormFwd(1e-12)(x.view(s0), w, b).view(s1)]

    def gelu_ln_stats(inp):
        x, w, b, s0, s1 = inp
        mean, rstd, y = eager.GeluLayerNormFwd(1e-7, with_stats=True)(x.view(s0), w, b)
        return [mean, rstd, y.view(s1)]

    def headmerge(inp):
        return [eager.HeadMergePermute()(*inp)]

    def qkv_views_kvq(inp):
        return list(eager.QkvSplitViews(768)(*inp, order=(1, 2, 0)))

    def cast_alias(inp):
        return list(eager.CastWithTransposedAlias()(inp[0]))

    def scale_view(inp):
        return [eager.ScaleIntoHeadView(0.125)(*inp)]

    def qkv_views(inp):
        return list(eager.QkvSplitViews(768)(*inp))

    return {
        "cast_alias_8bb40810003c": cast_alias, "scale_view_95ed2ef35da9": scale_view,
        "qkv_views_1611fb0c7845": qkv_views, "gelu_ln_af505388b035": gelu_ln,
        "dropout_add_4b076ed1ff41": dropout_add, "softmax_dropout_089fdab8f22b": softmax_dropout,
        "res_ln_0ada225c0a04": res_ln(1e-6, ("y2",)), "res_ln_sum_f4578c128d74": res_ln(1e-6, ("sum3", "y2")),
        "res_ln_alias_45f7dfd4a983": res_ln(1e-12, ("y3", "y2")), "res_ln_sum2_49afc8635b79": res_ln(1e-5, ("sum2", "y2")),
        "res_ln_stats_547bcc63004b": res_ln(1e-5, ("sum3", "mean", "rstd", "y2")),
        "cast_param_04d85912d998": lambda inp: [eager.ParameterCast(torch.float32)(inp[0])],
        "cast_param_ccd411f2a45d": lambda inp: [eager.ParameterCast(torch.bfloat16)(inp[0])],
        "relu_3abc926270f6": lambda inp: [eager.Relu()(inp[0])],
        "gelu_826ea0b5f6e4": lambda inp: [eager.GeluErf()(*inp)], "silu_795cdbe23b17": lambda inp: [eager.Silu()(inp[0])],
        "gelu_ln_stats_21faaccf749d": gelu_ln_stats, "headmerge_e87d6ebc9ded": headmerge,
        "qkv_views_d5a413a2c233": qkv_views_kvq,
        "dropout_ln_01fbd6c1b27f": dropout_ln,
        "dropout_rms_014afd4984e6": dropout_rms,
        "ln_fwd_f8ec553e339e": ln_fwd, "rmsnorm_fwd_f667cd8901af": rms_fwd,
        "softmax_bias_20ccc18dda60": softmax_bias, "bn_relu_42fad1ece813": bn_relu,
        "rms_bwd_2cd99e5eb23e": rms_bwd, "ln_bwd_3cac3bbf4e8f": ln_bwd,
        "colsum_eb86a17deab9": colsum, "headsplit_c0d19d490a2f": headsplit,
        "transpose_021e90d9c17d": transpose, "logsoftmax_d16035e7b826": logsoftmax,
        "softmax_long_7079889cfc04": softmax_long, "spatial_mean_c9e1a8113328": spatial_mean,
        "bn_bwd_leaky_12fc8ebf8180": bn_bwd_leaky,
    }


CASE_NAMES = sorted(p.stem for p in GOLDEN.glob("*.pt"))
STOCHASTIC = {"dropout_rms_014afd4984e6", "dropout_ln_01fbd6c1b27f", "dropout_add_4b076ed1ff41",
              "softmax_dropout_089fdab8f22b"}   # cases whose region draws random numbers


def _clone(inputs):
    return [i.clone() if isinstance(i, torch.Tensor) else i for i in inputs]


def test_every_fixture_has_a_case():
    assert set(CASE_NAMES) == set(golden_cases())


@pytest.mark.parametrize("name", CASE_NAMES)
def test_eager_oracle_reproduces_reference_outputs(name):
    data = _load(name)
    want = data["outputs"]
    if name in STOCHASTIC:   # the recorded masks stand in for the draws; the rest must follow from them
        got = golden_cases()[name](_clone(data["inputs"]), want)
    else:
        got = golden_cases()[name](_clone(data["inputs"]))
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert g.shape == w.shape, f"{name} output {i}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
        assert g.dtype == w.dtype, f"{name} output {i}: dtype {g.dtype} vs {w.dtype}"
        # Same ops on the same torch build: bit-exact here. The tolerance only absorbs a different
        # torch version reordering a CPU reduction.
        assert torch.allclose(g.float(), w.float(), rtol=2e-6, atol=2e-6, equal_nan=True), \
            f"{name} output {i}: max diff {(g.float() - w.float()).abs().max().item():.3e}"


@pytest.mark.parametrize("name", CASE_NAMES)
def test_byte_model_reproduces_reference_byte_counts(name):
    from better_benchmark_b200.byte_model import count_bytes_effective
    data = _load(name)
    fn = golden_cases()[name]

    class Region(torch.nn.Module):
        def forward(self, *inputs):
            return tuple(fn(list(inputs)))

    assert count_bytes_effective(Region(), _clone(data["inputs"])) == data["effective_bytes"]
