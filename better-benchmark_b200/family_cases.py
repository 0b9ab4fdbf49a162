"""One measured case per kernel family outside the five benchmark configurations: column
reductions, row statistics, log_softmax, RMSNorm forward, LayerNorm backward, BatchNorm backward,
permuting copies, transpose and cast. Same protocol as ``workloads.py`` (seeded synthetic inputs,
bytes = every input once + every output once); sizes are chosen above the 126 MB L2.
``bench.py`` times them next to the five configurations (key ``families`` of its JSON line).
"""
from __future__ import annotations

import torch

from . import kernels
from .families import batch_norm_bwd, column_sum, dropout_rms_norm, permute
from .workloads import Workload, _gen


def _nbytes(*tensors):
    return sum(t.numel() * t.element_size() for t in tensors)


def _randn(shape, dtype, seed, device):
    # generated on the device from a seeded generator: these cases are only timed on a GPU
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(dtype)


def _case(name, description, dtype, nbytes, make_inputs, forward):
    return Workload(name=name, canonical_id="", shape_hash="", description=description, dtype=dtype,
                    algorithmic_bytes=int(nbytes), make_inputs=make_inputs, oracle_forward=forward)


def _col_sum_inputs(device="cuda", seed=1):
    return [_randn((16384, 4096), torch.float32, seed, device)]


def _spatial_mean_inputs(device="cuda", seed=1):
    return [_randn((256, 64, 56, 56), torch.bfloat16, seed, device).contiguous(memory_format=torch.channels_last)]


def _row_amax_inputs(device="cuda", seed=1):
    return [_randn((65536, 1024), torch.bfloat16, seed, device)]


def _row_var_mean_inputs(device="cuda", seed=1):
    return [_randn((32768, 1024), torch.float32, seed, device)]


def _log_softmax_inputs(device="cuda", seed=1):
    return [_randn((32768, 1024), torch.bfloat16, seed, device)]


def _rms_fwd_inputs(device="cuda", seed=1):
    return [_randn((16384, 4096), torch.bfloat16, seed, device),
            (torch.rand(4096, generator=_gen(seed)) + 0.5).to(torch.bfloat16).to(device)]


def _dropout_rms_inputs(device="cuda", seed=1):
    rows, cols = 32768, 512          # eight times the rows of the reference's point, to exceed the L2
    seeds = torch.randint(0, 2 ** 62, (84,), generator=_gen(seed), dtype=torch.int64).to(device)
    return [_randn((rows, cols), torch.bfloat16, seed, device), seeds,
            _randn((256, 128, cols), torch.float32, seed + 100, device),
            (torch.rand(cols, generator=_gen(seed)) + 0.5).to(device),
            [256, 128, cols], [256, 128, cols], [256, 128, cols], [rows, cols]]


def _dropout_add_inputs(device="cuda", seed=1):
    rows, cols = 16384, 2560         # four times the rows of the reference's largest point
    seeds = torch.randint(0, 2 ** 62, (2,), generator=_gen(seed), dtype=torch.int64).to(device)
    return [_randn((rows, cols), torch.bfloat16, seed, device), seeds,
            _randn((128, 128, cols), torch.float32, seed + 100, device), [128, 128, cols], [128, 128, cols]]


def _dropout_ln_inputs(device="cuda", seed=1):
    rows, cols = 32768, 768          # four times the rows of the reference's point, to exceed the L2
    seeds = torch.randint(0, 2 ** 62, (36,), generator=_gen(seed), dtype=torch.int64).to(device)
    return [_randn((rows, cols), torch.bfloat16, seed, device), seeds,
            _randn((32, 1024, cols), torch.float32, seed + 100, device),
            (torch.rand(cols, generator=_gen(seed)) + 0.5).to(device),
            (torch.rand(cols, generator=_gen(seed + 1)) - 0.5).to(device),
            [32, 1024, cols], [32, 1024, cols]]


def _ln_bwd_inputs(device="cuda", seed=1):
    x = _randn((32768, 768), torch.bfloat16, seed, device)
    dy = _randn((32768, 768), torch.bfloat16, seed + 100, device)
    w = (torch.rand(768, generator=_gen(seed)) + 0.5).to(device)
    xf = x.float()
    mean = xf.mean(dim=1)
    rstd = torch.rsqrt(xf.var(dim=1, unbiased=False) + 1e-5)
    return [x, dy, w, mean, rstd]


def _bn_bwd_inputs(device="cuda", seed=1):
    shape = (256, 64, 56, 56)
    x = _randn(shape, torch.bfloat16, seed, device).contiguous(memory_format=torch.channels_last)
    dy = _randn(shape, torch.bfloat16, seed + 100, device).contiguous(memory_format=torch.channels_last)
    mean = torch.zeros(64, device=device)
    invstd = torch.ones(64, device=device)
    w = (torch.rand(64, generator=_gen(seed)) + 0.5).to(device)
    return [dy, x, mean, invstd, w]


def _head_split_inputs(device="cuda", seed=1):
    return [_randn((4 * 4096, 32 * 128), torch.bfloat16, seed, device), [4, 4096, 4096], [4, 4096, 32, 128],
            [128, 4096, 128]]


def _transpose_inputs(device="cuda", seed=1):
    return [_randn((64, 1024, 768), torch.bfloat16, seed, device), [64, 768, 1024]]


def _cast_inputs(device="cuda", seed=1):
    return [_randn((64 << 20,), torch.bfloat16, seed, device)]


def _softmax_long_inputs(device="cuda", seed=1):
    return [_randn((1024, 131072), torch.bfloat16, seed, device)]


def _log_softmax_ragged_inputs(device="cuda", seed=1):
    return [_randn((4096, 20008), torch.bfloat16, seed, device)]  # the softmax runs over the first 20005 columns


def _bn_nchw_inputs(device="cuda", seed=1):
    c = 128
    return [_randn((128, c, 56, 56), torch.bfloat16, seed, device), torch.zeros(c, device=device),
            torch.ones(c, device=device), (torch.rand(c, generator=_gen(seed)) + 0.5).to(device),
            (torch.rand(c, generator=_gen(seed + 1)) - 0.5).to(device)]


def _bn_bwd_nchw_inputs(device="cuda", seed=1):
    shape = (128, 128, 56, 56)
    x = _randn(shape, torch.bfloat16, seed, device)
    dy = _randn(shape, torch.bfloat16, seed + 100, device)
    return [dy, x, torch.zeros(128, device=device), torch.ones(128, device=device),
            (torch.rand(128, generator=_gen(seed)) + 0.5).to(device)]


def _gelu_ln_inputs(device="cuda", seed=1):
    return [_randn((65536, 768), torch.bfloat16, seed, device),
            (torch.rand(768, generator=_gen(seed)) + 0.5).to(torch.bfloat16).to(device),
            (torch.rand(768, generator=_gen(seed + 1)) - 0.5).to(torch.bfloat16).to(device)]


def _rms_bwd_scalar_inputs(device="cuda", seed=1):
    x = _randn((262144, 512), torch.bfloat16, seed, device)
    rstd = torch.rsqrt(x.float().pow(2).mean(dim=1) + 1e-6)
    return [x, torch.tensor(0.75, dtype=torch.bfloat16, device=device),
            (torch.rand(512, generator=_gen(seed)) + 0.5).to(device), rstd]


def _bn_nchw_small_inputs(device="cuda", seed=1):
    c = 384
    return [_randn((128, c, 8, 8), torch.bfloat16, seed, device), torch.zeros(c, device=device),
            torch.ones(c, device=device), (torch.rand(c, generator=_gen(seed)) + 0.5).to(device),
            (torch.rand(c, generator=_gen(seed + 1)) - 0.5).to(device)]


def _bn_cl_odd_inputs(device="cuda", seed=1):
    c = 92
    x = _randn((512, c, 14, 14), torch.bfloat16, seed, device).contiguous(memory_format=torch.channels_last)
    return [x, torch.zeros(c, device=device), torch.ones(c, device=device),
            (torch.rand(c, generator=_gen(seed)) + 0.5).to(device), (torch.rand(c, generator=_gen(seed + 1)) - 0.5).to(device)]


def _ln_bwd_scalar_inputs(device="cuda", seed=1):
    x = _randn((262144, 512), torch.bfloat16, seed, device)
    xf = x.float()
    mean = xf.mean(dim=1)
    rstd = torch.rsqrt(xf.var(dim=1, unbiased=False) + 1e-5)
    return [x, torch.tensor(0.75, dtype=torch.bfloat16, device=device),
            (torch.rand(512, generator=_gen(seed)) + 0.5).to(device), mean, rstd]


def _transpose_small_inputs(device="cuda", seed=1):
    return [_randn((16384, 49, 128), torch.bfloat16, seed, device), [16384, 128, 49]]


MB = 1 << 20
FAMILY_CASES = {c.name: c for c in [
    _case("col_sum_f32", "column sum: x f32 [16384, 4096] -> f32 [4096]", "f32",
          16384 * 4096 * 4 + 4096 * 4, _col_sum_inputs, lambda i: column_sum.oracle_forward(i)),
    _case("spatial_mean_cl_bf16", "mean over H,W: x bf16 channels_last [256,64,56,56] -> bf16 [256,64,1,1]", "bf16",
          256 * 64 * 3136 * 2 + 256 * 64 * 2, _spatial_mean_inputs, lambda i: column_sum.spatial_mean_forward(i)),
    _case("row_amax_bf16", "row amax: x bf16 [65536, 1024] -> bf16 [65536]", "bf16",
          65536 * 1024 * 2 + 65536 * 2, _row_amax_inputs, lambda i: kernels.row_reduce(i[0], "amax")),
    _case("row_var_mean_f32", "row var_mean: x f32 [32768, 1024] -> var, mean f32 [32768]", "f32",
          32768 * 1024 * 4 + 2 * 32768 * 4, _row_var_mean_inputs,
          lambda i: kernels.norm_fwd(i[0], None, None, eps=0.0, want_y=False, want_mean=True, want_var=True,
                                     correction=1.0)),
    _case("log_softmax_bf16_f32", "log_softmax: x bf16 [32768, 1024] -> f32", "bf16",
          32768 * 1024 * (2 + 4), _log_softmax_inputs,
          lambda i: kernels.softmax(i[0], log=True, out_dtype=torch.float32)),
    _case("rms_norm_fwd_bf16", "RMSNorm forward: x bf16 [16384, 4096], w bf16 -> y bf16", "bf16",
          2 * 16384 * 4096 * 2 + 4096 * 2, _rms_fwd_inputs,
          lambda i: kernels.norm_fwd(i[0], i[1], None, eps=1e-6, rms=True)[0]),
    _case("dropout_rms_norm_bf16",
          "dropout + residual -> RMSNorm -> dropout: x bf16 [32768, 512], residual f32 -> 2 masks, sum f32, rstd, y bf16",
          "bf16", 32768 * 512 * (2 + 4 + 1 + 4 + 1 + 2) + 32768 * 4 + 512 * 4, _dropout_rms_inputs,
          lambda i: dropout_rms_norm.oracle_forward(i)),
    _case("dropout_add_bf16", "dropout + residual: x bf16 [16384, 2560], residual f32 -> mask, sum f32", "bf16",
          16384 * 2560 * (2 + 4 + 1 + 4), _dropout_add_inputs, lambda i: dropout_rms_norm.add_forward(i)),
    _case("dropout_layer_norm_bf16",
          "dropout + residual -> LayerNorm: x bf16 [32768, 768], residual f32 -> mask, xhat f32, y f32, rstd/n",
          "bf16", 32768 * 768 * (2 + 4 + 1 + 4 + 4) + 32768 * 4 + 2 * 768 * 4, _dropout_ln_inputs,
          lambda i: dropout_rms_norm.layer_norm_forward(i)),
    _case("layer_norm_bwd_bf16", "LayerNorm backward: x, dy bf16 [32768, 768] -> dx bf16, dweight, dbias f32", "bf16",
          3 * 32768 * 768 * 2 + 768 * 4 * 3 + 2 * 32768 * 4, _ln_bwd_inputs,
          lambda i: kernels.norm_bwd(i[0], i[1], i[2], i[4], mean=i[3], rms=False, want_dbias=True)),
    _case("batch_norm_bwd_cl_bf16", "BatchNorm backward: dy, x bf16 channels_last [256,64,56,56] -> dx, dweight, dbias",
          "bf16", 3 * 256 * 64 * 3136 * 2 + 5 * 64 * 4, _bn_bwd_inputs, lambda i: batch_norm_bwd.oracle_forward(i)),
    _case("head_split_bf16", "[B*S, H*D] -> [B*H, S, D] copy: bf16, B=4 S=4096 H=32 D=128", "bf16",
          2 * 16384 * 4096 * 2, _head_split_inputs, lambda i: permute.head_split_forward(i)),
    _case("transpose_bf16", "[64, 1024, 768] -> [64, 768, 1024] contiguous copy, bf16", "bf16",
          2 * 64 * 1024 * 768 * 2, _transpose_inputs, lambda i: permute.transpose_forward(i)),
    _case("cast_bf16_f32", "cast bf16 -> f32, 64 Mi elements", "bf16",
          (64 << 20) * 6, _cast_inputs, lambda i: kernels.cast_scale(i[0], torch.float32)),
    _case("softmax_long_rows_bf16", "softmax over rows of 131072: x bf16 [1024, 131072] -> bf16", "bf16",
          2 * 1024 * 131072 * 2, _softmax_long_inputs, lambda i: kernels.softmax(i[0])),
    _case("log_softmax_ragged_bf16_f32", "log_softmax over 20005 of 20008 columns: x bf16 [4096, 20005] -> f32", "bf16",
          4096 * 20005 * (2 + 4), _log_softmax_ragged_inputs,
          lambda i: kernels.softmax(i[0][:, :20005], log=True, out_dtype=torch.float32)),
    _case("batch_norm_relu_nchw_bf16", "BatchNorm2d train fwd + ReLU: x bf16 NCHW [128,128,56,56]", "bf16",
          2 * 128 * 128 * 3136 * 2 + 6 * 128 * 4, _bn_nchw_inputs,
          lambda i: kernels.batch_norm_fwd(i[0], i[3], i[4], i[1], i[2], eps=1e-3, momentum=0.1, relu=True)),
    _case("batch_norm_bwd_nchw_bf16", "BatchNorm backward: dy, x bf16 NCHW [128,128,56,56] -> dx, dweight, dbias", "bf16",
          3 * 128 * 128 * 3136 * 2 + 5 * 128 * 4, _bn_bwd_nchw_inputs, lambda i: batch_norm_bwd.oracle_forward(i)),
    _case("gelu_layer_norm_bf16", "exact GELU -> bf16 -> LayerNorm: x bf16 [65536, 768], w/b bf16 -> y bf16", "bf16",
          2 * 65536 * 768 * 2 + 2 * 768 * 2, _gelu_ln_inputs,
          lambda i: kernels.norm_fwd(i[0], i[1], i[2], eps=1e-12, prologue="gelu_erf")[0]),
    _case("rms_norm_bwd_scalar_dy_bf16", "RMSNorm backward, dy a broadcast scalar: x bf16 [262144, 512] -> dx bf16, dweight f32",
          "bf16", 2 * 262144 * 512 * 2 + 262144 * 4 + 2 * 512 * 4, _rms_bwd_scalar_inputs,
          lambda i: kernels.norm_bwd(i[0], i[1], i[2], i[3], rms=True)),
    _case("batch_norm_relu_nchw_small_bf16", "BatchNorm2d train fwd + ReLU, channel in registers: x bf16 NCHW [128,384,8,8]", "bf16",
          2 * 128 * 384 * 64 * 2 + 6 * 384 * 4, _bn_nchw_small_inputs,
          lambda i: kernels.batch_norm_fwd(i[0], i[3], i[4], i[1], i[2], eps=1e-3, momentum=0.1, relu=True)),
    _case("batch_norm_relu_cl_c92_bf16", "BatchNorm2d train fwd + ReLU, 92 channels: x bf16 channels_last [512,92,14,14]", "bf16",
          2 * 512 * 92 * 196 * 2 + 6 * 92 * 4, _bn_cl_odd_inputs,
          lambda i: kernels.batch_norm_fwd(i[0], i[3], i[4], i[1], i[2], eps=1e-3, momentum=0.1, relu=True)),
    _case("layer_norm_bwd_scalar_dy_bf16", "LayerNorm backward, dy a broadcast scalar: x bf16 [262144, 512] -> dx bf16, dweight, dbias f32",
          "bf16", 2 * 262144 * 512 * 2 + 2 * 262144 * 4 + 3 * 512 * 4, _ln_bwd_scalar_inputs,
          lambda i: kernels.norm_bwd(i[0], i[1], i[2], i[4], mean=i[3], rms=False, want_dbias=True)),
    _case("transpose_small_bf16", "[16384, 49, 128] -> [16384, 128, 49] contiguous copy, bf16", "bf16",
          2 * 16384 * 49 * 128 * 2, _transpose_small_inputs, lambda i: permute.transpose_forward(i)),
]}
