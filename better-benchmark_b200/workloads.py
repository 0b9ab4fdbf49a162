"""The five benchmark configurations: seeded synthetic inputs, byte counts, oracle entry points.

These are synthetic stand-ins shaped like the reference's repro families (no such point exists
verbatim in its corpus): shapes, dtypes, memory formats and value distributions are fixed here,
and every tensor comes from a seeded ``torch.Generator`` so that any two processes build the same
bits. ``algorithmic_bytes`` is the minimum-bytes model of the region (each input once + each
output once, ``byte_model.count_bytes_effective``); tests recompute it from the eager module.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from .families import batch_norm_relu, layer_norm, masked_softmax, rms_norm_bwd_heads, row_mean


@dataclass(frozen=True)
class Workload:
    name: str
    canonical_id: str          # directory name under canonical/
    shape_hash: str
    description: str
    dtype: str                 # arithmetic/storage dtype string reported by the benchmark
    algorithmic_bytes: int
    make_inputs: Callable      # (device, seed, scale=1) -> list of inputs
    oracle_forward: Callable   # the product entry point for this family
    mutates_inputs: bool = False


def _gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def _c1(device="cuda", seed=1, rows=8192, cols=4096):
    g = _gen(seed)
    return [torch.randn(rows, cols, generator=g).to(device)]


def _c2(device="cuda", seed=1, rows=32768, hidden=768):
    g = _gen(seed)
    x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
    w = (torch.rand(hidden, generator=g) + 0.5).to(torch.bfloat16)
    b = (0.02 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    return [x.to(device), w.to(device), b.to(device)]


def _c3(device="cuda", seed=1, batch=16, heads=12, q=512, k=512):
    g = _gen(seed)
    scores = torch.randn(batch, heads, q, k, generator=g).to(torch.float16)
    lengths = torch.randint(k // 4, k + 1, (batch,), generator=g)
    keys = torch.arange(k)[None, :]
    mask = torch.where(keys < lengths[:, None], 0.0, -10000.0).to(torch.float16).view(batch, 1, 1, k)
    return [scores.to(device), mask.to(device)]


def _c4(device="cuda", seed=1, n=256, c=64, h=56, w=56):
    g = _gen(seed)
    x = (0.5 + 2.0 * torch.randn(n, c, h, w, generator=g)).to(torch.bfloat16)
    x = x.contiguous(memory_format=torch.channels_last)
    weight = torch.rand(c, generator=g) + 0.5
    bias = 0.1 * torch.randn(c, generator=g)
    running_mean, running_var = torch.zeros(c), torch.ones(c)
    return [x.to(device), running_mean.to(device), running_var.to(device), weight.to(device), bias.to(device)]


def _c5(device="cuda", seed=1, b=4, s=4096, h=32, d=128):
    g = _gen(seed)
    x = torch.randn(b, s, h, d, generator=g).to(torch.bfloat16)
    dy = torch.randn(b, s, h, d, generator=g).to(torch.bfloat16)
    w = (torch.rand(h * d, generator=g) + 0.5).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().view(b * s, h * d).pow(2).mean(-1) + 1e-6)
    return [x.to(device), dy.to(device), w.to(device), rstd.to(device)]


WORKLOADS = {
    "c1_row_mean": Workload(
        "c1_row_mean", "mean_b200c1a00001", "c1a00001",
        "row mean: x fp32 [8192, 4096] -> fp32 [8192]", "f32", 134_250_496, _c1,
        row_mean.oracle_forward),
    "c2_layer_norm_fwd": Workload(
        "c2_layer_norm_fwd", "var_mean_b200c2a00002", "c2a00002",
        "LayerNorm forward: x bf16 [32768, 768], w/b bf16 [768], eps 1e-12 -> y bf16, mean/rstd fp32 [32768]",
        "bf16", 100_928_512, _c2, layer_norm.oracle_forward),
    "c3_masked_softmax": Workload(
        "c3_masked_softmax", "amax_sum_b200c3a00003", "c3a00003",
        "masked scaled softmax: scores fp16 [16,12,512,512] * 0.125 + mask fp16 [16,1,1,512] -> fp16",
        "f16", 201_342_976, _c3, masked_softmax.oracle_forward),
    "c4_batch_norm_relu": Workload(
        "c4_batch_norm_relu", "var_mean_b200c4a00004", "c4a00004",
        "BatchNorm2d train fwd + ReLU: x bf16 channels_last [256,64,56,56], eps 1e-5, momentum 0.1",
        "bf16", 205_522_944, _c4, batch_norm_relu.oracle_forward, mutates_inputs=True),
    "c5_rms_norm_bwd": Workload(
        "c5_rms_norm_bwd", "sum_sum_b200c5a00005", "c5a00005",
        "RMSNorm backward + head transpose: x,dy bf16 [4,4096,32,128] -> dx bf16 [4,32,4096,128], dw fp32 [4096]",
        "bf16", 402_743_296, _c5, rms_norm_bwd_heads.oracle_forward),
}

# The configuration the headline metric is quoted on (second entry of the baseline's list).
HEADLINE = "c2_layer_norm_fwd"
