"""Regions whose outputs are VIEWS: what the harness compares is values, but what a consumer of the
region sees is also which outputs share storage, with which strides and offsets. These adapters
return exactly the aliasing structure of the eager graphs (family ``pointwise``, cast / scale /
split forms):

``cast_with_transposed_alias``  repros/canonical/pointwise_8bb40810003c/repro.py:23-29 - one cast
    f32 -> bf16, returned twice: as its transpose and as itself (two views of ONE buffer; the
    reference's kernel: oracle.py:11-15, the views: :102-119).
``scale_into_head_view``  repros/canonical/pointwise_95ed2ef35da9/repro.py:23-30 - ``x * 0.125`` into
    backing storage laid out like x, returned as the [B, H, S, D] permuted view of it (strided, not
    contiguous; reference: oracle.py:10-44).
``qkv_split_views``  repros/canonical/pointwise_1611fb0c7845/repro.py:23-37 - no arithmetic at all:
    three strided views of the INPUT (packed q, k, v -> [B, H, S, D] each; reference: oracle.py:23-50).
    No kernel is launched, nothing is allocated.
"""
import torch

from .. import kernels


def _resolve(shape, numel):
    """A lifted view shape with at most one -1, resolved against the number of elements."""
    dims = [int(d) for d in shape]
    if -1 in dims:
        known = 1
        for d in dims:
            if d != -1:
                known *= d
        dims[dims.index(-1)] = numel // known if known else 0
    return dims


def cast_with_transposed_alias(inputs, *, out_dtype=torch.bfloat16):
    x = inputs[0]
    base = kernels.cast_scale(x, out_dtype)          # one kernel, one buffer with x's layout
    return base.permute(1, 0), base                  # both outputs alias it


def scale_into_head_view(inputs, *, scale=0.125):
    x, shape3, shape4 = inputs[:3]
    scaled = kernels.cast_scale(x, x.dtype, scale=scale)   # backing storage, laid out like x
    b, s, hidden = _resolve(shape3, x.numel())
    _, _, h, d = _resolve(shape4, x.numel())
    return scaled.view(b, s, hidden).view(b, s, h, d).permute(0, 2, 1, 3)


def qkv_split_views(inputs, *, width=768, order=None):
    """``width``: the split size, a literal of the captured graph (repro.py:27). ``order``: which
    chunk each output is (default 0, 1, 2 ...; repros/canonical/pointwise_d5a413a2c233/repro.py:28-36
    returns chunks 1, 2, 0)."""
    x, shape3 = inputs[0], inputs[1]
    b, s, packed = _resolve(shape3, x.numel())
    chunks = packed // width
    _, _, h, d = _resolve(inputs[2], b * s * width)
    v = x.view(b, s, packed)
    picks = range(chunks) if order is None else order
    return tuple(v[:, :, i * width:(i + 1) * width].view(b, s, h, d).permute(0, 2, 1, 3) for i in picks)
