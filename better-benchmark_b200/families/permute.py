"""Permuting copies with pointwise epilogues (family ``pointwise`` with permute / clone / view).

``head_split_forward``: [B*S, H*D] -> [B*H, S, D] (reference graph
repros/canonical/pointwise_c0d19d490a2f/repro.py, replaced kernel .../oracle.py:10-33);
``transpose_forward``: [.., P, C] -> [.., C, P] contiguous, returned under a lifted view shape
(repros/canonical/pointwise_021e90d9c17d/repro.py, replaced kernel .../oracle.py:10-51)."""
from .. import kernels


def head_split_forward(inputs):
    x, _flat3, split4, out3 = inputs[:4]
    b, s, h, d = split4
    return kernels.permute_copy(x.view(b, s, h, d), (0, 2, 1, 3)).view(out3)


def head_merge_forward(inputs):
    """The inverse of the head split: [B*H, S, D] -> view [B, H, S, D] -> permute(0, 2, 1, 3) ->
    contiguous -> view [B, S, H*D] -> view [B*S, H*D]
    (repros/canonical/pointwise_e87d6ebc9ded/repro.py:24-31; lifted shapes may hold one -1)."""
    x, split4, merged3, flat2 = inputs[:4]
    y = kernels.permute_copy(x.view([int(d) for d in split4]), (0, 2, 1, 3))
    return y.view([int(d) for d in merged3]).view([int(d) for d in flat2])


def transpose_forward(inputs):
    x, out_shape = inputs[:2]
    nd = x.dim()
    dims = list(range(nd - 2)) + [nd - 1, nd - 2]
    return kernels.permute_copy(x, dims).view(out_shape)
