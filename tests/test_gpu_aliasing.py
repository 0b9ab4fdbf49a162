"""Regions whose outputs are views: beyond the values (tests/test_gpu_golden.py), the outputs must
alias each other and the inputs exactly as the eager graph's outputs do - same strides, same
storage offsets relative to the buffer they share, same sharing."""
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"


def _load_inputs(name):
    data = torch.load(GOLDEN / f"{name}.pt", weights_only=False)
    return [i.clone().cuda() if isinstance(i, torch.Tensor) else i for i in data["inputs"]]


def _structure(outputs, inputs):
    """Per output: (shape, stride, which buffer it lives in, element offset inside that buffer).
    Buffers are numbered in order of first appearance; an input's storage is named by its index."""
    owners = {i.untyped_storage().data_ptr(): f"input{k}" for k, i in enumerate(inputs) if isinstance(i, torch.Tensor)}
    fresh, desc = {}, []
    for o in outputs:
        key = o.untyped_storage().data_ptr()
        owner = owners.get(key)
        if owner is None:
            owner = fresh.setdefault(key, f"new{len(fresh)}")
        desc.append((tuple(o.shape), tuple(o.stride()), owner, o.storage_offset()))
    return desc


def _stub(dirname):
    from better_benchmark_b200 import harness
    root = Path(__file__).resolve().parents[1] / "better-benchmark_b200" / "canonical"
    harness.get_gpu_kind._cached = "B200"
    harness.reset_oracle_registry()
    _, fn, _ = harness._load_oracle_module(root / dirname)
    return fn


@pytest.mark.parametrize("fixture,dirname,module", [
    ("cast_alias_8bb40810003c", "pointwise_8bb40810003c", "CastWithTransposedAlias"),
    ("scale_view_95ed2ef35da9", "pointwise_95ed2ef35da9", "ScaleIntoHeadView"),
    ("qkv_views_1611fb0c7845", "pointwise_1611fb0c7845", "QkvSplitViews"),
])
def test_outputs_alias_like_the_eager_graph(fixture, dirname, module):
    from better_benchmark_b200 import harness, native
    from oracle import eager

    inputs = _load_inputs(fixture)
    fn = _stub(dirname)
    selected, _ = harness.resolve_oracle(fn, inputs)
    before = native.load().b200_launch_count()
    got = harness._normalize_outputs(selected(inputs))
    launched = native.load().b200_launch_count() - before
    eager_inputs = _load_inputs(fixture)
    with torch.no_grad():
        want = harness._normalize_outputs(getattr(eager, module)()(*eager_inputs))
    assert _structure(got, inputs) == _structure(want, eager_inputs)
    for g, w in zip(got, want):
        assert g.dtype == w.dtype and torch.equal(g, w)
    if module == "QkvSplitViews":
        assert launched == 0, "views of the input: nothing to launch"
        x = inputs[0]
        assert all(o.untyped_storage().data_ptr() == x.untyped_storage().data_ptr() for o in got)
    else:
        assert launched == 1
    if module == "CastWithTransposedAlias":
        assert got[0].data_ptr() == got[1].data_ptr()
        got[1][0, 1] = 7.0                      # writing through one view is seen through the other
        assert got[0][1, 0].item() == 7.0
