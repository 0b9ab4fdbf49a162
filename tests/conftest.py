"""pytest configuration: the ``gpu`` marker, import paths, shared tolerances and helpers."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Acceptance tolerances of the backend: outputs must match the eager module on the same inputs.
TOL = {
    "float32": dict(rtol=1.3e-6, atol=1e-5),
    "bfloat16": dict(rtol=1.6e-2, atol=1e-2),
    "float16": dict(rtol=1.6e-2, atol=1e-2),
}


def assert_close(actual, expected, what=""):
    """Compare one output against the eager result with the tolerance of the output dtype."""
    import torch

    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    assert actual.dtype == expected.dtype, f"{what}: dtype {actual.dtype} vs {expected.dtype}"
    if not expected.is_floating_point():
        assert torch.equal(actual.cpu(), expected.cpu()), f"{what}: integer outputs differ"
        return
    tol = TOL[str(expected.dtype).replace("torch.", "")]
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    if not torch.allclose(a, e, equal_nan=True, **tol):
        diff = (a - e).abs()
        diff = torch.where(torch.isnan(diff), torch.zeros_like(diff), diff)
        idx = int(diff.argmax())
        raise AssertionError(
            f"{what}: max abs diff {diff.max().item():.3e} at flat index {idx} "
            f"(got {a.flatten()[idx].item():.8g}, want {e.flatten()[idx].item():.8g}); tol {tol}")
