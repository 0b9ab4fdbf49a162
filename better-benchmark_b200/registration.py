"""Registration of one ``oracle_forward`` for every shape point of its canonical directory.

The reference keys an oracle registration on the 8-hex ``shape_hash`` of a point in the
``shapes.json`` next to the oracle file (``oracle_impl(hardware=, point=)``, oracle_harness.py:468-549);
a point registered that way dispatches as ``matched="hardware+shape"``, anything else is reported
as a fallback (oracle_harness.py:240-300). The kernels here are shape-general, so a stub registers
itself once per point listed in the sibling ``shapes.json`` and once more without a shape, for inputs
outside the list (reduced test shapes, new points):

    from better_benchmark_b200.registration import every_point

    @every_point(oracle_impl, hardware="B200", eps=1e-5)
    def oracle_forward(inputs, *, eps): ...

``oracle_impl`` is whichever harness the stub imported: the reference's, or this package's mirror.
Two points whose tensor shapes are equal (they differ in dtype only) share one registration.
"""
from __future__ import annotations

import inspect
import json
import sys
from pathlib import Path


def _points(stub_file) -> list:
    path = Path(stub_file).resolve().parent / "shapes.json"
    if not path.is_file():
        return []
    return [p for p in json.loads(path.read_text()).get("points", []) if p.get("shape_hash")]


def point_hashes(stub_file) -> list:
    """shape_hash of every point in the shapes.json next to ``stub_file`` ([] without one)."""
    return [p["shape_hash"] for p in _points(stub_file)]


def _tensor_shapes(point, harness):
    decode = getattr(harness, "spec_from_compact", None)
    if decode is None:
        from input_codec import spec_from_compact as decode  # the reference keeps it there
    specs = [decode(e) for e in point.get("inputs", [])]
    return tuple(tuple(s["shape"]) for s in specs if s.get("kind") == "tensor")


def every_point(oracle_impl, hardware="B200", **kwargs):
    harness = sys.modules[oracle_impl.__module__]

    def decorator(fn):
        stub_file = getattr(inspect.getmodule(fn), "__file__", None) or inspect.getfile(fn)
        seen = set()
        for point in _points(stub_file):
            shapes = _tensor_shapes(point, harness)
            if shapes in seen:
                continue  # same tensor shapes as an earlier point: one entry serves both
            seen.add(shapes)
            oracle_impl(hardware=hardware, point=point["shape_hash"], **kwargs)(fn)
        oracle_impl(hardware=hardware, **kwargs)(fn)  # shape-general: any other input of the family
        return fn

    return decorator
