"""shapes.json decoding and seeded input generation for canonical repro directories.

Read side of the reference's data format:
  * compact input entries (``input_codec.py:146-178``): ``[shape, dtype, opts?]`` tensors with
    optional ``st`` stride, ``dev`` device, ``off`` storage offset, ``gen`` generator;
    ``["S", dims]`` lifted shape parameters; ``["sc", v]`` scalars; ``["sym", v]`` symints
  * ``shapes.json`` points (``repro_harness.py:91-157``): each point has a ``shape_hash``,
    ``models`` and ``inputs``; the label of a point is ``<last component of first model>_<hash>``
  * input materialisation (``repro_harness.py:430-569``): ``randn`` for floating tensors (over the
    whole strided storage), bounded ``randint`` for integers, 0/1 for bool, generators for index,
    permutation, offsets and constant tensors.
Symbolic (dynamic-shape) points and alias groups are outside the families this backend covers
and raise ``NotImplementedError`` rather than being silently skipped.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

LONG_DTYPE = {
    "f32": "float32", "f16": "float16", "bf16": "bfloat16", "f64": "float64", "i64": "int64",
    "i32": "int32", "i16": "int16", "i8": "int8", "b8": "bool", "u8": "uint8",
}
SHORT_DTYPE = {v: k for k, v in LONG_DTYPE.items()}


def contiguous_stride(shape) -> list:
    stride = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        stride[i] = stride[i + 1] * max(int(shape[i + 1]), 1)
    return stride


def _gen_from_compact(c) -> dict:
    kind = c[0]
    if kind in ("index", "randint"):
        return {"kind": kind, "low": c[1], "high": c[2]}
    if kind == "perm":
        return {"kind": "permutation", "size": c[1] if len(c) > 1 else None}
    if kind == "offsets":
        return {"kind": "offsets", "high": c[1]}
    if kind == "const":
        return {"kind": "constant", "value": c[1]}
    return {"kind": kind}


def spec_from_compact(entry, name: str | None = None) -> dict:
    """One compact shapes.json entry -> the verbose per-input spec dict."""
    if entry and entry[0] == "S":
        return {"kind": "shape", "name": name, "dims": list(entry[1])}
    if entry and entry[0] == "sym":
        return {"kind": "symint", "name": name, "value": entry[1]}
    if entry and entry[0] == "sc":
        return {"kind": "scalar", "name": name, "value": entry[1]}
    if entry and entry[0] == "I":
        raise NotImplementedError("symbolic symint entries are not supported")
    shape = list(entry[0])
    if any(isinstance(d, str) for d in shape):
        raise NotImplementedError("symbolic dimensions are not supported")
    opts = entry[2] if len(entry) > 2 else {}
    spec = {
        "kind": "tensor",
        "name": name if name is not None else opts.get("n"),
        "shape": shape,
        "dtype": LONG_DTYPE.get(entry[1], entry[1]),
        "stride": list(opts.get("st", contiguous_stride(shape))),
        "device": opts.get("dev", "cuda"),
        "storage_offset": opts.get("off", 0),
    }
    if "gen" in opts:
        spec["gen"] = _gen_from_compact(opts["gen"])
    if "alias" in opts:
        spec["alias_group"] = opts["alias"]
    return spec


def compact_from_tensor(t: torch.Tensor) -> list:
    """The compact entry that describes a tensor (used to author shapes.json files)."""
    entry = [list(t.shape), SHORT_DTYPE[str(t.dtype).replace("torch.", "")]]
    if list(t.stride()) != contiguous_stride(t.shape):
        entry.append({"st": list(t.stride())})
    return entry


def point_label(point: dict) -> str:
    shape_hash = point.get("shape_hash", "unknown")
    first_model = next(iter(point.get("models", {})), "")
    short = first_model.rsplit("/", 1)[-1] if first_model else ""
    return f"{short}_{shape_hash}" if short else shape_hash


def load_shape_configs(repro_file) -> dict:
    """{label: {"inputs": [spec, ...]}} for the shapes.json next to ``repro_file``; {} if absent."""
    path = Path(repro_file).parent / "shapes.json"
    if not path.exists():
        return {}
    data = json.loads(path.read_text())
    if data.get("symbols"):
        raise NotImplementedError(f"{path}: dynamic-shape repros are not supported")
    configs = {}
    for point in data.get("points", []):
        compact = point.get("inputs")
        if compact is None:
            raise ValueError(f"{path}: point {point.get('shape_hash')} has no structured inputs")
        configs[point_label(point)] = {"inputs": [spec_from_compact(e) for e in compact]}
    return configs


def _storage_size(shape, stride) -> int:
    if any(int(s) == 0 for s in shape):
        return 0
    return 1 + sum((int(s) - 1) * int(st) for s, st in zip(shape, stride))


def _strided(make_flat, shape, stride, offset=0):
    numel = _storage_size(shape, stride) + int(offset)
    return make_flat(numel).as_strided(shape, stride, int(offset))


def make_inputs_from_config(config: dict, device: str | None = None) -> list:
    """Materialise the inputs of one shape point with torch's current RNG state.

    ``device`` overrides every tensor spec's device (the specs default to "cuda"); the CPU
    baseline and CPU tests pass "cpu".
    """
    out = []
    for spec in config["inputs"]:
        kind = spec.get("kind", "tensor")
        if kind == "shape":
            out.append(list(spec["dims"]))
            continue
        if kind == "symint":
            out.append(int(spec["value"]))
            continue
        if kind == "scalar":
            out.append(spec["value"])
            continue
        if spec.get("alias_group") is not None:
            raise NotImplementedError("alias-group inputs are not supported")
        shape = [int(s) for s in spec["shape"]]
        dtype = getattr(torch, spec["dtype"].replace("torch.", ""))
        dev = device or spec.get("device", "cuda")
        stride = spec.get("stride")
        if stride is not None and list(stride) == contiguous_stride(shape):
            stride = None
        offset = spec.get("storage_offset", 0)
        gen = spec.get("gen")

        def build(flat_factory):
            if stride or offset:
                return _strided(flat_factory, shape, stride or contiguous_stride(shape), offset)
            n = 1
            for s in shape:
                n *= s
            return flat_factory(n).reshape(shape)

        if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
            if gen and gen["kind"] == "constant":
                out.append(build(lambda n: torch.full((n,), int(gen.get("value", 0)), dtype=dtype, device=dev)))
            elif gen and gen["kind"] == "permutation":
                size = int(gen.get("size") or max(1, _numel(shape)))
                rows = max(1, _numel(shape) // size)
                vals = torch.stack([torch.randperm(size, device=dev) for _ in range(rows)]).to(dtype)
                t = torch.empty_strided(shape, stride or contiguous_stride(shape), dtype=dtype, device=dev)
                t.copy_(vals.reshape(shape))
                out.append(t)
            elif gen and gen["kind"] == "offsets":
                hi = max(int(gen.get("high", 1)), 1)
                vals, _ = torch.sort(torch.randint(0, hi, shape, dtype=dtype, device=dev))
                if vals.numel():
                    vals.reshape(-1)[0] = 0
                out.append(vals)
            else:
                low = int(gen.get("low", 0)) if gen else 0
                hi = int(gen.get("high", 100)) if gen else 100
                hi = max(hi, low + 1)
                out.append(build(lambda n: torch.randint(low, hi, (n,), dtype=dtype, device=dev)))
        elif dtype == torch.bool:
            out.append(build(lambda n: torch.randint(0, 2, (n,), dtype=torch.bool, device=dev)))
        else:
            if gen and gen["kind"] == "index":
                low, hi = int(gen.get("low", 0)), int(gen.get("high", 100))
                hi = max(hi, low + 1)
                out.append(build(lambda n: torch.randint(low, hi, (n,), dtype=torch.int64, device=dev).to(dtype)))
            else:
                out.append(build(lambda n: torch.randn(n, dtype=dtype, device=dev)))
    return out


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n
