"""The oracle contract: registration, dispatch, correctness check, CUDA-graph benchmark.

Host-side mirror of the reference's ``oracle_harness.py`` for the path this backend serves, with
the same names, argument meaning and error behaviour, so that an ``oracle.py`` written for one
runs under the other:

  oracle_impl / OracleRegistry / resolve_oracle   ``oracle_harness.py:96-369``, ``:468-577``
  check_oracle / check_oracle_all_shapes          ``:926-1050`` (eager module vs oracle, allclose)
  detect_stochastic_outputs                       ``:807-858``
  bench_oracle                                    ``:1057-1287`` (CUDA graph capture, warning trap,
                                                  fp64-anchored numerics gate, exclusive GPU lock,
                                                  interleaved min-of-rounds timing, status words)
  _anchored_numerics_gate                         ``:1479-1548``
  _runner_main                                    ``:1791-1913`` (``python -m ... <dir> --check/--bench``)

Differences, all additive: timing uses this module's own ``do_bench`` (same protocol as the one
the reference imports: flush a 256 MB buffer, record, replay, record, min over the repetitions)
so that no Triton is needed; ``bench_oracle`` also reports GB/s and the fraction of the measured
HBM peak when it is given the region's byte count; ``compile_reference=False`` skips the
``torch.compile`` arm (the comparison then has no ratio and the status is ``TIMED``).
"""
from __future__ import annotations

import copy
import importlib.util
import inspect
import json
import math
import re
import subprocess
import sys
import time
import warnings
from pathlib import Path

import torch

from .gpu_lock import gpu_exclusive_lock
from .inputs import load_shape_configs, make_inputs_from_config, spec_from_compact


# ---------------------------------------------------------------------------------------------
# Hardware and shape keys
# ---------------------------------------------------------------------------------------------
def get_shape_key(inputs) -> tuple:
    return tuple(tuple(t.shape) for t in inputs if isinstance(t, torch.Tensor))


def get_gpu_kind() -> str:
    """Short GPU name ("B200", "H100", ...) from nvidia-smi; "unknown" when it cannot be read.
    Cached on the function object (tests overwrite ``get_gpu_kind._cached``)."""
    if not hasattr(get_gpu_kind, "_cached"):
        try:
            name = subprocess.check_output(
                ["nvidia-smi", "--query-gpu=name", "--format=csv,noheader"], text=True,
                timeout=5).strip().split("\n")[0]
            for kind in ("B200", "H200", "H100", "A100", "V100"):
                if kind in name:
                    get_gpu_kind._cached = kind
                    break
            else:
                get_gpu_kind._cached = name.replace(" ", "_")[:20]
        except Exception:
            get_gpu_kind._cached = "unknown"
    return get_gpu_kind._cached


# ---------------------------------------------------------------------------------------------
# Registration and dispatch
# ---------------------------------------------------------------------------------------------
class OracleDispatchError(RuntimeError):
    """Registrations exist, but none matches the runtime inputs."""


class OracleRegistry:
    """Per-module list of (hardware, shape signature, kwargs) registrations; exact matching only."""

    def __init__(self):
        self._entries = []
        self.last_dispatch_info = None

    @staticmethod
    def _normalize_shape(shape):
        if shape is None:
            return None, False
        if callable(shape):
            raise TypeError("shape must be a concrete tuple, not a callable predicate")
        shape = tuple(shape)
        if len(shape) == 0:
            return (), True
        if all(isinstance(d, int) for d in shape):
            return (shape,), False
        if all(isinstance(s, (tuple, list, torch.Size)) for s in shape):
            return tuple(tuple(s) for s in shape), True
        raise TypeError(f"shape must be a tuple of ints or a tuple of tuples, got {shape!r}")

    def register(self, hardware=None, shape=None, configs=None, description=None):
        norm_shape, full_sig = self._normalize_shape(shape)
        if configs is not None and not isinstance(configs, dict):
            raise TypeError(f"configs must be a dict or None, got {type(configs).__name__}")

        def decorator(fn):
            for prev in self._entries:
                if prev["hardware"] == hardware and prev["shape"] == norm_shape:
                    print(f"WARNING: duplicate oracle registration for (hardware={hardware!r}, "
                          f"shape={norm_shape!r})", file=sys.stderr)
                    break
            self._entries.append({
                "hardware": hardware, "shape": norm_shape, "full_sig": full_sig, "fn": fn,
                "configs": dict(configs) if configs else None,
                "description": description or fn.__name__,
            })
            return fn
        return decorator

    @staticmethod
    def _matches(entry, actual):
        if entry["shape"] is None:
            return False
        if entry["full_sig"]:
            return tuple(entry["shape"]) == tuple(actual)
        return bool(actual) and tuple(entry["shape"][0]) == tuple(actual[0])

    def select(self, inputs):
        """First hit of: hardware+shape, shape, hardware (shape-general), any (shape-general)."""
        hw = get_gpu_kind()
        actual = get_shape_key(inputs)
        tiers = (
            ("hardware+shape", lambda e: self._matches(e, actual) and e["hardware"] == hw),
            ("shape", lambda e: self._matches(e, actual)),
            ("hardware", lambda e: e["shape"] is None and e["hardware"] == hw),
            ("any", lambda e: e["shape"] is None and e["hardware"] is None),
        )
        for matched, pred in tiers:
            for entry in self._entries:
                if pred(entry):
                    info = {
                        "matched": matched, "fallback": matched != "hardware+shape",
                        "fn_name": entry["fn"].__name__, "description": entry["description"],
                        "tuned_hardware": entry["hardware"], "registered_shape": entry["shape"],
                        "configs": entry["configs"], "current_hardware": hw, "actual_shapes": actual,
                    }
                    self.last_dispatch_info = info
                    return entry, info
        self.last_dispatch_info = None
        raise RuntimeError(f"No oracle registered for hardware={hw!r} shapes={actual!r}. Registry has "
                           f"{len(self._entries)} entries: {[e['description'] for e in self._entries]}")

    def dispatch(self, inputs):
        entry, _ = self.select(inputs)
        return entry["fn"](inputs, **entry["configs"]) if entry["configs"] else entry["fn"](inputs)

    def list_entries(self):
        return [{"hardware": e["hardware"], "shape": e["shape"], "fn_name": e["fn"].__name__,
                 "configs": e["configs"], "description": e["description"]} for e in self._entries]

    def clear(self):
        self._entries.clear()
        self.last_dispatch_info = None


_module_registries: dict = {}


def parse_shapes_signature(shapes):
    """``"(T([8, 4], bf16), S([32]))"`` -> ((8, 4),): tensor shapes only; tuples pass through."""
    if shapes is None:
        return None
    if not isinstance(shapes, str):
        return tuple(tuple(s) for s in shapes)
    found = re.findall(r"T\(\s*\[([^\]]*)\]", shapes)
    return tuple(tuple(int(d) for d in f.split(",") if d.strip()) for f in found)


def oracle_impl(hardware=None, shapes=None, point=None, description=None, **kwargs):
    """Register the decorated function as the oracle for one (hardware, shape point).

    ``point`` is the 8-hex ``shape_hash`` of a point in the shapes.json next to the oracle file
    (unknown hashes raise at import); ``shapes`` is an explicit signature; neither means
    shape-general. Extra keyword arguments are passed to the function at dispatch time. Returns
    the function unchanged, so one body can be registered many times.
    """
    if point is not None and shapes is not None:
        raise ValueError("oracle_impl: pass point= (hash) or shapes=, not both")
    parsed = parse_shapes_signature(shapes)

    def decorator(fn):
        reg = _module_registries.setdefault(fn.__module__, OracleRegistry())
        entry_shapes = parsed
        if point is not None:
            mod = inspect.getmodule(fn)
            fpath = Path(getattr(mod, "__file__", None) or inspect.getfile(fn))
            shapes_path = fpath.parent / "shapes.json"
            if not shapes_path.exists():
                raise OracleDispatchError(f"oracle_impl(point={point!r}): no shapes.json next to {fpath}")
            data = json.loads(shapes_path.read_text())
            match = next((p for p in data.get("points", []) if p.get("shape_hash") == point), None)
            if match is None:
                known = [p.get("shape_hash") for p in data.get("points", [])]
                raise OracleDispatchError(f"oracle_impl(point={point!r}): hash not in {shapes_path} "
                                          f"(known: {known[:8]})")
            specs = [spec_from_compact(e) for e in match.get("inputs", [])]
            entry_shapes = tuple(tuple(s["shape"]) for s in specs if s.get("kind") == "tensor")
        reg.register(hardware=hardware, shape=entry_shapes, configs=kwargs or None,
                     description=description)(fn)
        reg._entries[-1]["point"] = point
        return fn
    return decorator


def get_module_registry(module_name):
    return _module_registries.get(module_name)


def reset_oracle_registry(module_name=None):
    if module_name is None:
        _module_registries.clear()
    else:
        _module_registries.pop(module_name, None)


def resolve_oracle(oracle_forward, inputs):
    """(callable with kwargs bound, dispatch info) - or (oracle_forward, None) when its module
    registered nothing. Raises OracleDispatchError when registrations exist but none matches."""
    reg = _module_registries.get(getattr(oracle_forward, "__module__", None))
    if reg is None or not reg._entries:
        return oracle_forward, None
    try:
        entry, info = reg.select(inputs)
    except RuntimeError as e:
        raise OracleDispatchError(str(e)) from e
    if entry["configs"]:
        fn, cfg = entry["fn"], entry["configs"]
        return (lambda inp: fn(inp, **cfg)), info
    return entry["fn"], info


# ---------------------------------------------------------------------------------------------
# Loading canonical directories
# ---------------------------------------------------------------------------------------------
def _load_file(path: Path, module_name: str):
    spec = importlib.util.spec_from_file_location(module_name, path)
    if spec is None or spec.loader is None:
        raise RuntimeError(f"cannot load {path}")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_repro_module(repro_dir):
    repro_dir = Path(repro_dir)
    return _load_file(repro_dir / "repro.py", f"{repro_dir.name}_repro")


def get_repro_instance(repro_dir):
    return load_repro_module(repro_dir).Repro()


def get_inputs(repro_dir):
    mod = load_repro_module(repro_dir)
    if hasattr(mod, "make_inputs"):
        return mod.make_inputs()
    raise RuntimeError("repro has no make_inputs")


def _load_oracle_module(canonical_dir):
    d = Path(canonical_dir)
    path = d / "oracle.py"
    if not path.exists():
        raise FileNotFoundError(f"no oracle.py in {d}")
    mod = _load_file(path, f"_oracle_{d.name}")
    fn = getattr(mod, "oracle_forward", None)
    if fn is None:
        raise AttributeError(f"{path} defines no oracle_forward")
    return mod, fn, d


def load_numerics_optout(repro_dir):
    """The reviewed ``numerics_optout`` annotation of meta.json, or None (``oracle_harness.py:701-733``)."""
    meta_path = Path(repro_dir) / "meta.json"
    if not meta_path.exists():
        return None
    try:
        meta = json.loads(meta_path.read_text())
    except (OSError, ValueError):
        return None
    opt = meta.get("numerics_optout") if isinstance(meta, dict) else None
    if not isinstance(opt, dict) or opt.get("verified") is not True:
        return None
    reason = opt.get("reason")
    if not (isinstance(reason, str) and reason.strip()):
        return None
    return opt


# ---------------------------------------------------------------------------------------------
# Correctness
# ---------------------------------------------------------------------------------------------
def _normalize_outputs(out) -> list:
    if isinstance(out, torch.Tensor):
        return [out]
    flat = []
    if isinstance(out, (tuple, list)):
        for item in out:
            flat.extend(_normalize_outputs(item))
    return flat


def _seed_input_generation(seed: int) -> None:
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def detect_stochastic_outputs(instance, inputs) -> set:
    """Indices of outputs that differ between two runs on the same inputs (dropout and friends)."""
    torch.manual_seed(42)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(42)
    with torch.no_grad():
        first = _normalize_outputs(instance(*inputs))
        second = _normalize_outputs(instance(*inputs))
    stochastic = set()
    for i, (a, b) in enumerate(zip(first, second)):
        try:
            if a.is_floating_point():
                differs = not torch.allclose(a.float(), b.float(), atol=1e-6, rtol=0, equal_nan=True)
            else:
                differs = not torch.equal(a, b)
        except RuntimeError:
            differs = True
        if differs:
            stochastic.add(i)
    return stochastic


# acceptance tolerances of this backend per output dtype (atol, rtol); used when a caller passes
# atol=None / rtol=None instead of the reference's blanket 1e-2
DTYPE_TOLERANCE = {torch.float32: (1e-5, 1.3e-6), torch.float64: (1e-5, 1.3e-6),
                   torch.bfloat16: (1e-2, 1.6e-2), torch.float16: (1e-2, 1.6e-2)}


def _compare_oracle_outputs(eager, oracle_out, stochastic, *, atol, rtol) -> bool:
    eager_list, oracle_list = _normalize_outputs(eager), _normalize_outputs(oracle_out)
    if len(oracle_list) != len(eager_list):
        print(f"  SCOPE_MISMATCH: oracle produces {len(oracle_list)} outputs, eager produces {len(eager_list)}")
        return False
    ok_all = True
    for i, (e, o) in enumerate(zip(eager_list, oracle_list)):
        if i in stochastic:
            print(f"  output {i}: SKIP (stochastic)")
            continue
        if e.shape != o.shape:
            print(f"  output {i}: SCOPE_MISMATCH shape oracle={list(o.shape)} eager={list(e.shape)}")
            ok_all = False
            continue
        if e.dtype != o.dtype:
            print(f"  output {i}: WARNING dtype mismatch oracle={o.dtype} eager={e.dtype}")
        if not e.is_floating_point():
            ok = torch.equal(e, o)
            print(f"  output {i}: {'PASS' if ok else 'FAIL'} (exact, dtype={e.dtype})")
            ok_all &= ok
            continue
        ef, of = e.float(), o.float()
        diff = (ef - of).abs()
        diff = torch.where(torch.isnan(ef) & torch.isnan(of), torch.zeros_like(diff), diff)
        max_diff = diff.max().item() if diff.numel() else 0.0
        a, r = DTYPE_TOLERANCE.get(e.dtype, (1e-2, 1e-2))
        ok = torch.allclose(ef, of, atol=a if atol is None else atol, rtol=r if rtol is None else rtol, equal_nan=True)
        print(f"  output {i}: {'PASS' if ok else 'FAIL'} (shape={list(e.shape)} dtype={e.dtype} "
              f"max_diff={max_diff:.2e})")
        ok_all &= ok
    return ok_all


def check_oracle(oracle_forward, instance, inputs, *, atol=1e-2, rtol=1e-2, skip_stochastic=True) -> bool:
    """Eager module vs oracle on ``inputs``. Note that both run on the SAME input objects: for a
    repro that mutates its inputs use ``check_oracle_all_shapes`` or pass separate copies."""
    try:
        oracle_forward, _ = resolve_oracle(oracle_forward, inputs)
    except OracleDispatchError as e:
        print(f"  NO_ORACLE_FOR_SHAPE: {str(e)[:200]}")
        return False
    stochastic = detect_stochastic_outputs(instance, inputs) if skip_stochastic else set()
    with torch.no_grad():
        eager = instance(*inputs)
        oracle_out = oracle_forward(inputs)
    return _compare_oracle_outputs(eager, oracle_out, stochastic, atol=atol, rtol=rtol)


def check_oracle_all_shapes(oracle_forward, repro_dir, repro_id, *, skip_stochastic=True, point=None,
                            atol=1e-2, rtol=1e-2, device=None) -> dict:
    """check at every shapes.json point, with separately seeded input copies for eager and oracle."""
    repro_dir = Path(repro_dir)
    configs = load_shape_configs(repro_dir / "repro.py")
    if point is not None:
        configs = {k: v for k, v in configs.items() if k == point or k.endswith(f"_{point}")}
        if not configs:
            print(f"  NO_SHAPE_POINT: {point}")
            return {point: False}
    if not configs:
        return {"default": check_oracle(oracle_forward, get_repro_instance(repro_dir),
                                        get_inputs(repro_dir), atol=atol, rtol=rtol,
                                        skip_stochastic=skip_stochastic)}
    results = {}
    for label, config in configs.items():
        print(f"Checking {repro_id}_{label}...")
        instance = get_repro_instance(repro_dir)
        _seed_input_generation(0)
        probe = make_inputs_from_config(config, device)
        stochastic = detect_stochastic_outputs(instance, probe) if skip_stochastic else set()
        _seed_input_generation(1)
        eager_inputs = make_inputs_from_config(config, device)
        _seed_input_generation(1)
        oracle_inputs = make_inputs_from_config(config, device)
        try:
            selected, _ = resolve_oracle(oracle_forward, oracle_inputs)
        except OracleDispatchError as e:
            print(f"  NO_ORACLE_FOR_SHAPE: {str(e)[:200]}")
            results[label] = False
            continue
        with torch.no_grad():
            eager = instance(*eager_inputs)
            oracle_out = selected(oracle_inputs)
        results[label] = _compare_oracle_outputs(eager, oracle_out, stochastic, atol=atol, rtol=rtol)
    return results


# ---------------------------------------------------------------------------------------------
# fp64-anchored numerics gate
# ---------------------------------------------------------------------------------------------
def _anchored_numerics_gate(oracle_outs, compiled_outs, ref_outs, stochastic, *, ref_precision="f64") -> dict:
    """Per float output: err_oracle <= max(3 * err_compiled, 1e-5 * max(|ref|max, 1))."""
    result = {"pass": True, "per_output": [], "worst_output_idx": None, "ref_precision": ref_precision}
    worst = 0.0
    for i, (o, c, r) in enumerate(zip(oracle_outs, compiled_outs, ref_outs)):
        entry = {"idx": i}
        if i in stochastic:
            entry["skip"] = "stochastic"
        elif not r.is_floating_point():
            entry["skip"] = "non_float"
        else:
            r64 = r.double()
            err_o = (o.double() - r64).abs().max().item() if r64.numel() else 0.0
            err_c = (c.double() - r64).abs().max().item() if r64.numel() else 0.0
            absmax = r64.abs().max().item() if r64.numel() else 0.0
            threshold = max(3.0 * err_c, 1e-5 * max(absmax, 1.0))
            ok = err_o <= threshold
            entry.update(err_oracle=err_o, err_compiled=err_c, threshold=threshold, ref_absmax=absmax)
            entry["pass"] = ok
            if not ok:
                result["pass"] = False
                ratio = err_o / max(err_c, 1e-30)
                if ratio > worst:
                    worst, result["worst_output_idx"] = ratio, i
        result["per_output"].append(entry)
    return result


def _copy_input(t):
    if any(s == 0 for s in t.stride()):
        return t.clone()
    out = torch.empty_strided(t.size(), t.stride(), dtype=t.dtype, device=t.device)
    out.copy_(t)
    return out


def _clone_inputs(inputs):
    return [_copy_input(i) if isinstance(i, torch.Tensor) else i for i in inputs]


def _run_anchored_numerics_gate(oracle_forward, instance, compiled, inputs):
    """fp64 eager anchor vs oracle vs the comparison arm (``compiled``; the fp32 eager module when
    there is no compiled arm). Every run gets its own copy of the inputs."""
    stochastic = detect_stochastic_outputs(instance, _clone_inputs(inputs))
    ref_precision = "f64"
    try:
        inst64 = copy.deepcopy(instance).double()
        in64 = [i.double() if isinstance(i, torch.Tensor) and i.is_floating_point() else i
                for i in _clone_inputs(inputs)]
        _seed_input_generation(1)
        with torch.no_grad():
            ref = _normalize_outputs(inst64(*in64))
    except Exception:
        ref_precision = "f32"
        try:
            _seed_input_generation(1)
            with torch.no_grad():
                ref = _normalize_outputs(instance(*_clone_inputs(inputs)))
        except Exception:
            return None
    _seed_input_generation(1)
    with torch.no_grad():
        oracle_outs = _normalize_outputs(oracle_forward(_clone_inputs(inputs)))
    _seed_input_generation(1)
    with torch.no_grad():
        comp_outs = _normalize_outputs((compiled if compiled is not None else instance)(*_clone_inputs(inputs)))
    if len(oracle_outs) != len(ref) or len(comp_outs) != len(ref):
        return None
    return _anchored_numerics_gate(oracle_outs, comp_outs, ref, stochastic, ref_precision=ref_precision)


# ---------------------------------------------------------------------------------------------
# Timing
# ---------------------------------------------------------------------------------------------
_CUDAGRAPH_WARNING = re.compile(r"CUDAGraph|cuda.?graph|graph.?capture|stream.?capture", re.IGNORECASE)
_flush_buffers: dict = {}


def _flush_buffer(device):
    key = str(device)
    if key not in _flush_buffers:
        _flush_buffers[key] = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=device)
    return _flush_buffers[key]


def do_bench(fn, *, warmup=25, rep=100, return_mode="min", device="cuda"):
    """Time ``fn`` in milliseconds: ``warmup`` / ``rep`` are budgets in MILLISECONDS, converted to
    iteration counts from a first estimate; before every timed call a 256 MB buffer is zeroed so
    that the call starts from a flushed L2; each call is bracketed by CUDA events."""
    cache = _flush_buffer(device)
    fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(5):
        cache.zero_()
        fn()
    end.record()
    torch.cuda.synchronize()
    estimate = start.elapsed_time(end) / 5
    n_warmup = max(1, int(warmup / max(estimate, 1e-6)))
    n_repeat = max(1, int(rep / max(estimate, 1e-6)))
    for _ in range(n_warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_repeat):
        cache.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in zip(starts, ends))
    if return_mode == "min":
        return times[0]
    if return_mode == "median":
        return times[len(times) // 2]
    if return_mode == "mean":
        return sum(times) / len(times)
    raise ValueError(f"unknown return_mode {return_mode!r}")


def memcpy_sol_us(total_bytes: int, *, device="cuda", warmup=10, rep=50) -> float:
    """The reference's speed-of-light yardstick for a region of ``total_bytes`` (read + write):
    ``torch.add(src, 1, out=dst)`` over ``total_bytes // 8`` fp32 elements, i.e. half of the bytes
    read and half written, timed like everything else (CUDA-graph replay from a flushed L2, min).
    ``repro_harness.py:952-958``, ``scripts/bench_parallel.py:3712-3719``. Microseconds."""
    n = max(1, int(total_bytes) // 8)
    src = torch.empty(n, dtype=torch.float32, device=device)
    dst = torch.empty_like(src)
    torch.add(src, 1, out=dst)
    torch.cuda.synchronize()
    graph, _ = _capture_graph_checked(lambda: torch.add(src, 1, out=dst))
    return _time_graph(graph, warmup=warmup, rep=rep)


def _time_graph(graph, warmup, rep) -> float:
    """Microseconds of one graph replay from a flushed L2 (min over the repetitions)."""
    return do_bench(lambda: graph.replay(), warmup=warmup, rep=rep, return_mode="min") * 1000.0


def _capture_graph_checked(fn):
    """Capture ``fn`` into a CUDA graph; returns (graph, [CUDA-graph related warning texts])."""
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(graph):
            fn()
        torch.cuda.synchronize()
    return graph, [str(w.message) for w in caught if _CUDAGRAPH_WARNING.search(str(w.message))]


def _get_device(inputs) -> torch.device:
    for i in inputs:
        if isinstance(i, torch.Tensor):
            return i.device
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


_INVALID_STATUSES = frozenset({"UNVERIFIED_NUMERICS", "INVALID_CUDAGRAPH_WARNING",
                               "NUMERICS_WORSE_THAN_COMPILED", "NO_ORACLE_FOR_SHAPE", "DEVICE_WAIT"})


def bench_oracle(oracle_forward, instance, inputs, repro_id, *, warmup=25, rep=200, rounds=5,
                 _skip_numerics_gate=False, numerics_optout=None, disable_gpu_lock=False,
                 compile_reference=True, region_bytes=None, peak_gbps=None, memcpy_sol=False,
                 adaptive_rep=True) -> dict:
    """Time the oracle (and, by default, ``torch.compile`` of the eager module) as CUDA-graph
    replays from a flushed L2: min over ``rounds`` interleaved rounds, under the exclusive GPU lock.

    Returns {repro_id, oracle_us, compile_us, ratio, status, ...}. Status is GOOD (ratio > 1.05),
    AT_FLOOR, BAD_ORACLE (< 0.95), TIMED (no compile arm), or one of the invalid statuses, in
    which case there are no timings. ``region_bytes`` adds oracle_gbps (and sol_frac with
    ``peak_gbps``).
    """
    try:
        oracle_forward, dispatch = resolve_oracle(oracle_forward, inputs)
    except OracleDispatchError as e:
        result = {"repro_id": repro_id, "status": "NO_ORACLE_FOR_SHAPE", "error": str(e)[:300]}
        print(json.dumps(result))
        return result
    if _get_device(inputs).type != "cuda":
        raise RuntimeError("bench_oracle times CUDA kernels; the inputs are not on a CUDA device")

    def finish(result):
        if dispatch is not None:
            result["dispatch"] = {"matched": dispatch["matched"], "tuned_on": dispatch["tuned_hardware"],
                                  "running_on": dispatch["current_hardware"], "fallback": dispatch["fallback"]}
        print(json.dumps(result, default=str))
        return result

    compiled = g_compile = None
    if compile_reference:
        import torch._dynamo as dynamo
        import torch._inductor.config as inductor_config
        inductor_config.coordinate_descent_tuning = True
        dynamo.reset()
        compiled = torch.compile(instance)
        with torch.no_grad():
            for _ in range(5):
                compiled(*inputs)
            torch.cuda.synchronize()
        g_compile, warns = _capture_graph_checked(lambda: compiled(*inputs))
        if warns:
            return finish({"repro_id": repro_id, "status": "INVALID_CUDAGRAPH_WARNING",
                           "warning_source": "compiled", "warnings": warns[:5]})
    with torch.no_grad():
        for _ in range(3):
            oracle_forward(inputs)
        torch.cuda.synchronize()
    g_oracle, warns = _capture_graph_checked(lambda: oracle_forward(inputs))
    if warns:
        return finish({"repro_id": repro_id, "status": "INVALID_CUDAGRAPH_WARNING",
                       "warning_source": "oracle", "warnings": warns[:5]})

    gate = optout_verdict = None
    if not _skip_numerics_gate:
        gate = _run_anchored_numerics_gate(oracle_forward, instance, compiled, inputs)
        if gate is not None and not gate["pass"]:
            verdict = numerics_optout_applies(gate, numerics_optout)
            if verdict["accept"]:
                optout_verdict = verdict
            else:
                result = {"repro_id": repro_id, "status": "NUMERICS_WORSE_THAN_COMPILED", "numerics_gate": gate}
                if numerics_optout:
                    result["numerics_optout_refused"] = verdict
                return finish(result)

    quick = _time_graph(g_oracle, warmup=5, rep=10)
    if g_compile is not None:
        quick = min(quick, _time_graph(g_compile, warmup=5, rep=10))
    if adaptive_rep:  # the reference lengthens the timing window of fast kernels; a sweep may keep it fixed
        if quick < 50:
            rep = max(rep, 500)
        elif quick < 200:
            rep = max(rep, 300)

    best_oracle = best_compile = math.inf
    with gpu_exclusive_lock(repro_id, disabled=disable_gpu_lock):
        for _ in range(max(1, int(warmup))):
            g_oracle.replay()
            if g_compile is not None:
                g_compile.replay()
        torch.cuda.synchronize()
        for _ in range(rounds):
            best_oracle = min(best_oracle, _time_graph(g_oracle, warmup=warmup, rep=rep))
            if g_compile is not None:
                best_compile = min(best_compile, _time_graph(g_compile, warmup=warmup, rep=rep))

    gave_up = device_wait_failures()
    if gave_up:
        # a bounded device-side wait ran out somewhere in what was just timed: the kernel skipped
        # work, so the time means nothing (not a status of the reference; additive)
        return finish({"repro_id": repro_id, "status": "DEVICE_WAIT", "device_waits": gave_up})
    result = {"repro_id": repro_id, "oracle_us": round(best_oracle, 2)}
    if g_compile is not None:
        ratio = best_compile / best_oracle if best_oracle > 0 else 0.0
        result.update(compile_us=round(best_compile, 2), ratio=round(ratio, 3))
        status = "GOOD" if ratio > 1.05 else ("BAD_ORACLE" if ratio < 0.95 else "AT_FLOOR")
    else:
        status = "TIMED"
    if optout_verdict is not None:
        status = "NUMERICS_OPTOUT_ACCEPTED"
        result["numerics_optout"] = {"accepted": True, "verdict": optout_verdict, "annotation": numerics_optout}
    result["status"] = status
    if gate is not None:
        result["numerics_gate"] = gate
    if region_bytes and memcpy_sol:
        sol = memcpy_sol_us(region_bytes, device=_get_device(inputs))
        result["sol_us"] = round(sol, 2)
        result["gap"] = round(best_oracle / sol, 3) if sol > 0 else None
    if region_bytes:
        gbps = region_bytes / (best_oracle * 1e-6) / 1e9
        result["region_bytes"] = int(region_bytes)
        result["oracle_gbps"] = round(gbps, 1)
        if peak_gbps:
            result["sol_frac"] = round(gbps / peak_gbps, 4)
    return finish(result)


def device_wait_failures() -> dict:
    """Bounded device-side waits of this backend's kernels that ran out since the last call ({} in
    normal operation): the error word of the shared scratch buffer and the per-family counters.
    Synchronises; call it after a timed region, never inside one."""
    from . import kernels, native
    found = {}
    try:
        lib = native.load()
    except native.NativeLibraryError:
        return found
    try:
        kernels.check_scratch_status()
    except native.KernelArgumentError as e:
        found["grid_barrier"] = str(e)[:200]
    seen = getattr(device_wait_failures, "_seen", {})
    for name in ("b200_norm_fwd_wait_timeouts", "b200_norm_bwd_wait_timeouts", "b200_batch_norm_wait_timeouts"):
        total = int(getattr(lib, name)())
        if total > seen.get(name, 0):
            found[name] = total - seen.get(name, 0)
        seen[name] = total
    device_wait_failures._seen = seen
    return found


NUMERICS_OPTOUT_MAX_REL_DIFF = 0.05
NUMERICS_OPTOUT_ABS_FLOOR = 1e-2


def numerics_optout_applies(numerics_result, optout) -> dict:
    """May a verified opt-out accept this failing gate? Only if every violation is a plausible
    precision drift: finite and within max(5 % of |ref|max, 1e-2) (``oracle_harness.py:736-804``)."""
    if not optout:
        return {"accept": False, "reason": "no verified opt-out"}
    if numerics_result is None:
        return {"accept": False, "reason": "no numerics gate result to accept"}
    offenders, failing = [], 0
    for entry in numerics_result.get("per_output", []):
        if entry.get("pass") is not False:
            continue
        failing += 1
        err = entry.get("err_oracle")
        absmax = entry.get("ref_absmax", 0.0) or 0.0
        if not isinstance(err, (int, float)):
            continue
        if not math.isfinite(err):
            offenders.append({"idx": entry.get("idx"), "err_oracle": err, "non_finite": True})
            continue
        bound = max(NUMERICS_OPTOUT_MAX_REL_DIFF * max(absmax, 1e-12), NUMERICS_OPTOUT_ABS_FLOOR)
        if err > bound:
            offenders.append({"idx": entry.get("idx"), "err_oracle": err, "plausible_bound": bound})
    if offenders:
        worst = max(offenders, key=lambda e: math.inf if e.get("non_finite") else e["err_oracle"])
        return {"accept": False, "reason": f"opt-out REFUSED: output {worst['idx']} diff "
                f"{worst['err_oracle']} is not a plausible precision drift", "worst_offender": worst}
    return {"accept": True, "n_failing": failing,
            "reason": f"verified numerics opt-out: {failing} output(s) within plausible precision-drift bound"}


def bench_oracle_all_shapes(oracle_forward, repro_dir, repro_id, **kwargs) -> list:
    repro_dir = Path(repro_dir)
    kwargs.setdefault("numerics_optout", load_numerics_optout(repro_dir))
    configs = load_shape_configs(repro_dir / "repro.py")
    if not configs:
        return [bench_oracle(oracle_forward, get_repro_instance(repro_dir), get_inputs(repro_dir),
                             repro_id, **kwargs)]
    results = []
    for label, config in configs.items():
        inputs = make_inputs_from_config(config)
        results.append(bench_oracle(oracle_forward, get_repro_instance(repro_dir), inputs,
                                    f"{repro_id}_{label}", **kwargs))
    return results


# ---------------------------------------------------------------------------------------------
# CLI: python -m better_benchmark_b200.harness <canonical_dir> [--check] [--bench]
# ---------------------------------------------------------------------------------------------
def _runner_main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="python -m better_benchmark_b200.harness",
                                 description="check / bench the oracle.py of a canonical repro directory")
    ap.add_argument("canonical_dir")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--point", default=None)
    ap.add_argument("--warmup", type=int, default=25)
    ap.add_argument("--rep", type=int, default=200)
    ap.add_argument("--no-compile", action="store_true", help="skip the torch.compile comparison arm")
    ap.add_argument("--disable-gpu-lock", action="store_true")
    args = ap.parse_args(argv)
    if not (args.check or args.bench):
        args.check = args.bench = True
    _, fn, d = _load_oracle_module(args.canonical_dir)
    repro_id = d.name
    rc = 0
    checks = {}
    if args.check or args.bench:  # --bench implies --check
        checks = check_oracle_all_shapes(fn, d, repro_id, point=args.point)
        for label, ok in checks.items():
            print(f"CHECK {repro_id}_{label}: {'PASS' if ok else 'FAIL'}")
        if not all(checks.values()):
            rc = 1
    if args.bench:
        configs = load_shape_configs(d / "repro.py")
        if args.point is not None:
            configs = {k: v for k, v in configs.items() if k == args.point or k.endswith(f"_{args.point}")}
        optout = load_numerics_optout(d)
        for label, config in configs.items():
            point_id = f"{repro_id}_{label}"
            if not checks.get(label, False):
                print(json.dumps({"repro_id": point_id, "status": "UNVERIFIED_NUMERICS"}))
                rc = 1
                continue
            result = bench_oracle(fn, get_repro_instance(d), make_inputs_from_config(config), point_id,
                                  warmup=args.warmup, rep=args.rep, numerics_optout=optout,
                                  disable_gpu_lock=args.disable_gpu_lock,
                                  compile_reference=not args.no_compile)
            if result.get("status") in _INVALID_STATUSES:
                rc = 1
    return rc


if __name__ == "__main__":
    sys.exit(_runner_main())
