"""Registration and dispatch of oracle implementations (CPU, meta tensors).

Mirrors the cases of the reference's dispatch tests (tests/test_oracle_dispatch.py:61-222,
tests/test_canonical_invariants.py:1406-1449): every match tier, exact-only matching, kwargs
pass-through, hash-keyed registration against a sibling shapes.json.
"""
import json
import sys
import types

import pytest
import torch

from better_benchmark_b200 import harness


def meta(*shape):
    return torch.empty(shape, device="meta")


@pytest.fixture(autouse=True)
def _clean():
    harness.reset_oracle_registry()
    harness.get_gpu_kind._cached = "B200"
    yield
    harness.reset_oracle_registry()


def fake_fn(module, name="oracle_forward"):
    def fn(inputs, **kw):
        return (name, kw)
    fn.__module__ = module
    fn.__name__ = name
    return fn


def test_unregistered_function_passes_through():
    fn = fake_fn("plain_mod")
    assert harness.resolve_oracle(fn, [meta(4, 4)]) == (fn, None)


def test_hardware_and_shape_tier_wins_and_binds_kwargs():
    fn = fake_fn("m1")
    harness.oracle_impl(hardware="H100", shapes="(T([4, 8], bf16),)", BLOCK=1)(fn)
    harness.oracle_impl(hardware="B200", shapes="(T([4, 8], bf16),)", BLOCK=2)(fn)
    selected, info = harness.resolve_oracle(fn, [meta(4, 8)])
    assert info["matched"] == "hardware+shape" and info["fallback"] is False
    assert selected([meta(4, 8)]) == ("oracle_forward", {"BLOCK": 2})


def test_shape_tier_on_other_hardware_is_a_fallback():
    fn = fake_fn("m2")
    harness.oracle_impl(hardware="H100", shapes=((4, 8),))(fn)
    _, info = harness.resolve_oracle(fn, [meta(4, 8)])
    assert info["matched"] == "shape" and info["fallback"] is True and info["tuned_hardware"] == "H100"


def test_shape_general_tiers():
    fn = fake_fn("m3")
    harness.oracle_impl(hardware=None)(fn)
    harness.oracle_impl(hardware="B200")(fn)
    _, info = harness.resolve_oracle(fn, [meta(3, 3)])
    assert info["matched"] == "hardware"
    harness.get_gpu_kind._cached = "A100"
    _, info = harness.resolve_oracle(fn, [meta(3, 3)])
    assert info["matched"] == "any"


def test_matching_is_exact_only():
    fn = fake_fn("m4")
    harness.oracle_impl(hardware="B200", shapes=((4, 8), (8,)))(fn)
    with pytest.raises(harness.OracleDispatchError):
        harness.resolve_oracle(fn, [meta(4, 9), meta(8)])
    with pytest.raises(harness.OracleDispatchError):
        harness.resolve_oracle(fn, [meta(4, 8)])          # full signature: every tensor must match
    harness.resolve_oracle(fn, [meta(4, 8), [4, 8], meta(8), 3])  # non-tensors are ignored


def test_point_and_shapes_are_mutually_exclusive():
    with pytest.raises(ValueError):
        harness.oracle_impl(point="abcd1234", shapes="(T([1], f32),)")


def test_signature_string_parsing():
    sig = "(T([512, 256, 13, 13], f32), T([512, 128, 27, 27], b8, stride=(1, 2, 3, 4)), S([131072, 169]))"
    assert harness.parse_shapes_signature(sig) == ((512, 256, 13, 13), (512, 128, 27, 27))
    assert harness.parse_shapes_signature("(T([8192], bf16))") == ((8192,),)
    assert harness.parse_shapes_signature(None) is None


def _write_oracle_dir(tmp_path, point):
    d = tmp_path / "repros" / "canonical" / "mean_0123456789ab"
    d.mkdir(parents=True)
    (d / "shapes.json").write_text(json.dumps({"points": [
        {"shape_hash": "deadbeef", "models": {"x/y/Model": {"occurrences": 1}},
         "inputs": [[[4, 8], "f32"], ["S", [32]]]}]}))
    (d / "oracle.py").write_text(
        "from better_benchmark_b200.harness import oracle_impl\n"
        f"@oracle_impl(hardware='B200', point='{point}', scale=3)\n"
        "def oracle_forward(inputs, *, scale):\n    return inputs[0] * scale\n")
    return d


def test_hash_keyed_registration_resolves_shapes_from_sibling_json(tmp_path):
    d = _write_oracle_dir(tmp_path, "deadbeef")
    _, fn, _ = harness._load_oracle_module(d)
    x = torch.ones(4, 8)
    selected, info = harness.resolve_oracle(fn, [x, [32]])
    assert info["registered_shape"] == ((4, 8),) and torch.equal(selected([x, [32]]), x * 3)


def test_unknown_hash_fails_at_import(tmp_path):
    d = _write_oracle_dir(tmp_path, "00000000")
    with pytest.raises(harness.OracleDispatchError):
        harness._load_oracle_module(d)


def test_shipped_oracle_files_register_their_points(tmp_path):
    from conftest import assemble_canonical_dir
    from better_benchmark_b200.workloads import WORKLOADS
    for wl in WORKLOADS.values():
        harness.reset_oracle_registry()
        d = assemble_canonical_dir(wl.canonical_id, tmp_path)
        mod, fn, _ = harness._load_oracle_module(d)
        reg = harness.get_module_registry(fn.__module__)
        entries = reg.list_entries()
        assert len(entries) == 1 and entries[0]["hardware"] == "B200"
        assert reg._entries[0]["point"] == wl.shape_hash
        configs = harness.load_shape_configs(d / "repro.py")
        assert list(configs) == [f"{wl.name}_{wl.shape_hash}"]
