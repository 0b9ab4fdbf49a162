"""shapes.json decoding, seeded input generation and the byte model (CPU)."""
import json

import pytest
import torch

from better_benchmark_b200 import byte_model, inputs


def test_compact_entries_decode_to_specs():
    s = inputs.spec_from_compact([[128, 128, 28, 28], "bf16", {"st": [100352, 1, 3584, 128]}])
    assert s["kind"] == "tensor" and s["dtype"] == "bfloat16" and s["stride"] == [100352, 1, 3584, 128]
    assert s["device"] == "cuda" and s["storage_offset"] == 0
    s = inputs.spec_from_compact([[4096], "i64", {"gen": ["index", 0, 1000]}])
    assert s["gen"] == {"kind": "index", "low": 0, "high": 1000}
    assert inputs.spec_from_compact(["S", [128, 512, 1, 1]]) == {"kind": "shape", "name": None, "dims": [128, 512, 1, 1]}
    assert inputs.spec_from_compact(["sc", 0.5])["value"] == 0.5
    assert inputs.spec_from_compact(["sym", 128])["kind"] == "symint"
    assert inputs.spec_from_compact([[2, 3], "f32"])["stride"] == [3, 1]
    with pytest.raises(NotImplementedError):
        inputs.spec_from_compact([[64, "s16"], "f32"])


def test_labels_and_configs_from_shapes_json(tmp_path):
    (tmp_path / "shapes.json").write_text(json.dumps({"points": [
        {"shape_hash": "23d9c217", "models": {"hf/train/BlenderbotForCausalLM": {"occurrences": 1}},
         "inputs": [[[2, 3, 8], "f32"], [[8], "f32"], ["S", [6, 8]]]},
        {"shape_hash": "3d83c7c9", "models": {}, "inputs": []}]}))
    cfg = inputs.load_shape_configs(tmp_path / "repro.py")
    assert list(cfg) == ["BlenderbotForCausalLM_23d9c217", "3d83c7c9"]
    assert cfg["3d83c7c9"] == {"inputs": []}
    assert inputs.load_shape_configs(tmp_path / "nowhere" / "repro.py") == {}


def test_generation_is_seeded_and_respects_strides_and_bounds():
    cfg = {"inputs": [inputs.spec_from_compact(e) for e in [
        [[4, 6, 5, 5], "bf16", {"st": [150, 1, 30, 6]}], [[7], "i64", {"gen": ["index", 3, 9]}],
        [[5], "b8"], ["S", [4, -1]], ["sc", 2.5], ["sym", 12], [[3, 4], "f32"],
        [[16], "i32", {"gen": ["const", 7]}], [[2, 8], "i64", {"gen": ["perm", 8]}]]]}
    torch.manual_seed(1)
    a = inputs.make_inputs_from_config(cfg, "cpu")
    torch.manual_seed(1)
    b = inputs.make_inputs_from_config(cfg, "cpu")
    assert a[0].shape == (4, 6, 5, 5) and a[0].stride() == (150, 1, 30, 6) and a[0].dtype == torch.bfloat16
    assert a[0].is_contiguous(memory_format=torch.channels_last)
    assert a[1].min() >= 3 and a[1].max() < 9 and a[2].dtype == torch.bool
    assert a[3] == [4, -1] and a[4] == 2.5 and a[5] == 12
    assert torch.equal(a[7], torch.full((16,), 7, dtype=torch.int32))
    assert all(sorted(row.tolist()) == list(range(8)) for row in a[8])
    for x, y in zip(a, b):
        assert torch.equal(x, y) if isinstance(x, torch.Tensor) else x == y


def test_contiguous_randn_matches_torch_randn_stream():
    torch.manual_seed(5)
    got = inputs.make_inputs_from_config({"inputs": [inputs.spec_from_compact([[6, 10], "f32"])]}, "cpu")[0]
    torch.manual_seed(5)
    assert torch.equal(got, torch.randn(6, 10))


class _Region(torch.nn.Module):
    def __init__(self, fn):
        super().__init__()
        self.fn = fn

    def forward(self, *a):
        return self.fn(*a)


def test_byte_model_dense_views_sparse_and_aliases():
    f = byte_model.count_bytes_effective
    x = torch.randn(64, 32)
    assert f(_Region(lambda t: t * 2 + 1), [x]) == 2 * x.numel() * 4           # intermediates are free
    assert f(_Region(lambda t: t[:16] * 2), [x]) == 2 * 16 * 32 * 4            # a slice charges the slice
    assert f(_Region(lambda t: (t * 2).sum(-1)), [x]) == x.numel() * 4 + 64 * 4
    table, idx = torch.randn(1000, 16), torch.randint(0, 1000, (8,))
    assert f(_Region(lambda tb, i: torch.ops.aten.embedding.default(tb, i)), [table, idx]) == 8 * 16 * 4 * 2 + idx.numel() * 8
    # an input returned next to a computed output is not charged as a write ...
    assert f(_Region(lambda t: (t * 2, t)), [x]) == 2 * x.numel() * 4
    # ... but a region with no op at all never registers its input, and the tensor counts as an
    # output (the reference's counter behaves the same: 8192 for this case)
    assert f(_Region(lambda t: t), [x]) == x.numel() * 4
    out = f(_Region(lambda t: (lambda y: (y, y.view(-1)))(t + 1)), [x])
    assert out == 2 * x.numel() * 4                                            # aliases of one output count once
    assert byte_model.count_bytes_naive([x, 3, [x]], (x + 1, x + 1)) == 2 * x.numel() * 4 + 2 * x.numel() * 4


def test_byte_model_index_put_and_scatter_charge_the_update():
    f = byte_model.count_bytes_effective
    base, idx, vals = torch.zeros(1000, 8), torch.randint(0, 1000, (10,)), torch.randn(10, 8)
    got = f(_Region(lambda b, i, v: torch.ops.aten.index_put.default(b, [i], v)), [base, idx, vals])
    assert got == base.numel() * 4 + idx.numel() * 8 + vals.numel() * 4 + vals.numel() * 4


@pytest.mark.parametrize("name,kwargs,expected", [
    ("c1_row_mean", dict(rows=64, cols=128), 64 * 128 * 4 + 64 * 4),
    ("c2_layer_norm_fwd", dict(rows=32, hidden=768), 2 * 32 * 768 * 2 + 2 * 768 * 2 + 2 * 32 * 4),
    ("c3_masked_softmax", dict(batch=2, heads=3, q=8, k=64), 2 * 2 * 3 * 8 * 64 * 2 + 2 * 64 * 2),
    ("c4_batch_norm_relu", dict(n=2, c=8, h=4, w=4), 2 * 2 * 8 * 16 * 2 + 4 * 8 * 4 + 4 * 8 * 4),
    ("c5_rms_norm_bwd", dict(b=1, s=8, h=2, d=16), 3 * 8 * 32 * 2 + 32 * 2 + 8 * 4 + 32 * 4),
])
def test_configuration_byte_formula_matches_the_model(name, kwargs, expected):
    """The closed forms behind WORKLOADS[...].algorithmic_bytes, checked at small sizes; the same
    forms at full size give 134250496 / 100928512 / 201342976 / 205522944 / 402743296."""
    from better_benchmark_b200.harness import load_repro_module
    from better_benchmark_b200.workloads import WORKLOADS
    from pathlib import Path
    wl = WORKLOADS[name]
    mod = load_repro_module(Path(__file__).resolve().parents[1] / "oracle" / "canonical" / wl.canonical_id)
    assert byte_model.count_bytes_effective(mod.Repro(), wl.make_inputs("cpu", 1, **kwargs)) == expected


def test_full_size_byte_counts_of_the_five_configurations():
    from better_benchmark_b200.workloads import WORKLOADS
    full = {
        "c1_row_mean": 8192 * 4096 * 4 + 8192 * 4,
        "c2_layer_norm_fwd": 2 * 32768 * 768 * 2 + 2 * 768 * 2 + 2 * 32768 * 4,
        "c3_masked_softmax": 2 * 16 * 12 * 512 * 512 * 2 + 16 * 512 * 2,
        "c4_batch_norm_relu": 2 * 256 * 64 * 56 * 56 * 2 + 8 * 64 * 4,
        "c5_rms_norm_bwd": 3 * 16384 * 4096 * 2 + 4096 * 2 + 16384 * 4 + 4096 * 4,
    }
    for name, expected in full.items():
        assert WORKLOADS[name].algorithmic_bytes == expected
