"""Every shipped canonical directory has an oracle.py that loads through the harness mirror and
registers a B200 entry; the five synthetic configurations also bind their shape point."""
from pathlib import Path

import pytest

CANONICAL = Path(__file__).resolve().parents[1] / "better-benchmark_b200" / "canonical"
DIRS = sorted(p.name for p in CANONICAL.iterdir() if (p / "oracle.py").is_file())


def test_the_expected_directories_are_shipped():
    assert len(DIRS) == 48
    assert sum("b200c" in d for d in DIRS) == 5
    for needed in ("var_mean_f8ec553e339e", "sum_sum_183b124c731f", "pointwise_021e90d9c17d", "mean_c9e1a8113328",
                   "mean_014afd4984e6", "var_mean_01fbd6c1b27f", "pointwise_4b076ed1ff41",
                   "pointwise_7bd204513fbb", "pointwise_6e7efb08a440"):
        assert needed in DIRS


@pytest.mark.parametrize("name", DIRS)
def test_oracle_stub_loads_and_registers_for_b200(name):
    from better_benchmark_b200 import harness
    harness.reset_oracle_registry()
    mod, fn, d = harness._load_oracle_module(CANONICAL / name)
    assert callable(fn) and d.name == name
    reg = harness.get_module_registry(fn.__module__)
    entries = reg.entries if hasattr(reg, "entries") else reg._entries
    assert len(entries) >= 1
    assert all((e.get("hardware") if isinstance(e, dict) else getattr(e, "hardware", None)) == "B200" for e in entries)
    assert (mod.__doc__ or "").strip(), "the stub says what region it covers"
