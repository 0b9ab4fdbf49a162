"""Launch one benchmark configuration (or one of the per-family cases) a few times, each time from a flushed L2: the small, bounded
program to put under a profiler (``ncu -k regex:<kernel> -c 1..3 python -m
better_benchmark_b200.profile_case <workload>``). A few hundred MB on the device, a handful of
launches, ends by itself.

    python -m better_benchmark_b200.profile_case c2_layer_norm_fwd [--launches 3] [--no-flush]
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    import torch
    from .family_cases import FAMILY_CASES
    from .workloads import WORKLOADS

    cases = {**WORKLOADS, **FAMILY_CASES}

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("workload", choices=sorted(cases))
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true", help="do not overwrite L2 between launches")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("profile_case needs a CUDA device")
    wl = cases[args.workload]
    inputs = wl.make_inputs("cuda", 1)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(max(1, args.launches)):
        if flush is not None:
            flush.zero_()
        wl.oracle_forward(inputs)
    torch.cuda.synchronize()
    print(f"{wl.name}: {args.launches} launches, {wl.algorithmic_bytes} algorithmic bytes each")
    return 0


if __name__ == "__main__":
    sys.exit(main())
