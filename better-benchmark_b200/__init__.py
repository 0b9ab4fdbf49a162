"""B200-native oracle backend for the memory-bound fused-kernel families of better-benchmark.

Layout:
  csrc/        hand-written sm_100a CUDA kernels behind a C ABI (include/b200_oracles.h)
  native.py    ctypes loader for the built shared library (no CPU fallback: loading fails loudly)
  kernels.py   tensor-level wrappers: validate layout, allocate outputs with eager strides,
               launch on the current CUDA stream
  families/    ``oracle_forward(inputs)`` bodies for each repro family (the drop-in oracles)
  harness.py   the reference's oracle contract: oracle_impl / resolve_oracle / check_oracle /
               bench_oracle, with the fp64-anchored numerics gate and CUDA-graph timing
  inputs.py    shapes.json decoding and seeded input generation
  byte_model.py minimum-bytes (speed-of-light) accounting for a fused region
  gpu_lock.py  per-GPU advisory file lock that serialises timing windows
  sweep.py     shards (canonical dir, shape point) tasks over the GPUs of one box
"""
__version__ = "0.1.0"
