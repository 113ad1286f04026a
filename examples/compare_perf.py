"""Throughput of the hand-written GEMM against the library GEMM (counterpart of the reference's examples/compare_perf,
which prints GFLOPS of 64/256/512 matmuls)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))      # run from a source checkout

import time

import torch

if torch.cuda.is_available():
    from ronn_b200.ops.microbench import bench_gemm
    for n in (512, 2048, 8192):
        print(bench_gemm(n, n, n, iters=5))
else:
    from ronn_b200 import _native
    lib = _native.host()
    for n in (64, 256, 512):
        a, b, c = torch.randn(n, n), torch.randn(n, n), torch.empty(n, n)
        t = time.perf_counter()
        for _ in range(20):
            lib.ronn_cpu_gemm_f32(a.data_ptr(), b.data_ptr(), None, c.data_ptr(), n, n, n, 0)
        dt = (time.perf_counter() - t) / 20
        print(n, f"{2 * n ** 3 / dt / 1e9:.1f} GFLOP/s (native AVX kernel, 1 thread)")
