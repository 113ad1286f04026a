"""The C++ host runtime (scheduler / block manager, pooled allocator, graph algorithms) under AddressSanitizer and
UndefinedBehaviorSanitizer: a self-test executable drives the C entry points with a deterministic random workload."""
import subprocess

import pytest


def test_host_runtime_is_clean_under_asan_and_ubsan():
    from ronn_b200.utils import build
    try:
        exe = build.build_host_selftest("address,undefined")
    except build.BuildError as e:
        if "sanitizer runtime" in str(e):
            pytest.skip("no compiler with the sanitizer runtimes on this box")
        raise
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-500:], p.stderr[-3000:])
    assert "host_selftest: ok" in p.stdout
    assert "runtime error" not in p.stderr          # UBSan reports without aborting
