"""In-tree native builds.

Two shared libraries live next to the package (``ronn_b200/_lib``):

* ``libronn_host.so``  - host C++17 runtime (ONNX wire codec, graph algorithms,
  memory pools, block manager + continuous-batching scheduler, CPU SIMD and
  BitNet kernels); built with g++.
* ``libronn_sm100.so`` - every CUDA kernel, compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); built with nvcc.  The kernels
  are plain ``extern "C"`` launchers taking raw device pointers and a stream,
  so the library does not link against libtorch and compiles in seconds.

Both are rebuilt when a source file is newer than the library.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "_lib"
OBJDIR = LIBDIR / "obj"

HOST_LIB = LIBDIR / "libronn_host.so"
CUDA_LIB = LIBDIR / "libronn_sm100.so"

HOST_SOURCES = ["core/onnx_pb.cc", "core/graph.cc", "core/host_pool.cc", "serving/scheduler.cc",
                "cpu/simd_kernels.cc", "cpu/bitnet_cpu.cc"]

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


class BuildError(RuntimeError):
    pass


def _run(cmd, what):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(map(str, cmd))}\n{proc.stdout}\n{proc.stderr}")
    return proc.stdout + proc.stderr


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def cuda_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


def cuda_headers():
    return sorted(list((CSRC / "kernels").glob("*.cuh")) + list((CSRC / "kernels").glob("*.h")) +
                  list((CSRC / "comm").glob("*.cuh")) + list((CSRC / "comm").glob("*.h")))


def find_nvcc():
    for cand in (os.environ.get("RONN_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def build_host(force: bool = False, verbose: bool = False) -> Path:
    srcs = [CSRC / s for s in HOST_SOURCES]
    if not force and not _newer(HOST_LIB, srcs):
        return HOST_LIB
    LIBDIR.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    tmp = HOST_LIB.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wno-unused-function", "-Wno-stringop-overflow", "-pthread",
           "-o", str(tmp)] + [str(s) for s in srcs]
    out = _run(cmd, "host library build")
    os.replace(tmp, HOST_LIB)
    if verbose:
        print(out)
    return HOST_LIB


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    srcs = cuda_sources()
    hdrs = cuda_headers()
    if not srcs:
        raise BuildError("no CUDA sources found")
    if not force and not _newer(CUDA_LIB, list(srcs) + list(hdrs)):
        return CUDA_LIB
    nvcc = find_nvcc()
    if nvcc is None:
        raise BuildError("nvcc not found; cannot build the sm_100a kernel library")
    OBJDIR.mkdir(parents=True, exist_ok=True)
    flags = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
             "-I", str(CSRC / "kernels"), "-I", str(CSRC / "comm")] + NVCC_ARCH
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    hdr_sig = hashlib.sha1(b"".join(h.read_bytes() for h in hdrs)).hexdigest()[:12]

    def compile_one(src: Path):
        sig = hashlib.sha1(src.read_bytes() + hdr_sig.encode() + " ".join(flags).encode()).hexdigest()[:16]
        obj = OBJDIR / f"{src.stem}.{sig}.o"
        if obj.exists() and not force:
            return obj, ""
        for old in OBJDIR.glob(f"{src.stem}.*.o"):
            old.unlink()
        out = _run([nvcc, "-c", str(src), "-o", str(obj)] + flags, f"nvcc {src.name}")
        return obj, out

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = [str(o) for o, _ in results]
    log = "".join(o for _, o in results)
    tmp = CUDA_LIB.with_suffix(f".tmp{os.getpid()}.so")
    _run([nvcc, "-shared", "-o", str(tmp)] + objs + NVCC_ARCH + ["-Xcompiler", "-fPIC"], "nvcc link")
    os.replace(tmp, CUDA_LIB)
    if verbose or ptxas_info:
        print(log)
    return CUDA_LIB


def build_host_selftest(sanitize: str = "address,undefined") -> Path:
    """The host runtime (scheduler, block manager, pooled allocator, graph algorithms, model codec) linked with
    ``csrc/core/host_selftest.cc`` into an executable built with ``-fsanitize=<sanitize>``; running it on a CPU box
    checks the C++ code for out-of-bounds accesses, leaks and undefined behaviour."""
    srcs = [CSRC / s for s in HOST_SOURCES] + [CSRC / "core" / "host_selftest.cc"]
    exe = LIBDIR / ("host_selftest_" + sanitize.replace(",", "_"))
    if exe.exists() and not _newer(exe, srcs):
        return exe
    LIBDIR.mkdir(parents=True, exist_ok=True)
    # not every g++ of a box ships the sanitizer runtimes: try the configured compiler, then the system ones
    tried, last = [], None
    for cxx in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++"):
        if not cxx or cxx in tried:
            continue
        tried.append(cxx)
        cmd = [cxx, "-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", f"-fsanitize={sanitize}", "-Wall",
               "-Wno-unused-function", "-Wno-stringop-overflow", "-pthread", "-o", str(exe)] + [str(s) for s in srcs]
        try:
            _run(cmd, "sanitized host self-test build")
            return exe
        except BuildError as e:
            last = e
    raise BuildError(f"no compiler with the '{sanitize}' sanitizer runtime found (tried {tried}): {last}")


def build_all(force: bool = False, verbose: bool = False):
    return build_host(force, verbose), build_cuda(force, verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    info = "--ptxas-info" in sys.argv
    build_host(force, True)
    build_cuda(force, True, ptxas_info=info)
    print("built", HOST_LIB, CUDA_LIB)
