"""ctypes bindings for the two in-tree native libraries.

``host()`` returns ``libronn_host.so`` (built on demand with g++); ``cuda()``
returns ``libronn_sm100.so`` (the sm_100a kernel library).  On a machine with a
GPU the kernel library is mandatory: ops that need it raise instead of falling
back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
import threading

from .utils import build as _build

_lock = threading.Lock()
_host = None
_cuda = None

c_i32p = C.POINTER(C.c_int32)
c_i64p = C.POINTER(C.c_int64)
c_u64p = C.POINTER(C.c_uint64)
c_u8p = C.POINTER(C.c_uint8)
c_f32p = C.POINTER(C.c_float)


def _sig(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def host():
    global _host
    if _host is not None:
        return _host
    with _lock:
        if _host is not None:
            return _host
        path = _build.build_host()
        lib = C.CDLL(str(path))
        V, I32, I64, U64, F32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float
        S = C.c_char_p
        # ---- onnx decode
        _sig(lib, "ronn_onnx_parse", V, [V, U64])
        _sig(lib, "ronn_onnx_error", S, [V])
        _sig(lib, "ronn_onnx_json", V, [V, c_u64p])
        _sig(lib, "ronn_onnx_num_blobs", U64, [V])
        _sig(lib, "ronn_onnx_blob", V, [V, U64, c_u64p])
        _sig(lib, "ronn_onnx_free", None, [V])
        _sig(lib, "ronn_onnx_elem_size", C.c_int, [I32])
        # ---- onnx encode
        _sig(lib, "ronn_onnxw_begin", V, [I64, S, S, S])
        _sig(lib, "ronn_onnxw_opset", None, [V, S, I64])
        _sig(lib, "ronn_onnxw_metadata", None, [V, S, S])
        _sig(lib, "ronn_onnxw_node", None, [V, S, S, S, C.POINTER(S), C.c_int, C.POINTER(S), C.c_int])
        _sig(lib, "ronn_onnxw_attr_i", None, [V, S, I64])
        _sig(lib, "ronn_onnxw_attr_f", None, [V, S, F32])
        _sig(lib, "ronn_onnxw_attr_s", None, [V, S, S, U64])
        _sig(lib, "ronn_onnxw_attr_ints", None, [V, S, c_i64p, C.c_int])
        _sig(lib, "ronn_onnxw_attr_floats", None, [V, S, c_f32p, C.c_int])
        _sig(lib, "ronn_onnxw_attr_strings", None, [V, S, C.POINTER(S), C.c_int])
        _sig(lib, "ronn_onnxw_attr_tensor", None, [V, S, I32, c_i64p, C.c_int, V, U64])
        _sig(lib, "ronn_onnxw_initializer", None, [V, S, I32, c_i64p, C.c_int, V, U64])
        _sig(lib, "ronn_onnxw_value", None, [V, C.c_int, S, I32, C.c_int, c_i64p, C.POINTER(S)])
        _sig(lib, "ronn_onnxw_finish", V, [V, c_u64p])
        _sig(lib, "ronn_onnxw_free", None, [V])
        # ---- graph
        _sig(lib, "ronn_graph_new", V, [])
        _sig(lib, "ronn_graph_free", None, [V])
        _sig(lib, "ronn_graph_add_node", I32, [V, c_i32p, I32, c_i32p, I32])
        _sig(lib, "ronn_graph_toposort", I32, [V, c_i32p])
        _sig(lib, "ronn_graph_validate", I32, [V, c_i32p, I32, c_i32p, I32, c_i32p])
        _sig(lib, "ronn_graph_live", None, [V, c_i32p, I32, c_u8p])
        _sig(lib, "ronn_graph_depth", I32, [V])
        # ---- pools
        _sig(lib, "ronn_pool_new", V, [U64, U64, U64, U64, U64])
        _sig(lib, "ronn_pool_clear", None, [V])
        _sig(lib, "ronn_pool_free", None, [V])
        _sig(lib, "ronn_pool_alloc", V, [V, U64])
        _sig(lib, "ronn_pool_release", I32, [V, V])
        _sig(lib, "ronn_pool_stats", None, [V, c_u64p])
        _sig(lib, "ronn_pool_bucket_size", U64, [V, U64])
        # ---- scheduler
        _sig(lib, "ronn_sched_new", V, [I32] * 8)
        _sig(lib, "ronn_sched_free", None, [V])
        _sig(lib, "ronn_sched_add", I32, [V, I64, c_i32p, I32, I32, I32])
        _sig(lib, "ronn_sched_cancel", I32, [V, I64])
        _sig(lib, "ronn_sched_schedule", I32, [V])
        _sig(lib, "ronn_sched_plan_size", I32, [V])
        _sig(lib, "ronn_sched_plan_tokens", I32, [V])
        _sig(lib, "ronn_sched_fill", I32, [V, V, V, V, V, V, V, V, V, V, I32])
        _sig(lib, "ronn_sched_commit", I32, [V, V, I32, V])
        _sig(lib, "ronn_sched_abort_step", None, [V])
        for name in ("state", "num_tokens", "prompt_len", "preemptions", "num_computed"):
            _sig(lib, f"ronn_sched_{name}", I32, [V, I64])
        _sig(lib, "ronn_sched_get_tokens", I32, [V, I64, c_i32p, I32])
        _sig(lib, "ronn_sched_get_blocks", I32, [V, I64, c_i32p, I32])
        _sig(lib, "ronn_sched_get_cpu_blocks", I32, [V, I64, c_i32p, I32])
        _sig(lib, "ronn_sched_forget", None, [V, I64])
        for name in ("num_waiting", "num_running", "num_free_blocks"):
            _sig(lib, f"ronn_sched_{name}", I32, [V])
        _sig(lib, "ronn_sched_block_ref", I32, [V, I32])
        _sig(lib, "ronn_sched_stats", None, [V, c_i64p])
        _sig(lib, "ronn_sched_set_swap", I32, [V, I32, I32, I32])
        _sig(lib, "ronn_sched_swap_counts", None, [V, c_i32p])
        _sig(lib, "ronn_sched_get_swaps", None, [V, c_i32p, c_i32p, c_i32p, c_i32p])
        _sig(lib, "ronn_sched_swap_stats", None, [V, c_i64p])
        # ---- cpu kernels
        _sig(lib, "ronn_cpu_simd_level", I32, [])
        _sig(lib, "ronn_cpu_force_level", None, [I32])
        _sig(lib, "ronn_cpu_dot_f32", F32, [V, V, I64])
        _sig(lib, "ronn_cpu_binary_f32", None, [V, V, V, I64, I32, I32])
        _sig(lib, "ronn_cpu_relu_f32", None, [V, V, I64])
        _sig(lib, "ronn_cpu_gemm_f32", None, [V, V, V, V, I64, I64, I64, I32])
        _sig(lib, "ronn_cpu_softmax_f32", None, [V, V, I64, I64])
        _sig(lib, "ronn_cpu_run_chain", None, [V, I64, I64, I32, V, V, V, V, V, V, V, V])
        # ---- bitnet cpu
        _sig(lib, "ronn_bitnet_quantize_binary", F32, [V, I64, V])
        _sig(lib, "ronn_bitnet_dequantize_binary", None, [V, I64, F32, V])
        _sig(lib, "ronn_bitnet_binary_matmul", None, [V, V, V, I64, I64, I64, F32, F32])
        _sig(lib, "ronn_bitnet_quantize_ternary", F32, [V, I64, V, c_f32p])
        _sig(lib, "ronn_bitnet_quantize_absmean", F32, [V, I64, V])
        _sig(lib, "ronn_bitnet_pack_ternary_rows", None, [V, I64, I64, V])
        _sig(lib, "ronn_bitnet_unpack_ternary", None, [V, I64, V])
        _sig(lib, "ronn_bitnet_dequantize_ternary", None, [V, I64, F32, V])
        _sig(lib, "ronn_bitnet_ternary_matmul", None, [V, V, V, I64, I64, I64, F32, F32])
        _sig(lib, "ronn_bitnet_quantize_act_int8", None, [V, I64, I64, V, V])
        _sig(lib, "ronn_bitnet_ternary_int8_matmul", None, [V, V, V, F32, V, V, I64, I64, I64])
        _host = lib
        return lib


_NOT_LAUNCHERS = {"ronn_set_pdl", "ronn_set_rowwise_status", "ronn_no_alloc_scratch_floats", "ronn_no_alloc_strerror",
                  "ronn_gemm_fuse_state_ints", "ronn_gemm_fuse_flag_ints", "ronn_bitlinear_workspace_bytes"}


class _Counted:
    """A launcher of the kernel library that bumps its library's launch counter on every call; attribute access
    (``restype``, ``argtypes``) goes to the ctypes function itself."""
    __slots__ = ("_fn", "_owner")

    def __init__(self, fn, owner):
        object.__setattr__(self, "_fn", fn)
        object.__setattr__(self, "_owner", owner)

    def __call__(self, *args):
        self._owner.launches += 1
        return self._fn(*args)

    def __getattr__(self, k):
        return getattr(self._fn, k)

    def __setattr__(self, k, v):
        setattr(self._fn, k, v)


class _KernelLib:
    """The loaded kernel library plus ``launches``: how many of its kernel launchers have been called in this process
    (a launcher enqueues one kernel, a few enqueue two).  Replays of a captured CUDA graph call no launcher; whoever
    replays a graph adds the count it recorded during capture (see ``LLMEngine.kernel_launches``)."""

    def __init__(self, lib):
        self.__dict__["_lib"] = lib
        self.__dict__["launches"] = 0

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name.startswith("ronn_") and name not in _NOT_LAUNCHERS:
            fn = _Counted(fn, self)
        self.__dict__[name] = fn
        return fn


def cuda_available() -> bool:
    import torch
    return torch.cuda.is_available()


def cuda():
    """The sm_100a kernel library.  Raises when it cannot be built or loaded."""
    global _cuda
    if _cuda is not None:
        return _cuda
    with _lock:
        if _cuda is not None:
            return _cuda
        path = _build.CUDA_LIB
        if not path.exists() or _build.find_nvcc() is not None:
            path = _build.build_cuda()
        raw = C.CDLL(str(path))
        from .ops import _signatures
        _signatures.declare(raw)
        _cuda = _KernelLib(raw)
        return _cuda
