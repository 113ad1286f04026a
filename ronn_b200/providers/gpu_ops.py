"""Node -> kernel resolution of the GPU provider."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..graph.ir import GraphNode, ModelGraph
from ..onnx.registry import default_registry

_HALF = (torch.bfloat16, torch.float16)
_GEMM_OPS = ("MatMul", "Gemm", "FusedGemm")
# operators whose trailing inputs are shape/axis parameters read on the host
_SHAPE_PARAM_OPS = {"Reshape", "Expand", "Slice", "Squeeze", "Unsqueeze", "Tile", "Pad", "Split", "ConstantOfShape",
                    "Range", "ReduceMean", "ReduceSum", "ReduceMax", "ReduceMin", "ReduceProd", "ReduceL2", "Clip"}
_UNARY_KERNELS = {"Relu": "relu", "Gelu": "gelu", "FastGelu": "fast_gelu", "Sigmoid": "sigmoid", "Swish": "silu",
                  "SiLU": "silu", "Tanh": "tanh"}
_BINARY_KERNELS = {"Add": "add", "Mul": "mul", "Sub": "sub", "SwiGLU": "swiglu"}


def _aligned(t: torch.Tensor) -> bool:
    return t.is_contiguous() and t.data_ptr() % 16 == 0


class GpuOpTable:
    def __init__(self, provider, graph: ModelGraph, compute_dtype: Optional[torch.dtype]):
        from .. import ops as K
        self.K = K
        self.provider = provider
        self.device = provider.device
        self.cdt = compute_dtype
        self.reg = default_registry()
        self.graph = graph
        self.w_nk: Dict[str, bool] = {}
        self._pinned: list = []
        self.custom = provider.config.enable_custom_kernels

    def to_device(self, t: torch.Tensor) -> torch.Tensor:
        """Host tensors produced by shape arithmetic (Shape/Range/...) reach the device through pinned memory, which
        is also legal inside CUDA-graph capture; the pinned staging buffer is kept alive with the session."""
        if t.device.type == "cuda":
            return t
        p = t.contiguous().pin_memory()
        self._pinned.append(p)
        if len(self._pinned) > 4096:
            del self._pinned[:2048]
        return p.to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ constants
    def place_const(self, name: str, t: torch.Tensor, users: List[GraphNode]) -> torch.Tensor:
        if not t.is_floating_point() and t.numel() <= 64:
            return t                                   # shape / axis parameters stay on the host
        if t.is_floating_point() and self.cdt is not None:
            t = t.to(self.cdt)
        gemm_weight = (t.dim() == 2 and t.dtype in _HALF and users
                       and all(u.op_type in _GEMM_OPS and len(u.inputs) > 1 and u.inputs[1] == name
                               and u.inputs[0] != name and not int(u.attr("transA", 0)) for u in users))
        if gemm_weight and self.custom:
            trans = {bool(int(u.attr("transB", 0))) for u in users}
            if len(trans) == 1:
                already_nk = trans.pop()
                w = t if already_nk else t.t()
                if w.shape[1] % 8 == 0:
                    self.w_nk[name] = True
                    return w.contiguous().to(self.device)
        return t.to(self.device)

    # ------------------------------------------------------------------ resolution
    def resolve(self, node: GraphNode, graph: ModelGraph):
        op = node.op_type
        fallback = self._fallback(node)
        if not self.custom:
            return fallback
        if op in _GEMM_OPS and len(node.inputs) > 1 and self.w_nk.get(node.inputs[1]):
            return self._gemm(node, fallback)
        if op == "LayerNormalization" and int(node.attr("axis", -1)) == -1:
            return self._layernorm(node, fallback)
        if op == "RMSNorm":
            return self._rmsnorm(node, fallback)
        if op == "Softmax":
            return self._softmax(node, fallback)
        if op in _UNARY_KERNELS and (op != "Gelu" or node.attr("approximate", "tanh") == "tanh"):
            return self._unary(_UNARY_KERNELS[op], fallback)
        if op in _BINARY_KERNELS:
            return self._binary(_BINARY_KERNELS[op], fallback)
        if op in ("Gather", "Embedding"):
            return self._gather(node, fallback)
        if op in ("Conv", "FusedConv") and node.attr("data_format") == "NHWC":
            from .gpu_conv import conv_resolver
            return conv_resolver(self, node, fallback)
        if op in ("MaxPool", "GlobalAveragePool") and node.attr("data_format") == "NHWC":
            from .gpu_conv import pool_resolver
            return pool_resolver(self, node, fallback)
        return fallback

    def _fallback(self, node: GraphNode):
        fn = self.reg.get(node.op_type).fn
        dev = self.device
        shape_op = node.op_type in _SHAPE_PARAM_OPS

        def run(i, a, c):
            if any(t is not None and t.device.type == "cuda" for t in i):
                lim = 1 if shape_op else len(i)
                i = [self.to_device(t) if (k < lim and t is not None and t.device.type != "cuda") else t
                     for k, t in enumerate(i)]
            return fn(i, a, c)
        return run

    # ------------------------------------------------------------------ kernels
    def _gemm(self, node: GraphNode, fallback):
        K = self.K
        act = node.attr("activation", "") if node.op_type == "FusedGemm" else ""
        plain_gemm = node.op_type == "Gemm" and (float(node.attr("alpha", 1.0)) != 1.0 or float(node.attr("beta", 1.0)) != 1.0)
        wname = node.inputs[1]

        def run(i, a, c):
            x, w = i[0], i[1]
            if plain_gemm or x.dtype not in _HALF or x.dtype != w.dtype or x.dim() < 1:
                return _torch_gemm(x, w, i, a, act)
            lead = x.shape[:-1]
            x2 = x.reshape(-1, x.shape[-1])
            if not _aligned(x2):
                x2 = x2.contiguous()
            bias = i[2] if len(i) > 2 else None
            if bias is not None and (bias.dim() != 1 or bias.shape[0] != w.shape[0]):
                return _torch_gemm(x, w, i, a, act)
            res = i[3].reshape(-1, w.shape[0]) if len(i) > 3 and i[3] is not None else None
            if res is not None and not res.is_contiguous():
                res = res.contiguous()
            y = K.gemm(x2, w, bias, res, act)
            return [y.reshape(*lead, w.shape[0])]
        return run

    def _layernorm(self, node, fallback):
        K = self.K

        def run(i, a, c):
            x = i[0]
            if x.dtype not in _HALF or x.shape[-1] % 8 or x.shape[-1] > 32768:
                return fallback(i, a, c)
            return [K.layernorm(x, i[1] if len(i) > 1 else None, i[2] if len(i) > 2 else None,
                                float(a.get("epsilon", 1e-5)))]
        return run

    def _rmsnorm(self, node, fallback):
        K = self.K

        def run(i, a, c):
            x = i[0]
            if x.dtype not in _HALF or x.shape[-1] % 8:
                return fallback(i, a, c)
            return [K.rmsnorm(x, i[1], float(a.get("epsilon", 1e-5)))]
        return run

    def _softmax(self, node, fallback):
        K = self.K

        def run(i, a, c):
            x = i[0]
            axis = int(a.get("axis", -1))
            if axis not in (-1, x.dim() - 1) or x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
                return fallback(i, a, c)
            return [K.softmax(x)]
        return run

    def _unary(self, kname, fallback):
        K = self.K

        def run(i, a, c):
            x = i[0]
            if x.dtype not in _HALF or x.device.type != "cuda":
                return fallback(i, a, c)
            return [K.unary(x, kname)]
        return run

    def _binary(self, kname, fallback):
        K = self.K

        def run(i, a, c):
            x, y = i[0], i[1]
            if (x.dtype not in _HALF or y.dtype != x.dtype or x.shape != y.shape or x.device.type != "cuda"
                    or y.device.type != "cuda"):
                return fallback(i, a, c)
            return [K.binary(x, y, kname)]
        return run

    def _gather(self, node, fallback):
        K = self.K
        axis = int(node.attr("axis", 0))

        def run(i, a, c):
            table, idx = (i[0], i[1]) if i[0].is_floating_point() else (i[1], i[0])
            if (axis != 0 or table.dim() != 2 or table.dtype not in _HALF or table.shape[1] % 8
                    or table.device.type != "cuda" or idx.is_floating_point()):
                return fallback(i, a, c)
            idx = self.to_device(idx)
            y = K.embedding(idx, table)
            return [y.reshape(*idx.shape, table.shape[1])]
        return run


def _torch_gemm(x, w_nk, i, a, act):
    """Library path for operand types the tensor-core kernel does not take (weights are stored [N,K])."""
    y = torch.matmul(x, w_nk.t().to(x.dtype)) * float(a.get("alpha", 1.0))
    if len(i) > 2 and i[2] is not None:
        y = y + float(a.get("beta", 1.0)) * i[2]
    if act == "Relu":
        y = torch.relu(y)
    elif act == "Gelu":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if len(i) > 3 and i[3] is not None:
        y = y + i[3]
    return [y]
