"""Node -> kernel resolution of the GPU provider."""
from __future__ import annotations

import math

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
        if op == "SkipLayerNorm":
            return self._skip_layernorm(node, fallback)
        if op == "Softmax":
            return self._softmax(node, fallback)
        if op in _UNARY_KERNELS and (op != "Gelu" or node.attr("approximate", "none") == "tanh"):
            return self._unary(_UNARY_KERNELS[op], fallback)
        if op in _BINARY_KERNELS:
            return self._binary(_BINARY_KERNELS[op], fallback)
        if op in ("Gather", "Embedding"):
            return self._gather(node, fallback)
        if op == "FusedElementwise":
            return self._fused_elementwise(node, fallback)
        if op in ("Attention", "MultiHeadAttention"):
            return self._attention(node, fallback)
        if op == "ScaledDotProductAttention":
            return self._sdpa(node, fallback)
        if op == "PagedAttention":
            return self._paged_attention(node, fallback)
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

    def _skip_layernorm(self, node, fallback):
        """LayerNorm(x + skip) and the sum in one launch of the norm kernel."""
        K = self.K

        def run(i, a, c):
            x, skip = i[0], i[1]
            if (x.dtype not in _HALF or skip.dtype != x.dtype or x.shape != skip.shape or x.shape[-1] % 8
                    or x.shape[-1] > 32768 or (len(i) > 4 and i[4] is not None)):
                return fallback(i, a, c)
            y, s = K.layernorm(x, i[2], i[3] if len(i) > 3 else None, float(a.get("epsilon", 1e-5)), residual=skip,
                               return_sum=True)
            return [y, s]
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
            if (x.dtype not in (torch.bfloat16, torch.float16, torch.float32) or x.device.type != "cuda" or x.dim() == 0
                    or a.get("legacy_flatten") or not -x.dim() <= axis < x.dim()):
                return fallback(i, a, c)
            return [K.softmax(x, axis)]
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

    def _fused_elementwise(self, node, fallback):
        """A collapsed chain of element-wise nodes: one launch of the chain kernel when the operands fit it."""
        K = self.K
        names = list(node.attr("ops"))
        arity = [int(v) for v in node.attr("arity")]

        def run(i, a, c):
            x = i[0]
            operands, k = [], 1
            for n_in in arity:
                operands.append(i[k] if n_in == 2 else None)
                k += n_in - 1
            if not isinstance(x, torch.Tensor) or x.device.type != "cuda":
                return fallback(i, a, c)
            operands = [self.to_device(b) if (b is not None and b.device.type != "cuda") else b for b in operands]
            operands = [b.to(x.dtype) if (b is not None and b.dtype != x.dtype and b.is_floating_point()) else b for b in operands]
            plan = K.fused_elementwise_plan(x, names, operands)
            if plan is None:
                return fallback(i, a, c)
            return [K.fused_elementwise(x, names, operands, plan)]
        return run

    def _attention(self, node, fallback):
        """Attention / MultiHeadAttention on [B, S, H] tensors -> the tcgen05 attention kernel.  Q and K are read in
        place when they are column slices of one fused projection buffer (what the QKV fusion of the optimiser
        produces), otherwise they are packed side by side first.  Masks: none, causal, or a key-padding mask marked
        ``mask_type="key_padding"`` (additive [B, 1, 1, S] with the padding at the end of every row); anything else
        runs the operator's library form."""
        K = self.K
        heads = int(node.attr("num_heads", 0))
        causal = bool(int(node.attr("causal", 0)))
        mask_type = node.attr("mask_type", "")
        plans = {}

        def plan_for(B, S, dev):
            p = plans.get((B, S))
            if p is None:
                mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
                p = {"seq_start": mk([b * S for b in range(B)]),
                     "max_len": S, "n_seq": B, "q_len": torch.full((B,), S, dtype=torch.int32, device=dev),
                     "kv_len": torch.full((B,), S, dtype=torch.int32, device=dev)}
                plans[(B, S)] = p
            return p

        def run(i, a, c):
            q, k, v = i[0], i[1], i[2]
            mask = i[3] if len(i) > 3 else None
            ok = (heads > 0 and q.dim() == 3 and q.dtype in _HALF and k.dtype == q.dtype and v.dtype == q.dtype
                  and q.device.type == "cuda" and q.shape == k.shape == v.shape and q.shape[-1] % heads == 0
                  and q.shape[-1] // heads in (64, 128) and (mask is None or mask_type == "key_padding"))
            if not ok:
                return fallback(i, a, c)
            B, S, H = q.shape
            d = H // heads
            plan = plan_for(B, S, q.device)
            # column slices of one [B * S, ld] buffer?
            same = (q.untyped_storage().data_ptr() == k.untyped_storage().data_ptr() == v.untyped_storage().data_ptr()
                    and q.stride() == k.stride() == v.stride() and q.stride(2) == 1 and q.stride(0) == S * q.stride(1)
                    and q.stride(1) % 8 == 0)
            if same:
                ld = q.stride(1)
                offs = [t.storage_offset() for t in (q, k, v)]
                base = min(offs)
                row0 = base // ld * ld                       # start of the row that holds the lowest slice
                cols = [o - row0 for o in offs]
                same = all(0 <= cc and cc + H <= ld and cc % 8 == 0 for cc in cols) and (row0 * q.element_size()) % 16 == 0
            if same:
                buf = torch.as_strided(q, (B * S, ld), (ld, 1), row0)
                q_off, k_off, v_off = cols
            else:
                buf = torch.cat([q.reshape(B * S, H), k.reshape(B * S, H), v.reshape(B * S, H)], dim=1)
                q_off, k_off, v_off = 0, H, 2 * H
            if mask is not None:
                m = mask.reshape(B, -1, mask.shape[-1])[:, 0, :] if mask.dim() > 2 else mask.reshape(B, -1)
                kv_len = (m > -1e4).sum(dim=-1).clamp_(min=1).to(torch.int32)
                plan = dict(plan, kv_len=kv_len)
            out = K.dense_attention(buf, q_off, k_off, v_off, plan, heads, heads, d, causal, plan["q_len"], S)
            return [out.view(B, S, H)]
        return run

    def _paged_attention(self, node, fallback):
        """``com.ronn::PagedAttention`` on the decode attention kernel (16-bit q and caches, head size 64 or 128,
        default scale, context within the kernel's limit); anything else takes the operator's library form."""
        K = self.K
        heads = int(node.attr("num_heads", 0))
        kv_heads = int(node.attr("kv_heads", heads))
        scale = node.attr("scale", None)

        def run(i, a, c):
            q, kc, vc, bt, ctx = i[0], i[1], i[2], i[3], i[4]
            d = kc.shape[3] if kc.dim() == 4 else 0
            ok = (q.is_cuda and q.dtype in _HALF and kc.dtype == q.dtype and vc.dtype == q.dtype and d in (64, 128)
                  and q.dim() == 2 and q.stride(1) == 1 and q.stride(0) % 8 == 0 and kc.is_contiguous()
                  and vc.is_contiguous() and bt.dtype == torch.int32 and bt.is_contiguous() and ctx.dtype == torch.int32
                  and bt.shape[1] * 16 <= 4096 and heads > 0 and heads % max(kv_heads, 1) == 0
                  and (scale is None or abs(float(scale) * math.sqrt(d) - 1.0) < 1e-6)
                  and (len(i) < 6 or i[5].dtype == torch.int32))
            if not ok:
                return fallback(i, a, c)
            return [K.paged_attention(q, kc, vc, bt, ctx.contiguous(), heads, kv_heads, d, bt.shape[1] * 16,
                                      i[5].contiguous() if len(i) > 5 else None)]
        return run

    def _sdpa(self, node, fallback):
        """The fused attention core on head-split tensors (Q [B, h, S, d], K^T [B, h, d, S], V [B, h, S, d]).  Without
        a mask, with the usual 1 / sqrt(d) scale and d of 64 or 128 the three operands are laid side by side as rows of
        tokens and the tcgen05 attention kernel runs; its [B, S, h, d] result goes back as a transposed view, which the
        Transpose that exporters put behind the attention core undoes without a copy.  Everything else takes the
        library's fused attention."""
        K = self.K
        scale = float(node.attr("scale", 1.0))
        kt = bool(int(node.attr("k_transposed", 0)))
        plans = {}

        def plan_for(B, S, dev):
            p = plans.get((B, S))
            if p is None:
                mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
                full = torch.full((B,), S, dtype=torch.int32, device=dev)
                p = {"seq_start": mk([b * S for b in range(B)]), "max_len": S, "n_seq": B, "q_len": full, "kv_len": full}
                plans[(B, S)] = p
            return p

        def run(i, a, c):
            q, k, v = i[0], i[1], i[2]
            mask = i[3] if len(i) > 3 else None
            if q.device.type != "cuda" or q.dtype not in _HALF or q.dim() != 4 or (len(i) > 4 and i[4] is not None):
                return fallback(i, a, c)
            k_bhsd = k.transpose(-1, -2) if kt else k
            B, h, S, d = q.shape
            ok = (mask is None and d in (64, 128) and k_bhsd.shape == q.shape and v.shape == q.shape
                  and k.dtype == q.dtype and v.dtype == q.dtype and abs(scale * math.sqrt(d) - 1.0) < 1e-3)
            if not ok:
                m = None if mask is None else mask.to(q.dtype)
                return [torch.nn.functional.scaled_dot_product_attention(q, k_bhsd, v, attn_mask=m, scale=scale)]
            H = h * d
            buf = torch.cat([t.transpose(1, 2).reshape(B * S, H) for t in (q, k_bhsd, v)], dim=1)
            plan = plan_for(B, S, q.device)
            out = K.dense_attention(buf, 0, H, 2 * H, plan, h, h, d, False, plan["q_len"], S)
            return [out.view(B, S, h, d).transpose(1, 2)]
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
