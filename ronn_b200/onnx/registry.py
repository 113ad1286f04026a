"""Operator registry.

The reference registers 39 ONNX operators behind ``OnnxOperator{op_type, execute, validate}``
(crates/ronn-onnx/src/ops/mod.rs:22-139) and builds a new registry for every node it runs
(crates/ronn-api/src/session.rs:254).  Here the registry is a process-wide table resolved
once per session: each entry is a function ``(inputs, attrs, ctx) -> outputs`` over torch
tensors, so the same definition serves the CPU provider and, as the fallback for ops with
no hand-written kernel, the GPU provider.  Numeric definitions follow the reference
(GELU tanh form crates/ronn-core/src/ops/arithmetic.rs:281-296, LayerNorm population
variance eps 1e-5 crates/ronn-core/src/tensor.rs:566-611, attention
crates/ronn-core/src/tensor.rs:640-709); Softmax uses ONNX axis semantics (negative axes
count from the end) where the reference clamps them to 0
(crates/ronn-onnx/src/ops/activations.rs:105-109).

Operators the reference lacks but the benchmark graphs need (Gemm, Flatten,
GlobalAveragePool, Identity, Constant, Shape, Where, Erf, Expand, Slice, ...) and the
``com.ronn`` custom domain (FusedConv, FusedGemm, RMSNorm, RotaryEmbedding, SwiGLU,
BitLinear, ...) are registered too.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..api.errors import InvalidAttribute, InvalidGraph, UnsupportedOperator
from .dtypes import DataTypeMapper

OpFn = Callable[[List[Optional[torch.Tensor]], Dict[str, Any], Any], List[torch.Tensor]]


class OnnxOperator:
    def __init__(self, op_type: str, fn: OpFn, min_inputs: int, max_inputs: Optional[int], domain: str = ""):
        self.op_type = op_type
        self.fn = fn
        self.min_inputs = min_inputs
        self.max_inputs = max_inputs
        self.domain = domain

    def validate(self, inputs: Sequence[Optional[torch.Tensor]]) -> None:
        n = len(inputs)
        if n < self.min_inputs or (self.max_inputs is not None and n > self.max_inputs):
            if self.max_inputs == self.min_inputs:
                want = f"{self.min_inputs} input{'s' if self.min_inputs != 1 else ''}"
            elif self.max_inputs is None:
                want = f"at least {self.min_inputs} input{'s' if self.min_inputs != 1 else ''}"
            else:
                want = f"{self.min_inputs}-{self.max_inputs} inputs"
            raise InvalidGraph(f"{self.op_type} expects {want}, got {n}")

    def execute(self, inputs, attrs=None, ctx=None):
        self.validate(inputs)
        return self.fn(list(inputs), attrs or {}, ctx)


class OperatorRegistry:
    def __init__(self):
        self._ops: Dict[str, OnnxOperator] = {}

    def register(self, op: OnnxOperator) -> None:
        self._ops[op.op_type] = op

    def get(self, op_type: str) -> OnnxOperator:
        op = self._ops.get(op_type)
        if op is None:
            raise UnsupportedOperator(op_type)
        return op

    def has(self, op_type: str) -> bool:
        return op_type in self._ops

    def supported_ops(self) -> List[str]:
        return sorted(self._ops)

    def __len__(self):
        return len(self._ops)


_REGISTRY = OperatorRegistry()


def default_registry() -> OperatorRegistry:
    return _REGISTRY


def op(name: str, min_inputs: int, max_inputs: Optional[int] = -1, domain: str = ""):
    def deco(fn):
        mx = min_inputs if max_inputs == -1 else max_inputs
        _REGISTRY.register(OnnxOperator(name, fn, min_inputs, mx, domain))
        return fn
    return deco


# The 39 operators the reference registers (crates/ronn-onnx/src/ops/mod.rs:50-139).
REFERENCE_OPS = [
    "Relu", "Sigmoid", "Tanh", "Softmax", "Gelu", "LeakyRelu", "Elu", "Swish",
    "Add", "Sub", "Mul", "Div", "MatMul", "Sqrt", "Pow", "Exp", "Log", "Neg", "Abs", "Clip",
    "Conv", "MaxPool", "AveragePool", "BatchNormalization", "LayerNormalization", "Attention", "MultiHeadAttention",
    "Reshape", "Transpose", "Concat", "Split", "Gather", "Slice", "Squeeze", "Unsqueeze", "ReduceMean", "ReduceSum",
    "Cast", "Embedding",
]


# ------------------------------------------------------------------------------ helpers
def _ints(v) -> List[int]:
    if v is None:
        return []
    if isinstance(v, torch.Tensor):
        return [int(x) for x in v.reshape(-1).tolist()]
    if isinstance(v, (int, float)):
        return [int(v)]
    return [int(x) for x in v]


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


def _unary(name, fn):
    op(name, 1)(lambda i, a, c, _f=fn: [_f(i[0])])


def _binary(name, fn):
    op(name, 2)(lambda i, a, c, _f=fn: [_f(i[0], i[1])])


# ------------------------------------------------------------------------------ activations
_unary("Relu", torch.relu)
_unary("Sigmoid", torch.sigmoid)
_unary("Tanh", torch.tanh)
_unary("Swish", lambda x: x * torch.sigmoid(x))
_unary("Erf", torch.erf)
_unary("Softplus", F.softplus)
_unary("Identity", lambda x: x)
_unary("Not", torch.logical_not)
_unary("Floor", torch.floor)
_unary("Ceil", torch.ceil)
_unary("Reciprocal", torch.reciprocal)
_unary("Sign", torch.sign)


@op("Gelu", 1)
def _gelu(i, a, c):
    """ONNX semantics: ``approximate`` defaults to "none" (the exact erf form).  The reference always evaluates the tanh
    form (crates/ronn-core/src/ops/arithmetic.rs:281-296); the in-tree model builders ask for it explicitly."""
    approx = a.get("approximate", "none")
    approx = approx.decode() if isinstance(approx, bytes) else approx
    return [F.gelu(i[0], approximate="tanh" if approx == "tanh" else "none")]


@op("FastGelu", 1, 2, domain="com.ronn")
def _fast_gelu(i, a, c):
    x = i[0] if len(i) == 1 or i[1] is None else i[0] + i[1]
    return [x * torch.sigmoid(1.702 * x)]


@op("LeakyRelu", 1)
def _leaky(i, a, c):
    return [F.leaky_relu(i[0], float(a.get("alpha", 0.01)))]


@op("Elu", 1)
def _elu(i, a, c):
    return [F.elu(i[0], float(a.get("alpha", 1.0)))]


@op("HardSigmoid", 1)
def _hsig(i, a, c):
    return [torch.clamp(float(a.get("alpha", 0.2)) * i[0] + float(a.get("beta", 0.5)), 0.0, 1.0)]


def _softmax_like(fn, i, a):
    """Opset >= 13: along ``axis`` (default -1).  Below opset 13 (the loader marks such nodes ``legacy_flatten``): the
    input is coerced to 2-D at ``axis`` (default 1) and normalised over the whole trailing block."""
    x = i[0]
    if int(a.get("legacy_flatten", 0)):
        axis = int(a.get("axis", 1))
        axis = axis + x.dim() if axis < 0 else axis
        lead = 1
        for d in x.shape[:axis]:
            lead *= d
        return [fn(x.reshape(lead, -1), dim=1).reshape(x.shape)]
    return [fn(x, dim=int(a.get("axis", -1)))]


@op("Softmax", 1)
def _softmax(i, a, c):
    return _softmax_like(torch.softmax, i, a)


@op("LogSoftmax", 1)
def _log_softmax(i, a, c):
    return _softmax_like(torch.log_softmax, i, a)


@op("Dropout", 1, 3)
def _dropout(i, a, c):
    return [i[0]]


# ------------------------------------------------------------------------------ math
def _div(x, y):
    if not x.is_floating_point() and not y.is_floating_point():
        return torch.div(x, y, rounding_mode="trunc")
    return x / y


_binary("Add", torch.add)
_binary("Sub", torch.sub)
_binary("Mul", torch.mul)
_binary("Div", _div)
_binary("Pow", lambda x, y: torch.pow(x, y.to(x.dtype) if y.dtype != x.dtype and x.is_floating_point() else y))
_binary("Equal", torch.eq)
_binary("Less", torch.lt)
_binary("Greater", torch.gt)
_binary("LessOrEqual", torch.le)
_binary("GreaterOrEqual", torch.ge)
_binary("And", torch.logical_and)
_binary("Or", torch.logical_or)
_binary("Xor", torch.logical_xor)
_unary("Sqrt", torch.sqrt)
_unary("Exp", torch.exp)
_unary("Log", torch.log)
_unary("Neg", torch.neg)
_unary("Abs", torch.abs)


@op("Min", 1, None)
def _min(i, a, c):
    out = i[0]
    for t in i[1:]:
        out = torch.minimum(out, t)
    return [out]


@op("Max", 1, None)
def _max(i, a, c):
    out = i[0]
    for t in i[1:]:
        out = torch.maximum(out, t)
    return [out]


@op("Sum", 1, None)
def _sum(i, a, c):
    out = i[0]
    for t in i[1:]:
        out = out + t
    return [out]


@op("MatMul", 2)
def _matmul(i, a, c):
    x, w = i
    if x.dim() < 1 or w.dim() < 1:
        raise InvalidGraph("MatMul operands must have at least one dimension")
    return [torch.matmul(x, w)]


@op("Gemm", 2, 3)
def _gemm(i, a, c):
    x, w = i[0], i[1]
    if int(a.get("transA", 0)):
        x = x.transpose(-1, -2)
    if int(a.get("transB", 0)):
        w = w.transpose(-1, -2)
    y = torch.matmul(x, w) * float(a.get("alpha", 1.0))
    if len(i) > 2 and i[2] is not None:
        y = y + float(a.get("beta", 1.0)) * i[2]
    return [y]


@op("Clip", 1, 3)
def _clip(i, a, c):
    lo = i[1] if len(i) > 1 and i[1] is not None else a.get("min")
    hi = i[2] if len(i) > 2 and i[2] is not None else a.get("max")
    lo = lo.item() if isinstance(lo, torch.Tensor) else lo
    hi = hi.item() if isinstance(hi, torch.Tensor) else hi
    if lo is None and hi is None:
        return [i[0]]
    return [torch.clamp(i[0], min=lo, max=hi)]


@op("Where", 3)
def _where(i, a, c):
    return [torch.where(i[0].bool(), i[1], i[2])]


# ------------------------------------------------------------------------------ neural network
def _conv_pads(pads, nd):
    pads = list(pads) if pads else [0] * (2 * nd)
    if len(pads) != 2 * nd:
        raise InvalidAttribute(f"pads must have {2 * nd} entries, got {len(pads)}")
    begin, end = pads[:nd], pads[nd:]
    return begin, end


def conv2d(x, w, b, a):
    nd = w.dim() - 2
    strides = _ints(a.get("strides")) or [1] * nd
    dil = _ints(a.get("dilations")) or [1] * nd
    group = int(a.get("group", 1))
    begin, end = _conv_pads(_ints(a.get("pads")), nd)
    auto = a.get("auto_pad", "NOTSET")
    if auto in ("SAME_UPPER", "SAME_LOWER"):
        begin, end = [], []
        for d in range(nd):
            size = x.shape[2 + d]
            k = (w.shape[2 + d] - 1) * dil[d] + 1
            total = max((math.ceil(size / strides[d]) - 1) * strides[d] + k - size, 0)
            lo = total // 2 if auto == "SAME_UPPER" else total - total // 2
            begin.append(lo)
            end.append(total - lo)
    if begin != end:
        padarg = []
        for d in reversed(range(nd)):
            padarg += [begin[d], end[d]]
        x = F.pad(x, padarg)
        begin = [0] * nd
    if nd == 2:
        return F.conv2d(x, w, b, strides, begin, dil, group)
    if nd == 1:
        return F.conv1d(x, w, b, strides, begin, dil, group)
    if nd == 3:
        return F.conv3d(x, w, b, strides, begin, dil, group)
    raise InvalidGraph(f"Conv with {nd} spatial dims is not supported")


@op("Conv", 2, 3)
def _conv(i, a, c):
    return [conv2d(i[0], i[1], i[2] if len(i) > 2 else None, a)]


@op("FusedConv", 2, 4, domain="com.ronn")
def _fused_conv(i, a, c):
    """Conv with folded BatchNorm, optional residual input (4th) and activation."""
    y = conv2d(i[0], i[1], i[2] if len(i) > 2 else None, a)
    if len(i) > 3 and i[3] is not None:
        y = y + i[3]
    act = a.get("activation", "")
    if act == "Relu":
        y = torch.relu(y)
    elif act:
        raise InvalidAttribute(f"FusedConv activation '{act}' is not supported")
    return [y]


def _pool_args(x, a):
    k = _ints(a.get("kernel_shape")) or [2, 2]
    nd = len(k)
    strides = _ints(a.get("strides")) or [1] * nd
    begin, end = _conv_pads(_ints(a.get("pads")), nd)
    return k, strides, begin, end, bool(int(a.get("ceil_mode", 0)))


def _pad_spatial(x, begin, end, value):
    arg = []
    for d in reversed(range(len(begin))):
        arg += [begin[d], end[d]]
    return F.pad(x, arg, value=value)


@op("MaxPool", 1)
def _maxpool(i, a, c):
    x = i[0]
    k, s, begin, end, ceil = _pool_args(x, a)
    nd = len(k)
    if x.dim() != nd + 2 or nd not in (1, 2, 3):
        raise InvalidGraph(f"MaxPool over {nd} spatial dimensions on a {x.dim()}-D input")
    if begin != end:
        x = _pad_spatial(x, begin, end, float("-inf"))
        begin = [0] * nd
    fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd]
    return [fn(x, k, s, begin, _ints(a.get("dilations")) or 1, ceil)]


@op("AveragePool", 1)
def _avgpool(i, a, c):
    x = i[0]
    k, s, begin, end, ceil = _pool_args(x, a)
    nd = len(k)
    if x.dim() != nd + 2 or nd not in (1, 2, 3):
        raise InvalidGraph(f"AveragePool over {nd} spatial dimensions on a {x.dim()}-D input")
    include = bool(int(a.get("count_include_pad", 0)))
    fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
    if begin != end:
        # asymmetric padding: pad by hand, then divide by the number of VALID elements under each window unless the
        # operator counts the padding (sum = mean over the padded window * window size)
        xp = _pad_spatial(x, begin, end, 0.0)
        y = fn(xp, k, s, 0, ceil, True)
        if include:
            return [y]
        ones = _pad_spatial(torch.ones((1, 1) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device), begin, end, 0.0)
        frac = fn(ones, k, s, 0, ceil, True)              # valid fraction of every window
        return [y / frac.clamp_min(1e-12)]
    return [fn(x, k, s, begin, ceil, include)]


@op("GlobalAveragePool", 1)
def _gap(i, a, c):
    x = i[0]
    return [x.mean(dim=tuple(range(2, x.dim())), keepdim=True)]


@op("GlobalMaxPool", 1)
def _gmp(i, a, c):
    x = i[0]
    return [x.amax(dim=tuple(range(2, x.dim())), keepdim=True)]


@op("BatchNormalization", 5)
def _bn(i, a, c):
    x, g, b, mean, var = i
    eps = float(a.get("epsilon", 1e-5))
    shape = [1, -1] + [1] * (x.dim() - 2)
    inv = torch.rsqrt(var.float() + eps)
    y = (x.float() - mean.float().reshape(shape)) * (inv * g.float()).reshape(shape) + b.float().reshape(shape)
    return [y.to(x.dtype)]


@op("LayerNormalization", 1, 3)
def _ln(i, a, c):
    x = i[0]
    axis = int(a.get("axis", -1))
    if axis < 0:
        axis += x.dim()
    shape = list(x.shape[axis:])
    w = i[1] if len(i) > 1 else None
    b = i[2] if len(i) > 2 else None
    y = F.layer_norm(x.float(), shape, None if w is None else w.float().reshape(shape),
                     None if b is None else b.float().reshape(shape), float(a.get("epsilon", 1e-5)))
    return [y.to(x.dtype)]


@op("RMSNorm", 2, domain="com.ronn")
def _rmsnorm(i, a, c):
    x, w = i
    eps = float(a.get("epsilon", 1e-5))
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return [y.to(x.dtype)]


@op("SkipLayerNorm", 3, 5, domain="com.ronn")
def _skip_ln(i, a, c):
    """y = LayerNorm(x + skip [+ bias]); second output is the pre-norm sum."""
    s = i[0] + i[1]
    if len(i) > 4 and i[4] is not None:
        s = s + i[4]
    y = _ln([s, i[2], i[3] if len(i) > 3 else None], a, c)[0]
    return [y, s]


@op("ScaledDotProductAttention", 3, 5, domain="com.ronn")
def _sdpa(i, a, c):
    """softmax(fill(scale * Q K^T) + mask) V on already head-split tensors: Q [..., Sq, D], V [..., Sk, D], and K either
    as [..., Sk, D] or, with ``k_transposed = 1``, as the [..., D, Sk] operand exporters feed to the first MatMul.  What
    the fusion pass makes of MatMul -> (Div | Mul scalar) -> (Where fill) -> (Add mask) -> Softmax(last axis) -> MatMul.
    The optional 5th input is a condition: scores where it is true (``fill_when = 1``) or false (0) are replaced by
    ``fill_value`` (a masked_fill)."""
    q, k, v = i[0], i[1], i[2]
    mask = i[3] if len(i) > 3 else None
    kt = k if int(a.get("k_transposed", 0)) else k.transpose(-1, -2)
    scores = torch.matmul(q.float(), kt.float()) * float(a.get("scale", 1.0))
    if len(i) > 4 and i[4] is not None:
        cond = i[4].bool()
        scores = scores.masked_fill(cond if int(a.get("fill_when", 1)) else ~cond, float(a.get("fill_value", float("-inf"))))
    if mask is not None:
        scores = scores + mask.float()
    return [torch.matmul(torch.softmax(scores, dim=-1), v.float()).to(q.dtype)]


@op("PagedAttention", 5, 6, domain="com.ronn")
def _paged_attention(i, a, c):
    """Attention of query rows over a paged key / value cache, the serving path's decode operator as a graph node.
    Inputs: q [rows, num_heads * head_dim]; k_cache and v_cache [blocks, kv_heads, 16, head_dim]; block_tables
    [*, max_blocks] int32 (cache block of every 16 keys); context_lens [rows] int32 (keys each row attends to, 0 gives
    a zero row); optional table_rows [rows] int32 (row of block_tables per query row; default its own index).
    Attributes: num_heads, kv_heads (default num_heads), scale (default 1 / sqrt(head_dim)).  The scale of the
    kernels is fixed to the default, so another value is applied to q first."""
    from ..serving.ops_backend import TorchOps
    q, kc, vc, bt, ctx = i[0], i[1], i[2], i[3], i[4]
    rows_of = i[5] if len(i) > 5 else None
    heads = int(a["num_heads"])
    kv_heads = int(a.get("kv_heads", heads))
    if kc.dim() != 4 or kc.shape[2] != 16 or kc.shape[1] != kv_heads or heads % kv_heads:
        raise InvalidGraph("PagedAttention expects caches of shape [blocks, kv_heads, 16, head_dim]")
    d = kc.shape[3]
    if q.dim() != 2 or q.shape[1] < heads * d:
        raise InvalidGraph(f"PagedAttention expects q of shape [rows, {heads * d}], got {list(q.shape)}")
    scale = float(a.get("scale", 1.0 / math.sqrt(d)))
    if abs(scale * math.sqrt(d) - 1.0) > 1e-6:
        q = (q.float() * (scale * math.sqrt(d))).to(q.dtype)
    max_ctx = bt.shape[1] * 16
    return [TorchOps().paged_attention(q, kc, vc, bt, ctx.to(torch.int32), heads, kv_heads, d, max_ctx, rows_of)]


def attention(q, k, v, num_heads: int, mask=None, causal: bool = False):
    """softmax(QK^T/sqrt(d) + mask) V per head; q,k,v are [B, S, H]."""
    B, Sq, H = q.shape
    Sk = k.shape[1]
    if H % num_heads:
        raise InvalidGraph(f"hidden size {H} is not divisible by num_heads {num_heads}")
    d = H // num_heads
    qh = q.reshape(B, Sq, num_heads, d).transpose(1, 2)
    kh = k.reshape(B, Sk, num_heads, d).transpose(1, 2)
    vh = v.reshape(B, Sk, num_heads, d).transpose(1, 2)
    scores = torch.matmul(qh.float(), kh.float().transpose(-1, -2)) / math.sqrt(d)
    if mask is not None:
        m = mask.float()
        while m.dim() < 4:
            m = m.unsqueeze(0) if m.dim() >= 2 else m.reshape(1, -1)
        if m.dim() == 4 or True:
            scores = scores + m
    if causal:
        cm = torch.full((Sq, Sk), float("-inf"), device=q.device).triu(1 + Sk - Sq)
        scores = scores + cm
    p = torch.softmax(scores, dim=-1)
    out = torch.matmul(p, vh.float()).transpose(1, 2).reshape(B, Sq, H)
    return out.to(q.dtype)


@op("Attention", 3, 4)
def _attention(i, a, c):
    if "num_heads" not in a:
        raise InvalidAttribute("Attention requires the num_heads attribute")
    mask = i[3] if len(i) > 3 else None
    return [attention(i[0], i[1], i[2], int(a["num_heads"]), mask, bool(int(a.get("causal", 0))))]


_REGISTRY.register(OnnxOperator("MultiHeadAttention", _attention, 3, 4))


@op("Embedding", 2)
def _embedding(i, a, c):
    table, idx = (i[0], i[1]) if i[0].is_floating_point() else (i[1], i[0])
    return [F.embedding(idx.long(), table)]


# ------------------------------------------------------------------------------ tensor ops
@op("Reshape", 2)
def _reshape(i, a, c):
    x = i[0]
    shape = _ints(i[1])
    if not int(a.get("allowzero", 0)):
        shape = [x.shape[k] if s == 0 and k < x.dim() else s for k, s in enumerate(shape)]
    return [x.reshape(shape)]


@op("Flatten", 1)
def _flatten(i, a, c):
    x = i[0]
    axis = int(a.get("axis", 1))
    if axis < 0:
        axis += x.dim()
    lead = 1
    for s in x.shape[:axis]:
        lead *= s
    return [x.reshape(lead, -1)]


@op("Transpose", 1)
def _transpose(i, a, c):
    x = i[0]
    perm = _ints(a.get("perm")) or list(reversed(range(x.dim())))
    return [x.permute(perm)]


@op("Concat", 1, None)
def _concat(i, a, c):
    if "axis" not in a:
        raise InvalidAttribute("Concat requires the axis attribute")
    return [torch.cat([t for t in i if t is not None], dim=int(a["axis"]))]


@op("Split", 1, 2)
def _split(i, a, c):
    x = i[0]
    axis = int(a.get("axis", 0))
    sizes = _ints(i[1]) if len(i) > 1 and i[1] is not None else _ints(a.get("split"))
    if sizes:
        return list(torch.split(x, sizes, dim=axis))
    n = int(a.get("num_outputs", 0)) or (c.num_outputs if c is not None and getattr(c, "num_outputs", 0) else 2)
    size = -(-x.shape[axis] // n)
    return list(torch.split(x, size, dim=axis))


@op("Gather", 2)
def _gather(i, a, c):
    x, idx = i
    axis = int(a.get("axis", 0))
    idx = idx.long()
    idx = torch.where(idx < 0, idx + x.shape[axis], idx)
    if idx.dim() == 0:
        return [x.select(axis, int(idx))]
    out = torch.index_select(x, axis, idx.reshape(-1))
    shape = list(x.shape[:axis]) + list(idx.shape) + list(x.shape[axis + 1:] if axis != -1 else [])
    return [out.reshape(shape)]


@op("Slice", 1, 5)
def _slice(i, a, c):
    x = i[0]
    if len(i) > 1:
        starts, ends = _ints(i[1]), _ints(i[2])
        axes = _ints(i[3]) if len(i) > 3 and i[3] is not None else list(range(len(starts)))
        steps = _ints(i[4]) if len(i) > 4 and i[4] is not None else [1] * len(starts)
    else:
        starts, ends = _ints(a.get("starts")), _ints(a.get("ends"))
        axes = _ints(a.get("axes")) or list(range(len(starts)))
        steps = [1] * len(starts)
    for s, e, ax, st in zip(starts, ends, axes, steps):
        n = x.shape[ax]
        if st > 0:
            s = max(0, min(n, s + n if s < 0 else s))
            e = max(0, min(n, e + n if e < 0 else e))
            x = x.narrow(ax, s, max(e - s, 0))
            if st != 1:
                x = x.index_select(ax, torch.arange(0, x.shape[ax], st, device=x.device))
        else:
            s = max(-1, min(n - 1, s + n if s < 0 else s))
            e = max(-1, min(n - 1, e + n if e < 0 else e))
            idx = torch.arange(s, e, st, device=x.device)
            x = x.index_select(ax, idx)
    return [x]


@op("Squeeze", 1, 2)
def _squeeze(i, a, c):
    x = i[0]
    axes = _ints(i[1]) if len(i) > 1 and i[1] is not None else _ints(a.get("axes"))
    if not axes:
        return [x.squeeze()]
    for ax in sorted([ax + x.dim() if ax < 0 else ax for ax in axes], reverse=True):
        x = x.squeeze(ax)
    return [x]


@op("Unsqueeze", 1, 2)
def _unsqueeze(i, a, c):
    x = i[0]
    axes = _ints(i[1]) if len(i) > 1 and i[1] is not None else _ints(a.get("axes"))
    if not axes:
        raise InvalidAttribute("Unsqueeze requires axes")
    nd = x.dim() + len(axes)
    for ax in sorted(ax + nd if ax < 0 else ax for ax in axes):
        x = x.unsqueeze(ax)
    return [x]


def _reduce(fn):
    def run(i, a, c):
        x = i[0]
        axes = _ints(i[1]) if len(i) > 1 and i[1] is not None else _ints(a.get("axes"))
        keep = bool(int(a.get("keepdims", 1)))
        if not axes:
            if int(a.get("noop_with_empty_axes", 0)):
                return [x]
            axes = list(range(x.dim()))
        return [fn(x, axes, keep)]
    return run


op("ReduceMean", 1, 2)(_reduce(lambda x, ax, k: x.mean(dim=ax, keepdim=k)))
op("ReduceSum", 1, 2)(_reduce(lambda x, ax, k: x.sum(dim=ax, keepdim=k)))
op("ReduceMax", 1, 2)(_reduce(lambda x, ax, k: x.amax(dim=ax, keepdim=k)))
op("ReduceMin", 1, 2)(_reduce(lambda x, ax, k: x.amin(dim=ax, keepdim=k)))
op("ReduceProd", 1, 2)(_reduce(lambda x, ax, k: _prod(x, ax, k)))
op("ReduceL2", 1, 2)(_reduce(lambda x, ax, k: x.pow(2).sum(dim=ax, keepdim=k).sqrt()))


def _prod(x, axes, keep):
    for ax in sorted([a + x.dim() if a < 0 else a for a in axes], reverse=True):
        x = x.prod(dim=ax, keepdim=keep)
    return x


@op("ArgMax", 1)
def _argmax(i, a, c):
    return [torch.argmax(i[0], dim=int(a.get("axis", 0)), keepdim=bool(int(a.get("keepdims", 1))))]


@op("ArgMin", 1)
def _argmin(i, a, c):
    return [torch.argmin(i[0], dim=int(a.get("axis", 0)), keepdim=bool(int(a.get("keepdims", 1))))]


@op("Cast", 1)
def _cast(i, a, c):
    if "to" not in a:
        raise InvalidAttribute("Cast requires the 'to' attribute")
    return [i[0].to(DataTypeMapper.from_onnx(int(a["to"])).torch)]


@op("Shape", 1)
def _shape(i, a, c):
    s = list(i[0].shape)
    start, end = int(a.get("start", 0)), a.get("end")
    s = s[start: (int(end) if end is not None else None)]
    return [torch.tensor(s, dtype=torch.int64)]


@op("Constant", 0)
def _constant(i, a, c):
    if "value" in a:
        return [a["value"]]
    if "value_float" in a:
        return [torch.tensor(float(a["value_float"]), dtype=torch.float32)]
    if "value_int" in a:
        return [torch.tensor(int(a["value_int"]), dtype=torch.int64)]
    if "value_floats" in a:
        return [torch.tensor(a["value_floats"], dtype=torch.float32)]
    if "value_ints" in a:
        return [torch.tensor(a["value_ints"], dtype=torch.int64)]
    raise InvalidAttribute("Constant node carries no value")


@op("ConstantOfShape", 1)
def _const_of_shape(i, a, c):
    v = a.get("value")
    shape = _ints(i[0])
    if v is None:
        return [torch.zeros(shape, dtype=torch.float32)]
    return [torch.full(shape, v.reshape(-1)[0].item(), dtype=v.dtype)]


@op("Expand", 2)
def _expand(i, a, c):
    x = i[0]
    shape = _ints(i[1])
    nd = max(len(shape), x.dim())
    xs = [1] * (nd - x.dim()) + list(x.shape)
    shape = [1] * (nd - len(shape)) + shape
    return [x.expand([max(s, t) for s, t in zip(shape, xs)])]


@op("Range", 3)
def _range(i, a, c):
    s, e, d = (t.item() for t in i)
    return [torch.arange(s, e, d, dtype=i[0].dtype)]


@op("Tile", 2)
def _tile(i, a, c):
    return [i[0].repeat(_ints(i[1]))]


@op("Pad", 2, 4)
def _pad(i, a, c):
    """Modes constant / reflect / edge; ``axes`` (opset 18, 4th input) selects the padded dimensions; negative pads crop."""
    x = i[0]
    pads = _ints(i[1])
    val = i[2].item() if len(i) > 2 and i[2] is not None else 0.0
    nd = x.dim()
    axes = [ax + nd if ax < 0 else ax for ax in _ints(i[3])] if len(i) > 3 and i[3] is not None else list(range(nd))
    if len(pads) != 2 * len(axes) or len(set(axes)) != len(axes) or any(ax < 0 or ax >= nd for ax in axes):
        raise InvalidAttribute(f"Pad: {len(pads)} pad values for axes {axes} of a {nd}-D input")
    begin, end = [0] * nd, [0] * nd
    for k, ax in enumerate(axes):
        begin[ax], end[ax] = pads[k], pads[k + len(axes)]
    mode = a.get("mode", "constant")
    mode = mode.decode() if isinstance(mode, bytes) else mode
    if mode not in ("constant", "reflect", "edge"):
        raise InvalidAttribute(f"Pad mode '{mode}' is not supported")
    for d in range(nd):                                   # negative pads crop, in every mode
        if begin[d] < 0 or end[d] < 0:
            x = x.narrow(d, max(-begin[d], 0), x.shape[d] - max(-begin[d], 0) - max(-end[d], 0))
            begin[d], end[d] = max(begin[d], 0), max(end[d], 0)
    if mode == "constant":
        arg = []
        for d in reversed(range(nd)):
            arg += [begin[d], end[d]]
        return [F.pad(x, arg, mode="constant", value=val)]
    # reflect / edge: gather along one dimension at a time (works for any rank, any dtype)
    for d in range(nd):
        if begin[d] == 0 and end[d] == 0:
            continue
        n = x.shape[d]
        idx = torch.arange(-begin[d], n + end[d], device=x.device)
        if mode == "edge":
            idx = idx.clamp(0, n - 1)
        else:
            if n < 2 or begin[d] >= n or end[d] >= n:
                raise InvalidAttribute("Pad reflect: pads must be smaller than the padded dimension")
            idx = idx.abs()
            idx = torch.where(idx >= n, 2 * (n - 1) - idx, idx)
        x = x.index_select(d, idx)
    return [x]


# ------------------------------------------------------------------------------ com.ronn custom domain
@op("FusedGemm", 2, 4, domain="com.ronn")
def _fused_gemm(i, a, c):
    """y = act(x @ W^T(if transB) + bias) [+ residual]; produced by the MatMul+Add / Gemm+activation fusion."""
    x, w = i[0], i[1]
    if int(a.get("transB", 0)):
        w = w.transpose(-1, -2)
    y = torch.matmul(x, w)
    if len(i) > 2 and i[2] is not None:
        y = y + i[2]
    act = a.get("activation", "")
    if act == "Relu":
        y = torch.relu(y)
    elif act == "Gelu":
        y = gelu_tanh(y)
    elif act:
        raise InvalidAttribute(f"FusedGemm activation '{act}' is not supported")
    if len(i) > 3 and i[3] is not None:
        y = y + i[3]
    return [y]


@op("FusedElementwise", 1, None, domain="com.ronn")
def _fused_elementwise(i, a, c):
    """A chain of elementwise ops run back to back; ``ops`` lists them, ``arity`` their input counts.
    The running value is always the first operand."""
    ops = a["ops"]
    arity = _ints(a["arity"])
    x = i[0]
    k = 1
    for name, n in zip(ops, arity):
        extra = i[k:k + n - 1]
        k += n - 1
        x = _REGISTRY.get(name).fn([x] + list(extra), {}, c)[0]
    return [x]


@op("AllReduce", 1, domain="com.ronn")
def _all_reduce(i, a, c):
    """Sum over the ranks of the session's process group (inserted by the tensor-parallel pass); the identity in a
    single-process session."""
    import torch.distributed as dist
    x = i[0]
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        x = x.contiguous().clone()
        dist.all_reduce(x)
    return [x]


@op("SiLU", 1, domain="com.ronn")
def _silu(i, a, c):
    return [F.silu(i[0])]


@op("SwiGLU", 2, domain="com.ronn")
def _swiglu(i, a, c):
    return [F.silu(i[0]) * i[1]]


def rotary(x, positions, base: float = 10000.0, num_heads: Optional[int] = None):
    """Rotate pairs (i, i + d/2) of every head: theta_i = base^(-2i/d).  x: [..., T, heads*d] or [..., T, heads, d]."""
    shape = x.shape
    if num_heads is not None and x.dim() >= 2 and x.shape[-1] % num_heads == 0 and (x.dim() < 3 or True):
        d = x.shape[-1] // num_heads
        xh = x.reshape(*shape[:-1], num_heads, d)
    else:
        xh = x
        d = x.shape[-1]
    half = d // 2
    inv = base ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / d)
    ang = positions.to(torch.float32).unsqueeze(-1) * inv            # [..., T, half]
    cos, sin = torch.cos(ang).unsqueeze(-2), torch.sin(ang).unsqueeze(-2)
    xf = xh.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    return out.to(x.dtype).reshape(shape)


@op("RotaryEmbedding", 2, domain="com.ronn")
def _rotary(i, a, c):
    return [rotary(i[0], i[1], float(a.get("base", 10000.0)), int(a["num_heads"]) if "num_heads" in a else None)]


@op("BitLinear", 3, 4, domain="com.ronn")
def _bitlinear(i, a, c):
    """y = (int8(x) . ternary(W)) * x_scale * w_scale [+ bias].

    Inputs: x [..., K]; W packed uint8 [N, K/4] (2-bit codes 00=-1, 01=0, 10=+1, element i at
    bits 2*(i mod 4) of byte i/4); w_scale scalar; optional bias [N].  Activations are quantised
    per token to int8 with absmax scaling.  Integer accumulation is exact."""
    from ..providers.bitnet.quantization import bitlinear_reference
    return [bitlinear_reference(i[0], i[1], i[2], i[3] if len(i) > 3 else None, int(a["k"]), int(a["n"]))]


# ------------------------------------------------------------------------------ NHWC execution
def _wrap_nhwc(name: str, image_inputs: Sequence[int], weight_inputs: Sequence[int] = ()):
    """Let a spatial operator run on NHWC tensors when the layout pass tagged it ``data_format="NHWC"``.

    Image operands are viewed as NCHW (a permute of an NHWC tensor is channels-last memory, which
    the CPU/cuDNN paths accept without a copy), weights stored [Cout,R,S,Cin] are viewed back as
    [Cout,Cin,R,S], and results are returned as NHWC."""
    base = _REGISTRY.get(name)
    inner = base.fn

    def run(i, a, c):
        if a.get("data_format") != "NHWC":
            return inner(i, a, c)
        i = list(i)
        for k in image_inputs:
            if k < len(i) and i[k] is not None and i[k].dim() == 4:
                i[k] = i[k].permute(0, 3, 1, 2)
        for k in weight_inputs:
            if k < len(i) and i[k] is not None and i[k].dim() == 4:
                i[k] = i[k].permute(0, 3, 1, 2)
        a2 = {k: v for k, v in a.items() if k != "data_format"}
        outs = inner(i, a2, c)
        return [o.permute(0, 2, 3, 1) if o.dim() == 4 else o for o in outs]

    _REGISTRY.register(OnnxOperator(name, run, base.min_inputs, base.max_inputs, base.domain))


_wrap_nhwc("Conv", [0], [1])
_wrap_nhwc("FusedConv", [0, 3], [1])
for _n in ("MaxPool", "AveragePool", "GlobalAveragePool", "BatchNormalization"):
    _wrap_nhwc(_n, [0])


from . import registry_extra  # noqa: E402,F401  (registers the operators beyond the core set)
