"""Operator conformance matrix: every case builds a one-node graph, runs it through the public session API on the CPU
provider at O0 and O3, and compares with an independent PyTorch expression of the ONNX definition.  The reference keeps
one small test per operator and shape (crates/ronn-onnx/tests/test_operators.rs, crates/ronn-core/tests/ops_*.rs); this
is that list as a table."""
import math

import pytest
import torch
import torch.nn.functional as F

from ronn_b200 import Model, SessionOptions
from ronn_b200.core.types import DataType
from ronn_b200.graph.ir import GraphBuilder

G = torch.Generator().manual_seed(1234)


def rnd(*shape, lo=-2.0, hi=2.0):
    return torch.rand(*shape, generator=G) * (hi - lo) + lo


def run_node(op, inputs, attrs=None, n_out=1, consts=None, domain="", in_dtypes=None, level="O0"):
    """inputs: list of (name, tensor) run-time inputs; consts: list of (name, tensor) initializers (in input order the
    names are given by `order`)."""
    b = GraphBuilder()
    names = []
    for k, (name, t) in enumerate(inputs):
        dt = {torch.float32: DataType.F32, torch.int64: DataType.I64, torch.bool: DataType.BOOL,
              torch.int32: DataType.I32, torch.uint8: DataType.U8, torch.int8: DataType.I8}[t.dtype]
        b.add_input(name, list(t.shape), dt)
        names.append(name)
    for name, t in (consts or []):
        b.add_initializer(name, t)
        names.append(name)
    outs = [f"y{k}" for k in range(n_out)]
    for o in outs:
        b.add_output(o, [])
    b.add_op(op, names, outs, domain=domain, **(attrs or {}))
    sess = Model.from_graph(b.build()).create_session(SessionOptions().with_optimization_level(level))
    res = sess.run({n: t for n, t in inputs})
    return [res[o] for o in outs]


def check(got, want, atol=1e-5, rtol=1e-5):
    want = want if isinstance(want, (list, tuple)) else [want]
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert tuple(g.shape) == tuple(w.shape), (g.shape, w.shape)
        if w.is_floating_point():
            torch.testing.assert_close(g.float(), w.float(), atol=atol, rtol=rtol, equal_nan=True)
        else:
            assert torch.equal(g.to(w.dtype), w), (g, w)


SHAPES = [(7,), (3, 5), (2, 3, 4, 5)]

UNARY = {
    "Abs": (torch.abs, {}), "Neg": (torch.neg, {}), "Exp": (torch.exp, {}), "Sqrt": (torch.sqrt, {"pos": True}),
    "Log": (torch.log, {"pos": True}), "Reciprocal": (torch.reciprocal, {"pos": True}), "Relu": (torch.relu, {}),
    "Sigmoid": (torch.sigmoid, {}), "Tanh": (torch.tanh, {}), "Erf": (torch.erf, {}), "Sin": (torch.sin, {}),
    "Cos": (torch.cos, {}), "Floor": (torch.floor, {}), "Ceil": (torch.ceil, {}), "Round": (torch.round, {}),
    "Sign": (torch.sign, {}), "Softplus": (F.softplus, {}), "Softsign": (F.softsign, {}),
    "Identity": (lambda x: x, {}), "Mish": (F.mish, {}), "HardSwish": (F.hardswish, {}),
    "Gelu": (lambda x: F.gelu(x), {}), "SiLU": (F.silu, {"domain": "com.ronn"}), "Swish": (F.silu, {"domain": "com.ronn"}),
    "FastGelu": (lambda x: x * torch.sigmoid(1.702 * x), {"domain": "com.ronn"}),
}


@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("op", sorted(UNARY))
def test_unary(op, shape):
    fn, opt = UNARY[op]
    x = rnd(*shape, lo=0.1 if opt.get("pos") else -2.0)
    try:
        got = run_node(op, [("x", x)], domain=opt.get("domain", ""))
    except Exception as e:
        if opt.get("domain") and "not" in str(e).lower():
            pytest.skip(f"{op} is not registered under {opt['domain']}")
        raise
    check(got, fn(x), atol=opt.get("atol", 1e-5))


UNARY_ATTR = [
    ("LeakyRelu", {"alpha": 0.2}, lambda x: F.leaky_relu(x, 0.2)),
    ("LeakyRelu", {}, lambda x: F.leaky_relu(x, 0.01)),
    ("Elu", {"alpha": 1.5}, lambda x: F.elu(x, 1.5)),
    ("Celu", {"alpha": 2.0}, lambda x: F.celu(x, 2.0)),
    ("Selu", {}, F.selu),
    ("HardSigmoid", {"alpha": 0.25, "beta": 0.4}, lambda x: torch.clamp(0.25 * x + 0.4, 0, 1)),
    ("HardSigmoid", {}, lambda x: torch.clamp(0.2 * x + 0.5, 0, 1)),
    ("ThresholdedRelu", {"alpha": 0.7}, lambda x: torch.where(x > 0.7, x, torch.zeros_like(x))),
    ("Shrink", {"lambd": 0.5, "bias": 0.1}, lambda x: torch.where(x < -0.5, x + 0.1, torch.where(x > 0.5, x - 0.1, torch.zeros_like(x)))),
    ("Gelu", {"approximate": "tanh"}, lambda x: F.gelu(x, approximate="tanh")),
    ("Softmax", {"axis": -1}, lambda x: torch.softmax(x, -1)),
    ("Softmax", {"axis": 0}, lambda x: torch.softmax(x, 0)),
    ("LogSoftmax", {"axis": -1}, lambda x: torch.log_softmax(x, -1)),
    ("LogSoftmax", {"axis": 1}, lambda x: torch.log_softmax(x, 1)),
    ("Hardmax", {"axis": -1}, lambda x: F.one_hot(x.argmax(-1), x.shape[-1]).to(x.dtype)),
    ("LpNormalization", {"axis": -1, "p": 2}, lambda x: x / x.norm(dim=-1, keepdim=True)),
    ("LpNormalization", {"axis": 0, "p": 1}, lambda x: x / x.abs().sum(dim=0, keepdim=True)),
    ("Flatten", {"axis": 1}, lambda x: x.reshape(x.shape[0], -1)),
    ("Flatten", {"axis": 2}, lambda x: x.reshape(x.shape[0] * x.shape[1], -1)),
    ("Transpose", {"perm": [1, 0, 2]}, lambda x: x.permute(1, 0, 2)),
    ("Transpose", {}, lambda x: x.permute(2, 1, 0)),
    ("IsNaN", {}, torch.isnan),
    ("Not", {"bool_in": True}, torch.logical_not),
    ("Cast", {"to": 7}, lambda x: x.to(torch.int64)),
    ("Cast", {"to": 6}, lambda x: x.to(torch.int32)),
    ("Dropout", {}, lambda x: x),
    ("Trilu", {"upper": 1}, lambda x: torch.triu(x)),
    ("Trilu", {"upper": 0}, lambda x: torch.tril(x)),
    ("DepthToSpace", {"blocksize": 2, "shape": (1, 8, 2, 3)}, lambda x: F.pixel_shuffle(x, 2) if False else
     x.reshape(1, 2, 2, 2, 2, 3).permute(0, 3, 4, 1, 5, 2).reshape(1, 2, 4, 6)),
    ("SpaceToDepth", {"blocksize": 2, "shape": (1, 2, 4, 6)}, lambda x: x.reshape(1, 2, 2, 2, 3, 2).permute(0, 3, 5, 1, 2, 4).reshape(1, 8, 2, 3)),
    ("GlobalAveragePool", {"shape": (2, 3, 4, 5)}, lambda x: x.mean((2, 3), keepdim=True)),
    ("GlobalMaxPool", {"shape": (2, 3, 4, 5)}, lambda x: x.amax((2, 3), keepdim=True)),
    ("LRN", {"size": 3, "shape": (2, 5, 4, 4)}, lambda x: F.local_response_norm(x, 3, alpha=1e-4, beta=0.75, k=1.0)),
    ("Size", {}, lambda x: torch.tensor(x.numel())),
    ("Shape", {}, lambda x: torch.tensor(list(x.shape))),
    ("EyeLike", {"shape": (4, 6), "k": 1}, lambda x: torch.eye(4, 6).roll(1, 1).triu(1)),
]


@pytest.mark.parametrize("case", UNARY_ATTR, ids=lambda c: f"{c[0]}-{'-'.join(f'{k}{v}' for k, v in c[1].items() if k != 'shape')}")
def test_unary_with_attributes(case):
    op, attrs, fn = case
    attrs = dict(attrs)
    shape = attrs.pop("shape", (3, 4, 5))
    x = rnd(*shape)
    if attrs.pop("bool_in", False):
        x = x > 0
    if op == "IsNaN":
        x[0, 0, 0] = float("nan")
    check(run_node(op, [("x", x)], attrs), fn(x), atol=1e-5)


BINARY = {
    "Add": torch.add, "Sub": torch.sub, "Mul": torch.mul, "Div": torch.div, "Pow": lambda a, b: torch.pow(a.abs() + 0.1, b),
    "Max": torch.maximum, "Min": torch.minimum, "Greater": torch.gt, "Less": torch.lt, "GreaterOrEqual": torch.ge,
    "LessOrEqual": torch.le, "Equal": torch.eq, "PRelu": lambda a, b: torch.where(a >= 0, a, a * b),
}
PAIRS = [((3, 4), (3, 4)), ((2, 3, 4), (4,)), ((5, 1, 4), (1, 3, 1)), ((4,), ())]


@pytest.mark.parametrize("pair", PAIRS, ids=str)
@pytest.mark.parametrize("op", sorted(BINARY))
def test_binary_broadcasting(op, pair):
    a, b = rnd(*pair[0]), rnd(*pair[1]) if pair[1] else torch.tensor(0.7)
    if op == "Div":
        b = b.abs() + 0.5
    if op == "Pow":
        a = a.abs() + 0.1
        want = torch.pow(a, b)
    else:
        want = BINARY[op](a, b)
    if op == "Equal":
        b = b.clone()
        a.reshape(-1)[0] = float(b.reshape(-1)[0])
        want = torch.eq(a, b)
    check(run_node(op, [("a", a), ("b", b)]), want)


@pytest.mark.parametrize("op,fn", [("And", torch.logical_and), ("Or", torch.logical_or), ("Xor", torch.logical_xor)])
@pytest.mark.parametrize("pair", PAIRS[:3], ids=str)
def test_logical(op, fn, pair):
    a, b = rnd(*pair[0]) > 0, rnd(*pair[1]) > 0
    check(run_node(op, [("a", a), ("b", b)]), fn(a, b))


@pytest.mark.parametrize("fmod", [0, 1])
def test_mod(fmod):
    a, b = rnd(4, 5, lo=-7, hi=7), rnd(5, lo=1, hi=3)
    if fmod:
        check(run_node("Mod", [("a", a), ("b", b)], {"fmod": 1}), torch.fmod(a, b))
    else:
        ai, bi = a.to(torch.int64), b.to(torch.int64)
        check(run_node("Mod", [("a", ai), ("b", bi)]), torch.remainder(ai, bi))


@pytest.mark.parametrize("op,fn", [("Sum", lambda *t: sum(t)), ("Mean", lambda *t: sum(t) / len(t)),
                                   ("Max", lambda *t: torch.stack(torch.broadcast_tensors(*t)).amax(0)),
                                   ("Min", lambda *t: torch.stack(torch.broadcast_tensors(*t)).amin(0))])
@pytest.mark.parametrize("n", [1, 2, 4])
def test_variadic(op, fn, n):
    ts = [rnd(3, 4) if k % 2 == 0 else rnd(4) for k in range(n)]
    check(run_node(op, [(f"t{k}", t) for k, t in enumerate(ts)]), fn(*ts) if n > 1 or op not in ("Max", "Min") else ts[0])


REDUCE = {
    "ReduceSum": lambda x, d, k: x.sum(d, keepdim=k), "ReduceMean": lambda x, d, k: x.mean(d, keepdim=k),
    "ReduceMax": lambda x, d, k: x.amax(d, keepdim=k), "ReduceMin": lambda x, d, k: x.amin(d, keepdim=k),
    "ReduceProd": lambda x, d, k: torch.prod(x, d[0], keepdim=k) if len(d) == 1 else x.flatten().prod().reshape([1] * x.dim() if k else []),
    "ReduceL1": lambda x, d, k: x.abs().sum(d, keepdim=k), "ReduceL2": lambda x, d, k: x.pow(2).sum(d, keepdim=k).sqrt(),
    "ReduceLogSum": lambda x, d, k: x.sum(d, keepdim=k).log(),
    "ReduceLogSumExp": lambda x, d, k: torch.logsumexp(x, d, keepdim=k),
    "ReduceSumSquare": lambda x, d, k: x.pow(2).sum(d, keepdim=k),
}


@pytest.mark.parametrize("keep", [0, 1])
@pytest.mark.parametrize("axes", [(1,), (-1,), (0, 2), None], ids=str)
@pytest.mark.parametrize("op", sorted(REDUCE))
def test_reductions(op, axes, keep):
    x = rnd(2, 3, 4)
    if op == "ReduceLogSum":
        x = x.abs() + 0.1
    dims = list(axes) if axes is not None else [0, 1, 2]
    if op == "ReduceProd" and axes is not None and len(axes) > 1:
        pytest.skip("reference expression covers one axis or all")
    want = REDUCE[op](x, dims, bool(keep))
    attrs = {"keepdims": keep}
    consts = []
    if axes is not None:
        if op == "ReduceSum":
            consts = [("axes", torch.tensor(list(axes)))]          # opset 13: axes is an input
        else:
            attrs["axes"] = list(axes)
    check(run_node(op, [("x", x)], attrs, consts=consts), want, atol=1e-5)


@pytest.mark.parametrize("op,fn", [("ArgMax", torch.argmax), ("ArgMin", torch.argmin)])
@pytest.mark.parametrize("axis,keep", [(0, 1), (1, 0), (-1, 1)])
def test_arg_reductions(op, fn, axis, keep):
    x = rnd(4, 5, 6)
    check(run_node(op, [("x", x)], {"axis": axis, "keepdims": keep}), fn(x, dim=axis, keepdim=bool(keep)))


def test_matmul_family():
    a, b = rnd(2, 3, 4), rnd(4, 5)
    check(run_node("MatMul", [("a", a), ("b", b)]), a @ b)
    a4, b4 = rnd(2, 3, 4, 5), rnd(2, 3, 5, 6)
    check(run_node("MatMul", [("a", a4), ("b", b4)]), a4 @ b4)
    x, w, c = rnd(3, 4), rnd(5, 4), rnd(5)
    check(run_node("Gemm", [("x", x), ("w", w), ("c", c)], {"transB": 1, "alpha": 0.5, "beta": 2.0}), 0.5 * x @ w.t() + 2 * c)
    check(run_node("Gemm", [("x", x.t().contiguous()), ("w", w.t().contiguous())], {"transA": 1}), x @ w.t())
    check(run_node("Einsum", [("a", a), ("b", b)], {"equation": "bij,jk->bik"}), torch.einsum("bij,jk->bik", a, b))


@pytest.mark.parametrize("axis", [0, 1, -1])
def test_concat_split_roundtrip(axis):
    parts = [rnd(2, 3, 4), rnd(2, 3, 4), rnd(2, 3, 4)]
    cat = torch.cat(parts, dim=axis)
    check(run_node("Concat", [(f"p{k}", p) for k, p in enumerate(parts)], {"axis": axis}), cat)
    sizes = [parts[0].shape[axis]] * 3
    got = run_node("Split", [("x", cat)], {"axis": axis}, n_out=3, consts=[("s", torch.tensor(sizes))])
    check(got, parts)


SHAPE_CASES = [
    ("Reshape", [("x", (2, 3, 4))], [("s", torch.tensor([6, -1]))], {}, lambda x: x.reshape(6, 4)),
    ("Reshape", [("x", (2, 3, 4))], [("s", torch.tensor([0, -1]))], {}, lambda x: x.reshape(2, 12)),
    ("Squeeze", [("x", (2, 1, 4, 1))], [("a", torch.tensor([1, 3]))], {}, lambda x: x.reshape(2, 4)),
    ("Squeeze", [("x", (2, 1, 4, 1))], [], {}, lambda x: x.reshape(2, 4)),
    ("Unsqueeze", [("x", (2, 4))], [("a", torch.tensor([0, 3]))], {}, lambda x: x.reshape(1, 2, 4, 1)),
    ("Tile", [("x", (2, 3))], [("r", torch.tensor([2, 3]))], {}, lambda x: x.repeat(2, 3)),
    ("Expand", [("x", (3, 1))], [("s", torch.tensor([2, 3, 4]))], {}, lambda x: x.expand(2, 3, 4)),
    ("Slice", [("x", (4, 6))], [("st", torch.tensor([1, 0])), ("en", torch.tensor([3, 6])), ("ax", torch.tensor([0, 1])),
                                ("sp", torch.tensor([1, 2]))], {}, lambda x: x[1:3, 0:6:2]),
    ("Slice", [("x", (4, 6))], [("st", torch.tensor([-1])), ("en", torch.tensor([-5])), ("ax", torch.tensor([1])),
                                ("sp", torch.tensor([-1]))], {}, lambda x: x[:, [5, 4, 3, 2]]),
    ("Gather", [("x", (5, 4))], [("i", torch.tensor([[0, 2], [4, 1]]))], {"axis": 0}, lambda x: x[torch.tensor([[0, 2], [4, 1]])]),
    ("Gather", [("x", (5, 4))], [("i", torch.tensor([3, -1]))], {"axis": 1}, lambda x: x[:, [3, 3]]),
    ("GatherElements", [("x", (3, 4))], [("i", torch.tensor([[0, 1, 2, 3], [3, 2, 1, 0], [1, 1, 1, 1]]))], {"axis": 1},
     lambda x: torch.gather(x, 1, torch.tensor([[0, 1, 2, 3], [3, 2, 1, 0], [1, 1, 1, 1]]))),
    ("CumSum", [("x", (3, 4))], [("a", torch.tensor(1))], {}, lambda x: x.cumsum(1)),
    ("CumSum", [("x", (3, 4))], [("a", torch.tensor(0))], {"reverse": 1}, lambda x: x.flip(0).cumsum(0).flip(0)),
    ("Pad", [("x", (2, 3))], [("p", torch.tensor([1, 0, 0, 2])), ("v", torch.tensor(1.5))], {}, lambda x: F.pad(x, (0, 2, 1, 0), value=1.5)),
    ("Clip", [("x", (3, 4))], [("lo", torch.tensor(-0.5)), ("hi", torch.tensor(0.8))], {}, lambda x: x.clamp(-0.5, 0.8)),
    ("Where", [("x", (3, 4))], [], {"cond": True}, None),
    ("OneHot", [], [("i", torch.tensor([0, 2, 1])), ("d", torch.tensor(4)), ("v", torch.tensor([0.0, 1.0]))], {"axis": -1},
     lambda: F.one_hot(torch.tensor([0, 2, 1]), 4).float()),
    ("Range", [], [("s", torch.tensor(1.0)), ("l", torch.tensor(7.0)), ("d", torch.tensor(1.5))], {}, lambda: torch.arange(1.0, 7.0, 1.5)),
    ("ConstantOfShape", [], [("s", torch.tensor([2, 3]))], {"value": torch.tensor([2.5])}, lambda: torch.full((2, 3), 2.5)),
    ("NonZero", [("x", (3, 4))], [], {}, lambda x: torch.nonzero(x > 99).t() if False else torch.nonzero(x).t()),
]


@pytest.mark.parametrize("case", SHAPE_CASES, ids=lambda c: f"{c[0]}-{len(c[2])}c-{'-'.join(c[3])}")
def test_shape_and_index_operators(case):
    op, ins, consts, attrs, fn = case
    attrs = dict(attrs)
    inputs = [(n, rnd(*s)) for n, s in ins]
    if op == "Where":
        attrs.pop("cond")
        x = inputs[0][1]
        c, y = x > 0, rnd(*x.shape)
        check(run_node("Where", [("c", c), ("x", x), ("y", y)]), torch.where(c, x, y))
        return
    want = fn(*[t for _, t in inputs])
    check(run_node(op, inputs, attrs, consts=consts), want)


@pytest.mark.parametrize("largest", [1, 0])
def test_topk(largest):
    x = rnd(3, 10)
    v, i = torch.topk(x, 4, dim=-1, largest=bool(largest))
    got = run_node("TopK", [("x", x)], {"axis": -1, "largest": largest}, n_out=2, consts=[("k", torch.tensor([4]))])
    check(got, [v, i])


NORM_CASES = [
    ("LayerNormalization", (4, 6, 8), {"axis": -1, "epsilon": 1e-5}, lambda x, g, b: F.layer_norm(x, (8,), g, b, 1e-5), (8,)),
    ("InstanceNormalization", (2, 3, 5, 5), {"epsilon": 1e-5}, lambda x, g, b: F.instance_norm(x, weight=g, bias=b, eps=1e-5), (3,)),
    ("BatchNormalization", (2, 3, 4, 4), {"epsilon": 1e-5}, None, (3,)),
    ("GroupNormalization", (2, 6, 4, 4), {"num_groups": 3, "epsilon": 1e-5}, lambda x, g, b: F.group_norm(x, 3, g, b, 1e-5), (6,)),
]


@pytest.mark.parametrize("case", NORM_CASES, ids=lambda c: c[0])
def test_normalisations(case):
    op, shape, attrs, fn, pshape = case
    x, g, b = rnd(*shape), rnd(*pshape), rnd(*pshape)
    if op == "BatchNormalization":
        m, v = rnd(*pshape), rnd(*pshape).abs() + 0.5
        got = run_node(op, [("x", x)], attrs, consts=[("g", g), ("b", b), ("m", m), ("v", v)])
        check(got, F.batch_norm(x, m, v, g, b, False, 0.0, 1e-5), atol=1e-4)
        return
    check(run_node(op, [("x", x)], attrs, consts=[("g", g), ("b", b)]), fn(x, g, b), atol=1e-4)


CONV_CASES = [
    ({"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]}, (2, 3, 8, 8), (4, 3, 3, 3), dict(padding=1)),
    ({"kernel_shape": [3, 3], "strides": [2, 2]}, (1, 3, 9, 9), (5, 3, 3, 3), dict(stride=2)),
    ({"kernel_shape": [1, 1]}, (2, 4, 5, 5), (6, 4, 1, 1), {}),
    ({"kernel_shape": [3, 3], "group": 2, "pads": [1, 1, 1, 1]}, (1, 4, 6, 6), (6, 2, 3, 3), dict(padding=1, groups=2)),
    ({"kernel_shape": [3, 3], "dilations": [2, 2], "pads": [2, 2, 2, 2]}, (1, 2, 8, 8), (3, 2, 3, 3), dict(padding=2, dilation=2)),
]


@pytest.mark.parametrize("level", ["O0", "O3"])
@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c[0].items()))
def test_convolutions(case, level):
    attrs, xs, ws, kw = case
    x, w, bias = rnd(*xs), rnd(*ws), rnd(ws[0])
    check(run_node("Conv", [("x", x)], attrs, consts=[("w", w), ("b", bias)], level=level), F.conv2d(x, w, bias, **kw), atol=1e-4)


POOL_CASES = [
    ("MaxPool", {"kernel_shape": [2, 2], "strides": [2, 2]}, lambda x: F.max_pool2d(x, 2, 2)),
    ("MaxPool", {"kernel_shape": [3, 3], "strides": [2, 2], "pads": [1, 1, 1, 1]}, lambda x: F.max_pool2d(x, 3, 2, 1)),
    ("MaxPool", {"kernel_shape": [3, 3], "strides": [2, 2], "ceil_mode": 1}, lambda x: F.max_pool2d(x, 3, 2, ceil_mode=True)),
    ("AveragePool", {"kernel_shape": [2, 2], "strides": [2, 2]}, lambda x: F.avg_pool2d(x, 2, 2)),
    ("AveragePool", {"kernel_shape": [3, 3], "strides": [1, 1], "pads": [1, 1, 1, 1], "count_include_pad": 1},
     lambda x: F.avg_pool2d(x, 3, 1, 1, count_include_pad=True)),
    ("AveragePool", {"kernel_shape": [3, 3], "strides": [1, 1], "pads": [1, 1, 1, 1]},
     lambda x: F.avg_pool2d(x, 3, 1, 1, count_include_pad=False)),
]


@pytest.mark.parametrize("case", POOL_CASES, ids=lambda c: c[0] + "-" + "-".join(f"{k}{v}" for k, v in c[1].items()))
def test_pooling(case):
    op, attrs, fn = case
    x = rnd(2, 3, 9, 9)
    check(run_node(op, [("x", x)], attrs), fn(x), atol=1e-5)


def test_quantize_dequantize_roundtrip():
    x = rnd(4, 6, lo=-3, hi=3)
    scale, zp = torch.tensor(0.05), torch.tensor(3, dtype=torch.uint8)
    q = run_node("QuantizeLinear", [("x", x)], consts=[("s", scale), ("z", zp)])[0]
    want_q = torch.clamp(torch.round(x / 0.05) + 3, 0, 255).to(torch.uint8)
    assert torch.equal(q, want_q)
    d = run_node("DequantizeLinear", [("q", q)], consts=[("s", scale), ("z", zp)])[0]
    check([d], (want_q.float() - 3) * 0.05)
    inside = (x / 0.05 + 3 >= 0) & (x / 0.05 + 3 <= 255)                # values that do not saturate round-trip within half a step
    assert float((d - x)[inside].abs().max()) <= 0.05 / 2 + 1e-6


@pytest.mark.parametrize("op", ["Add", "Mul", "Relu", "MatMul", "Softmax", "LayerNormalization", "Concat"])
def test_results_do_not_depend_on_the_optimisation_level(op):
    x, y = rnd(4, 8), rnd(4, 8)
    cases = {"Add": ([("a", x), ("b", y)], {}, []), "Mul": ([("a", x), ("b", y)], {}, []), "Relu": ([("a", x)], {}, []),
             "MatMul": ([("a", x)], {}, [("w", rnd(8, 3))]), "Softmax": ([("a", x)], {"axis": -1}, []),
             "LayerNormalization": ([("a", x)], {"axis": -1}, [("g", rnd(8)), ("b", rnd(8))]),
             "Concat": ([("a", x), ("b", y)], {"axis": 0}, [])}
    ins, attrs, consts = cases[op]
    ref = run_node(op, ins, attrs, consts=consts, level="O0")
    for lvl in ("O1", "O2", "O3"):
        check(run_node(op, ins, attrs, consts=consts, level=lvl), ref, atol=1e-5)


def test_math_constants_are_exact_where_they_must_be():
    x = torch.tensor([0.0, 1.0, -1.0, math.pi / 2])
    check(run_node("Sin", [("x", x)]), torch.sin(x))
    check(run_node("Exp", [("x", torch.tensor([0.0]))]), torch.tensor([1.0]), atol=0, rtol=0)
    check(run_node("Relu", [("x", torch.tensor([-0.0, 0.0, 3.0]))]), torch.tensor([0.0, 0.0, 3.0]), atol=0, rtol=0)


@pytest.mark.parametrize("heads,kv_heads,d", [(4, 4, 8), (4, 2, 16)])
@pytest.mark.parametrize("level", ["O0", "O3"])
def test_paged_attention_operator(heads, kv_heads, d, level):
    """com.ronn::PagedAttention: every query row attends to the first context_lens[row] keys of the cache blocks its
    table row lists; an empty context gives a zero row, table_rows lets rows share a table row, a custom scale is
    honoured."""
    lens = [5, 16, 0, 33]
    rows, max_blocks = len(lens), 3
    nblocks = 7
    kc, vc = rnd(nblocks, kv_heads, 16, d), rnd(nblocks, kv_heads, 16, d)
    bt = torch.tensor([[1, 0, 0], [2, 0, 0], [0, 0, 0], [3, 4, 5]], dtype=torch.int32)
    q = rnd(rows, heads * d)
    ctx = torch.tensor(lens, dtype=torch.int32)

    def want(q, rows_of, scale):
        out = torch.zeros(q.shape[0], heads * d)
        for r in range(q.shape[0]):
            n = int(ctx[r])
            if n == 0:
                continue
            tb = bt[rows_of[r]]
            k = torch.stack([kc[int(tb[t // 16]), :, t % 16] for t in range(n)])      # [n, kv, d]
            v = torch.stack([vc[int(tb[t // 16]), :, t % 16] for t in range(n)])
            k, v = k.repeat_interleave(heads // kv_heads, 1), v.repeat_interleave(heads // kv_heads, 1)
            s = torch.einsum("hd,nhd->hn", q[r].view(heads, d), k) * scale
            out[r] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v).reshape(-1)
        return out
    ins = [("q", q), ("kc", kc), ("vc", vc), ("bt", bt), ("ctx", ctx)]
    got = run_node("PagedAttention", ins, {"num_heads": heads, "kv_heads": kv_heads}, domain="com.ronn", level=level)[0]
    torch.testing.assert_close(got, want(q, list(range(rows)), 1 / math.sqrt(d)), atol=1e-5, rtol=1e-4)
    assert float(got[2].abs().max()) == 0.0
    shared = torch.tensor([3, 3, 3, 3], dtype=torch.int32)
    got = run_node("PagedAttention", ins + [("rows_of", shared)], {"num_heads": heads, "kv_heads": kv_heads, "scale": 0.5},
                   domain="com.ronn", level=level)[0]
    torch.testing.assert_close(got, want(q, [3, 3, 3, 3], 0.5), atol=1e-5, rtol=1e-4)
