"""Operator matrix on the GPU provider (bf16 and fp16, sm_100a kernels where the provider has one, library operators
elsewhere): every case is a one-node graph run through the public session API and compared with the fp32 CPU session
of the same graph."""
import pytest
import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.graph.ir import GraphBuilder

pytestmark = pytest.mark.gpu

G = torch.Generator().manual_seed(99)


def rnd(*shape, lo=-2.0, hi=2.0):
    return torch.rand(*shape, generator=G) * (hi - lo) + lo


def both(op, inputs, attrs=None, consts=None, dtype="bf16", level="O3", domain=""):
    b = GraphBuilder()
    names = []
    for name, t in inputs:
        b.add_input(name, list(t.shape))
        names.append(name)
    for name, t in (consts or []):
        b.add_initializer(name, t)
        names.append(name)
    b.add_output("y", [])
    b.add_op(op, names, ["y"], domain=domain, **(attrs or {}))
    g = b.build()
    feeds = {n: t for n, t in inputs}
    want = Model.from_graph(g).create_session(SessionOptions().with_optimization_level("O0")).run(feeds)["y"]
    sess = Model.from_graph(g).create_session(SessionOptions().with_provider("gpu").with_optimization_level(level).with_dtype(dtype))
    got = sess.run(feeds)["y"]
    assert got.device.type == "cuda"
    return got.float().cpu(), want.float()


TOL = {"bf16": dict(atol=4e-2, rtol=4e-2), "fp16": dict(atol=6e-3, rtol=6e-3)}
SHAPES = [(8, 256), (3, 5, 64), (1000,), (64, 1024)]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("op,attrs", [("Relu", {}), ("Sigmoid", {}), ("Tanh", {}), ("Gelu", {"approximate": "tanh"}), ("Gelu", {}),
                                      ("Neg", {}), ("Abs", {}), ("Exp", {}), ("Sqrt", {}), ("Erf", {})],
                         ids=lambda v: v if isinstance(v, str) else "-".join(map(str, v.values())))
def test_unary_on_the_gpu_provider(op, attrs, shape, dtype):
    x = rnd(*shape, lo=0.1 if op == "Sqrt" else -2.0)
    got, want = both(op, [("x", x)], attrs, dtype=dtype)
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("pair", [((8, 256), (8, 256)), ((4, 6, 128), (128,)), ((16, 64), ()), ((5, 1, 64), (1, 7, 64))], ids=str)
@pytest.mark.parametrize("op", ["Add", "Sub", "Mul", "Div"])
def test_binary_on_the_gpu_provider(op, pair, dtype):
    a = rnd(*pair[0])
    b = rnd(*pair[1]) if pair[1] else torch.tensor(1.3)
    if op == "Div":
        b = b.abs() + 0.5
    got, want = both(op, [("a", a), ("b", b)], dtype=dtype)
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("shape,axis", [((16, 512), -1), ((4, 8, 128), -1), ((4, 8, 128), 1), ((3000, 64), -1), ((7, 1000), -1)], ids=str)
def test_softmax_on_the_gpu_provider(shape, axis, dtype):
    got, want = both("Softmax", [("x", rnd(*shape, lo=-4, hi=4))], {"axis": axis}, dtype=dtype)
    torch.testing.assert_close(got, want, atol=2e-2 if dtype == "bf16" else 2e-3, rtol=3e-2)


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("rows,h", [(4, 768), (256, 1024), (37, 2560), (4096, 256)])
@pytest.mark.parametrize("op", ["LayerNormalization", "RMSNorm"])
def test_norms_on_the_gpu_provider(op, rows, h, dtype):
    consts = [("g", rnd(h, lo=0.5, hi=1.5))] + ([("b", rnd(h))] if op == "LayerNormalization" else [])
    got, want = both(op, [("x", rnd(rows, h))], {"axis": -1, "epsilon": 1e-5} if op == "LayerNormalization" else {"epsilon": 1e-5},
                     consts=consts, dtype=dtype, domain="" if op == "LayerNormalization" else "com.ronn")
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("m,k,n", [(1, 64, 32), (7, 256, 136), (128, 1024, 512), (300, 72, 1000), (64, 2048, 64)])
@pytest.mark.parametrize("form", ["MatMul", "Gemm", "Gemm-transB"])
def test_linear_layers_on_the_gpu_provider(form, m, k, n, dtype):
    x, w, c = rnd(m, k, lo=-1, hi=1), rnd(k, n, lo=-0.1, hi=0.1), rnd(n)
    if form == "MatMul":
        got, want = both("MatMul", [("x", x)], consts=[("w", w)], dtype=dtype)
    elif form == "Gemm":
        got, want = both("Gemm", [("x", x)], consts=[("w", w), ("c", c)], dtype=dtype)
    else:
        got, want = both("Gemm", [("x", x)], {"transB": 1}, consts=[("w", w.t().contiguous()), ("c", c)], dtype=dtype)
    torch.testing.assert_close(got, want, atol=(6e-2 if dtype == "bf16" else 1e-2) * (k / 256) ** 0.5 + 1e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_gather_rows_on_the_gpu_provider(dtype):
    table = rnd(500, 256)
    idx = torch.randint(0, 500, (4, 9), generator=G)
    b = GraphBuilder().add_input("i", [4, 9]).add_output("y", [])
    from ronn_b200.core.types import DataType
    b.graph.inputs[0].data_type = DataType.I64
    b.add_initializer("t", table).add_op("Gather", ["t", "i"], ["y"], axis=0)
    g = b.build()
    want = Model.from_graph(g).create_session(SessionOptions().with_optimization_level("O0")).run({"i": idx})["y"]
    got = Model.from_graph(g).create_session(SessionOptions().with_provider("gpu").with_dtype(dtype)).run({"i": idx})["y"]
    torch.testing.assert_close(got.float().cpu(), want, **TOL[dtype])
