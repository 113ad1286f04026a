"""Operators beyond the reference's 39: ONNX semantics checked against hand-computed values or a direct formula."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from ronn_b200.api.errors import InvalidAttribute
from ronn_b200.onnx.registry import default_registry

R = default_registry()


def ex(op, inputs, **attrs):
    return R.get(op).execute(inputs, attrs)


def t(*v, dtype=torch.float32):
    return torch.tensor(v, dtype=dtype)


def test_elementwise_family():
    x = t(-2.0, -0.5, 0.0, 0.5, 2.0)
    torch.testing.assert_close(ex("HardSwish", [x])[0], x * torch.clamp(x / 6 + 0.5, 0, 1))
    torch.testing.assert_close(ex("Mish", [x])[0], x * torch.tanh(torch.log1p(torch.exp(x))))
    torch.testing.assert_close(ex("Selu", [x])[0], F.selu(x))
    torch.testing.assert_close(ex("Celu", [x], alpha=2.0)[0], F.celu(x, 2.0))
    torch.testing.assert_close(ex("ThresholdedRelu", [x], alpha=0.4)[0], t(0, 0, 0, 0.5, 2.0))
    torch.testing.assert_close(ex("Shrink", [x], lambd=1.0, bias=0.5)[0], t(-1.5, 0, 0, 0, 1.5))
    torch.testing.assert_close(ex("PRelu", [x, t(0.1)])[0], t(-0.2, -0.05, 0, 0.5, 2.0))
    torch.testing.assert_close(ex("Round", [t(0.5, 1.5, 2.5, -0.5)])[0], t(0.0, 2.0, 2.0, -0.0))
    assert ex("IsNaN", [t(1.0, float("nan"))])[0].tolist() == [False, True]
    inf = t(float("inf"), -float("inf"), 1.0)
    assert ex("IsInf", [inf])[0].tolist() == [True, True, False]
    assert ex("IsInf", [inf], detect_negative=0)[0].tolist() == [True, False, False]
    assert ex("Mod", [t(-7, 7, dtype=torch.int64), t(3, -3, dtype=torch.int64)])[0].tolist() == [2, -2]
    torch.testing.assert_close(ex("Mod", [t(-7.0, 7.0), t(3.0, -3.0)], fmod=1)[0], t(-1.0, 1.0))
    torch.testing.assert_close(ex("Mean", [t(1.0, 2.0), t(3.0, 4.0), t(5.0, 9.0)])[0], t(3.0, 5.0))
    assert ex("Hardmax", [t([1.0, 3.0, 2.0], [5.0, 5.0, 1.0])], axis=1)[0].tolist() == [[0, 1, 0], [1, 0, 0]]


def test_reductions_cumsum_topk():
    x = torch.arange(1.0, 7.0).reshape(2, 3)
    torch.testing.assert_close(ex("ReduceL1", [-x], axes=[1], keepdims=0)[0], t(6.0, 15.0))
    torch.testing.assert_close(ex("ReduceSumSquare", [x], axes=[0])[0], t([17.0, 29.0, 45.0]))
    torch.testing.assert_close(ex("ReduceLogSumExp", [x, t(1, dtype=torch.int64)], keepdims=0)[0], torch.logsumexp(x, 1))
    torch.testing.assert_close(ex("ReduceLogSum", [x], axes=[1], keepdims=0)[0], x.sum(1).log())
    ax = t(1, dtype=torch.int64)
    assert ex("CumSum", [x, ax])[0].tolist() == [[1, 3, 6], [4, 9, 15]]
    assert ex("CumSum", [x, ax], exclusive=1)[0].tolist() == [[0, 1, 3], [0, 4, 9]]
    assert ex("CumSum", [x, ax], reverse=1)[0].tolist() == [[6, 5, 3], [15, 11, 6]]
    assert ex("CumSum", [x, ax], reverse=1, exclusive=1)[0].tolist() == [[5, 3, 0], [11, 6, 0]]
    v, i = ex("TopK", [t([3.0, 1.0, 4.0, 1.5]), t(2, dtype=torch.int64)], axis=-1)
    assert v.tolist() == [[4.0, 3.0]] and i.tolist() == [[2, 0]] and i.dtype == torch.int64
    v, i = ex("TopK", [t([3.0, 1.0, 4.0, 1.5]), t(2, dtype=torch.int64)], largest=0)
    assert v.tolist() == [[1.0, 1.5]] and i.tolist() == [[1, 3]]
    torch.testing.assert_close(ex("LpNormalization", [t([3.0, 4.0])], axis=1, p=2)[0], t([0.6, 0.8]))
    torch.testing.assert_close(ex("LpNormalization", [t([3.0, -1.0])], axis=1, p=1)[0], t([0.75, -0.25]))


def test_normalisation_and_convolution_family():
    torch.manual_seed(0)
    x = torch.randn(2, 6, 5, 5)
    g, b = torch.randn(6), torch.randn(6)
    mean, var = x.mean((2, 3), keepdim=True), x.var((2, 3), unbiased=False, keepdim=True)
    ref = (x - mean) / torch.sqrt(var + 1e-5) * g.view(1, 6, 1, 1) + b.view(1, 6, 1, 1)
    torch.testing.assert_close(ex("InstanceNormalization", [x, g, b])[0], ref, atol=1e-5, rtol=1e-5)
    xg = x.reshape(2, 3, 2 * 25)
    refg = ((xg - xg.mean(2, keepdim=True)) / torch.sqrt(xg.var(2, unbiased=False, keepdim=True) + 1e-5)).reshape(x.shape)
    refg = refg * g.view(1, 6, 1, 1) + b.view(1, 6, 1, 1)
    torch.testing.assert_close(ex("GroupNormalization", [x, g, b], num_groups=3)[0], refg, atol=1e-5, rtol=1e-5)
    # one scale per group (the older form of the operator)
    gg, bg = t(2.0, 3.0, 4.0), t(0.5, 0.0, -0.5)
    per_group = ex("GroupNormalization", [x, gg, bg], num_groups=3)[0]
    torch.testing.assert_close(per_group, ex("GroupNormalization", [x, gg.repeat_interleave(2), bg.repeat_interleave(2)],
                                             num_groups=3)[0])
    w = torch.randn(6, 4, 3, 3)
    y = ex("ConvTranspose", [x, w, torch.randn(4)], strides=[2, 2], pads=[1, 1, 1, 1], output_padding=[1, 1])[0]
    assert y.shape == (2, 4, 10, 10)
    # transposed convolution is the adjoint of convolution: <conv(u), x> == <u, convT(x)>
    u = torch.randn(2, 4, 10, 10)
    yt = ex("ConvTranspose", [x, w], strides=[2, 2], pads=[1, 1, 1, 1], output_padding=[1, 1])[0]
    lhs = (F.conv2d(u, w, stride=2, padding=1) * x).sum()
    torch.testing.assert_close(lhs, (u * yt).sum(), atol=1e-3, rtol=1e-4)
    with pytest.raises(InvalidAttribute):
        ex("ConvTranspose", [x, w], pads=[0, 0, 1, 1])
    lr = ex("LRN", [x], size=3)[0]
    sq = F.pad(x.pow(2), (0, 0, 0, 0, 1, 1)).unfold(1, 3, 1).sum(-1)
    torch.testing.assert_close(lr, x / (1.0 + 1e-4 / 3 * sq).pow(0.75), atol=1e-5, rtol=1e-5)


def test_depth_space_resize():
    x = torch.arange(2 * 8 * 2 * 3, dtype=torch.float32).reshape(2, 8, 2, 3)
    dcr = ex("DepthToSpace", [x], blocksize=2)[0]
    crd = ex("DepthToSpace", [x], blocksize=2, mode="CRD")[0]
    assert dcr.shape == crd.shape == (2, 2, 4, 6)
    # DCR: out[n, c, h*2+i, w*2+j] = x[n, (i*2+j)*C' + c, h, w];  CRD: x[n, c*4 + i*2 + j, h, w]
    assert dcr[1, 1, 3, 4] == x[1, (1 * 2 + 0) * 2 + 1, 1, 2] and crd[1, 1, 3, 4] == x[1, 1 * 4 + 1 * 2 + 0, 1, 2]
    back = ex("SpaceToDepth", [dcr], blocksize=2)[0]
    torch.testing.assert_close(back, x)
    img = torch.arange(4.0).reshape(1, 1, 2, 2)
    up = ex("Resize", [img, None, t(1.0, 1.0, 2.0, 2.0)], mode="nearest", coordinate_transformation_mode="asymmetric")[0]
    assert up.tolist() == [[[[0, 0, 1, 1], [0, 0, 1, 1], [2, 2, 3, 3], [2, 2, 3, 3]]]]
    lin = ex("Resize", [img, None, None, t(1, 1, 4, 4, dtype=torch.int64)], mode="linear")[0]
    torch.testing.assert_close(lin, F.interpolate(img, size=(4, 4), mode="bilinear", align_corners=False))


def test_indexing_family():
    x = t([1.0, 2.0], [3.0, 4.0])
    idx = t([0, 0], [1, 0], dtype=torch.int64)
    assert ex("GatherElements", [x, idx], axis=1)[0].tolist() == [[1, 1], [4, 3]]
    assert ex("GatherElements", [x, t([-1, 0], dtype=torch.int64)], axis=0)[0].tolist() == [[3, 2]]
    base = torch.zeros(3, 3)
    upd = t([1.0, 1.1, 1.2], [2.0, 2.1, 2.2])
    sidx = t([1, 0, 2], [0, 2, 1], dtype=torch.int64)
    got = ex("ScatterElements", [base, sidx, upd], axis=0)[0]
    assert torch.allclose(got, t([2.0, 1.1, 0.0], [1.0, 0.0, 2.2], [0.0, 2.1, 1.2]))
    acc = ex("ScatterElements", [torch.ones(1, 3), t([0, 0, 2], dtype=torch.int64).reshape(1, 3), t([1.0, 2.0, 3.0])],
             axis=1, reduction="add")[0]
    assert acc.tolist() == [[4.0, 1.0, 4.0]]
    data = torch.arange(8.0).reshape(2, 2, 2)
    assert ex("GatherND", [data, t([0, 1], [1, 0], dtype=torch.int64)])[0].tolist() == [[2, 3], [4, 5]]
    assert ex("GatherND", [data, t([1, 1, 0], dtype=torch.int64)])[0].tolist() == [6]
    s = ex("ScatterND", [torch.arange(1.0, 9.0), t([4], [3], [1], [7], dtype=torch.int64), t(9.0, 10.0, 11.0, 12.0)])[0]
    assert s.tolist() == [1, 11, 3, 10, 9, 6, 7, 12]
    s = ex("ScatterND", [torch.zeros(4), t([1], [1], dtype=torch.int64), t(2.0, 3.0)], reduction="add")[0]
    assert s.tolist() == [0, 5, 0, 0]
    oh = ex("OneHot", [t(0, 2, -1, 5, dtype=torch.int64), t(3, dtype=torch.int64), t(0.0, 1.0)])[0]
    assert oh.tolist() == [[1, 0, 0], [0, 0, 1], [0, 0, 1], [0, 0, 0]]          # -1 wraps, 5 is out of range
    oh0 = ex("OneHot", [t(0, 2, dtype=torch.int64), t(3, dtype=torch.int64), t(-1.0, 7.0)], axis=0)[0]
    assert oh0.tolist() == [[7, -1], [-1, -1], [-1, 7]]
    nz = ex("NonZero", [t([1.0, 0.0], [0.0, 2.0])])[0]
    assert nz.tolist() == [[0, 1], [0, 1]] and nz.dtype == torch.int64
    m = torch.arange(1.0, 10.0).reshape(3, 3)
    assert ex("Trilu", [m], upper=0)[0].tolist() == [[1, 0, 0], [4, 5, 0], [7, 8, 9]]
    assert ex("Trilu", [m, t(1, dtype=torch.int64)])[0].tolist() == [[0, 2, 3], [0, 0, 6], [0, 0, 0]]
    assert ex("Size", [m])[0].item() == 9
    assert ex("EyeLike", [torch.zeros(2, 3)], k=1)[0].tolist() == [[0, 1, 0], [0, 0, 1]]
    assert ex("EyeLike", [torch.zeros(3, 2)])[0].tolist() == [[1, 0], [0, 1], [0, 0]]
    a_, b_ = torch.randn(2, 3, 4), torch.randn(2, 4, 5)
    torch.testing.assert_close(ex("Einsum", [a_, b_], equation="bij,bjk->bik")[0], a_ @ b_)


def test_quantize_dequantize_linear():
    x = t(-1.0, 0.0, 0.26, 1.0, 300.0)
    q = ex("QuantizeLinear", [x, t(0.5), t(128, dtype=torch.uint8)])[0]
    assert q.dtype == torch.uint8 and q.tolist() == [126, 128, 129, 130, 255]          # 0.52 -> round half to even
    d = ex("DequantizeLinear", [q, t(0.5), t(128, dtype=torch.uint8)])[0]
    torch.testing.assert_close(d, t(-1.0, 0.0, 0.5, 1.0, 63.5))
    w = t([1.0, -2.0], [30.0, 40.0])
    qs = ex("QuantizeLinear", [w, t(0.5, 10.0), t(0, 0, dtype=torch.int8)], axis=0)[0]
    assert qs.dtype == torch.int8 and qs.tolist() == [[2, -4], [3, 4]]
    torch.testing.assert_close(ex("DequantizeLinear", [qs, t(0.5, 10.0)], axis=0)[0], w)


def test_registry_size_and_session_use():
    assert len(R) >= 130
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.core.types import DataType
    from ronn_b200.graph.ir import GraphBuilder
    b = GraphBuilder().add_input("x", [1, 4, 2, 2], DataType.F32).add_output("y", [1, 1, 4, 4], DataType.F32)
    b.add_op("HardSwish", ["x"], ["h"]).add_op("DepthToSpace", ["h"], ["y"], blocksize=2)
    model = Model.from_bytes(Model.from_graph(b.build()).to_bytes())           # through the ONNX codec
    x = torch.randn(1, 4, 2, 2)
    for level in ("O0", "O3"):
        y = model.create_session(SessionOptions().with_optimization_level(level)).run({"x": x})["y"]
        torch.testing.assert_close(y, ex("DepthToSpace", [x * torch.clamp(x / 6 + 0.5, 0, 1)], blocksize=2)[0])


def test_integer_matmul_family():
    torch.manual_seed(0)
    a = torch.randint(0, 256, (3, 5), dtype=torch.uint8)
    b = torch.randint(-128, 128, (5, 4), dtype=torch.int8)
    az, bz = t(7, dtype=torch.uint8), t(1, -2, 3, 0, dtype=torch.int8)
    got = ex("MatMulInteger", [a, b, az, bz])[0]
    want = (a.to(torch.int64) - 7) @ (b.to(torch.int64) - bz.to(torch.int64).reshape(1, -1))
    assert got.dtype == torch.int32 and torch.equal(got.to(torch.int64), want)
    assert torch.equal(ex("MatMulInteger", [a, b])[0].to(torch.int64), a.to(torch.int64) @ b.to(torch.int64))
    x = t([0.0, 2.0, -3.0, -2.5], [1.34, 0.48, 7.0, -0.5])
    y, scale, zp = ex("DynamicQuantizeLinear", [x])
    assert y.dtype == torch.uint8 and zp.dtype == torch.uint8 and abs(scale.item() - 10.0 / 255) < 1e-7 and zp.item() == 76
    torch.testing.assert_close((y.float() - zp.float()) * scale, x, atol=scale.item() / 2 + 1e-6, rtol=0)
    # QLinearMatMul: dequantise, multiply, requantise
    sa, sb, sy = t(0.02), t(0.05), t(0.1)
    za, zb, zy = t(128, dtype=torch.uint8), t(0, dtype=torch.int8), t(3, dtype=torch.uint8)
    q = ex("QLinearMatMul", [a, sa, za, b, sb, zb, sy, zy])[0]
    real = ((a.float() - 128) * 0.02) @ (b.float() * 0.05)
    assert q.dtype == torch.uint8
    assert (q.float() - torch.clamp(torch.round(real / 0.1) + 3, 0, 255)).abs().max() <= 1       # ties may fall either way


def test_integer_convolutions():
    torch.manual_seed(1)
    x = torch.randint(0, 256, (1, 2, 5, 5), dtype=torch.uint8)
    w = torch.randint(-128, 128, (3, 2, 3, 3), dtype=torch.int8)
    xz, wz = t(10, dtype=torch.uint8), t(1, 0, -1, dtype=torch.int8)
    got = ex("ConvInteger", [x, w, xz, wz], pads=[1, 1, 1, 1], strides=[2, 2])[0]
    ref = F.conv2d(x.double() - 10, w.double() - wz.double().view(3, 1, 1, 1), stride=2, padding=1)
    assert got.dtype == torch.int32 and got.shape == (1, 3, 3, 3) and torch.equal(got.double(), ref)
    xs, ws, ys = t(0.02), t(0.01, 0.02, 0.03), t(0.05)
    yz = t(100, dtype=torch.uint8)
    bias = torch.tensor([5, -3, 0], dtype=torch.int32)
    q = ex("QLinearConv", [x, xs, xz, w, ws, wz, ys, yz, bias], pads=[1, 1, 1, 1])[0]
    real = F.conv2d((x.double() - 10) * 0.02, (w.double() - wz.double().view(3, 1, 1, 1)) * ws.double().view(3, 1, 1, 1),
                    bias.double() * 0.02 * ws.double(), padding=1)
    want = torch.clamp(torch.round(real / 0.05) + 100, 0, 255)
    assert q.dtype == torch.uint8 and q.shape == (1, 3, 5, 5) and (q.double() - want).abs().max() <= 1
    with pytest.raises(InvalidAttribute):
        ex("ConvInteger", [x, w], pads=[0, 1, 1, 1])


def test_operator_semantics_follow_the_onnx_specification():
    """Pad axes / edge / reflect / negative pads, ConvTranspose output_shape, AveragePool with asymmetric pads,
    1-D and 3-D pooling, Softmax below opset 13."""
    import numpy as np
    from ronn_b200.api.errors import InvalidAttribute
    from ronn_b200.onnx.registry import default_registry
    R = default_registry()
    ex = lambda op, ins, **a: R.get(op).execute(ins, a)
    x = torch.arange(24.0).reshape(2, 3, 4)
    # Pad: axes select the padded dimensions (opset 18); edge and reflect follow numpy's modes
    got = ex("Pad", [x, torch.tensor([1, 2]), None, torch.tensor([-1])], mode="constant")[0]
    assert got.shape == (2, 3, 7) and torch.equal(got[..., 1:5], x) and float(got[..., 0].abs().sum()) == 0
    for mode, npmode in (("edge", "edge"), ("reflect", "reflect")):
        got = ex("Pad", [x, torch.tensor([0, 1, 2, 0, 1, 1])], mode=mode)[0]
        want = torch.from_numpy(np.pad(x.numpy(), ((0, 0), (1, 1), (2, 1)), mode=npmode))
        assert torch.equal(got, want), mode
    got = ex("Pad", [x, torch.tensor([0, 0, -1, 0, 0, 2])], mode="constant")[0]          # negative pad crops
    assert got.shape == (2, 3, 5) and torch.equal(got[..., :3], x[..., 1:])
    with pytest.raises(InvalidAttribute):
        ex("Pad", [x, torch.tensor([1, 1])], mode="wrap")
    with pytest.raises(InvalidAttribute):
        ex("Pad", [x, torch.tensor([1, 1, 1])])
    # ConvTranspose: output_shape decides the output padding
    xi, w = torch.randn(1, 2, 5, 5), torch.randn(2, 3, 3, 3)
    y = ex("ConvTranspose", [xi, w], strides=[2, 2], pads=[1, 1, 1, 1], output_shape=[10, 10])[0]
    assert y.shape == (1, 3, 10, 10)
    torch.testing.assert_close(y, torch.nn.functional.conv_transpose2d(xi, w, stride=2, padding=1, output_padding=1))
    with pytest.raises(InvalidAttribute, match="not reachable"):
        ex("ConvTranspose", [xi, w], strides=[2, 2], pads=[1, 1, 1, 1], output_shape=[40, 40])
    # AveragePool, asymmetric pads: the divisor is the number of valid elements unless count_include_pad is set
    img = torch.arange(16.0).reshape(1, 1, 4, 4)
    y = ex("AveragePool", [img], kernel_shape=[2, 2], strides=[2, 2], pads=[0, 0, 1, 1])[0]
    assert y.shape == (1, 1, 2, 2) or y.shape == (1, 1, 3, 3)
    padded = torch.nn.functional.pad(img, [0, 1, 0, 1])
    ones = torch.nn.functional.pad(torch.ones_like(img), [0, 1, 0, 1])
    want = torch.nn.functional.avg_pool2d(padded, 2, 2) * 4 / (torch.nn.functional.avg_pool2d(ones, 2, 2) * 4)
    torch.testing.assert_close(y, want)
    y_inc = ex("AveragePool", [img], kernel_shape=[2, 2], strides=[2, 2], pads=[0, 0, 1, 1], count_include_pad=1)[0]
    torch.testing.assert_close(y_inc, torch.nn.functional.avg_pool2d(padded, 2, 2))
    # pooling over one and three spatial dimensions
    s1 = torch.randn(2, 3, 9)
    torch.testing.assert_close(ex("MaxPool", [s1], kernel_shape=[3], strides=[2])[0], torch.nn.functional.max_pool1d(s1, 3, 2))
    v3 = torch.randn(1, 2, 4, 6, 6)
    torch.testing.assert_close(ex("AveragePool", [v3], kernel_shape=[2, 2, 2], strides=[2, 2, 2])[0],
                               torch.nn.functional.avg_pool3d(v3, 2, 2))
    # Softmax below opset 13: coerced to 2-D at axis (default 1)
    t = torch.randn(2, 3, 4)
    legacy = ex("Softmax", [t], axis=1, legacy_flatten=1)[0]
    torch.testing.assert_close(legacy, torch.softmax(t.reshape(2, 12), 1).reshape(2, 3, 4))
    assert not torch.allclose(legacy, torch.softmax(t, 1))


def test_softmax_of_an_opset_11_model_uses_the_flattening_semantics():
    from ronn_b200 import Model
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.onnx.writer import model_to_bytes
    b = GraphBuilder().add_input("x", [2, 3, 4]).add_output("y", [2, 3, 4])
    b.add_op("Softmax", ["x"], ["y"])
    x = torch.randn(2, 3, 4)
    old = Model.from_bytes(model_to_bytes(b.build(), opset=11)).create_session().run({"x": x})["y"]
    new = Model.from_bytes(model_to_bytes(b.build(), opset=17)).create_session().run({"x": x})["y"]
    torch.testing.assert_close(old, torch.softmax(x.reshape(2, 12), 1).reshape(2, 3, 4))
    torch.testing.assert_close(new, torch.softmax(x, -1))


def test_add_followed_by_layernorm_becomes_one_skip_layernorm_node():
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.graph.ir import GraphBuilder
    g = torch.Generator().manual_seed(4)
    b = GraphBuilder().add_input("a", [3, 16]).add_input("r", [3, 16]).add_output("y", [3, 16]).add_output("z", [3, 16])
    b.add_initializer("gamma", torch.rand(16, generator=g) + 0.5).add_initializer("beta", torch.randn(16, generator=g))
    b.add_op("Add", ["a", "r"], ["s"]).add_op("LayerNormalization", ["s", "gamma", "beta"], ["y"], axis=-1, epsilon=1e-5)
    b.add_op("Relu", ["s"], ["z"])                       # the sum has a second consumer
    graph = b.build()
    feeds = {"a": torch.randn(3, 16, generator=g), "r": torch.randn(3, 16, generator=g)}
    ref = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level("O0")).run(feeds)
    s = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level("O2"))
    assert sorted(n.op_type for n in s.graph().nodes) == ["Relu", "SkipLayerNorm"]
    out = s.run(feeds)
    torch.testing.assert_close(out["y"], ref["y"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out["z"], ref["z"])
