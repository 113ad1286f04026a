"""Operator registry: the reference's 39 operators plus the additions, arity errors, numeric definitions."""
import math

import pytest
import torch
import torch.nn.functional as F

from ronn_b200.api.errors import InvalidAttribute, InvalidGraph, UnsupportedOperator
from ronn_b200.onnx.registry import REFERENCE_OPS, default_registry

R = default_registry()


def ex(op, inputs, **attrs):
    return R.get(op).execute(inputs, attrs)


def test_reference_ops_all_registered():
    assert len(REFERENCE_OPS) == 39
    for name in REFERENCE_OPS:
        assert R.has(name), name
    for name in ("Gemm", "Flatten", "GlobalAveragePool", "Identity", "Constant", "Shape", "Where", "Erf", "Expand",
                 "Equal", "Not", "Range", "ConstantOfShape", "ReduceMax", "ArgMax", "FusedConv", "FusedGemm", "RMSNorm",
                 "RotaryEmbedding", "SwiGLU", "BitLinear", "SiLU"):
        assert R.has(name), name
    with pytest.raises(UnsupportedOperator):
        R.get("NoSuchOp")


def test_arity_errors():
    with pytest.raises(InvalidGraph, match=r"Reshape expects 2 inputs, got 1"):
        ex("Reshape", [torch.zeros(2)])
    with pytest.raises(InvalidGraph, match=r"Relu expects 1 input, got 2"):
        ex("Relu", [torch.zeros(2), torch.zeros(2)])
    with pytest.raises(InvalidGraph, match="at least 1"):
        ex("Concat", [], axis=0)
    with pytest.raises(InvalidAttribute):
        ex("Concat", [torch.zeros(2)])
    with pytest.raises(InvalidAttribute):
        ex("Cast", [torch.zeros(2)])


def test_activations():
    x = torch.linspace(-4, 4, 41)
    assert torch.equal(ex("Relu", [x])[0], x.clamp(min=0))
    torch.testing.assert_close(ex("Sigmoid", [x])[0], 1 / (1 + torch.exp(-x)))
    ref_gelu = 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3)))
    torch.testing.assert_close(ex("Gelu", [x], approximate="tanh")[0], ref_gelu, atol=1e-6, rtol=1e-5)
    # ONNX default: the exact (erf) form
    torch.testing.assert_close(ex("Gelu", [x])[0], 0.5 * x * (1 + torch.erf(x / math.sqrt(2))), atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(ex("FastGelu", [x])[0], x * torch.sigmoid(1.702 * x))
    torch.testing.assert_close(ex("LeakyRelu", [x])[0], torch.where(x > 0, x, 0.01 * x))
    torch.testing.assert_close(ex("Elu", [x])[0], torch.where(x > 0, x, torch.exp(x) - 1))
    torch.testing.assert_close(ex("Swish", [x])[0], x * torch.sigmoid(x))
    m = torch.randn(3, 5)
    torch.testing.assert_close(ex("Softmax", [m])[0].sum(-1), torch.ones(3))
    torch.testing.assert_close(ex("Softmax", [m], axis=-2)[0], torch.softmax(m, 0))      # ONNX semantics for negative axes
    torch.testing.assert_close(ex("Softmax", [m * 1000])[0].sum(-1), torch.ones(3))       # max-shifted: no overflow


def test_math_and_broadcast():
    a, b = torch.randn(2, 3, 4), torch.randn(4)
    for op, fn in (("Add", torch.add), ("Sub", torch.sub), ("Mul", torch.mul), ("Div", torch.div)):
        torch.testing.assert_close(ex(op, [a, b])[0], fn(a, b))
    assert ex("Div", [torch.tensor([7, -7]), torch.tensor([2, 2])])[0].tolist() == [3, -3]
    torch.testing.assert_close(ex("MatMul", [a, torch.randn(4, 5)])[0].shape, torch.Size([2, 3, 5]))
    torch.testing.assert_close(ex("Pow", [a.abs(), torch.tensor(2.0)])[0], a.abs() ** 2)
    torch.testing.assert_close(ex("Clip", [a, torch.tensor(-0.5), torch.tensor(0.5)])[0], a.clamp(-0.5, 0.5))
    torch.testing.assert_close(ex("Clip", [a], min=0.0)[0], a.clamp(min=0))
    w, bias = torch.randn(5, 4), torch.randn(5)
    torch.testing.assert_close(ex("Gemm", [a[0], w, bias], transB=1, alpha=2.0, beta=0.5)[0], 2 * a[0] @ w.t() + 0.5 * bias)
    torch.testing.assert_close(ex("Where", [a > 0, a, -a])[0], a.abs())


def test_nn_ops():
    x = torch.randn(2, 3, 9, 9)
    w, b = torch.randn(4, 3, 3, 3), torch.randn(4)
    torch.testing.assert_close(ex("Conv", [x, w, b], strides=[2, 2], pads=[1, 1, 1, 1])[0], F.conv2d(x, w, b, 2, 1))
    torch.testing.assert_close(ex("Conv", [x, w])[0], F.conv2d(x, w))                    # defaults: stride 1, no pad
    torch.testing.assert_close(ex("Conv", [x, w], pads=[0, 1, 2, 1])[0], F.conv2d(F.pad(x, [1, 1, 0, 2]), w))
    torch.testing.assert_close(ex("MaxPool", [x], kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])[0], F.max_pool2d(x, 3, 2, 1))
    torch.testing.assert_close(ex("AveragePool", [x], kernel_shape=[3, 3], strides=[3, 3])[0], F.avg_pool2d(x, 3, 3))
    torch.testing.assert_close(ex("GlobalAveragePool", [x])[0], x.mean((2, 3), keepdim=True))
    g, be, mu, var = torch.rand(3) + 0.5, torch.randn(3), torch.randn(3), torch.rand(3) + 0.5
    torch.testing.assert_close(ex("BatchNormalization", [x, g, be, mu, var])[0], F.batch_norm(x, mu, var, g, be, False, 0.0, 1e-5), atol=1e-5, rtol=1e-5)
    h = torch.randn(4, 7, 16)
    torch.testing.assert_close(ex("LayerNormalization", [h, torch.ones(16), torch.zeros(16)])[0], F.layer_norm(h, (16,)), atol=1e-5, rtol=1e-5)
    q = torch.randn(2, 5, 16)
    att = ex("Attention", [q, q, q], num_heads=4)[0]
    ref = F.scaled_dot_product_attention(*(t.reshape(2, 5, 4, 4).transpose(1, 2) for t in (q, q, q))).transpose(1, 2).reshape(2, 5, 16)
    torch.testing.assert_close(att, ref, atol=1e-5, rtol=1e-5)
    catt = ex("MultiHeadAttention", [q, q, q], num_heads=4, causal=1)[0]
    cref = F.scaled_dot_product_attention(*(t.reshape(2, 5, 4, 4).transpose(1, 2) for t in (q, q, q)), is_causal=True).transpose(1, 2).reshape(2, 5, 16)
    torch.testing.assert_close(catt, cref, atol=1e-5, rtol=1e-5)
    with pytest.raises(InvalidAttribute):
        ex("Attention", [q, q, q])


def test_tensor_ops():
    x = torch.arange(24.0).reshape(2, 3, 4)
    assert ex("Reshape", [x, torch.tensor([0, -1])])[0].shape == (2, 12)
    assert ex("Transpose", [x])[0].shape == (4, 3, 2)
    assert torch.equal(ex("Transpose", [ex("Transpose", [x])[0]])[0], x)
    assert ex("Transpose", [x], perm=[1, 0, 2])[0].shape == (3, 2, 4)
    assert ex("Concat", [x, x], axis=1)[0].shape == (2, 6, 4)
    parts = ex("Split", [x, torch.tensor([1, 3])], axis=2)
    assert [p.shape[2] for p in parts] == [1, 3]
    assert [p.shape[1] for p in R.get("Split").execute([x], {"axis": 1, "num_outputs": 3})] == [1, 1, 1]
    assert torch.equal(ex("Gather", [x, torch.tensor([1, 0])])[0], x[[1, 0]])
    assert torch.equal(ex("Gather", [x, torch.tensor(2)], axis=2)[0], x[:, :, 2])
    assert torch.equal(ex("Slice", [x, torch.tensor([1]), torch.tensor([3]), torch.tensor([2])])[0], x[:, :, 1:3])
    assert torch.equal(ex("Slice", [x, torch.tensor([-1]), torch.tensor([-5]), torch.tensor([2]), torch.tensor([-1])])[0], x.flip(2))
    assert ex("Squeeze", [x[:, :1]], axes=[1])[0].shape == (2, 4)
    assert ex("Unsqueeze", [x], axes=[0, -1])[0].shape == (1, 2, 3, 4, 1)
    assert ex("ReduceMean", [x], axes=[1])[0].shape == (2, 1, 4)
    assert ex("ReduceSum", [x], keepdims=0)[0].shape == ()
    assert ex("Cast", [x], to=7)[0].dtype == torch.int64
    assert ex("Flatten", [x], axis=2)[0].shape == (6, 4)
    assert ex("Shape", [x])[0].tolist() == [2, 3, 4]
    assert ex("Expand", [torch.ones(3, 1), torch.tensor([2, 3, 4])])[0].shape == (2, 3, 4)
    assert ex("Range", [torch.tensor(0), torch.tensor(5), torch.tensor(2)])[0].tolist() == [0, 2, 4]
    assert ex("ConstantOfShape", [torch.tensor([2, 2])], value=torch.tensor([7], dtype=torch.int64))[0].tolist() == [[7, 7], [7, 7]]
    assert ex("ArgMax", [x], axis=2, keepdims=0)[0].tolist() == [[3, 3, 3], [3, 3, 3]]
    emb = torch.randn(10, 4)
    assert torch.equal(ex("Embedding", [emb, torch.tensor([[1, 2]])])[0], emb[[1, 2]].unsqueeze(0))


def test_custom_domain_ops():
    x = torch.randn(5, 8)
    w = torch.rand(8) + 0.5
    torch.testing.assert_close(ex("RMSNorm", [x, w], epsilon=1e-6)[0], x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w)
    torch.testing.assert_close(ex("SwiGLU", [x, x * 2])[0], F.silu(x) * x * 2)
    pos = torch.arange(5)
    r = ex("RotaryEmbedding", [x, pos], num_heads=2, base=10000.0)[0]
    assert r.shape == x.shape
    torch.testing.assert_close(r[0], x[0])                                  # position 0 is the identity rotation
    torch.testing.assert_close(r.reshape(5, 2, 4).norm(dim=-1), x.reshape(5, 2, 4).norm(dim=-1), atol=1e-5, rtol=1e-5)
    wt, bias, res = torch.randn(6, 8), torch.randn(6), torch.randn(5, 6)
    y = ex("FusedGemm", [x, wt, bias, res], transB=1, activation="Gelu")[0]
    torch.testing.assert_close(y, F.gelu(x @ wt.t() + bias, approximate="tanh") + res)
    img, cw, cb = torch.randn(1, 2, 6, 6), torch.randn(3, 2, 3, 3), torch.randn(3)
    rz = torch.randn(1, 3, 6, 6)
    yc = ex("FusedConv", [img, cw, cb, rz], pads=[1, 1, 1, 1], activation="Relu")[0]
    torch.testing.assert_close(yc, torch.relu(F.conv2d(img, cw, cb, 1, 1) + rz))
    # NHWC execution of the same node
    yn = ex("FusedConv", [img.permute(0, 2, 3, 1).contiguous(), cw.permute(0, 2, 3, 1).contiguous(), cb,
                          rz.permute(0, 2, 3, 1).contiguous()], pads=[1, 1, 1, 1], activation="Relu", data_format="NHWC")[0]
    torch.testing.assert_close(yn.permute(0, 3, 1, 2), yc, atol=1e-5, rtol=1e-5)


def test_bitlinear_op_exact():
    from ronn_b200.providers.bitnet.quantization import pack_ternary_rows
    torch.manual_seed(0)
    K_, N = 64, 12
    wq = torch.randint(-1, 2, (N, K_), dtype=torch.int8)
    x = torch.randn(3, K_)
    y = ex("BitLinear", [x, pack_ternary_rows(wq), torch.tensor(0.037)], k=K_, n=N)[0]
    s = x.abs().amax(-1, keepdim=True) / 127.0
    q = torch.round(x / s).clamp(-127, 127)
    ref = (q @ wq.float().t()) * s * 0.037
    torch.testing.assert_close(y, ref, atol=1e-5, rtol=1e-5)
