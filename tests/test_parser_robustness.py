"""Robustness matrix of the ONNX wire parser and loader: every malformed, extreme or odd input must end in a library
error or in a loaded model, never in a crash, a hang or an unbounded allocation (the reference's matrix:
crates/ronn-onnx/tests/test_parser_robustness.rs:39-615).  Models are hand-encoded protobuf."""
import struct

import numpy as np
import pytest
import torch

from ronn_b200 import Model
from ronn_b200.api.errors import OnnxError, RonnError
from ronn_b200.core.types import DataType
from ronn_b200.graph.ir import ModelGraph, TensorInfo
from ronn_b200.onnx.loader import ModelLoader
from ronn_b200.onnx.writer import model_to_bytes


def varint(v):
    out = bytearray()
    v &= (1 << 64) - 1
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def field(num, wt, payload):
    return varint((num << 3) | wt) + payload


def ld(num, data):
    return field(num, 2, varint(len(data)) + data)


def model(graph=b"", ir=8, extra=b""):
    return field(1, 0, varint(ir)) + ld(7, graph) + extra


def tensor(name=b"t", dims=(2,), dtype=1, raw=None, extra=b""):
    t = b"".join(field(1, 0, varint(d)) for d in dims) + field(2, 0, varint(dtype)) + ld(8, name)
    if raw is not None:
        t += ld(9, raw)
    return t + extra


def node(op=b"Relu", ins=(b"x",), outs=(b"y",), name=b"", attrs=b""):
    return b"".join(ld(1, i) for i in ins) + b"".join(ld(2, o) for o in outs) + (ld(3, name) if name else b"") + ld(4, op) + attrs


def load(data):
    return ModelLoader.load_from_bytes(data)


# ------------------------------------------------------------------ garbage in
@pytest.mark.parametrize("data", [
    b"", b"\x00", b"{", b'{"graph": {"node": [', b"\xff" * 64, bytes(range(256)) * 4,
    "modèle ☃ \udcff".encode("utf-8", "surrogatepass"), b"\x0a\xff\xff\xff\xff\xff\xff\xff\xff\xff\x01",
    b"\x3a\x80\x80\x80\x80\x10" + b"\x00" * 8,                                  # graph length far beyond the buffer
    np.random.default_rng(0).integers(0, 256, 4096, dtype=np.uint8).tobytes(),
])
def test_garbage_bytes_raise_a_library_error(data):
    with pytest.raises(RonnError):
        load(data)


@pytest.mark.parametrize("seed", range(12))
def test_bit_flips_and_truncations_of_a_valid_model_never_crash(seed):
    g = ModelGraph()
    g.inputs.append(TensorInfo("x", [1, 4], DataType.F32))
    g.outputs.append(TensorInfo("y", [1, 4], DataType.F32))
    g.initializers["w"] = torch.arange(16.0).reshape(4, 4)
    g.add_node("MatMul", ["x", "w"], ["h"], name="mm")
    g.add_node("Relu", ["h"], ["y"], {"f": 1.5, "ints": [1, 2, 3], "s": "abc"})
    good = bytearray(model_to_bytes(g))
    rng = np.random.default_rng(seed)
    for _ in range(40):
        data = bytearray(good)
        for pos in rng.integers(0, len(data), size=int(rng.integers(1, 6))):
            data[pos] ^= 1 << int(rng.integers(0, 8))
        if rng.random() < 0.5:
            data = data[: int(rng.integers(1, len(data)))]
        try:
            m = load(bytes(data))
        except RonnError:
            continue
        assert isinstance(m.graph.nodes, list)         # whatever parsed is a well-formed object


# ------------------------------------------------------------------ missing pieces
def test_missing_graph_name_and_empty_names_are_tolerated():
    m = load(model(ld(1, node()) + ld(11, ld(1, b"x")) + ld(12, ld(1, b"y"))))
    assert m.graph.nodes[0].op_type == "Relu" and m.graph.nodes[0].name == "node_0"
    m = load(model(ld(1, node(ins=(b"",), outs=(b"y",))) + ld(2, b"")))
    assert m.graph.nodes[0].inputs == [""]                # an omitted optional input stays an empty name


def test_missing_op_type_is_an_error_and_names_the_node():
    bad = ld(1, b"x") + ld(2, b"y") + ld(3, b"nameless_op")
    with pytest.raises(OnnxError, match="nameless_op|op_type"):
        load(model(ld(1, bad)))


def test_tensor_without_dims_is_a_scalar_and_without_data_is_an_error():
    m = load(model(ld(5, field(2, 0, varint(1)) + ld(8, b"s") + ld(9, struct.pack("<f", 2.5)))))
    assert m.initializers["s"].shape == () and float(m.initializers["s"]) == 2.5
    with pytest.raises(OnnxError, match="no data|carries"):
        load(model(ld(5, tensor(dims=(3,)))))


def test_attribute_kinds_that_do_not_match_their_payload():
    # declared FLOAT but only an int payload, declared INTS with a string payload, undefined kind 0, unknown kind 99
    a1 = ld(5, ld(1, b"alpha") + field(20, 0, varint(1)) + field(3, 0, varint(7)))
    a2 = ld(5, ld(1, b"axes") + field(20, 0, varint(7)) + ld(4, b"text"))
    a3 = ld(5, ld(1, b"undef") + field(20, 0, varint(0)))
    a4 = ld(5, ld(1, b"future") + field(20, 0, varint(99)))
    m = load(model(ld(1, node(attrs=a1 + a2 + a3 + a4))))
    at = m.graph.nodes[0].attributes
    assert at["alpha"] == 0.0 and at["axes"] == [] and at.get("undef") is None and at.get("future") is None


# ------------------------------------------------------------------ types and shapes
@pytest.mark.parametrize("code", [0, 4, 5, 8, 13, 14, 15, 17, 99, 2 ** 31 - 1])
def test_unknown_element_types_are_rejected_with_their_code(code):
    with pytest.raises(OnnxError, match=str(code)):
        load(model(ld(5, tensor(dtype=code, raw=b"\x00" * 16))))


def test_declared_shapes_that_would_need_absurd_memory_are_refused_not_allocated():
    huge = tensor(dims=(2 ** 31, 2 ** 31), raw=b"\x00" * 8)
    with pytest.raises(OnnxError):
        load(model(ld(5, huge)))
    overflow = tensor(dims=(2 ** 62, 8), raw=b"\x00" * 8)
    with pytest.raises(OnnxError):
        load(model(ld(5, overflow)))
    # as a declared INPUT shape (no data behind it) a huge shape is just metadata
    vi = ld(1, b"x") + ld(2, ld(1, field(1, 0, varint(1)) + ld(2, ld(1, field(1, 0, varint(10 ** 12))) + ld(1, field(1, 0, varint(10 ** 12))))))
    m = load(model(ld(11, vi)))
    assert m.inputs[0].shape == [10 ** 12, 10 ** 12]


def test_zero_and_negative_dimensions():
    m = load(model(ld(5, tensor(dims=(0, 4), raw=b""))))
    assert tuple(m.initializers["t"].shape) == (0, 4)
    with pytest.raises(OnnxError, match="negative"):
        load(model(ld(5, tensor(dims=(-3,), raw=b"\x00" * 12))))
    # a negative dim_value in a declared input shape is read as a dynamic dimension
    vi = ld(1, b"x") + ld(2, ld(1, field(1, 0, varint(1)) + ld(2, ld(1, field(1, 0, varint(-1))))))
    assert load(model(ld(11, vi))).inputs[0].shape in ([-1], [0])


def test_raw_data_shorter_or_longer_than_the_shape():
    with pytest.raises(OnnxError):
        load(model(ld(5, tensor(dims=(4,), raw=b"\x00" * 12))))
    with pytest.raises(OnnxError):
        load(model(ld(5, tensor(dims=(2,), raw=b"\x00" * 12))))


# ------------------------------------------------------------------ sizes and nesting
def test_deeply_nested_subgraphs_hit_a_depth_limit_not_the_stack():
    g = ld(1, node())
    for _ in range(5000):                               # a graph attribute inside a node inside a graph ...
        g = ld(1, node(op=b"If", attrs=ld(5, ld(1, b"then_branch") + field(20, 0, varint(5)) + ld(6, g))))
    try:
        m = load(model(g))
        assert len(m.graph.nodes) == 1
    except RonnError:
        pass


def test_very_long_names_special_characters_and_many_nodes():
    long = b"n" * 200_000
    weird = "a/b:c d\t\"quoted\"\\back\u2603\U0001F600".encode()
    nodes = b"".join(ld(1, node(ins=(b"x",), outs=(b"y%d" % i,), name=b"n%d" % i)) for i in range(20_000))
    m = load(model(nodes + ld(1, node(ins=(long,), outs=(weird,), name=weird))))
    assert len(m.graph.nodes) == 20_001 and m.graph.nodes[-1].inputs[0] == long.decode()
    assert m.graph.nodes[-1].name == weird.decode()


def test_empty_and_very_large_repeated_fields():
    empty = ld(5, ld(1, b"ints") + field(20, 0, varint(7)))                       # INTS with no elements
    big = ld(5, ld(1, b"big") + field(20, 0, varint(7)) + ld(8, b"".join(varint(i) for i in range(100_000))))
    fl = ld(5, ld(1, b"fl") + field(20, 0, varint(6)) + ld(7, np.arange(50_000, dtype=np.float32).tobytes()))
    m = load(model(ld(1, node(attrs=empty + big + fl))))
    at = m.graph.nodes[0].attributes
    assert at["ints"] == [] and at["big"][-1] == 99_999 and len(at["fl"]) == 50_000 and at["fl"][7] == 7.0


def test_node_that_consumes_its_own_output_loads_but_does_not_validate():
    m = load(model(ld(1, node(ins=(b"y",), outs=(b"y",))) + ld(12, ld(1, b"y"))))
    with pytest.raises(RonnError):
        m.graph.validate()
    with pytest.raises(RonnError):
        Model.from_bytes(model(ld(1, node(ins=(b"y",), outs=(b"y",))) + ld(12, ld(1, b"y")))).create_session()


def test_extreme_float_and_int_values_survive():
    vals = np.array([np.inf, -np.inf, np.nan, np.finfo(np.float32).max, np.finfo(np.float32).tiny, -0.0, 1e-45], dtype=np.float32)
    m = load(model(ld(5, tensor(dims=(7,), raw=vals.tobytes()))))
    got = m.initializers["t"].numpy()
    assert np.array_equal(got[[0, 1, 3, 4]], vals[[0, 1, 3, 4]]) and np.isnan(got[2]) and np.signbit(got[5]) and got[6] == vals[6]
    ints = np.array([np.iinfo(np.int64).min, np.iinfo(np.int64).max, 0, -1], dtype=np.int64)
    m = load(model(ld(5, tensor(dims=(4,), dtype=7, raw=ints.tobytes()))))
    assert m.initializers["t"].tolist() == ints.tolist()
    a = ld(5, ld(1, b"i") + field(20, 0, varint(2)) + field(3, 0, varint(-(2 ** 63)))) + \
        ld(5, ld(1, b"f") + field(20, 0, varint(1)) + field(2, 5, struct.pack("<f", float("-inf"))))
    at = load(model(ld(1, node(attrs=a)))).graph.nodes[0].attributes
    assert at["i"] == -(2 ** 63) and at["f"] == float("-inf")


def test_a_large_model_file_loads_without_copying_every_tensor_twice():
    w = np.zeros(8 * 1024 * 1024, dtype=np.float32)                                 # 32 MiB initializer
    w[-1] = 3.0
    data = model(ld(5, tensor(name=b"w", dims=(w.size,), raw=w.tobytes())))
    m = load(data)
    assert m.initializers["w"].numel() == w.size and float(m.initializers["w"][-1]) == 3.0


def test_large_initializers_of_a_model_file_are_views_of_its_mapping(tmp_path):
    """Loading from a path maps the file copy-on-write: initializers of 64 KB or more share the mapping (no second
    copy of the weights; the ranks of a tensor-parallel job share the pages), small ones are copied, and writing to a
    shared tensor never reaches the file."""
    import numpy as np
    import torch

    from ronn_b200 import Model
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.onnx.loader import ModelLoader
    b = GraphBuilder().add_input("x", [4, 512]).add_output("y", [4, 256])
    w, small = torch.randn(512, 256), torch.randn(256)
    b.add_initializer("w", w).add_initializer("small", small)
    b.add_op("MatMul", ["x", "w"], ["m"]).add_op("Add", ["m", "small"], ["y"])
    path = tmp_path / "m.onnx"
    Model.from_graph(b.build()).save(str(path))
    on_disk = path.read_bytes()
    loaded = ModelLoader.load_from_file(str(path))
    lw, ls = loaded.initializers["w"], loaded.initializers["small"]
    assert torch.equal(lw, w) and torch.equal(ls, small)
    assert loaded.shared_bytes == 512 * 256 * 4          # the large tensor is a view of the mapping, the small one a copy
    lw[0, 0] = 12345.0                                   # copy-on-write: private to this process
    assert path.read_bytes() == on_disk
    x = torch.randn(4, 512)
    out = Model.load(str(path)).create_session().run({"x": x})["y"]
    torch.testing.assert_close(out, x @ w + small, atol=1e-4, rtol=1e-4)
    # from bytes nothing is shared
    again = ModelLoader.load_from_bytes(on_disk)
    again.initializers["w"][0, 0] = -1.0
    assert torch.equal(ModelLoader.load_from_bytes(on_disk).initializers["w"], w)
