"""Loader / writer / type-mapper behaviour (models are synthesised in-process, as the reference's tests do
with prost structs: crates/ronn-onnx/tests/test_loader.py-equivalents test_loader.rs:9-70)."""
import numpy as np
import pytest
import torch

from ronn_b200.api.errors import (InvalidGraph, ModelLoadError, OnnxError, ProtobufDecodeError, TypeConversionError,
                                  UnsupportedIrVersion)
from ronn_b200.core.types import DataType
from ronn_b200.graph.ir import GraphBuilder, ModelGraph, TensorInfo
from ronn_b200.onnx.dtypes import DataTypeMapper
from ronn_b200.onnx.loader import ModelLoader
from ronn_b200.onnx.writer import model_to_bytes


def _varint(v):
    out = bytearray()
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _field(num, wt, payload):
    return _varint((num << 3) | wt) + payload


def _ld(num, data):
    return _field(num, 2, _varint(len(data)) + data)


def small_graph(dtype=torch.float32):
    b = GraphBuilder().add_input("x", [1, 4]).add_output("y", [1, 2])
    b.add_initializer("w", torch.randn(4, 2).to(dtype))
    b.add_op("MatMul", ["x", "w"], ["h"], name="mm").add_op("Relu", ["h"], ["y"])
    return b.build()


def test_roundtrip_all_dtypes():
    g = ModelGraph()
    g.inputs.append(TensorInfo("x", [2, 0], DataType.F32, [None, "seq"]))
    g.outputs.append(TensorInfo("x", [2, 0], DataType.F32, [None, "seq"]))
    vals = {"f32": torch.randn(3, 2), "f16": torch.randn(5).half(), "bf16": torch.randn(2, 2).bfloat16(),
            "f64": torch.randn(2).double(), "i8": torch.tensor([-3, 4], dtype=torch.int8),
            "u8": torch.tensor([3, 250], dtype=torch.uint8), "i32": torch.tensor([7, -9], dtype=torch.int32),
            "i64": torch.tensor([2 ** 40, -1]), "bool": torch.tensor([True, False]),
            "scalar": torch.tensor(3.5)}
    for k, v in vals.items():
        g.initializers[k] = v
        g.add_node("Identity", [k], [k + "_o"])
    m = ModelLoader.load_from_bytes(model_to_bytes(g, metadata={"k": "v"}))
    for k, v in vals.items():
        assert m.initializers[k].dtype == v.dtype and torch.equal(m.initializers[k], v), k
    assert m.metadata["k"] == "v"
    assert m.inputs[0].shape == [2, 0] and m.inputs[0].dim_params == [None, "seq"]


def test_attributes_and_names():
    g = ModelGraph()
    g.inputs.append(TensorInfo("x", [1], DataType.F32))
    g.outputs.append(TensorInfo("y", [1], DataType.F32))
    g.add_node("Foo", ["x"], ["y"], {"f": 1.5, "i": -7, "s": "héllo", "fs": [1.0, 2.5], "is": [1, -2, 3],
                                     "ss": ["a", "b"], "t": torch.arange(6).reshape(2, 3).float(),
                                     "big": 2 ** 62, "neg_inf": float("-inf")}, name="")
    m = ModelLoader.load_from_bytes(model_to_bytes(g))
    n = m.graph.nodes[0]
    assert n.name == "node_0"
    a = n.attributes
    assert a["f"] == 1.5 and a["i"] == -7 and a["s"] == "héllo" and a["fs"] == [1.0, 2.5] and a["is"] == [1, -2, 3]
    assert a["ss"] == ["a", "b"] and torch.equal(a["t"], torch.arange(6).reshape(2, 3).float())
    assert a["big"] == 2 ** 62 and a["neg_inf"] == float("-inf")


def test_typed_fields_and_unpacked_repeated():
    # TensorProto with float_data given UNPACKED (one fixed32 field per element) and int64 dims unpacked
    t = _field(1, 0, _varint(2)) + _field(2, 0, _varint(1)) + _ld(8, b"w")
    t += _field(4, 5, np.float32(1.5).tobytes()) + _field(4, 5, np.float32(-2.0).tobytes())
    graph = _ld(5, t) + _ld(2, b"g")
    model = _field(1, 0, _varint(8)) + _ld(7, graph)
    m = ModelLoader.load_from_bytes(model)
    assert torch.equal(m.initializers["w"], torch.tensor([1.5, -2.0]))
    # int32_data carrying fp16 bit patterns, packed
    h = np.array([1.0, -0.5], dtype=np.float16).view(np.uint16)
    t2 = _field(1, 0, _varint(2)) + _field(2, 0, _varint(10)) + _ld(8, b"h") + _ld(5, b"".join(_varint(int(x)) for x in h))
    m2 = ModelLoader.load_from_bytes(_field(1, 0, _varint(8)) + _ld(7, _ld(5, t2)))
    assert torch.equal(m2.initializers["h"], torch.tensor([1.0, -0.5], dtype=torch.float16))


def test_initializers_excluded_from_inputs_and_minimal_models():
    g = small_graph()
    g.inputs.append(TensorInfo("w", [4, 2], DataType.F32))       # old exporters list weights as inputs too
    m = ModelLoader.load_from_bytes(model_to_bytes(g))
    assert [i.name for i in m.inputs] == ["x"]
    empty = ModelGraph()
    m2 = ModelLoader.load_from_bytes(model_to_bytes(empty))
    assert m2.graph.nodes == [] and m2.ir_version == 8
    huge = ModelGraph()
    huge.inputs.append(TensorInfo("x", [10 ** 6, 10 ** 6], DataType.F32))
    assert ModelLoader.load_from_bytes(model_to_bytes(huge)).inputs[0].shape == [10 ** 6, 10 ** 6]


@pytest.mark.parametrize("data", [b"", b"\x00", b"\xff\xff\xff", b"not an onnx model at all", bytes(range(256)),
                                  b"\x08\x08\x3a\xff\xff\xff\xff\x0f"])
def test_malformed_bytes_raise(data):
    with pytest.raises(OnnxError):
        ModelLoader.load_from_bytes(data)


def test_truncated_and_missing_graph():
    data = model_to_bytes(small_graph())
    for cut in (len(data) // 2, len(data) - 3, 5):
        with pytest.raises(OnnxError):
            ModelLoader.load_from_bytes(data[:cut])
    with pytest.raises(InvalidGraph):
        ModelLoader.load_from_bytes(_field(1, 0, _varint(8)))
    with pytest.raises(UnsupportedIrVersion):
        ModelLoader.load_from_bytes(model_to_bytes(small_graph(), ir_version=2))
    assert ModelLoader.load_from_bytes(model_to_bytes(small_graph(), ir_version=3)).ir_version == 3


def test_missing_op_type_unknown_dtype_negative_dims():
    node = _ld(1, b"x") + _ld(2, b"y")
    with pytest.raises(InvalidGraph):
        ModelLoader.load_from_bytes(_field(1, 0, _varint(8)) + _ld(7, _ld(1, node)))
    t = _field(1, 0, _varint(1)) + _field(2, 0, _varint(15)) + _ld(8, b"c") + _ld(9, b"\x00" * 16)
    with pytest.raises(TypeConversionError, match="15"):
        ModelLoader.load_from_bytes(_field(1, 0, _varint(8)) + _ld(7, _ld(5, t)))
    neg = _field(1, 0, _varint((1 << 64) - 4)) + _field(2, 0, _varint(1)) + _ld(8, b"n")
    with pytest.raises(OnnxError):
        ModelLoader.load_from_bytes(_field(1, 0, _varint(8)) + _ld(7, _ld(5, neg)))


def test_type_mapper():
    pairs = {1: DataType.F32, 2: DataType.U8, 3: DataType.I8, 6: DataType.I32, 7: DataType.I64, 9: DataType.BOOL,
             10: DataType.F16, 11: DataType.F64, 12: DataType.U32, 16: DataType.BF16}
    for code, dt in pairs.items():
        assert DataTypeMapper.from_onnx(code) == dt and DataTypeMapper.to_onnx(dt) == code
    for bad in (0, -1, 4, 5, 8, 13, 14, 15, 99):
        with pytest.raises(TypeConversionError, match=str(bad)):
            DataTypeMapper.from_onnx(bad)


def test_special_names_and_long_names():
    g = ModelGraph()
    long = "n" * 5000
    weird = "tensor/with:odd\tchars\"\\ ☃"
    g.inputs.append(TensorInfo(weird, [1], DataType.F32))
    g.outputs.append(TensorInfo(long, [1], DataType.F32))
    g.add_node("Relu", [weird], [long], name=weird)
    m = ModelLoader.load_from_bytes(model_to_bytes(g))
    assert m.graph.nodes[0].inputs == [weird] and m.graph.nodes[0].outputs == [long] and m.graph.nodes[0].name == weird


def test_model_api_load_errors(tmp_path):
    from ronn_b200 import Model
    for bad in ("", str(tmp_path), str(tmp_path / "missing.onnx")):
        with pytest.raises(ModelLoadError) as e:
            Model.load(bad)
        assert str(e.value).startswith("Failed to load model: ")
    p = tmp_path / "m.txt"
    p.write_bytes(b"hello")
    with pytest.raises(ModelLoadError):
        Model.load(p)
    q = tmp_path / "ok.onnx"
    q.write_bytes(model_to_bytes(small_graph()))
    a, b = Model.load(q), Model.from_bytes(q.read_bytes())
    assert a.input_names() == b.input_names() == ["x"] and a.output_names() == ["y"]
    assert a.ir_version() == 8 and a.producer_name() == "ronn_b200" and a.metadata()["node_count"] == 2


def _external_model(location, offset=None, length=None, dims=(4,)):
    """A model with one float initializer whose bytes live in an external file named by `location` (hand-encoded)."""
    t = b"".join(_field(1, 0, _varint(d)) for d in dims) + _field(2, 0, _varint(1)) + _ld(8, b"w")
    entries = {"location": location}
    if offset is not None:
        entries["offset"] = str(offset)
    if length is not None:
        entries["length"] = str(length)
    for k, v in entries.items():
        t += _ld(13, _ld(1, k.encode()) + _ld(2, v.encode()))
    t += _field(14, 0, _varint(1))                               # data_location = EXTERNAL
    return _field(1, 0, _varint(8)) + _ld(7, _ld(5, t) + _ld(2, b"g"))


@pytest.mark.parametrize("location,offset,length,err", [
    ("../w.bin", None, None, "leaves the model directory"),
    ("sub/../../w.bin", None, None, "leaves the model directory"),
    ("/etc/passwd", None, None, "absolute path"),
    ("inside.bin", None, 4096, "exceeds"),
    ("inside.bin", 640, None, "exceeds"),
    ("inside.bin", 0, 32, "exceeds the 16 bytes"),
    ("inside.bin", "x", None, "not a number"),
    ("missing.bin", None, None, "not found"),
    ("link.bin", None, None, "symbolic link"),
])
def test_external_data_locations_are_confined_to_the_model_directory(tmp_path, location, offset, length, err):
    from ronn_b200.api.errors import RonnError
    sub = tmp_path / "model"
    sub.mkdir()
    (tmp_path / "w.bin").write_bytes(b"\0" * 64)
    (sub / "inside.bin").write_bytes(b"\0" * 64)
    (sub / "link.bin").symlink_to(tmp_path / "w.bin")
    with pytest.raises(RonnError, match=err):
        ModelLoader.load_from_bytes(_external_model(location, offset, length), base_dir=str(sub))


def test_external_data_inside_the_model_directory_loads(tmp_path):
    (tmp_path / "w.bin").write_bytes(np.arange(8, dtype=np.float32).tobytes())
    m = ModelLoader.load_from_bytes(_external_model("w.bin", 16, 16), base_dir=str(tmp_path))
    torch.testing.assert_close(m.initializers["w"], torch.arange(4, 8, dtype=torch.float32))
    m = ModelLoader.load_from_bytes(_external_model("w.bin", None, None, dims=(8,)), base_dir=str(tmp_path))
    torch.testing.assert_close(m.initializers["w"], torch.arange(8, dtype=torch.float32))
