"""The small fixture models round-trip through the ONNX codec and run at every optimisation level."""
import pytest
import torch
import torch.nn.functional as F

from ronn_b200 import Model, SessionOptions
from ronn_b200.models.test_models import BUILDERS, write_all


def test_fixture_models_round_trip_and_run(tmp_path):
    paths = write_all(str(tmp_path))
    assert set(paths) == set(BUILDERS)
    torch.manual_seed(0)
    for name, path in paths.items():
        model = Model.load(path)
        feeds = {t.name: torch.rand(*[int(s) for s in t.shape]) for t in model.inputs()}
        outs = {}
        for level in ("O0", "O3"):
            sess = model.create_session(SessionOptions().with_optimization_level(level).with_provider("cpu"))
            outs[level] = sess.run(feeds)
        for k in outs["O0"]:
            torch.testing.assert_close(outs["O0"][k], outs["O3"][k], atol=1e-4, rtol=1e-4)
        init = Model.load(path).graph.initializers
        got = next(iter(outs["O0"].values()))
        if name in ("simple_add", "add_model"):
            torch.testing.assert_close(got, feeds["a"] + feeds["b"])
        elif name == "simple_matmul":
            torch.testing.assert_close(got, feeds["a"] @ feeds["b"])
        elif name == "simple_relu":
            torch.testing.assert_close(got, torch.relu(feeds["x"]))
        elif name == "simple_model":
            torch.testing.assert_close(got, feeds["input"])
        elif name == "simple_linear":
            torch.testing.assert_close(got, feeds["input"] @ init["weight"] + init["bias"], atol=1e-5, rtol=1e-5)
        elif name == "simple_conv":
            ref = torch.relu(F.conv2d(feeds["input"], init["conv.weight"], stride=2, padding=3))
            torch.testing.assert_close(got, ref, atol=1e-4, rtol=1e-4)
        elif name == "resnet18_stub":
            ref = F.conv2d(feeds["input"], init["conv.weight"], stride=2, padding=3).mean(dim=(2, 3)) @ init["fc.weight"]
            torch.testing.assert_close(got, ref, atol=1e-4, rtol=1e-4)


def test_command_line_info_run_optimize(tmp_path, capsys):
    import json
    from ronn_b200.__main__ import main
    paths = write_all(str(tmp_path))
    assert main(["info", paths["simple_linear"]]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["inputs"] == [{"name": "input", "shape": [1, 10], "dtype": "f32"}] and info["operators"] == {"MatMul": 1, "Add": 1}
    assert main(["run", paths["resnet18_stub"], "--level", "O3", "--repeat", "1"]) == 0
    ran = json.loads(capsys.readouterr().out)
    assert ran["outputs"] == {"logits": {"shape": [1, 1000], "dtype": "float32"}} and ran["ms_per_run"] > 0
    out = str(tmp_path / "opt.onnx")
    assert main(["optimize", paths["simple_linear"], out, "--level", "O3"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["nodes_before"] == 2 and rep["nodes_after"] == 1 and rep["nodes_fused"] == 1 and len(rep["passes"]) == 6
    # the rewritten model loads and computes what the original computes
    x = {"input": torch.rand(1, 10)}
    a = Model.load(paths["simple_linear"]).create_session(SessionOptions().with_optimization_level("O0")).run(x)
    b = Model.load(out).create_session(SessionOptions().with_optimization_level("O0")).run(x)
    torch.testing.assert_close(a["output"], b["output"], atol=1e-5, rtol=1e-5)
