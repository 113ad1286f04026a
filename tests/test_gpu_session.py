"""GPU provider sessions against the CPU provider on the same ONNX graphs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_mlp_gpu_matches_cpu():
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.models.mlp784 import build_mlp784
    m = Model.from_graph(build_mlp784())
    x = torch.rand(4, 784)
    ref = m.create_session(SessionOptions().with_optimization_level("O0"))
    # batch dimension is free in the graph (MatMul broadcasting)
    want = ref.run({"input": x})["probs"]
    for lvl in ("O0", "O3"):
        s = m.create_session(SessionOptions().with_provider("gpu").with_optimization_level(lvl).with_dtype("bf16"))
        got = s.run({"input": x})["probs"].float().cpu()
        torch.testing.assert_close(got, want, atol=2e-2, rtol=5e-2)


def test_gpt2_session_gpu_matches_cpu():
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    cfg = GPT2Config.tiny(n_layer=2, n_embd=128, n_head=2, vocab_size=512, n_positions=64)
    m = Model.from_graph(build_gpt2(cfg, dtype=torch.float32, seed=2))
    ids = torch.randint(0, 512, (2, 24))
    want = m.create_session(SessionOptions().with_optimization_level("O0")).run({"input_ids": ids})["logits"]
    s = m.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3").with_dtype("bf16"))
    got = s.run({"input_ids": ids})["logits"].float().cpu()
    torch.testing.assert_close(got, want, atol=5e-2, rtol=5e-2)
    assert any(n.op_type == "FusedGemm" for n in s.graph().nodes)


def test_resnet18_gpu_o3_matches_cpu_o0():
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.models.resnet18 import build_resnet18
    m = Model.from_graph(build_resnet18(dtype=torch.float32, image=64, num_classes=40))
    x = torch.randn(4, 3, 64, 64)
    want = m.create_session(SessionOptions().with_optimization_level("O0")).run({"input": x})["logits"]
    s = m.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3").with_dtype("fp16"))
    got = s.run({"input": x})["logits"].float().cpu()
    assert sum(1 for n in s.graph().nodes if n.op_type == "FusedConv") == 17
    assert (got - want).abs().max() < 0.05 * want.abs().max()
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() >= 0.75
