"""Models written by PyTorch's own ONNX exporter (not by the in-tree encoder) load and run: a transformer block and a
small CNN, opset 17, compared with the eager module at O0 and O3."""
import collections
import io
import warnings

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from ronn_b200 import Model, SessionOptions


class Block(nn.Module):
    def __init__(self, d=32, h=4):
        super().__init__()
        self.h = h
        self.emb = nn.Embedding(50, d)
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.o = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.f1, self.f2 = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

    def forward(self, ids):
        x = self.emb(ids)
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).chunk(3, -1)
        split = lambda t: t.reshape(B, T, self.h, D // self.h).transpose(1, 2)
        att = torch.softmax(split(q) @ split(k).transpose(-1, -2) / (D // self.h) ** 0.5, -1) @ split(v)
        x = x + self.o(att.transpose(1, 2).reshape(B, T, D))
        return x + self.f2(F.gelu(self.f1(self.ln2(x))))


class CNN(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.bn, self.c2 = nn.Conv2d(3, 8, 3, 2, 1), nn.BatchNorm2d(8), nn.Conv2d(8, 16, 3, 1, 1)
        self.fc = nn.Linear(16, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.bn(self.c1(x))), 2)
        x = F.relu(self.c2(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def _export(module, example, dynamic_axes=None, opset=17) -> bytes:
    """TorchScript-based exporter; its last step (attaching onnxscript functions) needs the `onnx` package, which these
    graphs do not use, so it is stubbed out when that package is absent."""
    try:
        from torch.onnx._internal.torchscript_exporter import onnx_proto_utils
    except Exception:
        pytest.skip("this PyTorch has no TorchScript ONNX exporter")
    try:
        import onnx  # noqa: F401
    except ImportError:
        onnx_proto_utils._add_onnxscript_fn = lambda proto, custom_opsets: proto
    buf = io.BytesIO()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            torch.onnx.export(module, (example,), buf, input_names=["x"], output_names=["y"], opset_version=opset,
                              dynamo=False, dynamic_axes={"x": dynamic_axes} if dynamic_axes else None)
        except Exception as e:                     # exporter unavailable in this build: nothing to test against
            pytest.skip(f"torch.onnx.export failed: {type(e).__name__}")
    return buf.getvalue()


@pytest.mark.parametrize("name", ["block", "cnn"])
def test_models_from_the_pytorch_exporter_run(name):
    torch.manual_seed(0)
    module, example = (Block().eval(), torch.randint(0, 50, (2, 6))) if name == "block" else \
        (CNN().eval(), torch.randn(2, 3, 16, 16))
    model = Model.from_bytes(_export(module, example))
    ops = collections.Counter(n.op_type for n in model.graph.nodes)
    assert ("LayerNormalization" in ops and "Softmax" in ops) if name == "block" else ("Conv" in ops and "Gemm" in ops)
    with torch.no_grad():
        want = module(example)
    for level in ("O0", "O3"):
        got = model.create_session(SessionOptions().with_optimization_level(level)).run({"x": example})["y"]
        torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


class UNetish(nn.Module):
    def __init__(self):
        super().__init__()
        self.down, self.gn = nn.Conv2d(3, 8, 3, 2, 1), nn.GroupNorm(2, 8)
        self.up, self.out = nn.ConvTranspose2d(8, 4, 2, 2), nn.Conv2d(4 + 3, 2, 1)

    def forward(self, x):
        h = self.up(F.silu(self.gn(self.down(x))))
        return self.out(torch.cat([h, x], 1))


class Upsample(nn.Module):
    def forward(self, x):
        return F.interpolate(x, scale_factor=2, mode="nearest") + \
            F.interpolate(x, scale_factor=2, mode="bilinear", align_corners=False)


class Misc(nn.Module):
    def forward(self, x):
        a = x.clamp(-1, 1).abs().sqrt() + torch.where(x > 0, x, torch.zeros_like(x)).mean(-1, keepdim=True)
        b = torch.cumsum(x, 1) * F.hardswish(x) + F.leaky_relu(x, 0.1) + F.elu(x)
        v, _ = torch.topk(x, 2, dim=-1)
        return a + b + v.sum(-1, keepdim=True) + F.log_softmax(x, -1) + x.max(-1, keepdim=True).values + \
            torch.tril(x @ x.transpose(-1, -2))[..., :1]


class SelfAttention(nn.Module):
    def __init__(self):
        super().__init__()
        self.m = nn.MultiheadAttention(16, 4, batch_first=True)

    def forward(self, x):
        return self.m(x, x, x, need_weights=False)[0]


class PixelOps(nn.Module):
    def forward(self, x):
        return F.pixel_unshuffle(F.pixel_shuffle(x, 2), 2) + F.instance_norm(x) + \
            F.avg_pool2d(x, 2, 1, padding=1, count_include_pad=False)[..., :4, :4]


class Recurrent(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, x):
        out, state = self.m(x)
        h = state[0] if isinstance(state, tuple) else state
        return out + 0.0 * h.sum()                 # keeps the final-state output of the operator in the graph


WIDER = {
    "unet": (UNetish, (1, 3, 8, 8), {"ConvTranspose", "InstanceNormalization"}),
    "upsample": (Upsample, (1, 2, 4, 4), {"Resize"}),
    "misc": (Misc, (3, 5), {"CumSum", "TopK", "Trilu", "HardSwish"}),
    "attention": (SelfAttention, (2, 5, 16), {"Softmax", "Gemm"}),
    "pixel": (PixelOps, (1, 8, 4, 4), {"DepthToSpace", "AveragePool"}),
    "gru": (lambda: Recurrent(nn.GRU(8, 8, batch_first=True)), (3, 4, 8), {"GRU"}),
    "gru_bidirectional": (lambda: Recurrent(nn.GRU(8, 6, bidirectional=True)), (3, 4, 8), {"GRU"}),
    "lstm": (lambda: Recurrent(nn.LSTM(8, 8, batch_first=True)), (3, 4, 8), {"LSTM"}),
    "lstm_two_layers_bidirectional": (lambda: Recurrent(nn.LSTM(8, 5, num_layers=2, bidirectional=True)), (3, 4, 8), {"LSTM"}),
    "rnn_relu": (lambda: Recurrent(nn.RNN(8, 7, nonlinearity="relu", batch_first=True)), (3, 4, 8), {"RNN"}),
}


@pytest.mark.parametrize("name", sorted(WIDER))
def test_wider_operator_coverage_through_the_exporter(name):
    torch.manual_seed(1)
    make, shape, expect_ops = WIDER[name]
    module, example = make().eval(), torch.randn(*shape)
    model = Model.from_bytes(_export(module, example))
    ops = {n.op_type for n in model.graph.nodes}
    assert expect_ops <= ops, (expect_ops, ops)
    with torch.no_grad():
        want = module(example)
    for level in ("O0", "O3"):
        got = model.create_session(SessionOptions().with_optimization_level(level)).run({"x": example})["y"]
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-5)


def test_dynamic_axes_run_at_other_sizes():
    """Symbolic dimensions keep their names, load as 0, and the session runs shapes other than the traced one."""
    torch.manual_seed(2)
    block, cnn = Block().eval(), CNN().eval()
    m1 = Model.from_bytes(_export(block, torch.randint(0, 50, (2, 6)), {0: "batch", 1: "sequence"}))
    assert [(t.shape, t.dim_params) for t in m1.inputs()] == [([0, 0], ["batch", "sequence"])]
    m2 = Model.from_bytes(_export(cnn, torch.randn(2, 3, 16, 16), {0: "batch", 2: "height", 3: "width"}))
    assert m2.inputs()[0].shape == [0, 3, 0, 0] and m2.inputs()[0].dim_params == ["batch", None, "height", "width"]
    for level in ("O0", "O3"):
        s1 = m1.create_session(SessionOptions().with_optimization_level(level))
        s2 = m2.create_session(SessionOptions().with_optimization_level(level))
        for ids in (torch.randint(0, 50, (2, 6)), torch.randint(0, 50, (3, 9)), torch.randint(0, 50, (1, 1))):
            with torch.no_grad():
                torch.testing.assert_close(s1.run({"x": ids})["y"], block(ids), atol=1e-5, rtol=1e-5)
        for img in (torch.randn(2, 3, 16, 16), torch.randn(1, 3, 24, 20)):
            with torch.no_grad():
                torch.testing.assert_close(s2.run({"x": img})["y"], cnn(img), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ["block", "cnn", "lstm"])
def test_exporter_models_survive_the_in_tree_encoder(name):
    """Decode with the in-tree codec, encode again, decode again: same graph, same numbers."""
    torch.manual_seed(3)
    if name == "block":
        module, example = Block().eval(), torch.randint(0, 50, (2, 6))
    elif name == "cnn":
        module, example = CNN().eval(), torch.randn(2, 3, 16, 16)
    else:
        module, example = Recurrent(nn.LSTM(8, 8, batch_first=True)).eval(), torch.randn(3, 4, 8)
    first = Model.from_bytes(_export(module, example))
    second = Model.from_bytes(first.to_bytes())
    assert [n.op_type for n in first.graph.nodes] == [n.op_type for n in second.graph.nodes]
    assert sorted(first.graph.initializers) == sorted(second.graph.initializers)
    a = first.create_session(SessionOptions()).run({"x": example})["y"]
    b = second.create_session(SessionOptions()).run({"x": example})["y"]
    torch.testing.assert_close(a, b, atol=0, rtol=0)


def test_exact_gelu_chain_becomes_one_node():
    """The exporter writes the exact GELU as Div, Erf, Add, Mul, Mul; O2 and above fold the chain into one Gelu node."""
    from ronn_b200.graph.optimizer import Optimizer
    import copy
    torch.manual_seed(4)
    block, ids = Block().eval(), torch.randint(0, 50, (2, 6))
    model = Model.from_bytes(_export(block, ids))
    g = copy.deepcopy(model.graph)
    before = [n.op_type for n in g.nodes]
    assert "Erf" in before and "Gelu" not in before
    Optimizer("O2").optimize(g)
    after = [n.op_type for n in g.nodes]
    assert "Erf" not in after and after.count("Gelu") == 1
    gelu = next(n for n in g.nodes if n.op_type == "Gelu")
    assert gelu.attr("approximate") == "none"
    with torch.no_grad():
        want = block(ids)
    got = model.create_session(SessionOptions().with_optimization_level("O3")).run({"x": ids})["y"]
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    # the other multiplication order: (x * 0.5) * (1 + erf(x / sqrt 2))
    from ronn_b200.core.types import DataType
    from ronn_b200.graph.ir import GraphBuilder
    b = GraphBuilder().add_input("x", [2, 8], DataType.F32).add_output("y", [2, 8], DataType.F32)
    for name, v in (("half", 0.5), ("one", 1.0), ("rsqrt2", 0.7071067811865476)):
        b.add_initializer(name, torch.tensor(v))
    b.add_op("Mul", ["x", "half"], ["hx"]).add_op("Mul", ["rsqrt2", "x"], ["sx"]).add_op("Erf", ["sx"], ["e"])
    b.add_op("Add", ["one", "e"], ["e1"]).add_op("Mul", ["hx", "e1"], ["y"])
    g2 = b.build()
    Optimizer("O2").optimize(g2)
    assert [n.op_type for n in g2.nodes] == ["Gelu"]
    x = torch.randn(2, 8)
    y = Model.from_graph(g2).create_session(SessionOptions().with_optimization_level("O0")).run({"x": x})["y"]
    torch.testing.assert_close(y, F.gelu(x), atol=1e-6, rtol=1e-6)
    # a chain whose intermediate value is used elsewhere must stay
    b3 = GraphBuilder().add_input("x", [2, 8], DataType.F32).add_output("y", [2, 8], DataType.F32)
    b3.add_output("e", [2, 8], DataType.F32)
    for name, v in (("half", 0.5), ("one", 1.0), ("sqrt2", 1.4142135623730951)):
        b3.add_initializer(name, torch.tensor(v))
    b3.add_op("Div", ["x", "sqrt2"], ["sx"]).add_op("Erf", ["sx"], ["e"]).add_op("Add", ["e", "one"], ["e1"])
    b3.add_op("Mul", ["x", "e1"], ["m"]).add_op("Mul", ["m", "half"], ["y"])
    g3 = b3.build()
    Optimizer("O2").optimize(g3)
    assert "Erf" in [n.op_type for n in g3.nodes]


def test_opset13_layernorm_chain_becomes_one_node():
    """Below opset 17 exporters write LayerNorm as nine primitive nodes (the reference's export scripts use opset 13);
    O2 folds each chain back into a LayerNormalization node."""
    import copy
    from ronn_b200.graph.optimizer import Optimizer
    torch.manual_seed(5)
    block, ids = Block().eval(), torch.randint(0, 50, (2, 6))
    model = Model.from_bytes(_export(block, ids, opset=13))
    before = collections.Counter(n.op_type for n in model.graph.nodes)
    assert before["ReduceMean"] == 4 and "LayerNormalization" not in before
    g = copy.deepcopy(model.graph)
    Optimizer("O2").optimize(g)
    after = collections.Counter(n.op_type for n in g.nodes)
    assert after["LayerNormalization"] == 2 and "ReduceMean" not in after and "Pow" not in after and after["Gelu"] == 1
    ln = next(n for n in g.nodes if n.op_type == "LayerNormalization")
    assert ln.attr("axis") == -1 and abs(ln.attr("epsilon") - 1e-5) < 1e-9
    with torch.no_grad():
        want = block(ids)
    for level in ("O0", "O2", "O3"):
        got = model.create_session(SessionOptions().with_optimization_level(level)).run({"x": ids})["y"]
        torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    # a mean over another axis is not a LayerNorm over the last one: the chain stays
    from ronn_b200.core.types import DataType
    from ronn_b200.graph.ir import GraphBuilder
    b = GraphBuilder().add_input("x", [2, 4, 8], DataType.F32).add_output("y", [2, 4, 8], DataType.F32)
    for name, v in (("two", torch.tensor(2.0)), ("eps", torch.tensor(1e-5)), ("g", torch.ones(8)), ("b", torch.zeros(8))):
        b.add_initializer(name, v)
    b.add_op("ReduceMean", ["x"], ["m"], axes=[1]).add_op("Sub", ["x", "m"], ["d"]).add_op("Pow", ["d", "two"], ["p"])
    b.add_op("ReduceMean", ["p"], ["v"], axes=[1]).add_op("Add", ["v", "eps"], ["ve"]).add_op("Sqrt", ["ve"], ["s"])
    b.add_op("Div", ["d", "s"], ["n"]).add_op("Mul", ["n", "g"], ["ng"]).add_op("Add", ["ng", "b"], ["y"])
    g2 = b.build()
    Optimizer("O2").optimize(g2)
    assert "LayerNormalization" not in [n.op_type for n in g2.nodes]


class MaskedEncoder(nn.Module):
    """DistilBERT-shaped layer: embeddings + positions, padding mask applied with masked_fill, post-LayerNorm."""

    def __init__(self, d=32, h=4, vocab=60, max_pos=16):
        super().__init__()
        self.h = h
        self.wte, self.wpe, self.eln = nn.Embedding(vocab, d), nn.Embedding(max_pos, d), nn.LayerNorm(d, eps=1e-12)
        self.q, self.k, self.v, self.o = (nn.Linear(d, d) for _ in range(4))
        self.ln1, self.ln2 = nn.LayerNorm(d, eps=1e-12), nn.LayerNorm(d, eps=1e-12)
        self.f1, self.f2 = nn.Linear(d, 2 * d), nn.Linear(2 * d, d)

    def forward(self, input_ids, attention_mask):
        B, T = input_ids.shape
        pos = torch.arange(T, device=input_ids.device).unsqueeze(0).expand(B, T)
        x = self.eln(self.wte(input_ids) + self.wpe(pos))
        D = x.shape[-1]
        split = lambda t: t.view(B, T, self.h, D // self.h).transpose(1, 2)
        q, k, v = split(self.q(x)) / (D // self.h) ** 0.5, split(self.k(x)), split(self.v(x))
        scores = q @ k.transpose(2, 3)
        mask = (attention_mask == 0).view(B, 1, 1, T).expand_as(scores)
        scores = scores.masked_fill(mask, torch.finfo(scores.dtype).min)
        ctx = (torch.softmax(scores, -1) @ v).transpose(1, 2).contiguous().view(B, T, D)
        x = self.ln1(self.o(ctx) + x)
        return self.ln2(self.f2(F.gelu(self.f1(x))) + x)


@pytest.mark.parametrize("opset", [13, 17])
def test_masked_encoder_with_two_inputs(opset):
    torch.manual_seed(6)
    module = MaskedEncoder().eval()
    ids = torch.randint(0, 60, (2, 8))
    mask = torch.ones(2, 8, dtype=torch.int64)
    mask[1, 5:] = 0
    try:
        from torch.onnx._internal.torchscript_exporter import onnx_proto_utils
    except Exception:
        pytest.skip("this PyTorch has no TorchScript ONNX exporter")
    try:
        import onnx  # noqa: F401
    except ImportError:
        onnx_proto_utils._add_onnxscript_fn = lambda proto, custom_opsets: proto
    buf = io.BytesIO()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            torch.onnx.export(module, (ids, mask), buf, input_names=["input_ids", "attention_mask"],
                              output_names=["last_hidden_state"], opset_version=opset, dynamo=False)
        except Exception as e:
            pytest.skip(f"torch.onnx.export failed: {type(e).__name__}")
    model = Model.from_bytes(buf.getvalue())
    assert model.input_names() == ["input_ids", "attention_mask"]
    with torch.no_grad():
        want = module(ids, mask)
    for level in ("O0", "O3"):
        sess = model.create_session(SessionOptions().with_optimization_level(level))
        got = sess.run({"input_ids": ids, "attention_mask": mask})["last_hidden_state"]
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-5)
        if level == "O3":
            # the exporter's MatMul / Div / masked_fill (a Where whose condition was expanded to the scores' shape) /
            # Softmax / MatMul became one fused attention node
            ops = [n.op_type for n in sess.graph().nodes]
            assert ops.count("ScaledDotProductAttention") == 1 and "Softmax" not in ops
        # rows that differ only in padded positions give the same output on the valid positions
        ids2 = ids.clone()
        ids2[1, 5:] = 7
        again = sess.run({"input_ids": ids2, "attention_mask": mask})["last_hidden_state"]
        torch.testing.assert_close(again[1, :5], got[1, :5], atol=2e-5, rtol=1e-5)


class ExportedGPT2(nn.Module):
    """GPT-2 the way the Hugging Face implementation computes it (Conv1D projections as x @ W + b with W [in, out],
    heads split with view + permute, causal mask from a tril buffer, gelu_new written out), small enough to export."""

    def __init__(self, vocab=211, n_pos=64, d=64, n_head=4, n_layer=2):
        super().__init__()
        self.d, self.h = d, n_head
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(n_pos, d)
        mk = lambda i, o: (nn.Parameter(torch.randn(i, o) * 0.08), nn.Parameter(torch.randn(o) * 0.02))
        self.blocks = nn.ModuleList()
        for _ in range(n_layer):
            b = nn.Module()
            b.ln_1, b.ln_2 = nn.LayerNorm(d), nn.LayerNorm(d)
            b.attn_w, b.attn_b = mk(d, 3 * d)
            b.proj_w, b.proj_b = mk(d, d)
            b.fc_w, b.fc_b = mk(d, 4 * d)
            b.out_w, b.out_b = mk(4 * d, d)
            self.blocks.append(b)
        self.ln_f = nn.LayerNorm(d)
        self.register_buffer("tril", torch.tril(torch.ones(n_pos, n_pos, dtype=torch.bool)).view(1, 1, n_pos, n_pos))

    def forward(self, input_ids):
        B, T = input_ids.shape
        pos = torch.arange(T, device=input_ids.device).unsqueeze(0)
        x = self.wte(input_ids) + self.wpe(pos)
        for b in self.blocks:
            qkv = torch.addmm(b.attn_b, b.ln_1(x).view(-1, self.d), b.attn_w).view(B, T, 3 * self.d)
            q, k, v = qkv.split(self.d, dim=2)
            heads = lambda t: t.view(B, T, self.h, self.d // self.h).permute(0, 2, 1, 3)
            w = torch.matmul(heads(q), heads(k).transpose(-1, -2)) / float(self.d // self.h) ** 0.5
            w = torch.where(self.tril[:, :, :T, :T], w, torch.full_like(w, -1e9))
            a = torch.matmul(torch.softmax(w, dim=-1), heads(v)).permute(0, 2, 1, 3).contiguous().view(B, T, self.d)
            x = x + torch.addmm(b.proj_b, a.view(-1, self.d), b.proj_w).view(B, T, self.d)
            hdn = torch.addmm(b.fc_b, b.ln_2(x).view(-1, self.d), b.fc_w)
            hdn = 0.5 * hdn * (1.0 + torch.tanh(0.7978845608028654 * (hdn + 0.044715 * torch.pow(hdn, 3.0))))
            x = x + torch.addmm(b.out_b, hdn, b.out_w).view(B, T, self.d)
        return self.ln_f(x)


@pytest.mark.parametrize("opset", [13, 17])
def test_exporter_written_gpt2_is_served_by_the_engine_with_matching_logits(opset):
    """A decoder that carries no in-tree metadata and exporter-chosen names is recognised from its operators; the
    engine's logits (paged KV, prefill then decode) equal the session's logits of the same graph at fp32 tolerance."""
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
    from ronn_b200.serving.graph_match import decoder_from_graph
    torch.manual_seed(3)
    module = ExportedGPT2().eval()
    ids = torch.randint(0, 211, (2, 7))
    model = Model.from_bytes(_export(module, ids, dynamic_axes={0: "batch", 1: "sequence"}, opset=opset))
    assert "ronn.arch" not in model.graph.metadata
    arch, init = decoder_from_graph(model.graph)
    assert (arch.n_layer, arch.hidden, arch.n_head, arch.ffn, arch.vocab, arch.max_pos) == (2, 64, 4, 256, 211, 64)
    torch.testing.assert_close(init["h.1.mlp.c_fc.weight"], module.blocks[1].fc_w.detach())
    sess = model.create_session(SessionOptions().with_optimization_level("O0"))
    eng = LLMEngine(model, EngineConfig(max_num_seqs=4, max_batch_tokens=64, max_model_len=64, num_blocks=32, dtype="fp32",
                                        backend="torch"), device="cpu")
    prompt = [5, 17, 200, 3, 3, 9]
    generated = eng.generate([prompt], SamplingParams(max_new_tokens=5))[0]
    # teacher forcing through the session: the token the engine chose at every step is the arg max of the session's
    # logits, and the runner's logits for the whole sequence equal the session's
    seq = prompt + generated
    hidden = sess.run({"x": torch.tensor([seq[:-1]])})["y"][0]
    logits = hidden @ module.wte.weight.detach().t()
    assert logits[len(prompt) - 1:].argmax(-1).tolist() == generated
    runner = eng.runner
    T = len(seq) - 1
    b = {"token_ids": torch.tensor(seq[:-1], dtype=torch.int32), "positions": torch.arange(T, dtype=torch.int32),
         "slot_mapping": torch.arange(T, dtype=torch.int32) + 16 * 20, "token_item": torch.zeros(T, dtype=torch.int32),
         "ctx_per_token": torch.arange(1, T + 1, dtype=torch.int32), "seq_lens": torch.tensor([T], dtype=torch.int32),
         "sample_index_clamped": torch.arange(T, dtype=torch.int32),
         "block_tables": torch.tensor([[20, 21, 22, 23]], dtype=torch.int32)}
    mine = runner.forward(b, False, T, T, want_logits=True)
    torch.testing.assert_close(mine[:, :211], logits, atol=2e-4, rtol=2e-4)
    with pytest.raises(Exception, match="four linear layers|not a decoder|position"):
        decoder_from_graph(Model.from_bytes(_export(Block().eval(), torch.randint(0, 50, (2, 6)))).graph)
