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


def test_distilbert_gpu_graph_matches_cpu():
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert
    m = Model.from_graph(build_distilbert(DistilBertConfig.tiny(), dtype=torch.float32, seed=4))
    ids = torch.randint(0, 512, (3, 16))
    mask = torch.ones(3, 16, dtype=torch.int64)
    mask[1, 9:] = 0
    want = m.create_session(SessionOptions().with_optimization_level("O0")).run({"input_ids": ids, "attention_mask": mask})["last_hidden_state"]
    for graphed in (False, True):
        s = m.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3").with_dtype("bf16").with_cuda_graph(graphed))
        for _ in range(2):
            got = s.run({"input_ids": ids, "attention_mask": mask})["last_hidden_state"].float().cpu()
        torch.testing.assert_close(got, want, atol=8e-2, rtol=5e-2)


def test_bitnet_engine_gpu_kernels_vs_torch_backend():
    from ronn_b200 import Model
    from ronn_b200.models.bitnet_llama import BitNetConfig, build_bitnet_llama
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
    m = Model.from_graph(build_bitnet_llama(BitNetConfig.tiny(n_layer=2, hidden=256, n_head=2, ffn=512), dtype=torch.bfloat16, seed=9))
    prompts = [[1, 2, 3, 4, 5], list(range(30, 70)), [9] * 17]
    outs = {}
    for backend in ("kernels", "torch"):
        eng = LLMEngine(m, EngineConfig(max_num_seqs=4, max_batch_tokens=128, max_model_len=128, num_blocks=32, dtype="bf16",
                                        backend=backend, use_cuda_graph=(backend == "kernels")), device=torch.device("cuda", 0))
        outs[backend] = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    agree = sum(a == b for x, y in zip(outs["kernels"], outs["torch"]) for a, b in zip(x, y))
    assert agree >= 14, outs


def test_encoder_runner_kernels_match_operator_backend():
    from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert
    from ronn_b200.serving.encoder_runner import EncoderRunner
    graph = build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=256, n_heads=4, hidden_dim=512), dtype=torch.bfloat16, seed=4)
    ids = torch.randint(0, 512, (5, 48), device="cuda")
    mask = torch.ones(5, 48, dtype=torch.int64, device="cuda")
    mask[1, 30:] = 0
    mask[3, 5:] = 0
    got = EncoderRunner(graph, dtype=torch.bfloat16).forward(ids, mask)
    want = EncoderRunner(graph, dtype=torch.bfloat16, backend="torch").forward(ids, mask)
    for b, n in enumerate(mask.sum(1).tolist()):
        torch.testing.assert_close(got[b, :n].float(), want[b, :n].float(), atol=6e-2, rtol=5e-2)


@pytest.mark.parametrize("method", ["binary", "ternary", "asymmetric"])
def test_bitnet_provider_session_runs_the_bitlinear_kernel(method):
    """A BitNet-provider session compiles constant-weight MatMul / Gemm nodes to packed 2-bit weights and launches the
    tcgen05 integer kernel for them; the result equals the host integer oracle of the same quantised operands."""
    from ronn_b200 import Model, SessionOptions, _native
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.providers.bitnet.provider import BitNetExecutionProvider, BitNetProviderConfig
    from ronn_b200.providers.bitnet.quantization import QuantizationMethod, bitlinear_reference
    g = torch.Generator().manual_seed(11)
    K, H, N = 256, 320, 64
    b = GraphBuilder().add_input("x", [40, K]).add_output("y", [40, N])
    b.add_initializer("w1", torch.randn(K, H, generator=g) * 0.1).add_initializer("b1", torch.randn(H, generator=g) * 0.1)
    b.add_initializer("w2", torch.randn(H, N, generator=g) * 0.1)
    b.add_op("MatMul", ["x", "w1"], ["h0"]).add_op("Add", ["h0", "b1"], ["h1"]).add_op("Relu", ["h1"], ["h2"])
    b.add_op("MatMul", ["h2", "w2"], ["y"])
    x = torch.randn(40, K, generator=g).cuda().bfloat16()
    prov = BitNetExecutionProvider(BitNetProviderConfig(QuantizationMethod(method)))
    sess = Model.from_graph(b.build()).create_session(SessionOptions().with_provider(prov))
    lib = _native.cuda()
    calls = []
    real = lib.ronn_bitlinear
    lib.__dict__["ronn_bitlinear"] = lambda *a: (calls.append(1), real(*a))[1]
    try:
        y = sess.run({"x": x})["y"]
    finally:
        lib.__dict__["ronn_bitlinear"] = real
    assert len(calls) == 2                                  # one launch of the integer kernel per linear layer
    # oracle: the same packed weights and the same per-token int8 activations, evaluated exactly on the host
    p1, p2 = (prov.packed_weights[("w1", False)], prov.packed_weights[("w2", False)])
    h = bitlinear_reference(x.cpu(), p1.packed.cpu(), p1.scale, None, p1.k_padded, p1.n_padded)[:, :p1.n].float()
    h = torch.relu(h + b.build().initializers["b1"].float()).bfloat16()
    ref = bitlinear_reference(h, p2.packed.cpu(), p2.scale, None, p2.k_padded, p2.n_padded)[:, :p2.n].float()
    torch.testing.assert_close(y.float().cpu(), ref, atol=0.08 * float(ref.abs().max()), rtol=5e-2)


def test_hrm_system1_session_launches_bitlinear():
    """The HRM router's fast path is a BitNet-provider session: a low-complexity input is served by the packed kernel."""
    from ronn_b200 import Model, _native
    from ronn_b200.hrm.router import RoutingStrategy
    from ronn_b200.models.mlp784 import build_mlp784
    s = Model.from_graph(build_mlp784()).create_session(enable_hrm=True)
    s._router.hrm.router.set_strategy(RoutingStrategy.ALWAYS_SYSTEM1)
    lib = _native.cuda()
    calls = []
    real = lib.ronn_bitlinear
    lib.__dict__["ronn_bitlinear"] = lambda *a: (calls.append(1), real(*a))[1]
    try:
        out = s.run({"input": torch.rand(1, 784)})
    finally:
        lib.__dict__["ronn_bitlinear"] = real
    assert out["probs"].shape == (1, 10) and abs(float(out["probs"].float().sum()) - 1) < 1e-2
    assert len(calls) == 2


def test_gpu_session_runs_elementwise_chains_and_attention_on_kernels():
    """O3 on the GPU provider: a chain of element-wise nodes is ONE launch of the chain kernel, and Attention nodes with
    a key-padding mask run the tensor-core attention kernel on the fused QKV projection (no library attention)."""
    from ronn_b200 import Model, SessionOptions, _native
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert
    lib = _native.cuda()

    def counting(names):
        counts = {n: 0 for n in names}
        saved = {n: getattr(lib, n) for n in names}
        for n in names:
            lib.__dict__[n] = (lambda real, key: (lambda *a: (counts.__setitem__(key, counts[key] + 1), real(*a))[1]))(saved[n], n)
        return counts, saved

    g = torch.Generator().manual_seed(2)
    b = GraphBuilder().add_input("x", [64, 256]).add_output("y", [64, 256])
    b.add_initializer("bias", torch.randn(256, generator=g)).add_initializer("w", torch.randn(64, 256, generator=g))
    b.add_op("Add", ["x", "bias"], ["a"]).add_op("Relu", ["a"], ["r"]).add_op("Mul", ["r", "w"], ["m"]).add_op("Tanh", ["m"], ["y"])
    graph = b.build()
    x = torch.randn(64, 256, generator=g)
    want = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level("O0")).run({"x": x})["y"]
    sess = Model.from_graph(graph).create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3").with_dtype("bf16"))
    assert [n.op_type for n in sess.graph().nodes] == ["FusedElementwise"]
    counts, saved = counting(["ronn_fused_elementwise", "ronn_unary", "ronn_binary"])
    try:
        got = sess.run({"x": x})["y"].float().cpu()
    finally:
        for n, f in saved.items():
            lib.__dict__[n] = f
    assert counts == {"ronn_fused_elementwise": 1, "ronn_unary": 0, "ronn_binary": 0}
    torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)

    m = Model.from_graph(build_distilbert(DistilBertConfig.tiny(n_layers=2, dim=256, n_heads=4, hidden_dim=512), dtype=torch.bfloat16, seed=4))
    ids = torch.randint(0, 512, (5, 48))
    mask = torch.ones(5, 48, dtype=torch.int64)
    mask[1, 30:] = 0
    mask[3, 5:] = 0
    want = m.create_session(SessionOptions().with_optimization_level("O0")).run({"input_ids": ids, "attention_mask": mask})["last_hidden_state"]
    s = m.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3").with_dtype("bf16"))
    counts, saved = counting(["ronn_fmha", "ronn_gemm"])
    try:
        got = s.run({"input_ids": ids, "attention_mask": mask})["last_hidden_state"].float().cpu()
    finally:
        for n, f in saved.items():
            lib.__dict__[n] = f
    assert counts["ronn_fmha"] == 2 and counts["ronn_gemm"] == 2 * 4        # fused QKV + out + two MLP per layer
    for bi, n in enumerate(mask.sum(1).tolist()):
        torch.testing.assert_close(got[bi, :n], want[bi, :n].float(), atol=8e-2, rtol=5e-2)


def test_attention_core_written_in_primitives_runs_the_tensor_core_kernel():
    """A graph that spells attention out (projection, Reshape, Transpose, MatMul, Div, Softmax, MatMul, Transpose,
    Reshape: what exporters write) is fused to one ScaledDotProductAttention node at O2+, and on the GPU provider that
    node launches the tcgen05 attention kernel; with a mask it takes the library's fused attention.  Both against the
    fp32 CPU session of the unfused graph."""
    import math

    from ronn_b200 import Model, SessionOptions, _native
    from ronn_b200.graph.ir import GraphBuilder
    B, S, H, D = 3, 160, 4, 64
    g = torch.Generator().manual_seed(3)

    def build(masked):
        b = GraphBuilder().add_input("x", [B, S, H * D]).add_output("y", [B, S, H * D])
        if masked:
            b.add_input("m", [B, 1, 1, S])
        for nm in ("q", "k", "v"):
            b.add_initializer("w" + nm, torch.randn(H * D, H * D, generator=g) * 0.05)
            b.add_op("MatMul", ["x", "w" + nm], [nm + "0"])
            b.add_initializer("shape_" + nm, torch.tensor([B, S, H, D]))
            b.add_op("Reshape", [nm + "0", "shape_" + nm], [nm + "1"])
        b.add_op("Transpose", ["q1"], ["q2"], perm=[0, 2, 1, 3]).add_op("Transpose", ["k1"], ["k2"], perm=[0, 2, 3, 1])
        b.add_op("Transpose", ["v1"], ["v2"], perm=[0, 2, 1, 3])
        b.add_initializer("c", torch.tensor(math.sqrt(D)))
        b.add_op("MatMul", ["q2", "k2"], ["s0"]).add_op("Div", ["s0", "c"], ["s1"])
        cur = "s1"
        if masked:
            b.add_op("Add", ["s1", "m"], ["s2"])
            cur = "s2"
        b.add_op("Softmax", [cur], ["p"], axis=-1).add_op("MatMul", ["p", "v2"], ["o0"])
        b.add_op("Transpose", ["o0"], ["o1"], perm=[0, 2, 1, 3])
        b.add_initializer("shape_o", torch.tensor([B, S, H * D]))
        b.add_op("Reshape", ["o1", "shape_o"], ["y"])
        return b.build()

    lib = _native.cuda()
    x = torch.randn(B, S, H * D, generator=g)
    for masked in (False, True):
        graph = build(masked)
        feeds = {"x": x}
        if masked:
            m = torch.zeros(B, 1, 1, S)
            m[1, :, :, 100:] = -1e4
            feeds["m"] = m
        want = Model.from_graph(graph).create_session(SessionOptions().with_optimization_level("O0")).run(feeds)["y"]
        sess = Model.from_graph(graph).create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3").with_dtype("bf16"))
        ops = [n.op_type for n in sess.graph().nodes]
        assert ops.count("ScaledDotProductAttention") == 1 and "Softmax" not in ops
        calls = {"n": 0}
        real = lib.ronn_fmha
        lib.__dict__["ronn_fmha"] = lambda *a: (calls.__setitem__("n", calls["n"] + 1), real(*a))[1]
        try:
            got = sess.run(feeds)["y"].float().cpu()
        finally:
            lib.__dict__["ronn_fmha"] = real
        assert calls["n"] == (0 if masked else 1)
        torch.testing.assert_close(got, want, atol=4e-2, rtol=4e-2)


def test_paged_attention_node_runs_the_decode_kernel():
    """com.ronn::PagedAttention through a GPU session: the node takes the decode attention kernel (counted) and agrees
    with the operator's CPU definition."""
    import math
    from ronn_b200 import Model, SessionOptions, _native
    from ronn_b200.core.types import DataType
    from ronn_b200.graph.ir import GraphBuilder
    heads, kv_heads, d, rows, max_blocks, nblocks = 8, 4, 64, 6, 5, 40
    g = torch.Generator().manual_seed(3)
    kc = (torch.randn(nblocks, kv_heads, 16, d, generator=g) * 0.5).bfloat16()
    vc = (torch.randn(nblocks, kv_heads, 16, d, generator=g) * 0.5).bfloat16()
    bt = torch.randperm(nblocks, generator=g)[: rows * max_blocks].reshape(rows, max_blocks).to(torch.int32)
    ctx = torch.tensor([1, 16, 17, 80, 0, 45], dtype=torch.int32)
    q = torch.randn(rows, heads * d, generator=g).bfloat16()
    b = GraphBuilder()
    b.add_input("q", [rows, heads * d], DataType.BF16).add_input("kc", list(kc.shape), DataType.BF16)
    b.add_input("vc", list(vc.shape), DataType.BF16).add_input("bt", list(bt.shape), DataType.I32)
    b.add_input("ctx", [rows], DataType.I32).add_output("y", [rows, heads * d], DataType.BF16)
    b.add_op("PagedAttention", ["q", "kc", "vc", "bt", "ctx"], ["y"], domain="com.ronn", num_heads=heads, kv_heads=kv_heads)
    model = Model.from_graph(b.build())
    feeds = {"q": q, "kc": kc, "vc": vc, "bt": bt, "ctx": ctx}
    want = model.create_session(SessionOptions().with_optimization_level("O0")).run(feeds)["y"].float()
    sess = model.create_session(SessionOptions().with_provider("gpu").with_optimization_level("O3"))
    lib = _native.cuda()
    calls = {"n": 0}
    real = lib.ronn_paged_attention
    lib.__dict__["ronn_paged_attention"] = lambda *a: (calls.__setitem__("n", calls["n"] + 1), real(*a))[1]
    try:
        got = sess.run(feeds)["y"].float().cpu()
    finally:
        lib.__dict__["ronn_paged_attention"] = real
    assert calls["n"] == 1
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)
    assert float(got[4].abs().max()) == 0.0


def test_graph_session_inputs_live_in_the_provider_device_pool():
    """A CUDA-graph session stages its inputs in buffers from the provider's device pool, which counts them against
    ``memory_limit`` and reports them in its statistics."""
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.graph.ir import GraphBuilder
    from ronn_b200.providers.gpu import GpuExecutionProvider, GpuProviderConfig
    prov = GpuExecutionProvider(GpuProviderConfig(memory_limit=1 << 20))
    b = GraphBuilder().add_input("x", [32, 128]).add_output("y", [32, 128])
    b.add_op("Relu", ["x"], ["y"])
    sess = Model.from_graph(b.build()).create_session(
        SessionOptions().with_provider(prov).with_optimization_level("O1").with_cuda_graph(True))
    x = torch.randn(32, 128)
    for _ in range(3):
        y = sess.run({"x": x})["y"]
    torch.testing.assert_close(y.float().cpu(), torch.relu(x))
    pool = prov.get_allocator()
    st = pool.stats()
    assert st.live_buffers == 1 and st.allocated_bytes == 32 * 128 * 4          # one staging buffer, made once
    t = pool.tensor((256, 256), torch.float32)                                  # 256 KB more
    assert t.is_cuda and pool.get_memory_info().total_bytes == 1 << 20
    with pytest.raises(Exception, match="limit"):
        pool.tensor((1024, 1024), torch.float32)
    pool.release(t)
    prov.shutdown()
    assert pool.stats().pooled_buffers == 0
