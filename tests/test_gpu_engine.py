"""Serving engine on the GPU: kernel backend against the PyTorch operator backend."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(model, backend, graph=True, **kw):
    from ronn_b200.serving import EngineConfig, LLMEngine
    cfg = EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=256, num_blocks=128, dtype="bf16",
                       backend=backend, use_cuda_graph=graph, **kw)
    return LLMEngine(model, cfg, device=torch.device("cuda", 0))


def test_smoke_entry():
    import __graft_entry__ as g
    g.smoke()


def test_engine_matches_torch_backend():
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.serving import SamplingParams
    cfg = GPT2Config.tiny(n_layer=3, n_embd=256, n_head=4, vocab_size=1000, n_positions=256)
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16, seed=5))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 17, 64, 100, 33, 1, 16, 150, 9, 70)]
    outs = {}
    for backend in ("kernels", "torch"):
        eng = _engine(model, backend, graph=(backend == "kernels"))
        outs[backend] = eng.generate(prompts, SamplingParams(max_new_tokens=8))
    agree = sum(a == b for x, y in zip(outs["kernels"], outs["torch"]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs["kernels"])
    assert total == 80
    assert agree >= int(0.9 * total), (outs, agree)


def test_graph_and_eager_decode_agree():
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.serving import SamplingParams
    cfg = GPT2Config.tiny(n_layer=2, n_embd=128, n_head=2, vocab_size=512, n_positions=256)
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16, seed=6))
    prompts = [[3, 4, 5, 6], list(range(100, 140)), [9] * 17]
    a = _engine(model, "kernels", graph=True).generate(prompts, SamplingParams(max_new_tokens=10))
    b = _engine(model, "kernels", graph=False).generate(prompts, SamplingParams(max_new_tokens=10))
    assert a == b


def test_concurrent_part_batches_give_the_same_tokens():
    """A decode step split into part-batches on concurrent streams computes every row exactly as the single-batch
    step does (rows are independent and the per-row reduction order does not change)."""
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
    cfg = GPT2Config.tiny(n_layer=2, n_embd=256, n_head=4, vocab_size=1000, n_positions=128)
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16, seed=7))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1000, (int(n),), generator=g).tolist() for n in torch.randint(1, 40, (150,), generator=g)]
    outs = []
    for streams in (1, 2, 3):
        ecfg = EngineConfig(max_num_seqs=160, max_batch_tokens=2048, max_model_len=128, num_blocks=160 * 8, dtype="bf16",
                            backend="kernels", use_cuda_graph=True, decode_streams=streams, decode_split_min=32)
        eng = LLMEngine(model, ecfg, device=torch.device("cuda", 0))
        outs.append(eng.generate(prompts, SamplingParams(max_new_tokens=6)))
        if streams > 1:
            assert len(eng._part_streams) == streams
    assert outs[0] == outs[1] == outs[2]


def test_swap_preemption_on_the_device_cache():
    """With too few KV blocks for all sequences, preempted ones are copied to the host pool and back; the tokens match
    an engine that never preempts (up to bf16 ties: a resumed token goes through the prefill path)."""
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
    cfg = GPT2Config.tiny(n_layer=2, n_embd=128, n_head=2, vocab_size=512, n_positions=256)
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16, seed=8))
    prompts = [[3 + i] * 15 for i in range(4)]            # one block each at admission, three each by the end
    dev = torch.device("cuda", 0)
    roomy = LLMEngine(model, EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=256, num_blocks=64,
                                          dtype="bf16"), device=dev)
    want = roomy.generate(prompts, SamplingParams(max_new_tokens=30))
    tight = LLMEngine(model, EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=256, num_blocks=7,
                                          dtype="bf16", preemption="swap", num_cpu_blocks=16), device=dev)
    got = tight.generate(prompts, SamplingParams(max_new_tokens=30))
    st = tight.stats()
    assert st["swap_preemptions"] >= 1 and st["swapped_in_blocks"] == st["swapped_out_blocks"] > 0
    agree = sum(a == b for x, y in zip(got, want) for a, b in zip(x, y))
    assert agree >= int(0.9 * 120), (agree, got, want)


def test_non_greedy_decode_replays_a_cuda_graph_and_is_reproducible():
    """Sampling with temperature / top-k / top-p / repeat penalty runs on the device inside the decode graph: the
    engine never reads logits back, a seeded request draws the same tokens alone or in a batch, and a request with
    top_k = 1 equals the greedy one."""
    from ronn_b200 import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
    m = Model.from_graph(build_gpt2(GPT2Config.tiny(n_layer=2, n_embd=128, n_head=2), dtype=torch.bfloat16, seed=5))
    cfg = lambda: EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=128, num_blocks=64, dtype="bf16",
                               backend="kernels", use_cuda_graph=True)
    dev = torch.device("cuda", 0)
    prompt = [5, 9, 2, 7, 1, 3]
    sp = SamplingParams(max_new_tokens=12, temperature=0.9, top_k=40, top_p=0.95, repeat_penalty=1.2, seed=77)
    eng = LLMEngine(m, cfg(), device=dev)
    assert eng.device_sampling
    alone = eng.generate([prompt], sp)[0]
    assert any(k[2] for k in eng._graphs), "the non-greedy step must have been captured as a graph"
    eng2 = LLMEngine(m, cfg(), device=dev)
    others = SamplingParams(max_new_tokens=12, temperature=1.1, seed=3)
    ids = [eng2.add_request([4, 4, 8], others), eng2.add_request(prompt, sp), eng2.add_request([1, 2, 3, 4, 5, 6, 7], others)]
    while eng2.has_unfinished():
        eng2.step()
    assert eng2.requests[ids[1]].output_tokens == alone
    greedy = LLMEngine(m, cfg(), device=dev).generate([prompt], SamplingParams(max_new_tokens=12))[0]
    k1 = LLMEngine(m, cfg(), device=dev).generate([prompt], SamplingParams(max_new_tokens=12, temperature=0.8, top_k=1, seed=1))[0]
    assert k1 == greedy
    assert len(set(map(tuple, [alone, greedy]))) >= 1 and all(0 <= t < 512 for t in alone)


def test_engine_logits_match_an_fp32_reference_of_the_graph():
    """Not token agreement: the kernel backend's logits (prefill over paged KV, then a decode step on the cache it
    filled) against fp32 logits of the same ONNX graph computed by the CPU session, within bf16 rounding."""
    from ronn_b200 import SessionOptions
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    cfg = GPT2Config.tiny(n_layer=3, n_embd=256, n_head=4, vocab_size=1000, n_positions=256)
    g32 = build_gpt2(cfg, dtype=torch.float32, seed=5)
    ref = Model.from_graph(g32).create_session(SessionOptions().with_optimization_level("O0"))
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16, seed=5))
    eng = _engine(model, "kernels", graph=False)
    r = eng.runner
    gen = torch.Generator().manual_seed(2)
    for T in (37, 128):
        seq = torch.randint(0, 1000, (T + 1,), generator=gen)
        want = ref.run({"input_ids": seq[None, :]})["logits"][0]                    # [T + 1, vocab], fp32
        dev = torch.device("cuda", 0)
        nblk = (T + 1 + 15) // 16
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        blocks = list(range(40, 40 + nblk))
        slots = [blocks[p // 16] * 16 + p % 16 for p in range(T + 1)]
        b = {"token_ids": seq[:T].to(dev, torch.int32), "positions": torch.arange(T, dtype=torch.int32, device=dev),
             "slot_mapping": i32(slots[:T]), "token_item": torch.zeros(T, dtype=torch.int32, device=dev),
             "ctx_per_token": torch.arange(1, T + 1, dtype=torch.int32, device=dev), "seq_lens": i32([T]),
             "sample_index_clamped": torch.arange(T, dtype=torch.int32, device=dev),
             "block_tables": i32([blocks + [0] * (r.max_blocks_per_seq - nblk)])}
        got = r.forward(b, False, T, T, want_logits=True)[:, :1000].float().cpu()
        scale = float(want.abs().max())
        assert float((got - want[:T]).abs().max()) < 0.04 * scale, (T, float((got - want[:T]).abs().max()), scale)
        # one decode step on top of the cache the prefill wrote
        d = {"token_ids": seq[T:T + 1].to(dev, torch.int32), "positions": i32([T]), "slot_mapping": i32([slots[T]]),
             "token_item": i32([0]), "ctx_per_token": i32([T + 1]), "seq_lens": i32([T + 1]), "sample_index_clamped": i32([0]),
             "block_tables": b["block_tables"]}
        got1 = r.forward(d, True, 1, 1, want_logits=True)[:, :1000].float().cpu()
        assert float((got1[0] - want[T]).abs().max()) < 0.04 * scale
        assert int(got1[0].argmax()) == int(want[T].argmax()) or float(want[T].topk(2).values.diff().abs()) < 0.04 * scale


def test_chunked_prefill_and_prefix_hits_use_the_paged_tensor_core_kernel():
    """Prompts longer than a step's token budget continue in later steps, and a shared prefix is served from the
    cache: those steps attend through the paged tensor-core kernel and produce the tokens of the per-row paged kernel
    and of the operator backend."""
    from ronn_b200 import _native
    from ronn_b200.api.model import Model
    from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
    from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
    cfg = GPT2Config.tiny(n_layer=2, n_embd=256, n_head=4, vocab_size=1000, n_positions=1024)
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16, seed=11))
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 1000, (160,), generator=g).tolist()
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (700, 333, 129)]
    prompts += [shared + [5, 6, 7] * 20, shared + [9] * 70]
    outs = {}
    lib = _native.cuda()
    calls = {"n": 0}
    real = lib.ronn_fmha_paged
    lib.__dict__["ronn_fmha_paged"] = lambda *a: (calls.__setitem__("n", calls["n"] + 1), real(*a))[1]
    try:
        for name, backend, dense in (("tensor", "kernels", True), ("rows", "kernels", False), ("torch", "torch", False)):
            ec = EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=1024, num_blocks=512, dtype="bf16",
                              backend=backend, use_cuda_graph=(backend == "kernels"), enable_prefix_cache=True,
                              prefill_chunk=128, dense_prefill=dense)
            eng = LLMEngine(model, ec, device=torch.device("cuda", 0))
            outs[name] = eng.generate(prompts[:3], SamplingParams(max_new_tokens=6))
            outs[name] += eng.generate(prompts[3:4], SamplingParams(max_new_tokens=6))
            outs[name] += eng.generate(prompts[4:], SamplingParams(max_new_tokens=6))         # prefix hit
            if name == "tensor":
                assert calls["n"] >= 2 * 3, calls               # at least three continuation steps, two layers each
                n_tensor = calls["n"]
        assert calls["n"] == n_tensor                           # the other two engines never reach it
    finally:
        lib.__dict__["ronn_fmha_paged"] = real
    same = lambda a, b: sum(x == y for p, q in zip(outs[a], outs[b]) for x, y in zip(p, q))
    assert sum(len(x) for x in outs["tensor"]) == 30
    assert same("tensor", "rows") >= 27, outs
    assert same("tensor", "torch") >= 24, outs                  # a random tiny model has near ties in bf16
