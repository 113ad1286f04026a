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
