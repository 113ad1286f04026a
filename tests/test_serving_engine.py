"""Scheduler / block manager / continuous-batching engine on CPU (PyTorch operator backend)."""
import numpy as np
import pytest
import torch

from ronn_b200 import Model
from ronn_b200.api.errors import SessionError
from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
from ronn_b200.serving import EngineConfig, FinishReason, LLMEngine, Priority, RequestState, SamplingParams
from ronn_b200.serving.scheduler import PLAN_DECODE, PLAN_NONE, PLAN_PREFILL, HostBatchBuffers, Scheduler


@pytest.fixture(scope="module")
def tiny():
    return Model.from_graph(build_gpt2(GPT2Config.tiny(), dtype=torch.float32, seed=1))


def engine(model, **kw):
    cfg = dict(max_num_seqs=4, max_batch_tokens=64, max_model_len=128, num_blocks=32, dtype="fp32", backend="torch")
    cfg.update(kw)
    return LLMEngine(model, EngineConfig(**cfg), device="cpu")


def reference_greedy(model, prompt, n):
    sess = model.create_session(optimization_level="O0")
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(sess.run({"input_ids": torch.tensor([toks])})["logits"][0, -1].argmax()))
    return toks[len(prompt):]


def drain(s, buf, token=7):
    steps = []
    while True:
        k = s.schedule()
        if k == PLAN_NONE:
            break
        sb = s.fill(buf, k)
        steps.append((k, sb.n_items, sb.n_tokens))
        s.commit(np.full(sb.n_items, token, dtype=np.int32))
    return steps


def test_scheduler_plan_layout():
    s = Scheduler(16, 64, 4, 256)
    s.add(1, list(range(100, 120)), 3)
    s.add(2, list(range(5)), 2)
    buf = HostBatchBuffers(256, 4, 8, False)
    assert s.schedule() == PLAN_PREFILL
    sb = s.fill(buf, PLAN_PREFILL)
    assert (sb.n_items, sb.n_tokens) == (2, 25) and sb.req_ids.tolist() == [1, 2]
    assert buf.field("q_start")[:3].tolist() == [0, 20, 25] and buf.field("seq_lens")[:2].tolist() == [20, 5]
    assert buf.field("sample_index")[:2].tolist() == [19, 24]
    assert buf.field("token_ids")[:3].tolist() == [100, 101, 102] and buf.field("positions")[18:22].tolist() == [18, 19, 0, 1]
    b1, b2 = s.blocks(1), s.blocks(2)
    assert len(b1) == 2 and len(b2) == 1 and len(set(b1 + b2)) == 3
    slots = buf.field("slot_mapping")[:25]
    assert slots[0] == b1[0] * 16 and slots[16] == b1[1] * 16 and slots[20] == b2[0] * 16
    assert buf.field("token_item")[:25].tolist() == [0] * 20 + [1] * 5
    assert buf.field("block_tables")[:8].tolist()[:2] == b1 and buf.field("block_tables")[2] == -1
    fin = s.commit(np.array([55, 66], dtype=np.int32))
    assert fin.tolist() == [0, 0] and s.state(1) == RequestState.DECODING
    assert s.schedule() == PLAN_DECODE
    sb = s.fill(buf, PLAN_DECODE)
    assert sb.n_tokens == 2 and buf.field("token_ids")[:2].tolist() == [55, 66] and buf.field("positions")[:2].tolist() == [20, 5]
    fin = s.commit(np.array([1, 2], dtype=np.int32))
    assert fin.tolist() == [0, 2] and s.state(2) == RequestState.FINISHED and s.tokens(2) == [0, 1, 2, 3, 4, 66, 2]
    drain(s, buf)
    assert s.num_free_blocks == 64 and s.stats()["finished"] == 2


def test_scheduler_admission_limits_and_errors():
    s = Scheduler(16, 8, 2, 32, max_blocks_per_seq=4)
    with pytest.raises(SessionError, match="never fit"):
        s.add(1, list(range(60)), 10)                 # exceeds max_blocks_per_seq * 16
    with pytest.raises(SessionError, match="never fit"):
        s.add(1, list(range(30)), 10)                 # exceeds the token budget without chunking
    s.add(1, list(range(20)), 2)
    with pytest.raises(SessionError, match="already exists"):
        s.add(1, [1], 1)
    s.add(2, list(range(20)), 2)
    s.add(3, list(range(4)), 2)
    buf = HostBatchBuffers(64, 2, 4, False)
    assert s.schedule() == PLAN_PREFILL
    sb = s.fill(buf, PLAN_PREFILL)
    assert sb.n_items == 1                            # 20 + 20 > 32 tokens: only one prompt fits the budget
    s.commit(np.array([9], dtype=np.int32))
    s.schedule()
    sb = s.fill(buf, PLAN_PREFILL)
    assert sb.req_ids.tolist() == [2] and s.num_waiting == 1    # max_num_seqs = 2 keeps request 3 waiting
    s.commit(np.array([9], dtype=np.int32))
    assert s.schedule() == PLAN_DECODE


def test_scheduler_preemption_recompute_and_priority():
    s = Scheduler(16, 6, 4, 256, policy="priority")
    s.add(1, list(range(30)), 40, priority=int(Priority.LOW))
    s.add(2, list(range(30)), 40, priority=int(Priority.CRITICAL))
    buf = HostBatchBuffers(256, 4, 8, False)
    s.schedule()
    sb = s.fill(buf, PLAN_PREFILL)
    assert sb.req_ids.tolist() == [2, 1]              # critical first
    s.commit(np.array([5, 5], dtype=np.int32))
    pre = 0
    for _ in range(30):                               # both sequences need a fourth block at token 49: only 6 exist
        k = s.schedule()
        sb = s.fill(buf, k)
        s.commit(np.full(sb.n_items, 5, dtype=np.int32))
        pre = s.preemptions(1)
        if pre:
            break
    assert pre == 1 and s.state(1) == RequestState.PREEMPTED and s.preemptions(2) == 0
    assert s.stats()["preemptions"] == 1 and len(s.blocks(1)) == 0
    n_before = len(s.tokens(1))
    assert n_before > 30                              # generated tokens are kept and recomputed on resume
    s.cancel(2)
    assert s.state(2) == RequestState.CANCELLED
    assert s.schedule() == PLAN_PREFILL
    sb = s.fill(buf, PLAN_PREFILL)
    assert sb.req_ids.tolist() == [1] and sb.n_tokens == n_before


def test_scheduler_preemption_swap_keeps_the_cache():
    s = Scheduler(16, 6, 4, 256, policy="priority")
    s.set_preemption("swap", 8)
    s.add(1, list(range(30)), 40, priority=int(Priority.LOW))
    s.add(2, list(range(30)), 40, priority=int(Priority.CRITICAL))
    buf = HostBatchBuffers(256, 4, 8, False)
    s.schedule()
    s.fill(buf, PLAN_PREFILL)
    s.commit(np.array([5, 5], dtype=np.int32))
    blocks_before = []
    for _ in range(30):
        blocks_before = s.blocks(1)
        k = s.schedule()
        if s.preemptions(1):
            break
        sb = s.fill(buf, k)
        s.commit(np.full(sb.n_items, 5, dtype=np.int32))
    o_src, o_dst, i_src, i_dst = s.swaps()
    n_tok = len(s.tokens(1))
    # the victim's cached tokens (all but the one sampled last) went to the host pool, block by block
    assert s.state(1) == RequestState.PREEMPTED and len(s.blocks(1)) == 0
    assert o_src.tolist() == blocks_before[:len(o_src)] and len(o_src) == -(-(n_tok - 1) // 16) and len(i_src) == 0
    assert sorted(o_dst.tolist()) == sorted(set(o_dst.tolist())) and all(0 <= c < 8 for c in o_dst)
    st = s.swap_stats()
    assert st["swap_preemptions"] == 1 and st["swapped_out_blocks"] == len(o_src) and st["free_cpu_blocks"] == 8 - len(o_src)
    sb = s.fill(buf, PLAN_DECODE)
    s.commit(np.full(sb.n_items, 5, dtype=np.int32))
    s.cancel(2)
    # resume: the blocks come back and only the last token is computed (no recompute of the prompt)
    assert s.schedule() == PLAN_PREFILL
    o2, _, i_src2, i_dst2 = s.swaps()
    sb = s.fill(buf, PLAN_PREFILL)
    assert len(o2) == 0 and i_src2.tolist() == o_dst.tolist() and i_dst2.tolist() == s.blocks(1)[:len(i_dst2)]
    assert sb.req_ids.tolist() == [1] and sb.n_tokens == 1 and int(buf.field("positions")[0]) == n_tok - 1
    s.commit(np.array([5], dtype=np.int32))
    assert s.state(1) == RequestState.DECODING
    s.schedule()                                        # host blocks are reusable from the next step on
    assert s.swap_stats()["free_cpu_blocks"] == 8 and s.swap_stats()["swapped_in_blocks"] == len(i_src2)
    # cancelling a swapped-out request returns its host blocks; a full host pool falls back to recompute
    t = Scheduler(16, 6, 4, 256)
    t.set_preemption("swap", 1)
    t.add(1, list(range(30)), 40)
    t.add(2, list(range(30)), 40)
    t.schedule(); t.fill(buf, PLAN_PREFILL); t.commit(np.array([5, 5], dtype=np.int32))
    for _ in range(30):
        k = t.schedule()
        if t.stats()["preemptions"]:
            break
        sb = t.fill(buf, k)
        t.commit(np.full(sb.n_items, 5, dtype=np.int32))
    assert t.swap_stats()["swap_preemptions"] == 0 and len(t.swaps()[0]) == 0      # 3 blocks do not fit a pool of 1
    with pytest.raises(Exception):
        t.set_preemption("swap", 4)                     # not on a scheduler that has requests
    with pytest.raises(Exception):
        Scheduler(16, 6, 4, 256).set_preemption("sometimes", 4)


@pytest.mark.parametrize("mode", ["swap", "auto"])
def test_engine_swap_preemption_keeps_outputs(tiny, mode):
    grow = [[3 + i] * 15 for i in range(4)]            # one block each at admission, three each by the end
    want = [reference_greedy(tiny, p, 30) for p in grow]
    tight = engine(tiny, num_blocks=7, preemption=mode, num_cpu_blocks=16, swap_min_tokens=8)
    got = tight.generate(grow, SamplingParams(max_new_tokens=30))
    st = tight.stats()
    assert got == want and st["preemptions"] >= 1
    assert st["swap_preemptions"] >= 1 and st["swapped_in_blocks"] == st["swapped_out_blocks"] > 0
    assert st["swapped_blocks"] == 2 * st["swapped_out_blocks"] and st["free_cpu_blocks"] == 16
    # "auto" below its threshold recomputes instead
    lazy = engine(tiny, num_blocks=7, preemption="auto", num_cpu_blocks=16, swap_min_tokens=10_000)
    assert lazy.generate(grow, SamplingParams(max_new_tokens=30)) == want
    assert lazy.stats()["swap_preemptions"] == 0 and lazy.stats()["preemptions"] >= 1


def test_prefix_cache_shares_blocks():
    s = Scheduler(16, 32, 4, 256, enable_prefix_cache=True)
    common = list(range(40))
    s.add(1, common + [100, 101], 2)
    buf = HostBatchBuffers(256, 4, 8, False)
    drain(s, buf)
    s.add(2, common + [200, 201, 202], 2)
    assert s.schedule() == PLAN_PREFILL
    sb = s.fill(buf, PLAN_PREFILL)
    assert sb.n_tokens == 43 - 32                     # two full blocks (32 tokens) come from the cache
    assert buf.field("positions")[0] == 32 and s.stats()["prefix_hit_blocks"] == 2
    shared = s.blocks(2)[:2]
    s.add(3, common + [300], 2)
    s.commit(np.array([1], dtype=np.int32))
    s.schedule()
    s.fill(buf, PLAN_PREFILL)
    assert s.blocks(3)[:2] == shared and s.block_ref(shared[0]) == 2


def test_engine_matches_single_sequence_reference(tiny):
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7], list(range(20, 45)), [100, 101], [5] * 18, [7, 7, 7]]
    eng = engine(tiny)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    for p, o in zip(prompts, outs):
        assert o == reference_greedy(tiny, p, 6)
    st = eng.stats()
    assert st["requests_finished"] == 6 and st["generated_tokens"] == 36 and st["preemptions"] == 0
    assert all(r.finish_reason == FinishReason.MAX_TOKENS and r.ttft is not None for r in eng.requests.values())
    assert "ronn_generated_tokens 36" in eng.metrics.prometheus()


def test_engine_chunked_prefill_and_preemption_keep_outputs(tiny):
    prompts = [list(range(3, 40)), list(range(50, 75)), list(range(90, 120)), [4, 5, 6]]
    want = [reference_greedy(tiny, p, 12) for p in prompts]
    chunked = engine(tiny, prefill_chunk=8, max_batch_tokens=16).generate(prompts, SamplingParams(max_new_tokens=12))
    assert chunked == want
    grow = [[3 + i] * 15 for i in range(4)]            # one block each at admission, three each by the end
    want_grow = [reference_greedy(tiny, p, 30) for p in grow]
    tight = engine(tiny, num_blocks=7)                 # 12 blocks would be needed to finish all four together
    got = tight.generate(grow, SamplingParams(max_new_tokens=30))
    assert got == want_grow and tight.stats()["preemptions"] >= 1
    cached = engine(tiny, enable_prefix_cache=True)
    same = [list(range(3, 40)) + [7], list(range(3, 40)) + [9]]
    a = cached.generate([same[0]], SamplingParams(max_new_tokens=5))
    b = cached.generate([same[1]], SamplingParams(max_new_tokens=5))
    assert a[0] == reference_greedy(tiny, same[0], 5) and b[0] == reference_greedy(tiny, same[1], 5)
    assert cached.stats()["prefix_hit_blocks"] == 2


def test_engine_eos_stop_cancel_and_limits(tiny):
    first = reference_greedy(tiny, [1, 2, 3], 3)
    eng = engine(tiny, eos_token_id=first[0])
    rid = eng.add_request([1, 2, 3], SamplingParams(max_new_tokens=10))
    while eng.has_unfinished():
        eng.step()
    r = eng.requests[rid]
    assert r.output_tokens == first[:1] and r.finish_reason == FinishReason.EOS_TOKEN
    eng2 = engine(tiny)
    rid = eng2.add_request([1, 2, 3], SamplingParams(max_new_tokens=10, stop_sequences=[first[0:2]]))
    while eng2.has_unfinished():
        eng2.step()
    assert eng2.requests[rid].finish_reason == FinishReason.STOP_SEQUENCE and eng2.requests[rid].output_tokens == first[:2]
    eng3 = engine(tiny)
    rid = eng3.add_request([1, 2, 3], SamplingParams(max_new_tokens=50))
    eng3.step()
    assert eng3.cancel(rid) and not eng3.has_unfinished() and eng3.requests[rid].finish_reason == FinishReason.CANCELLED
    assert eng3.sched.num_free_blocks == 32
    with pytest.raises(SessionError, match="max_model_len"):
        eng3.add_request(list(range(120)), SamplingParams(max_new_tokens=20))
    with pytest.raises(SessionError, match="empty"):
        eng3.add_request([])
    seen = []
    eng3.on_token = lambda req, tok: seen.append(tok)
    out = eng3.generate([[5, 6]], SamplingParams(max_new_tokens=3))
    assert seen == out[0]


def test_engine_sampling_is_seeded(tiny):
    p = SamplingParams(max_new_tokens=8, temperature=0.9, top_k=20, top_p=0.9, repeat_penalty=1.1, seed=11)
    a = engine(tiny).generate([[1, 2, 3, 4]], p)
    b = engine(tiny).generate([[1, 2, 3, 4]], p)
    assert a == b and len(a[0]) == 8


def test_failed_step_requeues_requests(tiny):
    eng = engine(tiny)
    eng.add_request([1, 2, 3, 4], SamplingParams(max_new_tokens=4))
    orig = eng.runner.forward
    calls = {"n": 0}

    def flaky(*a, **k):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("injected host-side failure")
        return orig(*a, **k)
    eng.runner.forward = flaky
    eng.step()
    with pytest.raises(RuntimeError, match="injected"):
        eng.step()
    assert eng.metrics.failed_steps == 1 and eng.sched.num_waiting == 1      # back in the queue for recompute
    while eng.has_unfinished():
        eng.step()
    assert list(eng.requests.values())[0].output_tokens == reference_greedy(tiny, [1, 2, 3, 4], 4)


def test_dense_attention_plan_layout():
    from ronn_b200.ops.kernels import dense_attention_plan
    p = dense_attention_plan([1, 5, 128, 129], "cpu")
    assert p["seq_start"].tolist() == [0, 1, 6, 134]
    assert p["max_len"] == 129 and p["n_seq"] == 4
    q = dense_attention_plan([100, 7], "cpu", row_lens=[128, 128])   # padded batch: rows advance by the padded length
    assert q["seq_start"].tolist() == [0, 128] and q["kv_len"].tolist() == [100, 7]


def test_part_batch_split_is_off_on_cpu_and_for_small_batches():
    eng = _tiny_engine() if "_tiny_engine" in globals() else None
    if eng is None:
        import torch
        from ronn_b200.api.model import Model
        from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
        from ronn_b200.serving import EngineConfig, LLMEngine
        cfg = GPT2Config.tiny(n_layer=1, n_embd=64, n_head=2, vocab_size=128, n_positions=64)
        eng = LLMEngine(Model.from_graph(build_gpt2(cfg, dtype=torch.float32, seed=0)),
                        EngineConfig(max_num_seqs=8, max_batch_tokens=64, max_model_len=64, num_blocks=32, dtype="fp32",
                                     backend="torch", decode_streams=4), device="cpu")
    assert eng._split_rows(256) is None          # operator backend: one batch
    assert eng._dense_prefill_plan(4, 1) is None


def test_block_manager_view_follows_the_scheduler(tiny):
    from ronn_b200.serving import BlockLocation, CachePrecision
    eng = engine(tiny, num_blocks=7, preemption="swap", num_cpu_blocks=16)
    bm = eng.block_manager
    assert bm.block_size == 16 and bm.precision == CachePrecision.FP32
    assert bm.gpu_pool == {"total_blocks": 7, "free_blocks": 7} and bm.cpu_pool == {"total_blocks": 16, "free_blocks": 16}
    assert bm.vram_budget == 7 * bm.block_bytes and bm.utilization() == 0.0
    ids = [eng.add_request([3 + i] * 15, SamplingParams(max_new_tokens=30)) for i in range(4)]
    seen_cpu = False
    for _ in range(200):
        eng.step()
        table = bm.page_table.as_dict()
        for (rid, lb), (loc, phys) in table.items():
            md = bm.metadata(rid, lb)
            assert md.location == loc and 0 <= md.num_tokens <= 16 and md.ref_count >= 1
            if loc == BlockLocation.CPU:
                seen_cpu = True
                assert 0 <= phys < 16
            else:
                assert loc == BlockLocation.UNIFIED and 0 <= phys < 7          # a CPU engine reads its cache in place
        if not eng.has_unfinished():
            break
    assert seen_cpu and not eng.has_unfinished()
    assert bm.gpu_pool["free_blocks"] == 7 and bm.cpu_pool["free_blocks"] == 16
    with pytest.raises(SessionError):
        CachePrecision.INT4.require_supported()
    with pytest.raises(KeyError):
        bm.page_table.lookup(ids[0], 0)                   # finished: no blocks left


def test_closed_loop_serving_bench_runs_on_cpu():
    from ronn_b200.bench_models import bench_serving
    r = bench_serving(concurrency=(1, 4), prompt=12, new_tokens=5, model="gpt2-tiny", device="cpu")
    assert [x["concurrency"] for x in r["results"]] == [1, 4]
    for x in r["results"]:
        assert x["tokens_per_s"] > 0 and x["requests"] == 3 * x["concurrency"]
        assert 0 < x["ttft_ms"]["p50"] <= x["ttft_ms"]["p99"] and 0 < x["itl_ms"]["p50"] <= x["itl_ms"]["p99"]


def test_prefill_step_classification():
    """Whole prompts go to the dense tensor-core kernel, continuations and prefix hits to its paged form when the items
    are long enough, everything else to the per-row kernel."""
    import numpy as np
    from ronn_b200.serving.engine import classify_prefill_step
    item = np.repeat(np.arange(3), [40, 100, 64]).astype(np.int32)
    pos0 = np.concatenate([np.arange(40), np.arange(100), np.arange(64)]).astype(np.int32)
    kind = classify_prefill_step(item, pos0, 3)
    assert kind[0] == "dense" and kind[1].tolist() == [40, 100, 64]
    pos1 = pos0.copy()
    pos1[40:140] += 128                                   # the second item continues at position 128
    kind = classify_prefill_step(item, pos1, 3)
    assert kind[0] == "paged" and kind[1].tolist() == [0, 40, 140] and kind[2].tolist() == [40, 100, 64]
    assert kind[3].tolist() == [0, 128, 0]
    short = np.repeat(np.arange(4), 8).astype(np.int32)   # 8 tokens per item behind a prefix hit: per-row kernel
    assert classify_prefill_step(short, np.tile(np.arange(16, 24), 4).astype(np.int32), 4) is None
    assert classify_prefill_step(item, pos0, 4) is None   # token ranges do not match the item count
    assert classify_prefill_step(item[:0], pos0[:0], 0) is None
