"""HTTP front end over a CPU engine."""
import json

import torch
from fastapi.testclient import TestClient

from ronn_b200 import Model
from ronn_b200.models.gpt2 import GPT2Config, build_gpt2
from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams
from ronn_b200.serving.server import create_app


def test_completions_health_metrics_cancel_stream():
    model = Model.from_graph(build_gpt2(GPT2Config.tiny(), dtype=torch.float32, seed=1))
    ref = LLMEngine(model, EngineConfig(max_num_seqs=4, max_batch_tokens=64, max_model_len=128, num_blocks=32, dtype="fp32",
                                        backend="torch"), device="cpu").generate([[1, 2, 3, 4]], SamplingParams(max_new_tokens=5))[0]
    eng = LLMEngine(model, EngineConfig(max_num_seqs=4, max_batch_tokens=64, max_model_len=128, num_blocks=32, dtype="fp32",
                                        backend="torch"), device="cpu")
    app = create_app(eng)
    with TestClient(app) as c:
        assert c.get("/v1/health").json()["status"] == "ok"
        r = c.post("/v1/completions", json={"prompt_token_ids": [1, 2, 3, 4], "max_tokens": 5})
        assert r.status_code == 200
        body = r.json()
        assert body["choices"][0]["token_ids"] == ref and body["choices"][0]["finish_reason"] == "max_tokens"
        assert body["usage"] == {"prompt_tokens": 4, "completion_tokens": 5}
        assert c.post("/v1/completions", json={"prompt_token_ids": []}).status_code == 400
        assert c.post("/v1/completions", json={"prompt_token_ids": [1], "priority": "urgent"}).status_code == 400
        too_long = c.post("/v1/completions", json={"prompt_token_ids": list(range(200)), "max_tokens": 5})
        assert too_long.status_code == 400 and "max_model_len" in too_long.json()["detail"]
        with c.stream("POST", "/v1/completions", json={"prompt_token_ids": [1, 2, 3, 4], "max_tokens": 5, "stream": True}) as s:
            lines = [l for l in s.iter_lines() if l.startswith("data: ")]
        toks = [json.loads(l[6:])["token_id"] for l in lines if "token_id" in l]
        assert toks == ref and lines[-1] == "data: [DONE]"
        assert "ronn_generated_tokens" in c.get("/v1/metrics").text
        assert c.delete("/v1/requests/9999").status_code == 404
        # an answered request leaves nothing behind: no event, no token stream, no engine or scheduler record
        assert c.delete(f"/v1/requests/{body['id']}").status_code == 404
        h = c.get("/v1/health").json()
        assert h["tracked_requests"] == 0 and h["admission"]["in_flight"] == 0 and h["admission"]["answered"] >= 2
        assert eng.requests == {} and app.state.loop._streams == {}
    app.state.loop.stop()


def _engine(**kw):
    model = Model.from_graph(build_gpt2(GPT2Config.tiny(), dtype=torch.float32, seed=1))
    cfg = dict(max_num_seqs=4, max_batch_tokens=64, max_model_len=128, num_blocks=32, dtype="fp32", backend="torch")
    cfg.update(kw)
    return LLMEngine(model, EngineConfig(**cfg), device="cpu")


def test_admission_refuses_beyond_the_limits_and_deadline_cancels():
    from ronn_b200.core.session_manager import RequestAdmission
    adm = RequestAdmission(max_in_flight=2, max_per_client=1, timeout_seconds=60)
    t1 = adm.acquire("a")
    assert t1 is not None and adm.acquire("a") is None            # per-client cap
    t2 = adm.acquire("b")
    assert t2 is not None and adm.acquire("c") is None            # global cap
    adm.release(t1)
    adm.release(t1)                                               # releasing twice is harmless
    assert adm.acquire("c") is not None and adm.snapshot()["refused"] == 2
    # through HTTP: a server whose admission is full answers 429; a zero deadline answers 504 and cancels the request
    eng = _engine()
    full = RequestAdmission(max_in_flight=0)
    app = create_app(eng, admission=full)
    with TestClient(app) as c:
        assert c.post("/v1/completions", json={"prompt_token_ids": [1, 2], "max_tokens": 3}).status_code == 429
    app.state.loop.stop()
    eng2 = _engine()
    app2 = create_app(eng2, admission=RequestAdmission(timeout_seconds=-1.0))
    with TestClient(app2) as c:
        r = c.post("/v1/completions", json={"prompt_token_ids": [1, 2], "max_tokens": 40})
        assert r.status_code in (200, 504)                        # the engine may finish before the first deadline check
        import time
        for _ in range(200):
            if not eng2.has_unfinished() and app2.state.loop.tracked() == 0:
                break
            time.sleep(0.01)
        assert not eng2.has_unfinished() and app2.state.loop.tracked() == 0 and eng2.requests == {}
    app2.state.loop.stop()


def test_engine_loop_gives_up_after_repeated_failed_steps_and_forgets_released_requests():
    import time
    from ronn_b200.serving.request import FinishReason
    from ronn_b200.serving.server import EngineLoop
    eng = _engine()
    loop = EngineLoop(eng, max_failed_steps=3)
    try:
        # a client that goes away while its request runs: release() cancels it and every record disappears
        rid = loop.submit([1, 2, 3], SamplingParams(max_new_tokens=40, stop_sequences=[[7, 7, 7]]))
        for _ in range(200):
            if rid in eng.requests:
                break
            time.sleep(0.005)
        loop.release(rid)
        for _ in range(400):
            if loop.tracked() == 0 and rid not in eng.requests:
                break
            time.sleep(0.005)
        assert loop.tracked() == 0 and rid not in eng.requests and eng._watch_count == 0
        assert eng.sched.state(rid) is None                           # the native scheduler has forgotten it too
        # every step fails: after three in a row the waiting request is failed instead of being retried for ever
        def boom(*a, **k):
            raise RuntimeError("injected step failure")
        eng.runner.forward = boom
        rid2 = loop.submit([4, 5, 6], SamplingParams(max_new_tokens=4))
        assert loop.wait(rid2, timeout=10)
        r = loop.result(rid2)
        assert r.finish_reason == FinishReason.ERROR and "consecutive iterations failed" in r.error
        assert not eng.has_unfinished()
    finally:
        loop.stop()


def test_chat_completions_text_prompts_and_streaming():
    from ronn_b200.serving.tokenizer import ByteTokenizer, load_tokenizer, render_chat
    cfg = GPT2Config.tiny()
    model = Model.from_graph(build_gpt2(cfg, dtype=torch.float32, seed=2))
    ecfg = dict(max_num_seqs=4, max_batch_tokens=128, max_model_len=256, num_blocks=64, dtype="fp32", backend="torch")
    tok = load_tokenizer("bytes", cfg.vocab_size)
    assert isinstance(tok, ByteTokenizer) and tok.decode(tok.encode("héllo")) == "héllo"
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    prompt = tok.encode(render_chat(msgs))
    ref = LLMEngine(model, EngineConfig(**ecfg), device="cpu").generate([prompt], SamplingParams(max_new_tokens=6))[0]
    eng = LLMEngine(model, EngineConfig(**ecfg), device="cpu")
    app = create_app(eng, tok)
    with TestClient(app) as c:
        r = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 6})
        assert r.status_code == 200
        ch = r.json()["choices"][0]
        assert ch["token_ids"] == ref and ch["message"] == {"role": "assistant", "content": tok.decode(ref)}
        assert r.json()["usage"]["prompt_tokens"] == len(prompt)
        with c.stream("POST", "/v1/chat/completions", json={"messages": msgs, "max_tokens": 6, "stream": True}) as s_:
            lines = [l for l in s_.iter_lines() if l.startswith("data: ")]
        chunks = [json.loads(l[6:]) for l in lines[:-1]]
        streamed = [t for ch_ in chunks for t in ch_["choices"][0].get("token_ids", [])]
        text = "".join(ch_["choices"][0]["delta"].get("content", "") for ch_ in chunks)
        assert streamed == ref and text == tok.decode(ref) and lines[-1] == "data: [DONE]"
        assert chunks[-1]["choices"][0]["finish_reason"] == "max_tokens"
        # text prompt on the completions endpoint
        r2 = c.post("/v1/completions", json={"prompt": render_chat(msgs), "max_tokens": 6})
        assert r2.json()["choices"][0]["token_ids"] == ref and r2.json()["choices"][0]["text"] == tok.decode(ref)
        assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    app.state.loop.stop()
    # without a tokenizer the text endpoints refuse
    eng2 = LLMEngine(model, EngineConfig(**ecfg), device="cpu")
    app2 = create_app(eng2)
    with TestClient(app2) as c:
        assert c.post("/v1/chat/completions", json={"messages": msgs}).status_code == 400
        assert c.post("/v1/completions", json={"prompt": "hi"}).status_code == 400
    app2.state.loop.stop()
