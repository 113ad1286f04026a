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
        assert c.delete(f"/v1/requests/{body['id']}").json()["cancelled"] is True
    app.state.loop.stop()
