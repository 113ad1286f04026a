"""EncoderRunner against the graph session of the same DistilBERT model (CPU, operator backend)."""
import pytest
import torch


def _model(dtype=torch.float32, **kw):
    from ronn_b200.api.model import Model
    from ronn_b200.models.distilbert import DistilBertConfig, build_distilbert
    return Model.from_graph(build_distilbert(DistilBertConfig.tiny(**kw), dtype=dtype, seed=3))


def test_encoder_runner_matches_graph_session_cpu():
    from ronn_b200 import SessionOptions
    from ronn_b200.serving.encoder_runner import EncoderRunner
    model = _model()
    ids = torch.randint(0, 512, (3, 32))
    mask = torch.ones(3, 32, dtype=torch.int64)
    mask[1, 20:] = 0
    mask[2, 7:] = 0
    sess = model.create_session(SessionOptions().with_provider("cpu"))
    want = sess.run({"input_ids": ids, "attention_mask": mask})["last_hidden_state"]
    got = EncoderRunner(model.graph, device="cpu").forward(ids, mask)
    assert got.shape == want.shape
    for b, n in enumerate(mask.sum(1).tolist()):       # valid positions agree; padded rows are unspecified
        torch.testing.assert_close(got[b, :n], want[b, :n], atol=2e-4, rtol=1e-3)


def test_encoder_runner_rejects_other_architectures():
    from ronn_b200.api.errors import SessionError
    from ronn_b200.models.mlp784 import build_mlp784
    from ronn_b200.serving.encoder_runner import EncoderRunner
    with pytest.raises(SessionError):
        EncoderRunner(build_mlp784(), device="cpu")
