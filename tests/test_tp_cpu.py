"""Tensor-parallel engine logic on CPU ranks (gloo): sharding, replicated scheduling, sharded argmax."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def launch(nproc, script, args, port, timeout=300, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_workers", script)] + args
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)


@pytest.mark.parametrize("world", [2, 4])
def test_tp_engine_on_cpu_ranks_matches_single_rank(tmp_path, world):
    out = tmp_path / "r.json"
    p = launch(world, "tp_engine_worker.py", ["cpu", str(out)], 29610 + world)
    assert p.returncode == 0, p.stderr[-3000:]
    r = json.loads(out.read_text())
    assert r["world"] == world and r["same_across_ranks"]
    assert r["agree"] == r["total"] == 48          # fp32: sharded and unsharded runs pick the same tokens
    assert r["sampled_same_across_ranks"] and r["sampled_in_range"]        # non-greedy requests: gathered logits, one seed


def test_tp_bitnet_engine_with_a_ragged_ffn_shard(tmp_path):
    """Ternary decoder at two ranks whose FFN shard (176) is widened to 192 with zero weights: every rank produces the
    same tokens, and they agree with the single-rank run up to the effect of quantising each rank's activation shard
    with its own scale."""
    out = tmp_path / "r.json"
    p = launch(2, "tp_engine_worker.py", ["cpu", str(out)], 29619, env={"RONN_TEST_MODEL": "bitnet"})
    assert p.returncode == 0, p.stderr[-3000:]
    r = json.loads(out.read_text())
    assert r["same_across_ranks"] and r["sampled_same_across_ranks"] and r["sampled_in_range"]
    assert r["agree"] >= int(0.5 * r["total"]), r


def test_tp_engine_swap_preemption_on_cpu_ranks(tmp_path):
    """Every rank runs the same scheduler, so every rank swaps the same blocks of its own shard of the cache."""
    out = tmp_path / "r.json"
    p = launch(2, "tp_engine_worker.py", ["cpu", str(out)], 29617, env={"RONN_TEST_TIGHT_BLOCKS": "7"})
    assert p.returncode == 0, p.stderr[-3000:]
    r = json.loads(out.read_text())
    assert r["same_across_ranks"] and r["agree"] == r["total"] == 120
    assert r["swap_preemptions"] >= 1 and r["swapped_in_blocks"] >= 1


def test_head_and_vocab_sharding_cover_everything():
    from ronn_b200.serving.model_runner import shard_heads
    for heads, tp in ((12, 8), (20, 8), (16, 8), (16, 3), (4, 4)):
        spans = [shard_heads(heads, tp, r) for r in range(tp)]
        assert spans[0][0] == 0 and sum(n for _, n in spans) == heads
        for (s0, n0), (s1, _) in zip(spans, spans[1:]):
            assert s0 + n0 == s1
        assert max(n for _, n in spans) - min(n for _, n in spans) <= 1


def test_rank_that_never_joins_is_reported_not_hung(tmp_path):
    """Failure made on the host: one of two ranks exits before the rendezvous; the other gets an error from the
    process-group timeout instead of hanging."""
    script = tmp_path / "w.py"
    script.write_text(
        "import os, sys, datetime, torch.distributed as dist\n"
        "rank = int(os.environ['RANK'])\n"
        "if rank == 1:\n    sys.exit(0)\n"
        "try:\n"
        "    dist.init_process_group('gloo', rank=rank, world_size=2, timeout=datetime.timedelta(seconds=5))\n"
        "    dist.barrier()\n"
        "    print('UNEXPECTED')\n"
        "except Exception as e:\n"
        "    print('DETECTED', type(e).__name__)\n")
    procs = []
    for r in range(2):
        e = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29633")
        procs.append(subprocess.Popen([sys.executable, str(script)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=e))
    out0, _ = procs[0].communicate(timeout=120)
    procs[1].wait(timeout=30)
    assert "DETECTED" in out0 and "UNEXPECTED" not in out0


@pytest.mark.parametrize("world", [2, 4])
def test_tp_encoder_on_cpu_ranks_matches_single_rank(tmp_path, world):
    out = tmp_path / "e.json"
    p = launch(world, "tp_encoder_worker.py", [str(out)], 29640 + world)
    assert p.returncode == 0, p.stderr[-3000:]
    r = json.loads(out.read_text())
    assert r["world"] == world and r["same_across_ranks"]
    assert r["err"] < 1e-4
    assert r["err_sequence_parallel"] < 1e-4          # token-sharded layout: all-gather / reduce-scatter around the GEMMs


def test_space_to_depth_stem_weights_reproduce_the_7x7_stride2_convolution():
    import torch
    import torch.nn.functional as F
    from ronn_b200.providers.gpu_conv import stem_weights_s2d
    torch.manual_seed(0)
    x = torch.randn(2, 3, 16, 20)
    w = torch.randn(8, 7, 7, 3)
    ref = F.conv2d(x, w.permute(0, 3, 1, 2), stride=2, padding=3)
    n, c, h, wd = x.shape
    x2 = torch.zeros(n, h // 2, wd // 2, 16)
    for dy in range(2):
        for dx in range(2):
            q = dy * 2 + dx
            x2[..., q * c:(q + 1) * c] = x[:, :, dy::2, dx::2].permute(0, 2, 3, 1)
    w2 = stem_weights_s2d(w)
    out = F.conv2d(F.pad(x2.permute(0, 3, 1, 2), (2, 1, 2, 1)), w2.permute(0, 3, 1, 2))
    torch.testing.assert_close(out, ref, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("world", [2, 4])
def test_session_level_tensor_parallelism_on_cpu_ranks(tmp_path, world):
    """SessionOptions.tp_size: every rank holds 1 / world of the projection weights, AllReduce nodes sum the partial
    results, and the output equals the unsharded session's."""
    out = tmp_path / "r.json"
    p = launch(world, "tp_session_worker.py", [str(out)], 29630 + world)
    assert p.returncode == 0, p.stderr[-3000:]
    for rank, r in enumerate(json.loads(out.read_text())):
        for lvl in ("O0", "O3"):
            assert r[lvl]["err"] < 1e-4, r
            assert r[lvl]["all_reduce_nodes"] == 4 and r[lvl]["tp"] == f"{rank}/{world}"      # 2 layers x (attention, MLP)
            assert abs(r[lvl]["weight_fraction"] - 1.0 / world) < 0.08, r       # the position table stays replicated
        assert r["odd"]["err"] < 1e-5 and r["odd"]["all_reduce_nodes"] == 0


def test_tp_size_without_a_process_group_is_an_error():
    from ronn_b200 import Model, SessionOptions
    from ronn_b200.api.errors import SessionError
    from ronn_b200.models.mlp784 import build_mlp784
    with pytest.raises(SessionError, match="process group"):
        Model.from_graph(build_mlp784()).create_session(SessionOptions().with_tp_size(2))
