"""Property tests (the reference's only randomised suite is crates/ronn-core/tests/property_tests.rs:11-90: algebraic
laws on small shapes).  Here: operator algebra, optimiser equivalence and idempotence on generated graphs, the model
codec round trip, and block accounting of the serving scheduler under random request streams."""
import numpy as np
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

from ronn_b200 import Model, SessionOptions
from ronn_b200.graph.ir import GraphBuilder
from ronn_b200.graph.optimizer import Optimizer
from ronn_b200.onnx.registry import default_registry

R = default_registry()
SET = settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow])


def ex(op, inputs, **attrs):
    return R.get(op).execute(inputs, attrs)[0]


shapes = st.lists(st.integers(1, 6), min_size=1, max_size=3)


@SET
@given(shape=shapes, seed=st.integers(0, 2 ** 16))
def test_elementwise_algebra(shape, seed):
    g = torch.Generator().manual_seed(seed)
    a, b, c = (torch.randn(*shape, generator=g) for _ in range(3))
    torch.testing.assert_close(ex("Add", [a, b]), ex("Add", [b, a]))
    torch.testing.assert_close(ex("Mul", [a, b]), ex("Mul", [b, a]))
    torch.testing.assert_close(ex("Add", [ex("Add", [a, b]), c]), ex("Add", [a, ex("Add", [b, c])]), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(ex("Sub", [a, a]), torch.zeros_like(a))
    assert ex("Relu", [a]).min().item() >= 0
    assert ex("Add", [a, b]).shape == a.shape
    s = ex("Softmax", [a], axis=-1)
    torch.testing.assert_close(s.sum(-1), torch.ones(s.shape[:-1]), atol=1e-5, rtol=1e-5)


@SET
@given(m=st.integers(1, 5), k=st.integers(1, 6), n=st.integers(1, 5), seed=st.integers(0, 2 ** 16))
def test_matmul_shape_and_transpose_law(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    a, b = torch.randn(m, k, generator=g), torch.randn(k, n, generator=g)
    y = ex("MatMul", [a, b])
    assert y.shape == (m, n)
    yt = ex("MatMul", [ex("Transpose", [b], perm=[1, 0]), ex("Transpose", [a], perm=[1, 0])])
    torch.testing.assert_close(ex("Transpose", [yt], perm=[1, 0]), y, atol=1e-5, rtol=1e-5)


def _chain_graph(widths, acts, seed, dead_branch):
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder().add_input("x", [2, widths[0]]).add_output("y", [2, widths[-1]])
    cur = "x"
    for i, (k, n) in enumerate(zip(widths, widths[1:])):
        b.add_initializer(f"w{i}", torch.randn(k, n, generator=g) * 0.3)
        b.add_initializer(f"b{i}", torch.randn(n, generator=g) * 0.1)
        b.add_op("MatMul", [cur, f"w{i}"], [f"mm{i}"], name=f"mm{i}")
        b.add_op("Add", [f"mm{i}", f"b{i}"], [f"a{i}"], name=f"add{i}")
        last = i == len(widths) - 2
        out = "y" if last else f"h{i}"
        act = acts[i % len(acts)]
        if act == "none":
            b.add_op("Identity", [f"a{i}"], [out], name=f"id{i}")
        else:
            b.add_op(act, [f"a{i}"], [out], name=f"act{i}")
        cur = out
    if dead_branch:
        b.add_initializer("cst", torch.randn(3, generator=g))
        b.add_op("Relu", ["cst"], ["unused0"], name="dead0")
        b.add_op("Add", ["unused0", "cst"], ["unused1"], name="dead1")
    return b.build()


@SET
@given(widths=st.lists(st.integers(1, 9), min_size=2, max_size=5),
       acts=st.lists(st.sampled_from(["Relu", "Sigmoid", "Tanh", "none"]), min_size=1, max_size=3),
       seed=st.integers(0, 2 ** 16), dead=st.booleans())
def test_optimised_graph_is_equivalent_and_optimiser_is_idempotent(widths, acts, seed, dead):
    graph = _chain_graph(widths, acts, seed, dead)
    x = torch.randn(2, widths[0], generator=torch.Generator().manual_seed(seed + 1))
    outs = {}
    for level in ("O0", "O1", "O2", "O3"):
        sess = Model.from_graph(graph.clone()).create_session(
            SessionOptions().with_optimization_level(level).with_provider("cpu"))
        outs[level] = sess.run({"x": x})["y"]
    for level in ("O1", "O2", "O3"):
        torch.testing.assert_close(outs[level], outs["O0"], atol=1e-5, rtol=1e-5)
    once = graph.clone()
    Optimizer("O3").optimize(once)
    n_once = len(once.nodes)
    names = sorted(n.name for n in once.nodes)
    stats = Optimizer("O3").optimize(once)                       # a second run finds nothing more to do
    assert len(once.nodes) == n_once and sorted(n.name for n in once.nodes) == names
    assert stats.nodes_removed == 0 and stats.nodes_fused == 0
    once.validate()
    assert [t.name for t in once.inputs] == ["x"] and [t.name for t in once.outputs] == ["y"]
    if dead:
        assert all(not n.name.startswith("dead") for n in once.nodes)


@SET
@given(shape=shapes, dtype=st.sampled_from([torch.float32, torch.float16, torch.int64, torch.int32, torch.uint8]),
       seed=st.integers(0, 2 ** 16))
def test_model_codec_round_trip(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(*shape, generator=g) * 10).to(dtype)
    b = GraphBuilder().add_input("x", list(shape)).add_output("y", list(shape))
    b.add_initializer("w", w)
    b.add_op("Identity", ["x"], ["y"], name="id")
    model = Model.from_graph(b.build())
    again = Model.from_bytes(model.to_bytes())
    w2 = again.graph.initializers["w"]
    assert w2.dtype == dtype and tuple(w2.shape) == tuple(shape)
    assert torch.equal(w2, w)
    assert [n.op_type for n in again.graph.nodes] == ["Identity"]


@SET
@given(data=st.data())
def test_scheduler_never_leaks_blocks(data):
    from ronn_b200.serving.scheduler import PLAN_NONE, HostBatchBuffers, Scheduler
    num_blocks, max_seqs, max_tokens, max_blocks = 24, 4, 64, 8
    sched = Scheduler(16, num_blocks, max_seqs, max_tokens, 0, "fcfs", False, max_blocks)
    host = HostBatchBuffers(max_tokens, max_seqs, max_blocks, pin=False)
    n_req = data.draw(st.integers(1, 7))
    for rid in range(n_req):
        plen = data.draw(st.integers(1, 40))
        new = data.draw(st.integers(1, 12))
        sched.add(rid, list(range(plen)), new, 1)
    finished = 0
    for _ in range(2000):
        kind = sched.schedule()
        if kind == PLAN_NONE:
            break
        sb = sched.fill(host, kind)
        assert sb.n_tokens <= max_tokens and sb.n_items <= max_seqs
        fin = sched.commit(np.zeros(sb.n_items, dtype=np.int32), -1)
        finished += int((fin != 0).sum())
        assert 0 <= sched.num_free_blocks <= num_blocks
    assert finished == n_req
    assert sched.num_waiting == 0 and sched.num_running == 0
    assert sched.num_free_blocks == num_blocks                    # every block came back


@SET
@given(data=st.data())
def test_swap_preemption_keeps_every_sequence_on_its_own_blocks(data):
    """A model of the cache contents (the token whose key/value each slot of each device / host block holds) follows
    the scheduler's swap plan: whenever a sequence is scheduled, every position of its cached prefix must hold that
    sequence's token, whatever preemptions, swap-outs, swap-ins and prefix-cache sharing happened in between."""
    from ronn_b200.serving.scheduler import PLAN_NONE, HostBatchBuffers, Scheduler
    num_blocks, max_seqs, max_tokens, max_blocks = data.draw(st.integers(6, 12)), 4, 64, 6
    sched = Scheduler(16, num_blocks, max_seqs, max_tokens, data.draw(st.sampled_from([0, 16])), "fcfs",
                      data.draw(st.booleans()), max_blocks)
    n_cpu = data.draw(st.integers(0, 12))
    sched.set_preemption(data.draw(st.sampled_from(["swap", "auto"])), n_cpu, data.draw(st.integers(1, 40)))
    host = HostBatchBuffers(max_tokens, max_seqs, max_blocks, pin=False)
    n_req = data.draw(st.integers(2, 7))
    for rid in range(n_req):
        # prompts share prefixes (0, 1, 2, ...), so the prefix cache has something to share
        sched.add(rid, list(range(data.draw(st.integers(1, 30)))), data.draw(st.integers(1, 30)), 1)
    gpu, cpu = {}, {}                                         # block -> 16 slots, each the token stored there
    finished = idle = 0
    for step in range(4000):
        kind = sched.schedule()
        o_src, o_dst, i_src, i_dst = sched.swaps()
        for s_, d_ in zip(o_src.tolist(), o_dst.tolist()):
            assert 0 <= d_ < n_cpu and d_ not in cpu
            cpu[d_] = list(gpu[s_])
        for s_, d_ in zip(i_src.tolist(), i_dst.tolist()):
            gpu[d_] = cpu.pop(s_)
        if kind == PLAN_NONE:
            if sched.num_waiting == 0 and sched.num_running == 0:
                break
            idle += 1
            assert idle < 50                                  # an all-preempted step is followed by progress
            continue
        idle = 0
        sb = sched.fill(host, kind)
        q_start, pos = host.field("q_start"), host.field("positions")
        for i, rid in enumerate(sb.req_ids.tolist()):
            start, count = int(pos[q_start[i]]), int(q_start[i + 1] - q_start[i])
            blocks, toks = sched.blocks(rid), sched.tokens(rid)
            for p_ in range(start):                           # the cached prefix holds this sequence's tokens
                assert gpu[blocks[p_ // 16]][p_ % 16] == toks[p_], (rid, p_, blocks)
            for p_ in range(start, start + count):
                gpu.setdefault(blocks[p_ // 16], [None] * 16)[p_ % 16] = toks[p_]
        fin = sched.commit(np.full(sb.n_items, 100 + step % 7, dtype=np.int32), -1)
        finished += int((fin != 0).sum())
    assert finished == n_req and not cpu
    assert sched.num_free_blocks == num_blocks and sched.swap_stats()["free_cpu_blocks"] == n_cpu
    st_ = sched.swap_stats()
    assert st_["swapped_in_blocks"] == st_["swapped_out_blocks"]
