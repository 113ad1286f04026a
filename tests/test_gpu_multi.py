"""Multi-GPU tests (child processes, one per GPU): fused GEMM + collective kernel and the TP engine."""
import json
import os

import pytest
import torch

from test_tp_cpu import launch

pytestmark = pytest.mark.gpu

need2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


@need2
def test_fused_gemm_allreduce_and_reduce_scatter(tmp_path):
    out = tmp_path / "r.json"
    p = launch(_world(), "fused_gemm_worker.py", [str(out)], 29650, env={"NCCL_NVLS_ENABLE": "0"})
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-4000:])
    for per_rank in json.loads(out.read_text()):
        for r in per_rank:
            assert r["identical"], r
            assert r["err"] < 0.15, r            # bf16 partials of O(10) magnitude summed over ranks


@need2
def test_sequence_parallel_encoder_on_fused_kernels_matches_single_gpu(tmp_path):
    out = tmp_path / "sp.json"
    # two or four ranks: the sizes this layout has been measured at (one head and 64-deep K slices per rank at eight)
    p = launch(min(_world(), 4), "sp_encoder_worker.py", [str(out)], 29670, env={"NCCL_NVLS_ENABLE": "0"})
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-4000:])
    r = json.loads(out.read_text())
    assert r["same_across_ranks"]
    assert r["fused_calls"] == 2 * 4, r              # per layer: two gather-GEMMs and two GEMM-reduce-scatters
    assert r["err"] < 0.12, r                        # bf16 activations of O(1) through two layers


@need2
@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_tp_engine_matches_single_gpu(tmp_path, mode):
    out = tmp_path / "r.json"
    p = launch(_world(), "tp_engine_worker.py", [mode, str(out)], 29660,
               env={"NCCL_NVLS_ENABLE": "0"})
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-4000:])
    r = json.loads(out.read_text())
    assert r["same_across_ranks"]
    assert r["agree"] >= int(0.85 * r["total"]), r
    assert r["sampled_same_across_ranks"] and r["sampled_in_range"], r      # device sampler on gathered vocabulary shards
    if mode == "fused":
        assert r["fused_calls"] > 0


def test_peer_wait_runs_out_and_context_survives():
    """A flag that nothing sets: the fused kernel gives up after its limit, reports STATUS_WAIT_PEER through the status
    word, and the CUDA context stays usable.  Both 'ranks' point at buffers of this one GPU."""
    import ctypes as C
    from ronn_b200 import _native
    from ronn_b200.api.errors import CommTimeoutError
    from ronn_b200.ops import kernels as K
    dev = torch.device("cuda", 0)
    M, N, Kd = 128, 256, 64
    a = torch.randn(M, Kd, device=dev).bfloat16()
    w = torch.randn(N, Kd, device=dev).bfloat16()
    stride = M * N * 2
    parts = [torch.zeros(2 * stride, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]
    state = torch.zeros(8, dtype=torch.int32, device=dev)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    pp = (C.c_void_p * 8)(*[parts[0].data_ptr(), parts[1].data_ptr()] + [None] * 6)
    fp = (C.c_void_p * 8)(*[flags[0].data_ptr(), flags[1].data_ptr()] + [None] * 6)
    K.check_status(dev)
    rc = _native.cuda().ronn_gemm_reduce(a.data_ptr(), w.data_ptr(), M, N, Kd, Kd, Kd, pp, fp, stride, state.data_ptr(),
                                         0, 2, 0, M, out.data_ptr(), N, None, None, 0, 0.3, 0, 0, None, None, None, 0.0, 0,
                                         K.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(CommTimeoutError, match="peer"):
        K.check_status(dev)
    # rank 0 raised its own flags on both "ranks"; rank 1 never did
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1 and int(flags[0][1]) == 0
    y = K.gemm(a, w)                                # the context is alive and later kernels run
    torch.testing.assert_close(y.float(), a.float() @ w.float().t(), atol=0.5, rtol=0.05)
    K.check_status(dev)


def test_push_mode_wait_runs_out_and_context_survives():
    """Push mode carries the call's sequence number inside the data words.  Words that never arrive (the second 'rank'
    writes nothing) make the bounded poll give up with STATUS_WAIT_PEER; the context stays usable."""
    import ctypes as C
    from ronn_b200 import _native
    from ronn_b200.api.errors import CommTimeoutError
    from ronn_b200.ops import kernels as K
    dev = torch.device("cuda", 0)
    M, N, Kd = 128, 256, 64
    a = torch.randn(M, Kd, device=dev).bfloat16()
    w = torch.randn(N, Kd, device=dev).bfloat16()
    stride = M * N * 2
    parts = [torch.zeros(2 * stride, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]
    src_stride = M * N * 4
    recv = [torch.zeros(2 * 2 * src_stride, dtype=torch.uint8, device=dev) for _ in range(2)]
    state = torch.zeros(8, dtype=torch.int32, device=dev)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    pp = (C.c_void_p * 8)(*[parts[0].data_ptr(), parts[1].data_ptr()] + [None] * 6)
    fp = (C.c_void_p * 8)(*[flags[0].data_ptr(), flags[1].data_ptr()] + [None] * 6)
    rp = (C.c_void_p * 8)(*[recv[0].data_ptr(), recv[1].data_ptr()] + [None] * 6)
    K.check_status(dev)
    rc = _native.cuda().ronn_gemm_reduce_push(a.data_ptr(), w.data_ptr(), M, N, Kd, Kd, Kd, pp, fp, stride,
                                              state.data_ptr(), 0, 2, 0, M, out.data_ptr(), N, None, None, 0, 0.3, 0, 0,
                                              None, None, None, 0.0, 0, rp, 2 * src_stride, src_stride,
                                              K.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(CommTimeoutError, match="peer"):
        K.check_status(dev)
    # rank 0 delivered its words (data + sequence number 1) to both receive areas, slot [parity 0][source 0]
    words = recv[1][:src_stride].view(torch.int32).view(-1, 2)
    assert bool((words[:, 1] == 1).all())
    assert bool((recv[0][src_stride:2 * src_stride] == 0).all())      # nothing ever came from 'rank 1'
    y = K.gemm(a, w)
    torch.testing.assert_close(y.float(), a.float() @ w.float().t(), atol=0.5, rtol=0.05)
    K.check_status(dev)


def test_two_shot_wait_runs_out_and_context_survives():
    """Two-shot protocol, peer-load mode, with a second 'rank' that never runs: the row-tile counters never complete,
    the bounded wait gives up with STATUS_WAIT_PEER and the context stays usable.  Both 'ranks' are buffers of this GPU."""
    import ctypes as C
    from ronn_b200.api.errors import CommTimeoutError
    from ronn_b200.ops import fuse as F
    from ronn_b200.ops import kernels as K
    dev = torch.device("cuda", 0)
    M, N, Kd = 128, 256, 64
    a = torch.randn(M, Kd, device=dev).bfloat16()
    w = torch.randn(N, Kd, device=dev).bfloat16()
    lib = F._lib()
    parts = [torch.zeros(2 * M * N, dtype=torch.float32, device=dev) for _ in range(2)]
    flags = [torch.zeros(lib.ronn_gemm_fuse_flag_ints(), dtype=torch.int32, device=dev) for _ in range(2)]
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    state = torch.zeros(lib.ronn_gemm_fuse_state_ints(), dtype=torch.int32, device=dev)
    p = F.FuseParams()
    p.A, p.W, p.M, p.N, p.K, p.lda, p.ldw = a.data_ptr(), w.data_ptr(), M, N, Kd, Kd, Kd
    p.splitk, p.bn, p.dtype = 1, 0, 0
    for r in range(2):
        p.part[r], p.flags[r], p.out[r] = parts[r].data_ptr(), flags[r].data_ptr(), outs[r].data_ptr()
    p.parity_stride, p.state = M * N, state.data_ptr()
    p.rank, p.world, p.nvls, p.scatter, p.ld_out = 0, 2, 0, 0, N
    p.wait_seconds = 0.3
    K.check_status(dev)
    rc = lib.ronn_gemm_fuse(C.byref(p), K.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(CommTimeoutError, match="peer"):
        K.check_status(dev)
    # rank 0 raised the counter of row tile 0 on both 'ranks', but a call completes a counter only with every rank's arrivals
    assert int(flags[0][0]) == int(flags[1][0]) != 0
    assert int(flags[0][0]) % 65536 != 0
    y = K.gemm(a, w)                                # the context is alive and later kernels run
    torch.testing.assert_close(y.float(), a.float() @ w.float().t(), atol=0.5, rtol=0.05)
    K.check_status(dev)
