"""Fused skinny GEMM (split-K GEMM + row reduction + bias / activation / residual + norm in one launch), single GPU:
numerics against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rand(*shape, dtype=torch.bfloat16, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(dtype)


def _ref(a, w, bias, res, act, norm, gamma, beta, eps=1e-5):
    x = a.float() @ w.float().t()
    if bias is not None:
        x = x + bias.float()
    if act == "gelu":
        x = F.gelu(x, approximate="tanh")
    elif act == "relu":
        x = torch.relu(x)
    if res is not None:
        x = x + res.float()
    xs = x.to(a.dtype).float()                       # the norm sees the stored (rounded) residual stream
    if norm == "layernorm":
        h = F.layer_norm(xs, (xs.shape[-1],), gamma.float(), beta.float(), eps)
    elif norm == "rmsnorm":
        h = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    else:
        h = None
    return x, h


@pytest.mark.parametrize("M,N,K_,S,bn", [
    (256, 1024, 1024, 4, 0), (256, 1024, 4096, 8, 64), (256, 1024, 4096, 4, 32), (200, 264, 320, 2, 32),
    (37, 136, 1024, 3, 0), (1, 1024, 1024, 0, 0), (128, 2560, 6912, 0, 128), (1024, 1024, 256, 1, 0),
    (256, 768, 3072, 4, 0)])
@pytest.mark.parametrize("norm", ["", "layernorm", "rmsnorm"])
def test_gemm_fuse_rows(M, N, K_, S, bn, norm):
    from ronn_b200.ops import kernels as K
    from ronn_b200.ops.fuse import gemm_fuse
    a, w = _rand(M, K_), _rand(N, K_, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    gamma, beta = _rand(N), _rand(N)
    for it in range(3):                               # consecutive calls alternate the parity slots and advance the counters
        r = gemm_fuse(a, w, bias, res, norm=(norm, gamma, beta if norm == "layernorm" else None, 1e-5) if norm else None,
                      splitk=S, bn=bn)
        K.check_status()
        x, h = (r if norm else (r, None))
        xr, hr = _ref(a, w, bias, res, "", norm, gamma, beta)
        tol = 3e-2 * math.sqrt(K_ / 64)
        torch.testing.assert_close(x.float(), xr, atol=tol, rtol=2e-2)
        if norm:
            # compare the norm against the norm of the kernel's own stored x: isolates it from GEMM rounding
            _, hr2 = _ref(a, w, bias, res, "", norm, gamma, beta)
            xs = x.float()
            if norm == "layernorm":
                hk = F.layer_norm(xs, (N,), gamma.float(), beta.float(), 1e-5)
            else:
                hk = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
            torch.testing.assert_close(h.float(), hk, atol=4e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K_,S,act", [(256, 3072, 1024, 2, ""), (256, 4096, 1024, 4, "gelu"), (100, 6000, 512, 2, "relu"),
                                           (256, 50264, 256, 1, "")])
def test_gemm_fuse_flat(M, N, K_, S, act):
    """Rows wider than 4096 values (and any row without a norm above that width) take the flat path of phase 2."""
    from ronn_b200.ops import kernels as K
    from ronn_b200.ops.fuse import gemm_fuse
    a, w = _rand(M, K_), _rand(N, K_, scale=0.05)
    bias = _rand(N)
    for it in range(2):
        x = gemm_fuse(a, w, bias, None, activation=act, splitk=S)
        K.check_status()
        xr, _ = _ref(a, w, bias, None, act, "", None, None)
        torch.testing.assert_close(x.float(), xr, atol=3e-2 * math.sqrt(K_ / 64), rtol=2e-2)


def test_gemm_fuse_graph_replay():
    """The counters and the call parity live on the device: replays of a captured chain need no new arguments."""
    from ronn_b200.ops import kernels as K
    from ronn_b200.ops.fuse import gemm_fuse
    M, N = 256, 1024
    a, w1, w2 = _rand(M, N), _rand(N, N, scale=0.03), _rand(N, N, scale=0.03)
    gamma, beta = _rand(N), _rand(N)
    gemm_fuse(a, w1, None, a, norm=("layernorm", gamma, beta, 1e-5))
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        gemm_fuse(a, w1, None, a, norm=("layernorm", gamma, beta, 1e-5))      # scratch of the capture stream
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        x1, h1 = gemm_fuse(a, w1, None, a, norm=("layernorm", gamma, beta, 1e-5))
        x2, h2 = gemm_fuse(h1, w2, None, x1, norm=("layernorm", gamma, beta, 1e-5))
        x3 = gemm_fuse(h2, w1, None, x2)
    for _ in range(7):                                 # an odd number of calls per replay: the parity alternates between replays
        g.replay()
    torch.cuda.synchronize()
    K.check_status()
    r1, hr1 = _ref(a, w1, None, a, "", "layernorm", gamma, beta)
    torch.testing.assert_close(x1.float(), r1, atol=0.15, rtol=2e-2)
    r2, hr2 = _ref(h1, w2, None, x1, "", "layernorm", gamma, beta)
    torch.testing.assert_close(x2.float(), r2, atol=0.15, rtol=2e-2)
    torch.testing.assert_close(h2.float(), F.layer_norm(x2.float(), (N,), gamma.float(), beta.float(), 1e-5), atol=4e-2, rtol=2e-2)
    r3, _ = _ref(h2, w1, None, x2, "", "", None, None)
    torch.testing.assert_close(x3.float(), r3, atol=0.15, rtol=2e-2)


@pytest.mark.parametrize("world,S", [(2, 1), (2, 4), (4, 1), (4, 2), (8, 1)])
@pytest.mark.parametrize("M,N,Kr", [(148, 1024, 128), (37, 1024, 512), (8, 2048, 64), (300, 256, 192)])
def test_gemm_ll_many_ranks_emulated_on_one_gpu(world, S, M, N, Kr):
    """The low-latency tensor-parallel projection at 2, 4 and 8 ranks on ONE device: every rank's receive and result
    areas live in this GPU's memory and the three parts of a call run as separate launches (all ranks' GEMM + scatter,
    then all owners' reduce + broadcast, then all ranks' unpack + norm), so no launch waits for a later one.  Checks the
    owner / source-slot / parity arithmetic for every world size against an fp32 reference of the summed product."""
    import ctypes as C

    from ronn_b200.ops import fuse as FU
    from ronn_b200.ops import kernels as K
    dev = torch.device("cuda", 0)
    owner_rows = (M + world - 1) // world
    sc_stride = world * S * owner_rows * N * 4
    rs_stride = M * N * 4
    scatter = [torch.zeros(2 * sc_stride, dtype=torch.uint8, device=dev) for _ in range(world)]
    result = [torch.zeros(2 * rs_stride, dtype=torch.uint8, device=dev) for _ in range(world)]
    state = [torch.zeros(4, dtype=torch.int64, device=dev) for _ in range(world)]
    bias, res, gamma, beta = _rand(N), _rand(M, N), _rand(N), _rand(N)
    lib = FU._lib()
    for it in range(3):                                    # both parities, then the first again
        a = [_rand(M, Kr) for _ in range(world)]
        w = [_rand(N, Kr, scale=0.05) for _ in range(world)]
        outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        hs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        for phase in (1, 2, 4):
            for r in range(world):
                p = FU.LLParams()
                p.A, p.W = a[r].data_ptr(), w[r].data_ptr()
                p.M, p.N, p.K, p.lda, p.ldw = M, N, Kr, Kr, Kr
                p.bn, p.splitk, p.dtype = 0, S, 0
                for q in range(world):
                    p.scatter_area[q] = scatter[q].data_ptr()
                    p.result_area[q] = result[q].data_ptr()
                p.scatter_parity_stride, p.result_parity_stride = sc_stride, rs_stride
                p.state, p.rank, p.world, p.nvls = state[r].data_ptr(), r, world, 0
                p.out, p.norm_out, p.ld_out = outs[r].data_ptr(), hs[r].data_ptr(), N
                p.bias, p.residual, p.ld_res = bias.data_ptr(), res.data_ptr(), N
                p.gamma, p.beta, p.eps, p.norm_mode = gamma.data_ptr(), beta.data_ptr(), 1e-5, 1
                p.wait_seconds, p.phases = 0.25, phase
                rc = lib.ronn_gemm_ll(C.byref(p), K.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
                assert rc == 0, rc
        K.check_status()
        x32 = sum(a[r].float() @ w[r].float().t() for r in range(world)) + bias.float() + res.float()
        tol = 3e-2 * math.sqrt(world * Kr / 64) + 2e-2
        for r in range(world):
            assert torch.equal(outs[r], outs[0]) and torch.equal(hs[r], hs[0])      # only the owner computes a row
        torch.testing.assert_close(outs[0].float(), x32, atol=tol, rtol=2e-2)
        hk = F.layer_norm(outs[0].float(), (N,), gamma.float(), beta.float(), 1e-5)
        torch.testing.assert_close(hs[0].float(), hk, atol=6e-2, rtol=3e-2)
        assert all(int(s[0]) == (it + 1) << 16 for s in state)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("M,N,Kr", [(128, 2560, 320), (37, 512, 256), (200, 1024, 896)])
def test_bitlinear_ll_many_ranks_emulated_on_one_gpu(world, M, N, Kr):
    """Row-parallel BitLinear fused with the low-latency all-reduce, 2 to 8 ranks on ONE device (every rank's areas in
    this GPU's memory, the three parts of a call as separate launches): against the sum of the ranks' bf16 partial
    products from the stand-alone BitLinear kernel plus the residual."""
    import ctypes as C

    from ronn_b200.ops import bitnet as KB
    from ronn_b200.ops import fuse as FU
    from ronn_b200.ops import kernels as K
    dev = torch.device("cuda", 0)
    owner_rows = (M + world - 1) // world
    sc_stride, rs_stride = world * owner_rows * N * 4, M * N * 4
    scatter = [torch.zeros(2 * sc_stride, dtype=torch.uint8, device=dev) for _ in range(world)]
    result = [torch.zeros(2 * rs_stride, dtype=torch.uint8, device=dev) for _ in range(world)]
    state = [torch.zeros(4, dtype=torch.int64, device=dev) for _ in range(world)]
    res = _rand(M, N)
    gamma = (_rand(N).float().abs() + 0.5).bfloat16()
    nq = [torch.zeros(M, N, dtype=torch.int8, device=dev) for _ in range(world)]
    nscale = [torch.zeros(M, dtype=torch.float32, device=dev) for _ in range(world)]
    lib = FU._lib()
    for it in range(3):
        qs, ss, ws = [], [], []
        for r in range(world):
            q, s = KB.act_quant_int8(_rand(M, Kr))
            qs.append(q)
            ss.append(s)
            ws.append(KB.ternary_pack(torch.randint(-1, 2, (N, Kr), device=dev, dtype=torch.int8)))
        outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        for phase in (1, 2, 4):
            for r in range(world):
                bp = FU.BitLinearLLParams()
                bp.xq, bp.w_packed, bp.x_scale, bp.w_scale, bp.ldx = qs[r].data_ptr(), ws[r].data_ptr(), ss[r].data_ptr(), 0.05, Kr
                p = bp.ll
                p.M, p.N, p.K, p.dtype = M, N, Kr, 0
                for w in range(world):
                    p.scatter_area[w] = scatter[w].data_ptr()
                    p.result_area[w] = result[w].data_ptr()
                p.scatter_parity_stride, p.result_parity_stride = sc_stride, rs_stride
                p.state, p.rank, p.world, p.nvls = state[r].data_ptr(), r, world, 0
                p.out, p.ld_out = outs[r].data_ptr(), N
                p.residual, p.ld_res = res.data_ptr(), N
                p.wait_seconds, p.phases = 0.25, phase
                if it == 2:                               # the unpack pass also normalises and quantises for the next layer
                    p.norm_mode, p.gamma, p.eps = 3, gamma.data_ptr(), 1e-5
                    p.quant_out, p.quant_scale = nq[r].data_ptr(), nscale[r].data_ptr()
                rc = lib.ronn_bitlinear_ll(C.byref(bp), K.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
                assert rc == 0, rc
        K.check_status()
        want = sum(KB.bitlinear_q(qs[r], ss[r], ws[r], 0.05, None, N, Kr, torch.bfloat16).float() for r in range(world)) + res.float()
        for r in range(world):
            assert torch.equal(outs[r], outs[0])
        scale = float(want.abs().max())
        torch.testing.assert_close(outs[0].float(), want, atol=1e-2 * scale, rtol=1e-2)
        if it == 2:
            q2, s2 = KB.rmsnorm_quant_int8(outs[0], gamma, 1e-5)          # the stand-alone kernel on the same rows
            for r in range(world):
                assert torch.equal(nq[r], nq[0]) and torch.equal(nscale[r], nscale[0])
            torch.testing.assert_close(nscale[0], s2, rtol=2e-2, atol=0)
            assert float((nq[0].float() * nscale[0][:, None] - q2.float() * s2[:, None]).abs().max()) <= 3 * float(s2.max())
