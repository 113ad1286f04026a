"""Numerics of every hand-written kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from ronn_b200 import ops
    return ops


def _rand(*shape, dtype=torch.bfloat16, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("M,N,K_,bn", [(128, 128, 64, 0), (256, 1024, 1024, 0), (200, 264, 320, 32), (256, 3072, 1024, 64),
                                       (300, 512, 4096, 128), (128, 256, 128, 256), (1, 50264, 256, 0), (77, 72, 136, 0)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_plain(K, M, N, K_, bn, dtype):
    a, w = _rand(M, K_, dtype=dtype), _rand(N, K_, dtype=dtype, scale=0.05)
    y = K.gemm(a, w, bn=bn)
    K.check_status()
    ref = a.float() @ w.float().t()
    assert y.shape == (M, N)
    torch.testing.assert_close(y.float(), ref, atol=2e-2 * math.sqrt(K_ / 64), rtol=2e-2)


@pytest.mark.parametrize("act", ["", "relu", "gelu"])
def test_gemm_epilogue(K, act):
    M, N, K_ = 256, 1024, 512
    a, w = _rand(M, K_), _rand(N, K_, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    y = K.gemm(a, w, bias, res, act)
    K.check_status()
    ref = a.float() @ w.float().t() + bias.float()
    if act == "relu":
        ref = torch.relu(ref)
    elif act == "gelu":
        ref = F.gelu(ref, approximate="tanh")
    ref = ref + res.float()
    torch.testing.assert_close(y.float(), ref, atol=6e-2, rtol=2e-2)
    y32 = K.gemm(a, w, bias, None, act, out_fp32=True)
    assert y32.dtype == torch.float32
    torch.testing.assert_close(y32, ref - res.float(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K_,S,bn", [(256, 1024, 4096, 4, 64), (64, 1024, 4096, 8, 0), (37, 136, 1024, 3, 32),
                                         (128, 768, 3072, 4, 128)])
@pytest.mark.parametrize("norm", ["", "layernorm", "rmsnorm"])
def test_gemm_splitk_and_finalize(K, M, N, K_, S, bn, norm):
    a, w = _rand(M, K_), _rand(N, K_, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    gamma, beta = _rand(N), _rand(N)
    ws, s_eff = K.gemm_splitk(a, w, S, bn=bn)
    K.check_status()
    assert 1 <= s_eff <= S
    part = ws[:s_eff * M * N].view(s_eff, M, N)
    ref = a.float() @ w.float().t()
    torch.testing.assert_close(part.sum(0), ref, atol=2e-2 * math.sqrt(K_ / 64), rtol=2e-2)
    total, y = K.splitk_finalize(ws, s_eff, M, N, torch.bfloat16, bias=bias, residual=res, gamma=gamma,
                                 beta=beta if norm == "layernorm" else None, norm=norm)
    full = ref + bias.float() + res.float()
    torch.testing.assert_close(total.float(), full, atol=0.15, rtol=2e-2)
    if norm:
        t = total.float()
        if norm == "layernorm":
            want = F.layer_norm(t, (N,), gamma.float(), beta.float(), 1e-5)
        else:
            want = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
        torch.testing.assert_close(y.float(), want, atol=6e-2, rtol=3e-2)
    else:
        assert y is None


@pytest.mark.parametrize("H", [128, 768, 1024, 2560])
def test_layernorm_rmsnorm(K, H):
    x, r = _rand(37, H), _rand(37, H)
    g, b = _rand(H), _rand(H)
    y = K.layernorm(x, g, b, 1e-5)
    ref = F.layer_norm(x.float(), (H,), g.float(), b.float(), 1e-5)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    y2, s2 = K.layernorm(x, g, b, 1e-5, residual=r, return_sum=True)
    sref = (x.float() + r.float())
    torch.testing.assert_close(s2.float(), sref, atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(y2.float(), F.layer_norm(sref, (H,), g.float(), b.float(), 1e-5), atol=5e-2, rtol=2e-2)
    y3 = K.rmsnorm(x, g, 1e-6)
    xf = x.float()
    torch.testing.assert_close(y3.float(), xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float(),
                               atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("cols", [10, 128, 1000, 5000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax(K, cols, dtype):
    x = _rand(19, cols, dtype=dtype, scale=3.0)
    y = K.softmax(x)
    torch.testing.assert_close(y.float(), torch.softmax(x.float(), -1), atol=1e-2 if dtype != torch.float32 else 1e-5,
                               rtol=2e-2 if dtype != torch.float32 else 1e-4)


def test_elementwise(K):
    x, y = _rand(1000, 77), _rand(1000, 77)
    torch.testing.assert_close(K.unary(x, "relu").float(), torch.relu(x.float()))
    torch.testing.assert_close(K.unary(x, "gelu").float(), F.gelu(x.float(), approximate="tanh"), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(K.unary(x, "fast_gelu").float(), x.float() * torch.sigmoid(1.702 * x.float()), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(K.unary(x, "sigmoid").float(), torch.sigmoid(x.float()), atol=1e-2, rtol=2e-2)
    torch.testing.assert_close(K.unary(x, "silu").float(), F.silu(x.float()), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(K.unary(x, "tanh").float(), torch.tanh(x.float()), atol=1e-2, rtol=2e-2)
    torch.testing.assert_close(K.binary(x, y, "add").float(), (x.float() + y.float()), atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(K.binary(x, y, "mul").float(), (x.float() * y.float()), atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(K.binary(x, y, "add_relu").float(), torch.relu(x.float() + y.float()), atol=2e-2, rtol=1e-2)
    z = _rand(33, 256)
    torch.testing.assert_close(K.swiglu_fused(z).float(), F.silu(z[:, :128].float()) * z[:, 128:].float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(K.cast(x, torch.float32), x.float())


@pytest.mark.parametrize("H,rows", [(768, 8192), (1024, 4099), (2560, 2048), (4096, 2050), (136, 3001)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_many_rows_streaming_norms(K, H, rows, dtype):
    """Row counts that take the shared-memory ring path (one warp per row, bulk-copy loads)."""
    x, r = _rand(rows, H, dtype=dtype), _rand(rows, H, dtype=dtype)
    g, b = _rand(H, dtype=dtype), _rand(H, dtype=dtype)
    y = K.layernorm(x, g, b, 1e-5)
    ref = F.layer_norm(x.float(), (H,), g.float(), b.float(), 1e-5)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    y2, s2 = K.layernorm(x, g, b, 1e-5, residual=r, return_sum=True)
    sref = (x.float() + r.float()).to(dtype).float()
    torch.testing.assert_close(s2.float(), sref, atol=0, rtol=0)
    torch.testing.assert_close(y2.float(), F.layer_norm(sref, (H,), g.float(), b.float(), 1e-5), atol=5e-2, rtol=2e-2)
    y3 = K.rmsnorm(x, g, 1e-6)
    xf = x.float()
    torch.testing.assert_close(y3.float(), xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float(),
                               atol=3e-2, rtol=2e-2)
    y4, s4 = K.rmsnorm(x, g, 1e-6, residual=r, return_sum=True)
    torch.testing.assert_close(s4.float(), sref, atol=0, rtol=0)
    torch.testing.assert_close(y4.float(), sref * torch.rsqrt(sref.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float(),
                               atol=5e-2, rtol=2e-2)
    K.check_status()


def test_many_rows_layernorm_with_a_large_mean(K):
    """The streaming kernel takes its statistics in one pass around a per-row shift: rows whose mean dwarfs their spread
    must not lose the variance to cancellation."""
    rows, H = 4096, 1024
    x = (torch.randn(rows, H, device="cuda") * 0.5 + torch.linspace(-300, 300, rows, device="cuda")[:, None]).to(torch.float16)
    g, b = _rand(H, dtype=torch.float16), _rand(H, dtype=torch.float16)
    y = K.layernorm(x, g, b, 1e-5)
    ref = F.layer_norm(x.float(), (H,), g.float(), b.float(), 1e-5)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    small = K.layernorm(x[:64].contiguous(), g, b, 1e-5)          # the few-rows kernel (two-pass statistics)
    torch.testing.assert_close(y[:64].float(), small.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("cols,rows", [(128, 5000), (1024, 2048), (1000, 4097), (5000, 2100)])
def test_many_rows_streaming_softmax(K, cols, rows):
    x = _rand(rows, cols, scale=3.0)
    y = K.softmax(x)
    torch.testing.assert_close(y.float(), torch.softmax(x.float(), -1), atol=1e-2, rtol=2e-2)
    K.check_status()


@pytest.mark.parametrize("H,rows", [(2560, 4096), (6912, 2048), (1024, 3000)])
def test_many_rows_streaming_quantisers(K, H, rows):
    from ronn_b200.ops import bitnet as B
    x, g = _rand(rows, H), _rand(H)
    q, s = B.act_quant_int8(x)
    xf = x.float()
    sref = xf.abs().amax(-1).clamp_min(1e-5) / 127
    torch.testing.assert_close(s, sref, rtol=1e-6, atol=0)
    qref = torch.clamp(torch.round(xf * (127.0 / xf.abs().amax(-1, keepdim=True).clamp_min(1e-5))), -127, 127)
    assert (q.float() - qref).abs().max() <= 1
    # small-row kernel and streaming kernel agree bit for bit
    q_small, s_small = B.act_quant_int8(x[:64].contiguous())
    assert torch.equal(q_small, q[:64]) and torch.equal(s_small, s[:64])
    q2, s2 = B.rmsnorm_quant_int8(x, g, 1e-5)
    q2_small, s2_small = B.rmsnorm_quant_int8(x[:64].contiguous(), g, 1e-5)
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()).bfloat16().float()
    sref2 = normed.abs().amax(-1) / 127
    torch.testing.assert_close(s2, sref2, rtol=2e-2, atol=1e-6)
    torch.testing.assert_close(q2.float() * s2[:, None], normed, atol=float(sref2.max()) * 1.5, rtol=0)
    torch.testing.assert_close(s2[:64], s2_small, rtol=1e-2, atol=1e-7)
    assert (q2[:64].float() - q2_small.float()).abs().max() <= 1
    K.check_status()


def test_elementwise_large_and_unaligned_argmax(K):
    """Sizes that reach the four-way unrolled loops, and argmax rows that start off a 16-byte boundary."""
    n = 148 * 8 * 256 * 8 * 5 + 24 + 3                       # five full turns of the resident wave + a tail
    x, y = _rand(n), _rand(n)
    torch.testing.assert_close(K.unary(x, "relu").float(), torch.relu(x.float()))
    torch.testing.assert_close(K.binary(x, y, "add").float(), (x.float() + y.float()).bfloat16().float())
    torch.testing.assert_close(K.cast(x, torch.float32), x.float())
    xf = torch.randn(n, device="cuda")
    assert torch.equal(K.cast(xf, torch.bfloat16), xf.bfloat16())
    assert torch.equal(K.cast(xf[:1003].contiguous(), torch.float16), xf[:1003].half())
    assert torch.equal(K.cast(x[:1003].contiguous().half(), torch.float32), x[:1003].half().float())
    z = _rand(40000, 512)
    torch.testing.assert_close(K.swiglu_fused(z).float(), (F.silu(z[:, :256].float()) * z[:, 256:].float()),
                               atol=3e-2, rtol=2e-2)
    for cols in (50257, 50264, 1001, 7):
        lb = torch.randn(33, cols, device="cuda").bfloat16()
        idx, mx = K.argmax(lb, return_max=True)
        ref_max = lb.float().max(-1).values
        torch.testing.assert_close(mx, ref_max)
        first = (lb.float() == ref_max[:, None]).float().argmax(-1)          # lowest index among ties
        assert torch.equal(idx.long(), first)


def test_embedding_argmax(K):
    table, ptab = _rand(1000, 256), _rand(64, 256)
    ids = torch.randint(0, 1000, (50,), device="cuda", dtype=torch.int32)
    pos = torch.randint(0, 64, (50,), device="cuda", dtype=torch.int32)
    y = K.embedding(ids, table, pos, ptab)
    torch.testing.assert_close(y.float(), table[ids.long()].float() + ptab[pos.long()].float(), atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(K.embedding(ids, table), table[ids.long()])
    lg = torch.randn(37, 50257, device="cuda")
    idx, mx = K.argmax(lg, return_max=True)
    assert torch.equal(idx.long(), lg.argmax(-1))
    torch.testing.assert_close(mx, lg.max(-1).values)
    lb = lg.bfloat16()
    idx_b = K.argmax(lb)
    assert torch.equal(lb.float().gather(1, idx_b.long()[:, None])[:, 0], lb.float().max(-1).values)
    vals = torch.stack([mx, mx - 1.0])
    comb = K.argmax_combine(vals, torch.stack([idx, idx + 7]))
    assert torch.equal(comb, idx)


def _fill_cache(tokens_per_seq, heads, d, nblocks, dtype):
    kc = torch.zeros(nblocks, heads, 16, d, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    return kc, vc


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 4, 4), (128, 4, 2), (64, 16, 16)])
def test_kv_append_and_paged_attention(K, d, heads, kv_heads):
    torch.manual_seed(0)
    dtype = torch.bfloat16
    lens = [1, 15, 16, 17, 100, 333]
    B = len(lens)
    max_blocks = 24
    nblocks = B * max_blocks
    perm = torch.randperm(nblocks)[: B * max_blocks].reshape(B, max_blocks).to(torch.int32).cuda()
    kc, vc = _fill_cache(lens, kv_heads, d, nblocks, dtype)
    ld = (heads + 2 * kv_heads) * d
    ks, vs, last_q = [], [], []
    for b, L in enumerate(lens):
        qkv = _rand(L, ld, dtype=dtype)
        slots = torch.tensor([int(perm[b, t // 16]) * 16 + t % 16 for t in range(L)], device="cuda", dtype=torch.int32)
        K.kv_append(qkv, heads * d, (heads + kv_heads) * d, slots, kc, vc, heads, kv_heads, d)
        ks.append(qkv[:, heads * d:(heads + kv_heads) * d].reshape(L, kv_heads, d).float())
        vs.append(qkv[:, (heads + kv_heads) * d:].reshape(L, kv_heads, d).float())
        last_q.append(qkv[-1:].clone())
    q = torch.cat(last_q)
    ctx = torch.tensor(lens, device="cuda", dtype=torch.int32)
    out = K.paged_attention(q, kc, vc, perm, ctx, heads, kv_heads, d, max_ctx=384)
    rep = heads // kv_heads
    for b, L in enumerate(lens):
        qh = q[b, :heads * d].reshape(heads, d).float()
        kk = ks[b].repeat_interleave(rep, dim=1)
        vv = vs[b].repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,lhd->hl", qh, kk) / math.sqrt(d)
        ref = torch.einsum("hl,lhd->hd", torch.softmax(s, -1), vv).reshape(-1)
        torch.testing.assert_close(out[b].float(), ref, atol=2e-2, rtol=2e-2)
    # ragged causal rows: every token of the longest sequence, length = position + 1
    b, L = B - 1, lens[-1]
    # rebuild that sequence's queries
    torch.manual_seed(1)
    qs = _rand(L, heads * d, dtype=dtype)
    ctx_t = torch.arange(1, L + 1, device="cuda", dtype=torch.int32)
    bt_row = torch.full((L,), b, device="cuda", dtype=torch.int32)
    out2 = K.paged_attention(qs, kc, vc, perm, ctx_t, heads, kv_heads, d, max_ctx=384, bt_row=bt_row)
    kk = ks[b].repeat_interleave(rep, dim=1)
    vv = vs[b].repeat_interleave(rep, dim=1)
    s = torch.einsum("qhd,lhd->hql", qs.reshape(L, heads, d).float(), kk) / math.sqrt(d)
    s = s + torch.full((L, L), float("-inf"), device="cuda").triu(1)
    ref2 = torch.einsum("hql,lhd->qhd", torch.softmax(s, -1), vv).reshape(L, -1)
    torch.testing.assert_close(out2.float(), ref2, atol=2e-2, rtol=2e-2)


def test_kv_append_rope(K):
    from ronn_b200.onnx.registry import rotary
    heads, kv_heads, d, T = 4, 2, 128, 9
    ld = (heads + 2 * kv_heads) * d
    qkv = _rand(T, ld)
    ref_q = rotary(qkv[:, :heads * d].clone(), torch.arange(T, device="cuda"), 10000.0, heads)
    ref_k = rotary(qkv[:, heads * d:(heads + kv_heads) * d].clone(), torch.arange(T, device="cuda"), 10000.0, kv_heads)
    kc = torch.zeros(2, kv_heads, 16, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.arange(T, device="cuda", dtype=torch.int32)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    K.kv_append(qkv, heads * d, (heads + kv_heads) * d, slots, kc, vc, heads, kv_heads, d, pos, 10000.0)
    torch.testing.assert_close(qkv[:, :heads * d].float(), ref_q.float(), atol=3e-2, rtol=2e-2)
    got_k = kc[0, :, :T, :].permute(1, 0, 2).reshape(T, -1)
    torch.testing.assert_close(got_k.float(), ref_k.float(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 4, 4), (128, 4, 2), (64, 2, 2)])
@pytest.mark.parametrize("splits", [2, 3, 8])
def test_paged_attention_split_over_cache_blocks(K, d, heads, kv_heads, splits):
    """Several CTAs per (row, head), combined by the last one to finish: same result as one CTA, for contexts shorter
    than the number of splits, empty rows, and twice in a row (the tickets return to zero)."""
    torch.manual_seed(4)
    dtype = torch.bfloat16
    lens = [0, 1, 15, 16, 17, 33, 100, 333, 640, 48]
    B, max_blocks = len(lens), 40
    nblocks = B * max_blocks
    perm = torch.randperm(nblocks).reshape(B, max_blocks).to(torch.int32).cuda()
    kc = (torch.randn(nblocks, kv_heads, 16, d, device="cuda") * 0.5).to(dtype)
    vc = (torch.randn(nblocks, kv_heads, 16, d, device="cuda") * 0.5).to(dtype)
    q = _rand(B, heads * d, dtype=dtype)
    ctx = torch.tensor(lens, device="cuda", dtype=torch.int32)
    one = K.paged_attention(q, kc, vc, perm, ctx, heads, kv_heads, d, max_ctx=640, splits=1)
    for _ in range(2):
        many = K.paged_attention(q, kc, vc, perm, ctx, heads, kv_heads, d, max_ctx=640, splits=splits)
        K.check_status()
        torch.testing.assert_close(many.float(), one.float(), atol=4e-3, rtol=1e-2)
    assert float(many[0].abs().max()) == 0.0
    # fp32 restatement of one long row
    b, n = 8, lens[8]
    kk = torch.stack([kc[int(perm[b, t // 16]), :, t % 16] for t in range(n)]).float()
    vv = torch.stack([vc[int(perm[b, t // 16]), :, t % 16] for t in range(n)]).float()
    rep = heads // kv_heads
    s_ = torch.einsum("hd,lhd->hl", q[b].float().view(heads, d), kk.repeat_interleave(rep, dim=1)) / math.sqrt(d)
    want = torch.einsum("hl,lhd->hd", torch.softmax(s_, -1), vv.repeat_interleave(rep, dim=1)).reshape(-1)
    torch.testing.assert_close(many[b].float(), want, atol=2e-2, rtol=2e-2)
    # with the fused append and rotary embedding
    qkv = _rand(B, (heads + 2 * kv_heads) * d, dtype=dtype)
    pos = torch.tensor([max(n - 1, 0) for n in lens], device="cuda", dtype=torch.int32)
    slots = torch.tensor([int(perm[i, max(n - 1, 0) // 16]) * 16 + max(n - 1, 0) % 16 if n > 0 else -1
                          for i, n in enumerate(lens)], device="cuda", dtype=torch.int32)
    kc1, vc1 = kc.clone(), vc.clone()
    a1 = K.paged_attention(qkv, kc1, vc1, perm, ctx, heads, kv_heads, d, max_ctx=640,
                           append=(heads * d, (heads + kv_heads) * d, slots), rope=(pos, 10000.0), splits=1)
    kc2, vc2 = kc.clone(), vc.clone()
    a2 = K.paged_attention(qkv, kc2, vc2, perm, ctx, heads, kv_heads, d, max_ctx=640,
                           append=(heads * d, (heads + kv_heads) * d, slots), rope=(pos, 10000.0), splits=splits)
    K.check_status()
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    torch.testing.assert_close(a2.float(), a1.float(), atol=4e-3, rtol=1e-2)


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 4, 4), (128, 8, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rope_append_attention_in_one_launch(K, d, heads, kv_heads, dtype):
    """Decode rows with rotary embedding: the one-launch form (rotate q and the new k, append, attend) against the
    rotate-and-append kernel followed by plain paged attention, and against an fp32 restatement."""
    from ronn_b200.onnx.registry import rotary
    torch.manual_seed(3)
    lens = [1, 16, 17, 130]
    B, max_blocks = len(lens), 12
    nblocks = B * max_blocks
    perm = torch.randperm(nblocks).reshape(B, max_blocks).to(torch.int32).cuda()
    kc = (torch.randn(nblocks, kv_heads, 16, d, device="cuda") * 0.5).to(dtype)      # earlier tokens: any values
    vc = (torch.randn(nblocks, kv_heads, 16, d, device="cuda") * 0.5).to(dtype)
    ld = (heads + 2 * kv_heads) * d
    qkv = _rand(B, ld, dtype=dtype)
    pos = torch.tensor([n - 1 for n in lens], device="cuda", dtype=torch.int32)
    slots = torch.tensor([int(perm[b, (n - 1) // 16]) * 16 + (n - 1) % 16 for b, n in enumerate(lens)],
                         device="cuda", dtype=torch.int32)
    ctx = torch.tensor(lens, device="cuda", dtype=torch.int32)
    kc2, vc2, qkv2 = kc.clone(), vc.clone(), qkv.clone()
    out = K.paged_attention(qkv, kc, vc, perm, ctx, heads, kv_heads, d, max_ctx=144,
                            append=(heads * d, (heads + kv_heads) * d, slots), rope=(pos, 10000.0))
    assert torch.equal(qkv, qkv2)                      # the fused form leaves the qkv row as it was
    K.kv_append(qkv2, heads * d, (heads + kv_heads) * d, slots, kc2, vc2, heads, kv_heads, d, pos, 10000.0)
    ref = K.paged_attention(qkv2, kc2, vc2, perm, ctx, heads, kv_heads, d, max_ctx=144)
    from ronn_b200 import ops
    ops.check_status()
    torch.testing.assert_close(kc.float(), kc2.float(), atol=1e-2, rtol=1e-2)
    assert torch.equal(vc, vc2)
    torch.testing.assert_close(out.float(), ref.float(), atol=1e-2, rtol=1e-2)
    # fp32 restatement for the longest row
    b, n = B - 1, lens[-1]
    qr = rotary(qkv[b:b + 1, :heads * d].float(), pos[b:b + 1], 10000.0, heads).reshape(heads, d)
    kk = torch.stack([kc[int(perm[b, t // 16]), :, t % 16] for t in range(n)]).float()      # [n, kv, d]
    vv = torch.stack([vc[int(perm[b, t // 16]), :, t % 16] for t in range(n)]).float()
    rep = heads // kv_heads
    s_ = torch.einsum("hd,lhd->hl", qr, kk.repeat_interleave(rep, dim=1)) / math.sqrt(d)
    want = torch.einsum("hl,lhd->hd", torch.softmax(s_, -1), vv.repeat_interleave(rep, dim=1)).reshape(-1)
    torch.testing.assert_close(out[b].float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("shape", [
    # N, H, W, C, Cout, R, stride, pad
    (2, 16, 16, 64, 64, 3, 1, 1), (2, 17, 19, 16, 72, 3, 2, 1), (1, 56, 56, 64, 128, 1, 2, 0),
    (2, 32, 32, 8, 64, 7, 2, 3), (3, 7, 7, 256, 512, 3, 1, 1), (1, 9, 9, 128, 32, 3, 1, 0)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_conv_igemm(shape, dtype):
    from ronn_b200.providers.gpu_conv import conv2d_nhwc
    N, H, W, C, Co, R, st, pad = shape
    torch.manual_seed(0)
    x = _rand(N, H, W, C, dtype=dtype)
    w = _rand(Co, R, R, C, dtype=dtype, scale=1.0 / math.sqrt(R * R * C))
    b = _rand(Co, dtype=dtype)
    ref = F.conv2d(x.permute(0, 3, 1, 2).float(), w.permute(0, 3, 1, 2).float(), b.float(), st, pad)
    y = conv2d_nhwc(x, w, b, None, st, pad, 1, relu=False)
    from ronn_b200 import ops
    ops.check_status()
    torch.testing.assert_close(y.permute(0, 3, 1, 2).float(), ref, atol=3e-2, rtol=3e-2)
    res = _rand(*y.shape, dtype=dtype)
    y2 = conv2d_nhwc(x, w, b, res, st, pad, 1, relu=True)
    torch.testing.assert_close(y2.permute(0, 3, 1, 2).float(), torch.relu(ref + res.permute(0, 3, 1, 2).float()), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("shape,axis", [((4, 8, 128), 1), ((4, 8, 128), 0), ((2, 3, 5, 7), 2), ((3000, 64), 0), ((6, 1000, 9), 1),
                                        ((16, 512), -1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_softmax_over_any_axis(K, shape, axis, dtype):
    """Softmax over an inner or leading axis runs on the tensor as it lies in memory (strides), no transpose."""
    x = (torch.randn(*shape, device="cuda") * 3).to(dtype)
    y = K.softmax(x, axis)
    ref = torch.softmax(x.float(), dim=axis)
    tol = {torch.bfloat16: 1e-2, torch.float16: 2e-3, torch.float32: 1e-5}[dtype]
    torch.testing.assert_close(y.float(), ref, atol=tol, rtol=3e-2 if dtype != torch.float32 else 1e-4)
    torch.testing.assert_close(y.float().sum(axis), torch.ones_like(ref.sum(axis)), atol=2e-2, rtol=0)


def test_pool_kernels():
    from ronn_b200.providers.gpu_conv import global_avgpool_nhwc, maxpool_nhwc
    x = _rand(3, 23, 21, 72, dtype=torch.float16)
    y = maxpool_nhwc(x, 3, 2, 1)
    ref = F.max_pool2d(x.permute(0, 3, 1, 2).float(), 3, 2, 1).permute(0, 2, 3, 1)
    torch.testing.assert_close(y.float(), ref)
    g = global_avgpool_nhwc(x)
    torch.testing.assert_close(g.float().reshape(3, 72), x.float().mean((1, 2)), atol=2e-3, rtol=2e-3)
    for shape, dt in (((5, 7, 7, 512), torch.float16), ((2, 9, 5, 264), torch.bfloat16), ((3, 1, 1, 1024), torch.float16),
                      ((2, 30, 3, 776), torch.bfloat16)):
        xw = _rand(*shape, dtype=dt)                      # wide maps: one CTA per 512-channel slab
        gw = global_avgpool_nhwc(xw)
        torch.testing.assert_close(gw.float().reshape(shape[0], shape[3]), xw.float().mean((1, 2)), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M,N,K_", [(128, 2560, 2560), (128, 320, 6912), (37, 72, 256), (130, 96, 128), (1, 32000, 2560),
                                     (64, 200, 1040), (9, 40, 48), (256, 4096, 832), (300, 130, 2112)])
def test_bitlinear_exact_against_host_oracle(M, N, K_):
    from ronn_b200.ops import bitnet as B
    from ronn_b200.providers.bitnet.quantization import bitlinear_reference, pack_ternary_rows
    torch.manual_seed(M + N)
    wq = torch.randint(-1, 2, (N, K_), dtype=torch.int8)
    packed = pack_ternary_rows(wq)
    x = (torch.randn(M, K_) * 2).bfloat16()
    ref = bitlinear_reference(x.float(), packed, torch.tensor(0.043), None, K_, N)
    y = B.bitlinear(x.cuda(), packed.cuda(), 0.043, None, K_, N)
    from ronn_b200 import ops
    ops.check_status()
    # integer accumulation is exact; only the final bf16 rounding differs from the fp32 oracle
    torch.testing.assert_close(y.float().cpu(), ref, atol=2e-2, rtol=1e-2)
    q, s = B.act_quant_int8(x.cuda())
    sref = x.float().abs().amax(-1).clamp_min(1e-5) / 127
    torch.testing.assert_close(s.cpu(), sref, rtol=1e-6, atol=0)
    qref = torch.round(x.float() * (127.0 / x.float().abs().amax(-1, keepdim=True).clamp_min(1e-5))).clamp(-127, 127)
    assert (q.cpu().float() - qref).abs().max() <= 1          # rint ties / reciprocal rounding
    acc = (q.cpu().to(torch.int32) @ wq.to(torch.int32).t()).float() * s.cpu()[:, None] * 0.043
    torch.testing.assert_close(y.float().cpu(), acc, atol=1e-2, rtol=1e-2)
    assert torch.equal(B.ternary_pack(wq.cuda()).cpu(), packed)


@pytest.mark.parametrize("rows,F_", [(128, 6912), (37, 864), (1, 3456), (300, 1728)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_swiglu_quant_fused_equals_swiglu_then_quant(rows, F_, dtype):
    """SwiGLU + per-token int8 quantisation in one kernel against the two-kernel form (bit-identical: the fused kernel
    rounds the product through the storage type as the stand-alone SwiGLU stores it) and against an fp32 reference."""
    from ronn_b200.ops import bitnet as B
    from ronn_b200.ops import kernels as K
    x = (torch.randn(rows, 2 * F_, device="cuda") * 1.5).to(dtype)
    q, s = B.swiglu_quant_int8(x)
    y = K.swiglu_fused(x)
    q2, s2 = B.act_quant_int8(y)
    assert torch.equal(s, s2)
    assert int((q.int() - q2.int()).abs().max()) == 0
    ref = torch.nn.functional.silu(x[:, :F_].float()) * x[:, F_:].float()
    deq = q.float() * s[:, None]
    step = ref.abs().amax(-1, keepdim=True) / 127
    assert bool(((deq - ref).abs() <= step * 0.51 + ref.abs() * (8e-3 if dtype == torch.bfloat16 else 2e-3) + 1e-6).all())


def test_rmsnorm_quant_fused():
    from ronn_b200.ops import bitnet as B
    x = _rand(19, 2560)
    g = _rand(2560)
    q, s = B.rmsnorm_quant_int8(x, g, 1e-5)
    xf = x.float()
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()).bfloat16().float()
    sref = normed.abs().amax(-1) / 127
    torch.testing.assert_close(s, sref, rtol=2e-2, atol=1e-6)
    deq = q.float() * s[:, None]
    torch.testing.assert_close(deq, normed, atol=float(sref.max()) * 1.5, rtol=0)


def _sdpa_ref(q, k, v, causal, shift=0):
    # q [Lq, H, d], k/v [Lk, Hkv, d] fp32
    H, Hkv = q.shape[1], k.shape[1]
    k = k.repeat_interleave(H // Hkv, dim=1)
    v = v.repeat_interleave(H // Hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(q.shape[-1])
    if causal:
        Lq, Lk = q.shape[0], k.shape[0]
        mask = torch.arange(Lk, device=q.device)[None, :] > (torch.arange(Lq, device=q.device)[:, None] + shift)
        s = s.masked_fill(mask[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), v)


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 4, 4), (64, 8, 2), (128, 4, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dense_attention_ragged_causal(K, d, heads, kv_heads, dtype):
    lens = [1, 5, 128, 129, 300, 64, 517]
    T = sum(lens)
    hn, kn = heads * d, kv_heads * d
    qkv = _rand(T, hn + 2 * kn, dtype=dtype)
    plan = K.dense_attention_plan(lens, "cuda")
    out = K.dense_attention(qkv, 0, hn, hn + kn, plan, heads, kv_heads, d, causal=True)
    K.check_status()
    t = 0
    for n in lens:
        rows = qkv[t:t + n].float()
        ref = _sdpa_ref(rows[:, :hn].view(n, heads, d), rows[:, hn:hn + kn].view(n, kv_heads, d),
                        rows[:, hn + kn:].view(n, kv_heads, d), True)
        torch.testing.assert_close(out[t:t + n].float().view(n, heads, d), ref, atol=2e-2, rtol=2e-2)
        t += n


def test_dense_attention_padded_encoder(K):
    B, S, heads, d = 6, 128, 12, 64
    lens = [128, 100, 1, 37, 128, 64]
    hn = heads * d
    qkv = _rand(B * S, 3 * hn)
    plan = K.dense_attention_plan(lens, "cuda", row_lens=[S] * B)
    q_len = torch.full((B,), S, dtype=torch.int32, device="cuda")
    out = K.dense_attention(qkv, 0, hn, 2 * hn, plan, heads, heads, d, causal=False, q_len=q_len, max_q_len=S)
    K.check_status()
    for b, n in enumerate(lens):
        rows = qkv[b * S:(b + 1) * S].float()
        ref = _sdpa_ref(rows[:, :hn].view(S, heads, d), rows[:n, hn:2 * hn].view(n, heads, d),
                        rows[:n, 2 * hn:].view(n, heads, d), False)
        torch.testing.assert_close(out[b * S:(b + 1) * S].float().view(S, heads, d), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 4, 4), (64, 8, 2), (128, 4, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_prefill_attention_cached_context(K, d, heads, kv_heads, dtype):
    """Query chunks over the paged cache: (cached context, new tokens) per sequence; the new tokens' K / V are in the
    cache already, every query sees the context and the new tokens up to itself."""
    torch.manual_seed(7)
    cases = [(0, 37), (16, 1), (100, 128), (300, 200), (517, 3), (128, 129), (0, 256)]
    max_blocks = 48
    nblocks = len(cases) * max_blocks + 1
    perm = (torch.randperm(nblocks - 1)[: len(cases) * max_blocks] + 1).reshape(len(cases), max_blocks).to(torch.int32).cuda()
    kc = torch.zeros(nblocks, kv_heads, 16, d, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    hn = heads * d
    T = sum(c for _, c in cases)
    qbuf = _rand(T, hn + 24, dtype=dtype)                 # queries at column 8 of a wider buffer
    ks, vs, starts, t = [], [], [], 0
    for b, (ctx, new) in enumerate(cases):
        n = ctx + new
        k, v = _rand(n, kv_heads, d, dtype=dtype), _rand(n, kv_heads, d, dtype=dtype)
        for tok in range(n):
            blk = int(perm[b, tok // 16])
            kc[blk, :, tok % 16] = k[tok]
            vc[blk, :, tok % 16] = v[tok]
        ks.append(k.float())
        vs.append(v.float())
        starts.append(t)
        t += new
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    out = K.paged_prefill_attention(qbuf, 8, kc, vc, perm, mk(starts), mk([c for _, c in cases]),
                                    mk([a + c for a, c in cases]), max(c for _, c in cases), heads, kv_heads, d)
    K.check_status()
    for b, (ctx, new) in enumerate(cases):
        q = qbuf[starts[b]:starts[b] + new, 8:8 + hn].float().view(new, heads, d)
        ref = _sdpa_ref(q, ks[b], vs[b], True, shift=ctx)
        torch.testing.assert_close(out[starts[b]:starts[b] + new].float().view(new, heads, d), ref, atol=2e-2, rtol=2e-2)
    # a table row shared by two sequences (bt_row) and full visibility (no causal mask)
    bt_row = mk([3, 3])
    out2 = K.paged_prefill_attention(qbuf[:40], 8, kc, vc, perm, mk([0, 20]), mk([20, 20]), mk([500, 321]), 20, heads,
                                     kv_heads, d, causal=False, bt_row=bt_row)
    K.check_status()
    for i, n in enumerate((500, 321)):
        q = qbuf[i * 20:(i + 1) * 20, 8:8 + hn].float().view(20, heads, d)
        ref = _sdpa_ref(q, ks[3][:n], vs[3][:n], False)
        torch.testing.assert_close(out2[i * 20:(i + 1) * 20].float().view(20, heads, d), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K_", [(256, 1024, 1024), (256, 1024, 4096), (100, 384, 512), (130, 128, 64), (1, 768, 3072)])
@pytest.mark.parametrize("norm", ["layernorm", "rmsnorm"])
def test_gemm_rownorm_cluster(K, M, N, K_, norm):
    a, w = _rand(M, K_), _rand(N, K_, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    gamma, beta = _rand(N), _rand(N)
    x, y = K.gemm_rownorm(a, w, bias, res, gamma, beta if norm == "layernorm" else None, 1e-5, norm)
    K.check_status()
    ref = a.float() @ w.float().t() + bias.float() + res.float()
    torch.testing.assert_close(x.float(), ref, atol=2e-2 * math.sqrt(K_ / 64) + 0.06, rtol=2e-2)
    t = x.float()                                      # the norm is taken over the stored (rounded) sums
    if norm == "layernorm":
        want = F.layer_norm(t, (N,), gamma.float(), beta.float(), 1e-5)
    else:
        want = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
    torch.testing.assert_close(y.float(), want, atol=6e-2, rtol=3e-2)
    # no residual, no bias
    x2, y2 = K.gemm_rownorm(a, w, None, None, gamma, None, 1e-5, "rmsnorm")
    K.check_status()
    torch.testing.assert_close(x2.float(), a.float() @ w.float().t(), atol=2e-2 * math.sqrt(K_ / 64) + 0.03, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_elementwise_chain(K, dtype):
    """Eight element-wise operators in one launch, with a full-size, a last-dimension-vector and a scalar operand."""
    x = _rand(512, 768, dtype=dtype)
    bias, full, scal = _rand(768, dtype=dtype), _rand(512, 768, dtype=dtype), torch.tensor([0.5], device="cuda", dtype=dtype)
    names = ["Add", "Gelu", "Mul", "Sub", "Sigmoid", "Abs", "Sqrt", "Div"]
    operands = [bias, None, full, scal, None, None, None, full.abs() + 1]
    y = K.fused_elementwise(x, names, operands)
    r = F.gelu(x.float() + bias.float(), approximate="tanh") * full.float() - 0.5
    r = torch.sqrt(torch.sigmoid(r).abs()) / (full.abs() + 1).float()
    torch.testing.assert_close(y.float(), r, atol=2e-2, rtol=2e-2)
    for name, ref in (("Relu", torch.relu), ("Tanh", torch.tanh), ("Neg", torch.neg), ("Exp", torch.exp),
                      ("Swish", lambda t: t * torch.sigmoid(t))):
        got = K.fused_elementwise(x, [name, "Neg", "Neg"], [None, None, None])
        torch.testing.assert_close(got.float(), ref(x.float()), atol=3e-2, rtol=2e-2)
    # what does not fit is reported by the planner, not launched
    assert K.fused_elementwise_plan(x[:, :100], ["Relu"], [None]) is None              # not contiguous
    assert K.fused_elementwise_plan(x, ["Add"], [_rand(512, 1, dtype=dtype)]) is None   # broadcast along the rows
    assert K.fused_elementwise_plan(x, ["Erf"], [None]) is None


def _sample_setup(K, rows, temperature=1.0, top_k=0, top_p=1.0, penalty=1.0, seed=7, recent=None):
    buf = bytearray(rows * K.SAMPLE_RECORD_BYTES)
    for r in range(rows):
        K.pack_sample_params(buf, r, temperature, top_k, top_p, penalty, seed + r, 0 if recent is None else len(recent[r]))
    params = torch.frombuffer(buf, dtype=torch.uint8).cuda()
    rec = None
    if recent is not None:
        R = max(len(x) for x in recent)
        rec = torch.full((rows, R), -1, dtype=torch.int32)
        for r, x in enumerate(recent):
            rec[r, :len(x)] = torch.tensor(x, dtype=torch.int32)
        rec = rec.cuda()
    return params, rec, torch.zeros(rows, dtype=torch.int64, device="cuda")


def test_device_sampler_limits_match_argmax(K):
    logits = torch.randn(64, 50257, device="cuda")
    want = logits.argmax(-1).int()
    for kw in (dict(temperature=0.0), dict(top_k=1), dict(top_p=1e-6), dict(temperature=1e-4)):
        params, rec, ctr = _sample_setup(K, 64, **kw)
        got = K.sample(logits.clone(), params, rec, ctr)
        assert torch.equal(got, want), kw


def test_device_sampler_distribution_top_k_top_p_and_penalty(K):
    """Empirical token frequencies of 20 000 draws per setting against the probabilities the pipeline defines
    (penalty -> temperature -> top-k -> softmax -> top-p, computed in fp32 with torch)."""
    V, draws = 50, 20000
    base = torch.tensor([3.0, 2.5, 2.5, 2.0, 1.0, 0.5, 0.0, -0.5, -1.0, -3.0] + [-4.0 - 0.1 * i for i in range(V - 10)], device="cuda")

    def expected(temperature, top_k, top_p, penalty, recent):
        l = base.clone()
        if penalty != 1.0:
            idx = torch.tensor(sorted(set(recent)), device="cuda")
            l[idx] = torch.where(l[idx] > 0, l[idx] / penalty, l[idx] * penalty)
        l = l / temperature
        if top_k:
            kth = torch.topk(l, top_k).values[-1]
            l = torch.where(l < kth, torch.full_like(l, float("-inf")), l)
        p = torch.softmax(l, -1)
        if top_p < 1.0:
            sp, si = torch.sort(p, descending=True)
            drop = torch.cumsum(sp, 0) - sp > top_p
            sp = torch.where(drop, torch.zeros_like(sp), sp)
            p = torch.zeros_like(p).scatter_(0, si, sp)
            p = p / p.sum()
        return p

    for (t, k, pp, pen, rec) in [(1.0, 0, 1.0, 1.0, None), (0.7, 5, 1.0, 1.0, None), (1.3, 0, 0.8, 1.0, None),
                                 (1.0, 8, 0.9, 1.5, [0, 0, 3, 7])]:
        logits = base[None, :].repeat(draws, 1).contiguous()
        params, recent, ctr = _sample_setup(K, draws, t, k, pp, pen, seed=1234, recent=None if rec is None else [rec] * draws)
        tok = K.sample(logits, params, recent, ctr)
        freq = torch.bincount(tok.long(), minlength=V).float() / draws
        exp = expected(t, k, pp, pen, rec or [])
        assert float((freq[exp == 0]).sum()) == 0.0, (t, k, pp)            # nothing outside the kept set is ever drawn
        assert float((freq - exp).abs().max()) < 0.015, (t, k, pp, (freq - exp).abs().max())
    # the draw counter advances: a second call with the same seeds gives other tokens, the same counters the same tokens
    logits = base[None, :].repeat(256, 1).contiguous()
    params, _, ctr = _sample_setup(K, 256, 1.0)
    a = K.sample(logits.clone(), params, None, ctr)
    b = K.sample(logits.clone(), params, None, ctr)
    ctr.zero_()
    c = K.sample(logits.clone(), params, None, ctr)
    assert torch.equal(a, c) and not torch.equal(a, b)


def test_kernel_checks_refuse_a_bad_block_table_before_the_launch(K, monkeypatch):
    """With RONN_KERNEL_CHECKS=1 a block-table entry past the cache raises on the host and nothing is launched; the
    same call with valid indices runs as usual."""
    from ronn_b200 import _native
    monkeypatch.setenv("RONN_KERNEL_CHECKS", "1")
    kc = torch.zeros(8, 2, 16, 64, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = _rand(2, 4 * 64)
    bt = torch.tensor([[0, 1], [2, 3]], device="cuda", dtype=torch.int32)
    ctx = torch.tensor([20, 32], device="cuda", dtype=torch.int32)
    out = K.paged_attention(q, kc, vc, bt, ctx, 4, 2, 64, max_ctx=32)
    assert out.shape == (2, 256)
    lib = _native.cuda()
    calls = {"n": 0}
    real = lib.ronn_paged_attention
    lib.__dict__["ronn_paged_attention"] = lambda *a: (calls.__setitem__("n", calls["n"] + 1), real(*a))[1]
    try:
        bad = bt.clone()
        bad[1, 1] = 8
        with pytest.raises(K.KernelError, match="block_tables"):
            K.paged_attention(q, kc, vc, bad, ctx, 4, 2, 64, max_ctx=32)
        with pytest.raises(K.KernelError, match="slots"):
            K.kv_append(_rand(2, 8 * 64), 4 * 64, 6 * 64, torch.tensor([0, 128], device="cuda", dtype=torch.int32), kc, vc, 4, 2, 64)
    finally:
        lib.__dict__["ronn_paged_attention"] = real
    assert calls["n"] == 0
    K.check_status()
