"""Thin launch wrappers: torch tensors in, raw pointers + current stream into the native library.

Every wrapper raises ``KernelError`` when the native launcher reports a bad configuration; nothing
here falls back to PyTorch.  A status word on the device records abandoned waits inside the
tensor-core kernels; ``check_status`` reads it (one small device-to-host copy) and raises.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import _native
from . import checks as _checks
from ..api.errors import CommTimeoutError, RonnError


class KernelError(RonnError):
    prefix = "Kernel error: "


_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_ACT = {"": 0, None: 0, "none": 0, "Relu": 1, "relu": 1, "Gelu": 2, "gelu": 2}
_STATUS = {}
_STATUS_NAMES = {1: "TMA stage never arrived", 2: "pipeline stage never released", 3: "accumulator never committed",
                 4: "peer flag never raised", 5: "epilogue never drained",
                 0x5201: "row load of a streaming row-wise kernel never completed"}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _check(rc: int, what: str):
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def status_word(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _STATUS.get(dev)
    if w is None:
        w = torch.zeros(4, dtype=torch.int32, device=dev)
        _STATUS[dev] = w
        lib = _native.cuda()
        if hasattr(lib, "ronn_set_rowwise_status"):          # launchers without a status parameter report here too
            with torch.cuda.device(dev):
                lib.ronn_set_rowwise_status(w.data_ptr())
    return w


def check_status(device=None) -> None:
    """Raise if a bounded wait inside a kernel gave up since the last check."""
    w = status_word(device)
    code = int(w[0].item())
    if code:
        w.zero_()
        raise CommTimeoutError(f"a device-side wait was abandoned: {_STATUS_NAMES.get(code, code)}")


def gemm(a: torch.Tensor, w_nk: torch.Tensor, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, activation: str = "", out: Optional[torch.Tensor] = None,
         out_fp32: bool = False, bn: int = 0) -> torch.Tensor:
    """out[M,N] = act(a[M,K] @ w_nk[N,K]^T + bias) + residual on the tcgen05 tensor cores."""
    if a.dim() != 2 or w_nk.dim() != 2 or a.shape[1] != w_nk.shape[1]:
        raise KernelError(f"gemm shape mismatch: a {tuple(a.shape)} w {tuple(w_nk.shape)}")
    if a.dtype not in (torch.bfloat16, torch.float16) or w_nk.dtype != a.dtype:
        raise KernelError(f"gemm needs bf16/fp16 operands of one dtype, got {a.dtype} and {w_nk.dtype}")
    if a.stride(1) != 1 or w_nk.stride(1) != 1:
        raise KernelError("gemm operands must be K-contiguous")
    M, K = a.shape
    N = w_nk.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32 if out_fp32 else a.dtype, device=a.device)
    if residual is not None and (residual.stride(0) != out.stride(0) or residual.stride(1) != 1):
        residual = residual.contiguous()
        if residual.stride(0) != out.stride(0):
            raise KernelError("gemm residual must share the output's row stride")
    if bias is not None and bias.dtype != a.dtype:
        bias = bias.to(a.dtype)
    rc = _native.cuda().ronn_gemm(a.data_ptr(), w_nk.data_ptr(), out.data_ptr(), _ptr(bias), _ptr(residual), M, N, K,
                                  a.stride(0), w_nk.stride(0), out.stride(0), _DT[a.dtype], _ACT[activation],
                                  1 if out.dtype == torch.float32 else 0, bn, status_word(a.device).data_ptr(),
                                  _stream())
    _check(rc, "gemm")
    return out


def _norm(x, gamma, beta, residual, eps, rms, sum_out):
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    y = torch.empty((rows, H), dtype=x.dtype, device=x.device)
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, H)
        if r2.stride(1) != 1:
            r2 = r2.contiguous()
    s = torch.empty_like(y) if sum_out else None
    status_word(x.device)                                    # the many-rows kernel reports abandoned waits there
    rc = _native.cuda().ronn_norm(x2.data_ptr(), _ptr(r2), _ptr(gamma), _ptr(beta), y.data_ptr(), _ptr(s), rows, H,
                                  x2.stride(0), r2.stride(0) if r2 is not None else 0, y.stride(0), float(eps),
                                  1 if rms else 0, _DT[x.dtype], _stream())
    _check(rc, "norm")
    y = y.reshape(x.shape)
    return (y, s.reshape(x.shape)) if sum_out else y


def layernorm(x, gamma=None, beta=None, eps: float = 1e-5, residual=None, return_sum: bool = False):
    """LayerNorm over the last axis of (x + residual); optionally also returns the sum."""
    return _norm(x, gamma, beta, residual, eps, False, return_sum)


def rmsnorm(x, gamma, eps: float = 1e-5, residual=None, return_sum: bool = False):
    return _norm(x, gamma, None, residual, eps, True, return_sum)


def softmax(x: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """Softmax over ``axis`` (the last one by default; any other axis is reduced in place through strides, without
    a transpose)."""
    xc = x.contiguous()
    y = torch.empty_like(xc)
    if axis < 0:
        axis += xc.dim()
    if axis != xc.dim() - 1 and xc.numel():
        outer = 1
        for d in xc.shape[:axis]:
            outer *= int(d)
        n = int(xc.shape[axis])
        inner = xc.numel() // (outer * n)
        _check(_native.cuda().ronn_softmax_strided(xc.data_ptr(), y.data_ptr(), outer, n, inner, _DT[x.dtype], _stream()),
               "softmax_strided")
        return y
    cols = xc.shape[-1]
    status_word(x.device)
    _check(_native.cuda().ronn_softmax(xc.data_ptr(), y.data_ptr(), xc.numel() // cols, cols, _DT[x.dtype], _stream()),
           "softmax")
    return y


_UNARY = {"relu": 0, "gelu": 1, "fast_gelu": 2, "sigmoid": 3, "silu": 4, "tanh": 5}
_BINARY = {"add": 0, "mul": 1, "sub": 2, "swiglu": 3, "add_relu": 4}


def unary(x: torch.Tensor, op: str) -> torch.Tensor:
    xc = x.contiguous()
    y = torch.empty_like(xc)
    _check(_native.cuda().ronn_unary(xc.data_ptr(), y.data_ptr(), xc.numel(), _UNARY[op], _DT[x.dtype], _stream()),
           f"unary {op}")
    return y


def binary(a: torch.Tensor, b: torch.Tensor, op: str) -> torch.Tensor:
    if a.shape != b.shape or a.dtype != b.dtype:
        raise KernelError("binary kernel needs operands of one shape and dtype")
    ac, bc = a.contiguous(), b.contiguous()
    y = torch.empty_like(ac)
    _check(_native.cuda().ronn_binary(ac.data_ptr(), bc.data_ptr(), y.data_ptr(), ac.numel(), _BINARY[op],
                                      _DT[a.dtype], _stream()), f"binary {op}")
    return y


_FEW_CODES = {"Relu": 0, "Gelu": 1, "Sigmoid": 2, "Tanh": 3, "Neg": 4, "Abs": 5, "Exp": 6, "Sqrt": 7, "Swish": 8, "SiLU": 8,
              "Add": 16, "Mul": 17, "Sub": 18, "Div": 19}


def fused_elementwise_plan(x: torch.Tensor, op_names, operands):
    """Checks that a chain of element-wise operators fits the one-launch kernel and returns its launch plan, or None.
    ``operands[k]`` is the second operand of binary operator k (None for unary ones): a tensor of x's shape, a vector
    over the last dimension, or a one-element tensor."""
    if len(op_names) < 1 or len(op_names) > 8 or x.dtype not in (torch.bfloat16, torch.float16) or not x.is_cuda:
        return None
    if x.numel() == 0 or x.numel() % 8 or not x.is_contiguous() or x.data_ptr() % 16:
        return None
    codes, modes, ops = [], [], []
    for name, b in zip(op_names, operands):
        code = _FEW_CODES.get(name)
        if code is None:
            return None
        mode = 0
        if code >= 16:
            if b is None or not b.is_cuda or b.dtype != x.dtype:
                return None
            if b.numel() == 1:
                mode = 2
            elif b.shape == x.shape and b.is_contiguous() and b.data_ptr() % 16 == 0:
                mode = 0
            elif (b.numel() == x.shape[-1] and b.shape[-1] == x.shape[-1] and x.shape[-1] % 8 == 0 and b.is_contiguous()
                  and b.data_ptr() % 16 == 0):
                mode = 1
            else:
                return None
        codes.append(code)
        modes.append(mode)
        ops.append(b if code >= 16 else None)
    return codes, modes, ops


def fused_elementwise(x: torch.Tensor, op_names, operands, plan=None) -> torch.Tensor:
    """y = op_n(...op_1(x, b_1)..., b_n) in one launch (see ``fused_elementwise_plan`` for what fits)."""
    import ctypes as C
    plan = plan or fused_elementwise_plan(x, op_names, operands)
    if plan is None:
        raise KernelError("this element-wise chain does not fit the fused kernel")
    codes, modes, ops = plan
    n = len(codes)
    y = torch.empty_like(x)
    rc = _native.cuda().ronn_fused_elementwise(x.data_ptr(), y.data_ptr(), x.numel(), n, (C.c_int * n)(*codes),
                                               (C.c_int * n)(*modes),
                                               (C.c_void_p * n)(*[None if b is None else b.data_ptr() for b in ops]),
                                               x.shape[-1], _DT[x.dtype], _stream())
    _check(rc, "fused_elementwise")
    return y


def swiglu_fused(x: torch.Tensor) -> torch.Tensor:
    """x = [rows, 2F] (gate | up) -> silu(gate) * up."""
    F2 = x.shape[-1]
    xc = x.reshape(-1, F2).contiguous()
    y = torch.empty((xc.shape[0], F2 // 2), dtype=x.dtype, device=x.device)
    _check(_native.cuda().ronn_swiglu_fused(xc.data_ptr(), y.data_ptr(), xc.shape[0], F2 // 2, _DT[x.dtype], _stream()),
           "swiglu")
    return y.reshape(*x.shape[:-1], F2 // 2)


def embedding(ids: torch.Tensor, table: torch.Tensor, positions: Optional[torch.Tensor] = None,
              pos_table: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    ids32 = ids.reshape(-1).to(torch.int32)
    pos32 = positions.reshape(-1).to(torch.int32) if positions is not None else None
    T, H = ids32.numel(), table.shape[1]
    if _checks.enabled():
        _run_check(_checks.embedding, ids32, table, pos32, pos_table)
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    _check(_native.cuda().ronn_embedding(ids32.data_ptr(), _ptr(pos32), table.data_ptr(), _ptr(pos_table),
                                         out.data_ptr(), T, H, table.shape[0],
                                         pos_table.shape[0] if pos_table is not None else 0, out.stride(0),
                                         _DT[table.dtype], _stream()), "embedding")
    return out


def argmax(x: torch.Tensor, col_offset: int = 0, return_max: bool = False, out: Optional[torch.Tensor] = None):
    """Row argmax of a 2-D tensor (lowest index wins ties) as int32."""
    rows, cols = x.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=x.device)
    mx = torch.empty(rows, dtype=torch.float32, device=x.device) if return_max else None
    _check(_native.cuda().ronn_argmax(x.data_ptr(), out.data_ptr(), _ptr(mx), rows, cols, x.stride(0), col_offset,
                                      _DT[x.dtype], _stream()), "argmax")
    return (out, mx) if return_max else out


SAMPLE_RECORD_BYTES = 32      # {float temperature, top_p, repeat_penalty; int top_k; uint64 seed; int n_recent, use_counter}


def pack_sample_params(buf, row: int, temperature: float, top_k: int, top_p: float, repeat_penalty: float, seed: int,
                       n_recent: int, use_counter: bool = True) -> None:
    """Writes the sampling record of one row into ``buf`` (a writable bytes-like host buffer of 32-byte records).
    ``use_counter``: mix the row's device-side draw counter into the seed (fresh draws on every graph replay); off,
    the draw is a function of ``seed`` alone."""
    import struct
    struct.pack_into("<fffiQii", buf, row * SAMPLE_RECORD_BYTES, float(temperature), float(top_p), float(repeat_penalty),
                     int(top_k), int(seed) & 0xFFFFFFFFFFFFFFFF, int(n_recent), 1 if use_counter else 0)


def sample(logits: torch.Tensor, params: torch.Tensor, recent: Optional[torch.Tensor], counters: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token per row of fp32 ``logits`` [rows, vocab] (row stride free) on the device: repeat penalty (in place) ->
    temperature -> top-k -> softmax -> top-p -> draw.  ``params``: uint8 tensor of 32-byte records
    (``pack_sample_params``), ``recent``: int32 [rows, R] token ids the penalty applies to (or None), ``counters``:
    int64 [rows] draw counters advanced by the kernel.  Rows with temperature <= 0 return the arg max."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample needs fp32 logits [rows, vocab] with unit column stride")
    rows, vocab = logits.shape
    if params.numel() < rows * SAMPLE_RECORD_BYTES or counters.numel() < rows:
        raise KernelError("sample: parameter or counter buffer too small")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(_native.cuda().ronn_sample(logits.data_ptr(), logits.stride(0), vocab, rows, params.data_ptr(), _ptr(recent),
                                      recent.shape[1] if recent is not None else 0, counters.data_ptr(), out.data_ptr(),
                                      _stream()), "sample")
    return out


def argmax_combine(vals: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    shards, rows = vals.shape
    out = torch.empty(rows, dtype=torch.int32, device=vals.device)
    _check(_native.cuda().ronn_argmax_combine(vals.data_ptr(), idx.data_ptr(), out.data_ptr(), shards, rows, _stream()),
           "argmax_combine")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    xc = x.contiguous()
    y = torch.empty(xc.shape, dtype=dtype, device=x.device)
    _check(_native.cuda().ronn_cast(xc.data_ptr(), y.data_ptr(), xc.numel(), _DT[x.dtype], _DT[dtype], _stream()), "cast")
    return y


def kv_append(qkv: torch.Tensor, k_off: int, v_off: int, slots: torch.Tensor, kcache: torch.Tensor,
              vcache: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
              positions: Optional[torch.Tensor] = None, rope_base: float = 0.0) -> None:
    """Scatter the K/V columns of a fused QKV activation into the paged cache (optionally after rotary)."""
    T = qkv.shape[0]
    if _checks.enabled():
        _run_check(_checks.kv_append, qkv, slots, kcache, positions)
    use_rope = 1 if rope_base > 0 and positions is not None else 0
    _check(_native.cuda().ronn_kv_append(qkv.data_ptr(), qkv.stride(0), k_off, v_off, slots.data_ptr(),
                                         _ptr(positions), kcache.data_ptr(), vcache.data_ptr(), T, heads, kv_heads,
                                         head_dim, float(rope_base), use_rope, _DT[qkv.dtype], _stream()), "kv_append")


def _run_check(fn, *args) -> None:
    try:
        fn(*args)
    except _checks.IndexCheckError as e:
        raise KernelError(f"RONN_KERNEL_CHECKS: {e}") from None


_ATTN_SPLIT_WS = {}


def attention_split_workspace(device, items: int, splits: int, head_dim: int):
    """(partials, tickets) of the split decode attention, one pair per (device, stream): fp32 partial sums and the
    int32 ticket of every (row, head), zero between launches (the kernel resets what it used)."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    need = items * splits * (head_dim + 2)
    ws = _ATTN_SPLIT_WS.get(key)
    if ws is None or ws[0].numel() < need or ws[1].numel() < items:
        ws = (torch.empty(max(need, 1 << 20), dtype=torch.float32, device=dev),
              torch.zeros(max(items, 1 << 14), dtype=torch.int32, device=dev))
        _ATTN_SPLIT_WS[key] = ws
    return ws


def attention_splits(rows: int, heads: int, max_ctx: int) -> int:
    """CTAs per (row, head) of the decode attention kernel.  One, at every size measured (256 rows, mean context 416,
    2 to 16 heads per GPU): a split CTA pays its start-up, the ticket and the combining pass for a fraction of the
    work, and lost 10-50 % against one CTA per (row, head) once the kernel prefetched its next cache block.
    ``RONN_ATTN_SPLITS`` overrides (long single sequences, few rows)."""
    env = os.environ.get("RONN_ATTN_SPLITS")
    if env:
        return max(1, min(16, int(env)))
    return 1


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                    ctx_len: torch.Tensor, heads: int, kv_heads: int, head_dim: int, max_ctx: int,
                    bt_row: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                    scale: Optional[float] = None, append=None, rope=None, splits: Optional[int] = None) -> torch.Tensor:
    """q: [rows, >= heads*head_dim] (row stride free).  Returns [rows, heads*head_dim].
    ``append=(k_off, v_off, slots)`` (decode, one row per sequence): the new K/V columns of the fused QKV row are
    written to their cache slots by the same kernel.  ``rope=(positions int32 [rows], base)`` with ``append``: q and the
    new k are rotated by the same kernel too (the q row in memory stays as it is).  ``splits`` CTAs share the cache
    blocks of one (row, head) and the last to finish combines them (default: ``attention_splits``)."""
    rows = q.shape[0]
    if out is None:
        out = torch.empty((rows, heads * head_dim), dtype=q.dtype, device=q.device)
    sc = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if _checks.enabled():
        _run_check(_checks.paged_attention, q, kcache, block_tables, ctx_len, heads, head_dim, int(max_ctx), bt_row,
                   append[2] if append else None, rope[0] if rope else None)
    if splits is None:
        splits = attention_splits(rows, heads, int(max_ctx))
    part, tickets = attention_split_workspace(q.device, rows * heads, splits, head_dim) if splits > 1 else (None, None)
    _check(_native.cuda().ronn_paged_attention(q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(),
                                               block_tables.data_ptr(), block_tables.shape[1], ctx_len.data_ptr(),
                                               _ptr(bt_row), out.data_ptr(), out.stride(0), rows, heads, kv_heads,
                                               head_dim, int(max_ctx), float(sc), _DT[q.dtype],
                                               append[0] if append else 0, append[1] if append else 0,
                                               append[2].data_ptr() if append else None,
                                               rope[0].data_ptr() if rope else None, float(rope[1]) if rope else 0.0,
                                               int(splits), _ptr(part), _ptr(tickets), _stream()),
           "paged_attention")
    return out


def gemm_rownorm_ok(n: int, k: int) -> bool:
    """Shapes the cluster GEMM + row-norm kernel takes: a row of at most 8 tiles of 128 columns."""
    return n % 128 == 0 and 128 <= n <= 1024 and k % 8 == 0


def gemm_rownorm(a: torch.Tensor, w_nk: torch.Tensor, bias, residual, gamma, beta=None, eps: float = 1e-5,
                 norm: str = "layernorm"):
    """x = a @ w_nk^T + bias + residual and y = LayerNorm / RMSNorm(x) in ONE kernel: the CTAs that share a row block
    form a thread-block cluster and exchange the row statistics over distributed shared memory.  Returns (x, y)."""
    M, Kd = a.shape
    N = w_nk.shape[0]
    if not gemm_rownorm_ok(N, Kd):
        raise KernelError(f"gemm_rownorm needs N a multiple of 128 up to 1024 (got N={N}, K={Kd})")
    x = torch.empty((M, N), dtype=a.dtype, device=a.device)
    y = torch.empty((M, N), dtype=a.dtype, device=a.device)
    if residual is not None and residual.stride(1) != 1:
        residual = residual.contiguous()
    rc = _native.cuda().ronn_gemm_rownorm(a.data_ptr(), w_nk.data_ptr(), x.data_ptr(), y.data_ptr(), _ptr(bias),
                                          _ptr(residual), gamma.data_ptr(), _ptr(beta), M, N, Kd, a.stride(0),
                                          w_nk.stride(0), residual.stride(0) if residual is not None else 0, float(eps),
                                          {"layernorm": 1, "rmsnorm": 2}[norm], _DT[a.dtype],
                                          status_word(a.device).data_ptr(), _stream())
    _check(rc, "gemm_rownorm")
    return x, y


def dense_attention_plan(kv_lens, device, row_lens=None) -> dict:
    """Per-sequence index tensors of ``dense_attention`` for sequences stored back to back in the token buffer.
    ``kv_lens``: host list of sequence lengths; ``row_lens``: rows each sequence occupies in the buffer when that is
    more than its length (padded batches)."""
    starts, t = [], 0
    for i, n in enumerate(kv_lens):
        starts.append(t)
        t += int(n if row_lens is None else row_lens[i])
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return {"seq_start": mk(starts), "kv_len": mk([int(n) for n in kv_lens]),
            "max_len": max(int(n) for n in kv_lens), "n_seq": len(kv_lens)}


def dense_attention(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, plan: dict, heads: int, kv_heads: int,
                    head_dim: int, causal: bool, q_len: Optional[torch.Tensor] = None, max_q_len: Optional[int] = None,
                    out: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Tensor-core attention over the fused qkv buffer [tokens, ld] of whole sequences (prefill without cached
    context, encoders): one kernel per (128 queries, head, sequence) runs S = Q K^T and O = P V on tcgen05 with an
    online softmax in between; K and V are read where the QKV projection wrote them.  ``plan`` comes from
    ``dense_attention_plan``; ``q_len`` defaults to the key lengths (set it to the padded row count for encoders whose
    padded rows must still be produced).  Returns [tokens, heads * head_dim]."""
    tokens = qkv.shape[0]
    if out is None:
        out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    ql = q_len if q_len is not None else plan["kv_len"]
    mq = int(max_q_len if max_q_len is not None else plan["max_len"])
    sc = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if _checks.enabled():
        _run_check(_checks.sequences, tokens, plan["seq_start"], ql, plan["kv_len"], True)
    _check(_native.cuda().ronn_fmha(qkv.data_ptr(), qkv.stride(0), tokens, q_off, k_off, v_off,
                                    plan["seq_start"].data_ptr(), ql.data_ptr(), plan["kv_len"].data_ptr(),
                                    out.data_ptr(), out.stride(0), plan["n_seq"], mq, heads, kv_heads, head_dim,
                                    1 if causal else 0, float(sc), _DT[qkv.dtype],
                                    status_word(qkv.device).data_ptr(), _stream()), "fmha")
    return out


def paged_prefill_attention(q: torch.Tensor, q_off: int, kcache: torch.Tensor, vcache: torch.Tensor,
                            block_tables: torch.Tensor, seq_start: torch.Tensor, q_len: torch.Tensor,
                            kv_len: torch.Tensor, max_q_len: int, heads: int, kv_heads: int, head_dim: int,
                            causal: bool = True, bt_row: Optional[torch.Tensor] = None,
                            out: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Tensor-core attention of query chunks over the paged KV cache (chunked prefill, prefix hits): sequence s has its
    ``q_len[s]`` queries at rows ``seq_start[s] ..`` of ``q`` ([tokens, ld], head h at column q_off + h * head_dim) and
    attends to the ``kv_len[s]`` keys its block-table row lists; the queries are the last positions of that context.
    The new tokens' K / V must already be in the cache.  Returns [tokens, heads * head_dim]."""
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, heads * head_dim), dtype=q.dtype, device=q.device)
    sc = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if _checks.enabled():
        _run_check(_checks.sequences, tokens, seq_start, q_len, kv_len, False, block_tables.shape[1] * 16)
        rows_of = bt_row if bt_row is not None else torch.arange(seq_start.numel(), device=q.device, dtype=torch.int32)
        _run_check(_checks.paged_attention, q[: seq_start.numel()], kcache, block_tables, kv_len, 0, 0,
                   block_tables.shape[1] * 16, rows_of)
    _check(_native.cuda().ronn_fmha_paged(q.data_ptr(), q.stride(0), tokens, q_off, kcache.data_ptr(), vcache.data_ptr(),
                                          kcache.shape[0], block_tables.data_ptr(), block_tables.stride(0), _ptr(bt_row),
                                          seq_start.data_ptr(), q_len.data_ptr(), kv_len.data_ptr(), out.data_ptr(),
                                          out.stride(0), seq_start.numel(), int(max_q_len), heads, kv_heads, head_dim,
                                          1 if causal else 0, float(sc), _DT[q.dtype],
                                          status_word(q.device).data_ptr(), _stream()), "fmha_paged")
    return out


_WORKSPACES = {}


def splitk_workspace(device, nfloats: int) -> torch.Tensor:
    """fp32 scratch for split-K partial sums, one per (device, stream) so that launches on concurrent streams never
    share it; grown on demand and reused by every call on that stream."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    w = _WORKSPACES.get(key)
    if w is None or w.numel() < nfloats:
        w = torch.empty(max(nfloats, 1 << 22), dtype=torch.float32, device=dev)
        _WORKSPACES[key] = w
    return w


def gemm_splitk(a: torch.Tensor, w_nk: torch.Tensor, splitk: int, bn: int = 0,
                workspace: Optional[torch.Tensor] = None):
    """Partial products of a[M,K] @ w_nk[N,K]^T over `splitk` K-slices as fp32 [S, M, N] in the workspace.
    Returns (workspace, S) with S the effective number of slices."""
    import ctypes as C
    M, K = a.shape
    N = w_nk.shape[0]
    if workspace is None:
        workspace = splitk_workspace(a.device, splitk * M * N)
    if workspace.numel() < splitk * M * N:
        raise KernelError("split-K workspace too small")
    s_out = C.c_int(0)
    rc = _native.cuda().ronn_gemm_splitk(a.data_ptr(), w_nk.data_ptr(), workspace.data_ptr(), M, N, K, a.stride(0),
                                         w_nk.stride(0), _DT[a.dtype], bn, splitk, C.addressof(s_out),
                                         status_word(a.device).data_ptr(), _stream())
    _check(rc, "gemm_splitk")
    return workspace, s_out.value


def splitk_finalize(ws: torch.Tensor, S: int, rows: int, N: int, dtype: torch.dtype, bias=None, residual=None,
                    gamma=None, beta=None, eps: float = 1e-5, activation: str = "", norm: str = "",
                    want_sum: bool = True):
    """sum = sum_s ws[s] + bias (+act) + residual ; y = norm(sum).  Returns (sum or None, y or None)."""
    nm = {"": 0, "none": 0, "layernorm": 1, "rmsnorm": 2}[norm]
    dev = ws.device
    sum_out = torch.empty((rows, N), dtype=dtype, device=dev) if (want_sum or nm == 0) else None
    y = torch.empty((rows, N), dtype=dtype, device=dev) if nm else None
    rc = _native.cuda().ronn_splitk_finalize(ws.data_ptr(), S, _ptr(bias), _ptr(residual), _ptr(sum_out), _ptr(gamma),
                                             _ptr(beta), _ptr(y), rows, N, float(eps), _ACT[activation], nm,
                                             _DT[dtype], _stream())
    _check(rc, "splitk_finalize")
    return sum_out, y
