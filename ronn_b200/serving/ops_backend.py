"""Operator backends of the decoder runner.

``KernelOps`` launches the hand-written sm_100a kernels.  ``TorchOps`` expresses the same
operators with PyTorch library calls (cuBLAS matmul, SDPA-style attention on gathered KV): it is
the CPU path of the engine tests and, on a GPU, the measured library baseline - never the product
path.  Both work on the same paged KV layout [num_blocks, kv_heads, 16, head_dim].
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from ..onnx.registry import rotary

KV_BLOCK = 16


class TorchOps:
    name = "torch"

    def gemm(self, a, w_nk, bias=None, residual=None, activation="", out_fp32=False):
        y = torch.matmul(a, w_nk.t())
        if bias is not None:
            y = y + bias
        if activation in ("gelu", "Gelu"):
            y = F.gelu(y.float(), approximate="tanh").to(y.dtype)
        elif activation in ("relu", "Relu"):
            y = torch.relu(y)
        if residual is not None:
            y = y + residual
        return y.float() if out_fp32 else y

    def lm_head(self, x, w_nk):
        return self.gemm(x, w_nk, out_fp32=True)

    def layernorm(self, x, w, b, eps):
        return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)

    def rmsnorm(self, x, w, eps):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)

    def embedding(self, ids, table, positions=None, pos_table=None):
        y = F.embedding(ids.long(), table)
        if pos_table is not None:
            y = y + F.embedding(positions.long(), pos_table)
        return y

    def gather_rows(self, x, idx):
        return x.index_select(0, idx.long())

    def swiglu_fused(self, x):
        f = x.shape[-1] // 2
        return (F.silu(x[..., :f].float()) * x[..., f:].float()).to(x.dtype)

    def kv_append(self, qkv, k_off, v_off, slots, kcache, vcache, heads, kv_heads, d, positions=None, rope_base=0.0):
        T = qkv.shape[0]
        if rope_base > 0 and positions is not None:
            q = rotary(qkv[:, :heads * d], positions, rope_base, heads)
            k = rotary(qkv[:, k_off:k_off + kv_heads * d], positions, rope_base, kv_heads)
            qkv[:, :heads * d] = q
            qkv[:, k_off:k_off + kv_heads * d] = k
        k = qkv[:, k_off:k_off + kv_heads * d].reshape(T, kv_heads, d)
        v = qkv[:, v_off:v_off + kv_heads * d].reshape(T, kv_heads, d)
        # rows without a slot (padding) go to the spare last block, so no data-dependent shapes are needed
        trash = (kcache.shape[0] - 1) * KV_BLOCK
        s = torch.where(slots >= 0, slots, torch.full_like(slots, trash)).long()
        blk, off = s // KV_BLOCK, s % KV_BLOCK
        kcache[blk, :, off, :] = k
        vcache[blk, :, off, :] = v

    def paged_attention(self, q, kcache, vcache, block_tables, ctx_len, heads, kv_heads, d, max_ctx, bt_row=None):
        """Gather each row's pages into a dense [rows, heads, L, d] tensor and call the library SDPA."""
        rows = q.shape[0]
        cdt = torch.float32 if q.device.type == "cpu" else q.dtype
        qh = q[:, :heads * d].reshape(rows, heads, 1, d).to(cdt)
        bt = block_tables if bt_row is None else block_tables.index_select(0, bt_row.long())
        nb = min((max_ctx + KV_BLOCK - 1) // KV_BLOCK, bt.shape[1])
        idx = bt[:, :nb].long().clamp_min(0)                                   # [rows, nb]
        k = kcache[idx].permute(0, 2, 1, 3, 4).reshape(rows, kv_heads, nb * KV_BLOCK, d).to(cdt)
        v = vcache[idx].permute(0, 2, 1, 3, 4).reshape(rows, kv_heads, nb * KV_BLOCK, d).to(cdt)
        if kv_heads != heads:
            rep = heads // kv_heads
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        pos = torch.arange(nb * KV_BLOCK, device=q.device)
        keep = pos[None, :] < ctx_len[:, None].long()                             # [rows, L]
        empty = ~keep.any(dim=1)
        keep = keep | empty[:, None]                                              # avoid all-masked rows (NaN)
        v = torch.where(keep[:, None, :, None], v, torch.zeros((), device=v.device, dtype=cdt))
        out = F.scaled_dot_product_attention(qh, k, v, attn_mask=keep[:, None, None, :])
        out = torch.where(empty[:, None, None, None], torch.zeros((), device=out.device, dtype=cdt), out)
        return out.reshape(rows, heads * d).to(q.dtype)

    def argmax(self, logits, col_offset=0, return_max=False):
        m, i = logits.float().max(dim=-1)
        idx = (i + col_offset).to(torch.int32)
        return (idx, m) if return_max else idx

    def argmax_combine(self, vals, idx):
        # largest value wins, lowest index on ties
        best = vals.max(dim=0).values
        cand = torch.where(vals == best[None, :], idx, torch.full_like(idx, 2 ** 31 - 1))
        return cand.min(dim=0).values.to(torch.int32)

    def check(self):
        pass

    def status_tensor(self):
        return None


class KernelOps:
    name = "kernels"

    def __init__(self):
        from .. import ops as K
        self.K = K

    def gemm(self, a, w_nk, bias=None, residual=None, activation="", out_fp32=False):
        return self.K.gemm(a, w_nk, bias, residual, activation, out_fp32=out_fp32)

    def lm_head(self, x, w_nk):
        """fp32 logits [rows, vocab].  The buffer's row stride is padded to a multiple of 8 values: with an odd
        vocabulary (50257) as the stride every row would start off a 16-byte boundary and the GEMM epilogue would fall
        back to scalar stores (measured: 113 us instead of about 30 for 256 x 50257 x 1024)."""
        n = w_nk.shape[0]
        buf = torch.empty((x.shape[0], -(-n // 8) * 8), dtype=torch.float32, device=x.device)
        return self.K.gemm(x, w_nk, out=buf[:, :n], out_fp32=True)

    def layernorm(self, x, w, b, eps):
        return self.K.layernorm(x, w, b, eps)

    def gemm_splitk_norm(self, a, lw, residual, norm_params, norm_kind, eps, splitk):
        """Skinny GEMM as split-K partial sums, then ONE pass that adds bias + residual, writes the new residual
        stream and (optionally) the normalised input of the next block."""
        ws, S = self.K.gemm_splitk(a, lw.w, splitk, 64)
        gamma = norm_params[0] if norm_params is not None else None
        beta = norm_params[1] if (norm_params is not None and len(norm_params) > 1) else None
        return self.K.splitk_finalize(ws, S, a.shape[0], lw.w.shape[0], a.dtype, bias=lw.bias, residual=residual,
                                      gamma=gamma, beta=beta, eps=eps,
                                      norm=(norm_kind if norm_params is not None else ""))

    def gemm_rownorm(self, a, lw, residual, norm_params, norm_kind, eps):
        """Projection + bias + residual + the next block's norm in one cluster kernel; (new residual stream, normed)."""
        beta = norm_params[1] if len(norm_params) > 1 else None
        return self.K.gemm_rownorm(a, lw.w, lw.bias, residual, norm_params[0], beta, eps, norm_kind)

    def rmsnorm(self, x, w, eps):
        return self.K.rmsnorm(x, w, eps)

    def embedding(self, ids, table, positions=None, pos_table=None):
        return self.K.embedding(ids, table, positions, pos_table)

    def gather_rows(self, x, idx):
        return self.K.embedding(idx, x)

    def swiglu_fused(self, x):
        return self.K.swiglu_fused(x)

    def kv_append(self, qkv, k_off, v_off, slots, kcache, vcache, heads, kv_heads, d, positions=None, rope_base=0.0):
        self.K.kv_append(qkv, k_off, v_off, slots, kcache, vcache, heads, kv_heads, d, positions, rope_base)

    def paged_attention(self, q, kcache, vcache, block_tables, ctx_len, heads, kv_heads, d, max_ctx, bt_row=None):
        return self.K.paged_attention(q, kcache, vcache, block_tables, ctx_len, heads, kv_heads, d, max_ctx, bt_row)

    def append_attention(self, qkv, k_off, v_off, slots, kcache, vcache, block_tables, ctx_len, heads, kv_heads, d, max_ctx,
                         positions=None, rope_base=0.0):
        """Decode step: (rotary embedding,) cache append and attention in one launch."""
        rope = (positions, rope_base) if rope_base > 0 and positions is not None else None
        return self.K.paged_attention(qkv, kcache, vcache, block_tables, ctx_len, heads, kv_heads, d, max_ctx,
                                      append=(k_off, v_off, slots), rope=rope)

    def dense_attention(self, qkv, q_off, k_off, v_off, plan, heads, kv_heads, d, causal, q_len=None, max_q_len=None):
        """Whole-sequence attention on the tensor cores, straight from the fused qkv buffer."""
        return self.K.dense_attention(qkv, q_off, k_off, v_off, plan, heads, kv_heads, d, causal, q_len, max_q_len)

    def paged_prefill_attention(self, q, kcache, vcache, block_tables, plan, heads, kv_heads, d):
        """Causal attention of this step's query chunks over the paged cache, on the tensor cores."""
        return self.K.paged_prefill_attention(q, 0, kcache, vcache, block_tables, plan["seq_start"], plan["q_len"],
                                              plan["kv_len"], plan["max_q_len"], heads, kv_heads, d, causal=True)

    def argmax(self, logits, col_offset=0, return_max=False):
        return self.K.argmax(logits, col_offset, return_max)

    def argmax_combine(self, vals, idx):
        return self.K.argmax_combine(vals, idx)

    def check(self):
        self.K.check_status()

    def status_tensor(self):
        """Device word that the kernels' bounded waits write; lets a caller fetch it with its own copy."""
        return self.K.status_word()


def make_ops(backend: str, device: torch.device):
    if backend == "kernels":
        if device.type != "cuda":
            raise RuntimeError("the 'kernels' backend needs a CUDA device; use backend='torch' on CPU")
        return KernelOps()
    if backend == "torch":
        return TorchOps()
    raise ValueError(f"unknown backend '{backend}'")
