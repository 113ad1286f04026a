"""Encoder runner: DistilBERT-style post-LayerNorm transformer encoder over the kernel operator backend, with
tensor parallelism.

The reference serves encoder models through its generic graph session, one library call per node
(crates/ronn-providers/src/gpu/provider.rs:1135-1436; example examples/onnx-model/src/main.rs).  Here the
initializers of the DistilBERT graph (names of models/export_distilbert.py's HuggingFace export) are turned into
fused device weights once: Q, K and V projections become one column-parallel GEMM, attention runs on the tensor-core attention
kernel straight from the fused QKV buffer (head sizes 64 / 128; others use the paged kernel over a scratch K/V layout), and every block ends in ONE kernel that does the row-parallel GEMM, the cross-rank
reduction, the bias, the residual and the LayerNorm (``FusedComm.gemm_allreduce(norm=...)``) when tensor parallelism is
on.  Without tensor parallelism the GEMM epilogue adds bias + residual and the LayerNorm kernel follows.

``sequence_parallel=True`` keeps the activations between the row-parallel and the column-parallel projections sharded
by token: every rank embeds and normalises 1/W of the tokens, the column-parallel GEMMs (QKV, MLP-up) read the
gathered activations tile by tile from the peers' shards (``FusedComm.ag_gemm``), and the row-parallel GEMMs
(attention output, MLP-down) end in a reduce-scatter that leaves each rank its own tokens
(``FusedComm.gemm_reduce_scatter``), so LayerNorm, bias and residual touch T / W rows.  With library collectives (or
token counts that are not a multiple of 128 per rank) the same layout runs on all-gather / reduce-scatter calls.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..api.errors import SessionError
from .model_runner import KV_BLOCK, LinearW, NoComm, shard_heads
from .ops_backend import make_ops


class EncoderRunner:
    def __init__(self, graph, device=None, dtype: torch.dtype = torch.bfloat16, comm=None, backend: str = "kernels",
                 sequence_parallel: bool = False):
        md = graph.metadata
        if md.get("ronn.arch") != "distilbert":
            raise SessionError(f"EncoderRunner needs a DistilBERT graph (ronn.arch={md.get('ronn.arch')!r})")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        if self.device.type == "cpu":
            backend, dtype = "torch", torch.float32
        self.dtype = dtype
        self.ops = make_ops(backend, self.device)
        self.comm = comm or NoComm()
        self.tp, self.rank = self.comm.world, self.comm.rank
        self.sequence_parallel = bool(sequence_parallel) and self.comm.world > 1
        self.n_layers, self.hidden = int(md["ronn.n_layers"]), int(md["ronn.dim"])
        self.n_heads, self.ffn = int(md["ronn.n_heads"]), int(md["ronn.hidden_dim"])
        self.max_pos, self.eps = int(md["ronn.max_pos"]), float(md["ronn.eps"])
        self.head_dim = self.hidden // self.n_heads
        self.h0, self.heads_local = shard_heads(self.n_heads, self.tp, self.rank)
        if self.heads_local == 0:
            raise SessionError("tensor-parallel size exceeds the number of attention heads")
        if self.ffn % self.tp:
            raise SessionError("FFN width must divide by the tensor-parallel size")
        self.ffn_local = self.ffn // self.tp
        self._load(graph.initializers)
        self._scratch: Dict[tuple, tuple] = {}

    def _dev(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device, self.dtype).contiguous()

    def _load(self, init: Dict[str, torch.Tensor]) -> None:
        d = self.head_dim
        c0, c1 = self.h0 * d, (self.h0 + self.heads_local) * d
        f0, f1 = self.rank * self.ffn_local, (self.rank + 1) * self.ffn_local
        self.wte = self._dev(init["embeddings.word_embeddings.weight"])
        self.wpe = self._dev(init["embeddings.position_embeddings.weight"])
        self.emb_ln = (self._dev(init["embeddings.LayerNorm.weight"]), self._dev(init["embeddings.LayerNorm.bias"]))
        self.layers = []
        for i in range(self.n_layers):
            p = f"transformer.layer.{i}"
            w = lambda n: init[f"{p}.{n}.weight"]          # stored [in, out]
            b = lambda n: init[f"{p}.{n}.bias"]
            wqkv = torch.cat([w("attention.q_lin")[:, c0:c1], w("attention.k_lin")[:, c0:c1],
                              w("attention.v_lin")[:, c0:c1]], dim=1)
            bqkv = torch.cat([b("attention.q_lin")[c0:c1], b("attention.k_lin")[c0:c1], b("attention.v_lin")[c0:c1]])
            self.layers.append({
                "qkv": LinearW(self._dev(wqkv.t()), self._dev(bqkv)),
                "out": LinearW(self._dev(w("attention.out_lin")[c0:c1, :].t()), self._dev(b("attention.out_lin"))),
                "ln1": (self._dev(w("sa_layer_norm")), self._dev(b("sa_layer_norm"))),
                "up": LinearW(self._dev(w("ffn.lin1")[:, f0:f1].t()), self._dev(b("ffn.lin1")[f0:f1])),
                "down": LinearW(self._dev(w("ffn.lin2")[f0:f1, :].t()), self._dev(b("ffn.lin2"))),
                "ln2": (self._dev(w("output_layer_norm")), self._dev(b("output_layer_norm"))),
            })

    # ------------------------------------------------------------------ per-shape scratch (index tensors, K/V layout)
    def _plan(self, B: int, S: int):
        key = (B, S)
        plan = self._scratch.get(key)
        if plan is None:
            nb = (S + KV_BLOCK - 1) // KV_BLOCK
            dev = self.device
            tok_seq = torch.arange(B, device=dev, dtype=torch.int32).repeat_interleave(S)
            pos = torch.arange(S, device=dev, dtype=torch.int32).repeat(B)
            slots = (tok_seq * (nb * KV_BLOCK) + pos).to(torch.int32)
            bt = torch.arange(B * nb, device=dev, dtype=torch.int32).view(B, nb)
            shape = (B * nb + 1, self.heads_local, KV_BLOCK, self.head_dim)
            kc = torch.zeros(shape, dtype=self.dtype, device=dev)
            vc = torch.zeros(shape, dtype=self.dtype, device=dev)
            mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            dense = {"seq_start": mk([b * S for b in range(B)]), "max_len": S, "n_seq": B,
                     "q_len": torch.full((B,), S, dtype=torch.int32, device=dev)}
            plan = (tok_seq, pos, slots, bt, kc, vc, nb * KV_BLOCK, dense)
            self._scratch[key] = plan
        return plan

    def _row_parallel(self, inp, lw: LinearW, residual, ln):
        """LayerNorm(inp @ W^T (summed over ranks) + bias + residual)."""
        ops = self.ops
        if self.tp > 1 and getattr(self.comm, "fused", False) and ops.name == "kernels" and self.hidden <= 1024:
            return self.comm.gemm_allreduce(inp, lw.w, lw.bias, residual, norm=("layernorm", ln[0], ln[1], self.eps))[1]
        if self.tp > 1:
            y = self.comm.all_reduce(ops.gemm(inp, lw.w)) + lw.bias + residual
        else:
            y = ops.gemm(inp, lw.w, lw.bias, residual)
        return ops.layernorm(y, ln[0], ln[1], self.eps)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """input_ids [B, S] (any integer dtype), attention_mask [B, S] of 0/1 with the padding at the end of each row
        (or None for no padding).  Returns last_hidden_state [B, S, hidden]; rows of padded positions are computed
        like any other row but attend only to the valid prefix."""
        ops = self.ops
        B, S = input_ids.shape
        if S > self.max_pos:
            raise SessionError(f"sequence length {S} exceeds the position table ({self.max_pos})")
        tok_seq, pos, slots, bt, kc, vc, max_ctx, dense = self._plan(B, S)
        ids = input_ids.to(self.device).reshape(-1).to(torch.int32)
        if attention_mask is None:
            lens = torch.full((B,), S, dtype=torch.int32, device=self.device)
        else:
            lens = attention_mask.to(self.device).sum(dim=1).clamp_(min=1).to(torch.int32)
        tensor_core = ops.name == "kernels" and self.head_dim in (64, 128)
        if tensor_core:
            dense = dict(dense, kv_len=lens)           # key lengths stay on the device: no host round trip
        else:
            ctx = lens.repeat_interleave(S)
        d, hl = self.head_dim, self.heads_local
        hn = hl * d
        if self.sequence_parallel and (B * S) % self.tp == 0:
            return self._forward_token_sharded(ids, pos, B, S, tensor_core, dense,
                                               None if tensor_core else (slots, kc, vc, bt, ctx, max_ctx, tok_seq))
        x = ops.embedding(ids, self.wte, pos, self.wpe)
        x = ops.layernorm(x, self.emb_ln[0], self.emb_ln[1], self.eps)
        for L in self.layers:
            qkv = ops.gemm(x, L["qkv"].w, L["qkv"].bias)
            if tensor_core:
                att = ops.dense_attention(qkv, 0, hn, 2 * hn, dense, hl, hl, d, False, dense["q_len"], S)
            else:
                ops.kv_append(qkv, hn, 2 * hn, slots, kc, vc, hl, hl, d)
                att = ops.paged_attention(qkv, kc, vc, bt, ctx, hl, hl, d, max_ctx, tok_seq)
            x = self._row_parallel(att, L["out"], x, L["ln1"])
            f = ops.gemm(x, L["up"].w, L["up"].bias, None, "gelu")
            x = self._row_parallel(f, L["down"], x, L["ln2"])
        return x.view(B, S, self.hidden)

    def _forward_token_sharded(self, ids, pos, B, S, tensor_core, dense, paged):
        """The sequence-parallel layout: this rank owns tokens [rank * T / W, (rank + 1) * T / W) between the
        projections; attention still sees every token of the local heads."""
        ops, comm = self.ops, self.comm
        T = B * S
        per = T // self.tp
        r0 = self.rank * per
        d, hl, H = self.head_dim, self.heads_local, self.hidden
        hn = hl * d
        fused = getattr(comm, "fused", False) and ops.name == "kernels" and per % 128 == 0

        def column_parallel(x_local, lw, act=""):
            if fused:
                shard = comm.shard_buffer(per, H, x_local.dtype)
                shard.copy_(x_local)
                comm.signal_shard_ready()
                return comm.ag_gemm(per, H, lw.w, lw.bias, act)
            return ops.gemm(comm.all_gather_rows(x_local), lw.w, lw.bias, None, act)

        def row_parallel(inp, lw, residual_local, ln):
            if fused:
                y = comm.gemm_reduce_scatter(inp, lw.w, lw.bias, residual_local)
            else:
                y = comm.reduce_scatter_rows(ops.gemm(inp, lw.w)) + lw.bias + residual_local
            return ops.layernorm(y, ln[0], ln[1], self.eps)

        x = ops.embedding(ids[r0:r0 + per].contiguous(), self.wte, pos[r0:r0 + per].contiguous(), self.wpe)
        x = ops.layernorm(x, self.emb_ln[0], self.emb_ln[1], self.eps)
        for L in self.layers:
            qkv = column_parallel(x, L["qkv"])
            if tensor_core:
                att = ops.dense_attention(qkv, 0, hn, 2 * hn, dense, hl, hl, d, False, dense["q_len"], S)
            else:
                slots, kc, vc, bt, ctx, max_ctx, tok_seq = paged
                ops.kv_append(qkv, hn, 2 * hn, slots, kc, vc, hl, hl, d)
                att = ops.paged_attention(qkv, kc, vc, bt, ctx, hl, hl, d, max_ctx, tok_seq)
            x = row_parallel(att, L["out"], x, L["ln1"])
            f = column_parallel(x, L["up"], "gelu")
            x = row_parallel(f, L["down"], x, L["ln2"])
        return comm.all_gather_rows(x).view(B, S, H)
