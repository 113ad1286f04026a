"""Paged-KV decoder runner: turns the initializers of a GPT-2 or Llama/BitNet-style ONNX model into
sharded device weights and runs prefill / decode steps over the operator backend.

Tensor parallelism (Megatron layout): QKV and MLP-up are column-parallel (heads / FFN columns
sharded), attention-out and MLP-down are row-parallel; the vocabulary of the LM head is sharded
and the greedy token is chosen by a cross-rank (max, index) combine.  The collective after a
row-parallel GEMM is delegated to ``self.comm`` (library all-reduce on the baseline path, fused
in-kernel exchange on the product path).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..api.errors import SessionError
from .config import EngineConfig
from .ops_backend import make_ops

KV_BLOCK = 16


@dataclass
class DecoderArch:
    name: str
    n_layer: int
    hidden: int
    n_head: int
    n_kv_head: int
    head_dim: int
    ffn: int
    vocab: int
    max_pos: int
    norm: str = "layernorm"        # "layernorm" | "rmsnorm"
    mlp: str = "gelu"              # "gelu" | "swiglu"
    rope_base: float = 0.0         # 0 = learned absolute positions
    eps: float = 1e-5
    bitlinear: bool = False

    @staticmethod
    def from_metadata(md: Dict[str, str]) -> "DecoderArch":
        arch = md.get("ronn.arch")
        if arch == "gpt2":
            H, nh = int(md["ronn.n_embd"]), int(md["ronn.n_head"])
            return DecoderArch("gpt2", int(md["ronn.n_layer"]), H, nh, nh, H // nh, 4 * H, int(md["ronn.vocab_size"]),
                               int(md["ronn.n_positions"]), eps=float(md.get("ronn.eps", 1e-5)))
        if arch in ("llama", "bitnet"):
            H, nh = int(md["ronn.hidden"]), int(md["ronn.n_head"])
            return DecoderArch(arch, int(md["ronn.n_layer"]), H, nh, int(md.get("ronn.n_kv_head", nh)),
                               int(md.get("ronn.head_dim", H // nh)), int(md["ronn.ffn"]), int(md["ronn.vocab_size"]),
                               int(md.get("ronn.max_pos", 4096)), norm="rmsnorm", mlp="swiglu",
                               rope_base=float(md.get("ronn.rope_base", 10000.0)), eps=float(md.get("ronn.eps", 1e-5)),
                               bitlinear=(arch == "bitnet"))
        raise SessionError(f"model metadata does not describe a decoder architecture (ronn.arch={arch!r})")


def shard_heads(n_head: int, tp: int, rank: int):
    """Contiguous head ranges; the first (n_head % tp) ranks take one extra head."""
    base, extra = divmod(n_head, tp)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


class NoComm:
    world = 1
    rank = 0

    def all_reduce(self, x):
        return x

    def all_gather_small(self, x):
        return x.unsqueeze(0)

    def barrier(self):
        pass


class LinearW:
    """A dense [N,K] weight (+ optional bias) or a packed ternary BitLinear weight."""
    __slots__ = ("w", "bias", "scale", "packed", "n", "k", "_dense")

    def __init__(self, w=None, bias=None, packed=None, scale=None, n=0, k=0):
        self.w, self.bias, self.packed, self.scale, self.n, self.k = w, bias, packed, scale, n, k
        self._dense = None


class QuantAct:
    """Activations already quantised per token for a packed (ternary) projection: int8 values, fp32 scales and the
    dtype the projection should produce."""
    __slots__ = ("q", "s", "dtype")

    def __init__(self, q, s, dtype):
        self.q, self.s, self.dtype = q, s, dtype

    @property
    def shape(self):
        return self.q.shape


class DecoderRunner:
    def __init__(self, arch: DecoderArch, initializers: Dict[str, torch.Tensor], cfg: EngineConfig,
                 device: torch.device, comm=None, num_blocks: Optional[int] = None):
        self.arch, self.cfg, self.device = arch, cfg, device
        self.comm = comm or NoComm()
        self.tp, self.rank = self.comm.world, self.comm.rank
        self.dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[cfg.dtype]
        self.ops = make_ops(cfg.backend, device)
        if cfg.backend == "kernels" and self.dtype == torch.float32:
            raise SessionError("the kernel backend computes in bf16 or fp16")
        a = arch
        self.h0, self.n_head_local = shard_heads(a.n_head, self.tp, self.rank)
        if a.n_kv_head == a.n_head:
            self.kv0, self.n_kv_local = self.h0, self.n_head_local
        else:
            if a.n_kv_head % self.tp:
                raise SessionError("grouped KV heads must divide by the tensor-parallel size")
            self.kv0, self.n_kv_local = shard_heads(a.n_kv_head, self.tp, self.rank)
        if self.n_head_local == 0:
            raise SessionError("tensor-parallel size exceeds the number of attention heads")
        if a.ffn % self.tp:
            raise SessionError("FFN width must divide by the tensor-parallel size")
        self.ffn_local = a.ffn // self.tp
        vs = -(-a.vocab // self.tp)
        vs = (vs + 7) // 8 * 8
        self.vocab_shard = vs
        self.vocab_start = min(self.rank * vs, a.vocab)
        self.vocab_local = max(min(vs, a.vocab - self.vocab_start), 0)
        self._load_weights(initializers)
        self.num_blocks = num_blocks or cfg.num_blocks
        self.max_blocks_per_seq = (cfg.max_model_len + KV_BLOCK - 1) // KV_BLOCK
        self._alloc_cache()
        self.launches = 0
        self.step_ctx = 0

    # ------------------------------------------------------------------ weights
    def _dev(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device, self.dtype).contiguous()

    def _load_weights(self, init: Dict[str, torch.Tensor]) -> None:
        a, d = self.arch, self.arch.head_dim
        hs, hn = self.h0 * d, self.n_head_local * d
        ks, kn = self.kv0 * d, self.n_kv_local * d
        self.layers: List[Dict[str, object]] = []
        if a.name == "gpt2":
            self.wte = self._dev(init["wte"])
            self.wpe = self._dev(init["wpe"])
            self.lnf = (self._dev(init["ln_f.weight"]), self._dev(init["ln_f.bias"]))
            H = a.hidden
            for i in range(a.n_layer):
                p = f"h.{i}"
                wqkv, bqkv = init[f"{p}.attn.c_attn.weight"], init[f"{p}.attn.c_attn.bias"]      # [H, 3H] (K,N)
                cols = torch.cat([torch.arange(hs, hs + hn), H + torch.arange(hs, hs + hn),
                                  2 * H + torch.arange(hs, hs + hn)])
                wo = init[f"{p}.attn.c_proj.weight"]                                              # [H(in), H(out)]
                wfc, bfc = init[f"{p}.mlp.c_fc.weight"], init[f"{p}.mlp.c_fc.bias"]              # [H, 4H]
                wpr = init[f"{p}.mlp.c_proj.weight"]                                              # [4H, H]
                f0, f1 = self.rank * self.ffn_local, (self.rank + 1) * self.ffn_local
                self.layers.append({
                    "ln1": (self._dev(init[f"{p}.ln_1.weight"]), self._dev(init[f"{p}.ln_1.bias"])),
                    "ln2": (self._dev(init[f"{p}.ln_2.weight"]), self._dev(init[f"{p}.ln_2.bias"])),
                    "qkv": LinearW(self._dev(wqkv[:, cols].t()), self._dev(bqkv[cols])),
                    "out": LinearW(self._dev(wo[hs:hs + hn, :].t()), self._dev(init[f"{p}.attn.c_proj.bias"])),
                    "up": LinearW(self._dev(wfc[:, f0:f1].t()), self._dev(bfc[f0:f1])),
                    "down": LinearW(self._dev(wpr[f0:f1, :].t()), self._dev(init[f"{p}.mlp.c_proj.bias"])),
                })
            self.lm_head = self.wte[self.vocab_start:self.vocab_start + self.vocab_local]
        else:
            from ..models.bitnet_llama import load_decoder_weights
            load_decoder_weights(self, init)

    def _alloc_cache(self) -> None:
        a = self.arch
        if self.num_blocks <= 0:
            per_block = a.n_layer * 2 * self.n_kv_local * KV_BLOCK * a.head_dim * torch.finfo(self.dtype).bits // 8
            want = self.cfg.max_num_seqs * self.max_blocks_per_seq
            if self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                cap = int(free * self.cfg.gpu_memory_utilization) // per_block
                want = min(want, cap)
            self.num_blocks = max(want, 1)
        # one spare block past the pool: padded rows of the library backend scatter there
        shape = (self.num_blocks + 1, self.n_kv_local, KV_BLOCK, a.head_dim)
        self.kcache = [torch.zeros(shape, dtype=self.dtype, device=self.device) for _ in range(a.n_layer)]
        self.vcache = [torch.zeros(shape, dtype=self.dtype, device=self.device) for _ in range(a.n_layer)]

    # ------------------------------------------------------------------ forward
    def _linear(self, x, lw: LinearW, residual=None, activation="", reduce=False, comm=None, norm_quant=None):
        """``norm_quant=(gamma, eps)`` (packed row-parallel projections on the fused communicator): the reduction also
        produces RMSNorm(result) quantised for the next packed projection; the return value is then
        (result, QuantAct or None)."""
        ops = self.ops
        comm = comm or self.comm
        if lw.packed is not None:
            from ..providers.bitnet import kernels as BK
            pre = x if isinstance(x, QuantAct) else None          # quantised by the kernel that produced the activations
            out_dtype = pre.dtype if pre is not None else x.dtype
            ws = float(lw.scale.reshape(-1)[0]) if isinstance(lw.scale, torch.Tensor) else float(lw.scale)
            if reduce and self.tp > 1 and getattr(comm, "fused", False) and ops.name == "kernels" and lw.bias is None:
                # ternary GEMM + cross-rank reduction over NVLink (one launch under the low-latency protocol)
                from ..ops import bitnet as KB
                q, s = (pre.q, pre.s) if pre is not None else KB.act_quant_int8(x)
                r = comm.bitlinear_allreduce(q, s, lw.packed, ws, lw.n, lw.k, out_dtype, residual, norm_quant=norm_quant)
                if norm_quant is None:
                    return r
                return (r[0], QuantAct(r[1], r[2], out_dtype)) if isinstance(r, tuple) else (r, None)
            if pre is not None:
                from ..ops import bitnet as KB
                y = KB.bitlinear_q(pre.q, pre.s, lw.packed, ws, lw.bias, lw.n, lw.k, out_dtype)
            else:
                y = BK.bitlinear(x, lw, backend=ops.name)
            if reduce and self.tp > 1:
                y = comm.all_reduce(y)
            if residual is not None:
                y = y + residual
            return y
        if reduce and self.tp > 1 and getattr(comm, "fused", False) and ops.name == "kernels":
            # one kernel: partial GEMM on the tensor cores + cross-rank reduction over NVLink + bias + residual
            return comm.gemm_allreduce(x, lw.w, lw.bias, residual)
        if reduce and self.tp > 1:
            # bias and residual are applied once, after the partial sums are combined
            y = ops.gemm(x, lw.w)
            y = comm.all_reduce(y)
            if lw.bias is not None:
                y = y + lw.bias
            if residual is not None:
                y = y + residual
            return y
        return ops.gemm(x, lw.w, lw.bias, residual, activation)

    def _norm_linear(self, x, norm_p, lw: LinearW):
        """norm(x) followed by a column-parallel projection.  For packed ternary weights on the kernel backend the
        RMSNorm and the per-token int8 quantisation run as ONE kernel that feeds the ternary GEMM directly."""
        if (lw.packed is not None and self.ops.name == "kernels" and self.arch.norm == "rmsnorm" and lw.bias is None
                and x.is_cuda):
            from ..ops import bitnet as KB
            q, s = KB.rmsnorm_quant_int8(x, norm_p[0], self.arch.eps)
            ws = float(lw.scale.reshape(-1)[0]) if isinstance(lw.scale, torch.Tensor) else float(lw.scale)
            return KB.bitlinear_q(q, s, lw.packed, ws, None, lw.n, lw.k, x.dtype)
        return self._linear(self._norm(x, norm_p), lw)

    def _norm(self, x, p):
        if self.arch.norm == "layernorm":
            return self.ops.layernorm(x, p[0], p[1], self.arch.eps)
        return self.ops.rmsnorm(x, p[0], self.arch.eps)

    def forward(self, b: Dict[str, torch.Tensor], decode: bool, n_tokens: int, n_items: int,
                want_logits: bool = False, comm=None, local_argmax: bool = False, on_first_attention=None):
        """Runs one step over device-side batch tensors (already sliced to n_tokens / n_items) and returns the
        greedy token of every item as int32 [n_items] (or, with ``want_logits`` and TP=1, the fp32 logits).
        ``comm`` replaces the runner's communicator (concurrent part-batches each need their own); with
        ``local_argmax`` a tensor-parallel rank returns its (index, max) pair and the caller combines the ranks.
        ``on_first_attention()`` is called right after the first layer's attention has been enqueued."""
        a, ops, d = self.arch, self.ops, self.arch.head_dim
        comm = comm or self.comm
        ids, pos, slots = b["token_ids"], b["positions"], b["slot_mapping"]
        if a.rope_base > 0:
            x = ops.embedding(ids, self.wte)
        else:
            x = ops.embedding(ids, self.wte, pos, self.wpe)
        if decode:
            ctx, bt_row = b["seq_lens"], None
        else:
            ctx, bt_row = b["ctx_per_token"], b["token_item"]
        hn, kn = self.n_head_local * d, self.n_kv_local * d
        dense_plan = b.get("dense_plan") if (not decode and ops.name == "kernels" and d in (64, 128)) else None
        # the library backend gathers dense KV, so it is sized by the longest context of this step
        max_ctx = self.step_ctx if (ops.name == "torch" and self.step_ctx) else self.cfg.max_model_len
        split_down = (ops.name == "kernels" and self.tp == 1 and x.shape[0] <= 512 and not a.bitlinear
                      and self.layers[0]["down"].w is not None and self.layers[0]["down"].w.shape[1] >= 2048)
        # one rank, prefill-sized batches: the projections that end a half block run as a cluster GEMM whose epilogue
        # also applies the next norm.  Not for decode: with one or two row tiles only 8-16 CTAs would stream the whole
        # weight matrix (measured 2x slower than split-K + finalize there).
        cluster_norm = (ops.name == "kernels" and self.tp == 1 and not a.bitlinear and self.cfg.cluster_norm
                        and a.hidden % 128 == 0 and a.hidden <= 1024)
        cluster_norm_rows = 1024
        fused_tp = (ops.name == "kernels" and self.tp > 1 and getattr(comm, "fused", False) and not a.bitlinear
                    and a.hidden <= 1024)

        def row_parallel(inp, lw, residual, norm_params, allow_split, quant_next=False):
            """Row-parallel projection + residual.  Returns (new residual stream, normalised copy or None): on the
            fused paths the reduction pass already holds whole rows, so it applies the next norm as well."""
            if fused_tp:
                if norm_params is None:
                    return comm.gemm_allreduce(inp, lw.w, lw.bias, residual), None
                beta = norm_params[1] if len(norm_params) > 1 else None
                return comm.gemm_allreduce(inp, lw.w, lw.bias, residual, norm=(a.norm, norm_params[0], beta, a.eps))
            if cluster_norm and norm_params is not None and lw.w is not None and inp.shape[0] >= cluster_norm_rows:
                return ops.gemm_rownorm(inp, lw, residual, norm_params, a.norm, a.eps)
            if allow_split and split_down:
                return ops.gemm_splitk_norm(inp, lw, residual, norm_params, a.norm, a.eps, 4)
            if (quant_next and lw.packed is not None and norm_params is not None and a.norm == "rmsnorm" and self.tp > 1
                    and getattr(comm, "fused", False) and ops.name == "kernels" and lw.bias is None):
                # the reduction's unpack pass also normalises and quantises for the packed projection that reads next
                return self._linear(inp, lw, residual=residual, reduce=True, comm=comm, norm_quant=(norm_params[0], a.eps))
            return self._linear(inp, lw, residual=residual, reduce=True, comm=comm), None

        h_next = None
        for li, L in enumerate(self.layers):
            if h_next is None and L["qkv"].packed is not None:
                qkv = self._norm_linear(x, L["ln1"], L["qkv"])
            else:
                h = h_next if h_next is not None else self._norm(x, L["ln1"])
                qkv = self._linear(h, L["qkv"])
            if decode and ops.name == "kernels":
                att = ops.append_attention(qkv, hn, hn + kn, slots, self.kcache[li], self.vcache[li], b["block_tables"],
                                           ctx, self.n_head_local, self.n_kv_local, d, max_ctx, pos, a.rope_base)
            else:
                ops.kv_append(qkv, hn, hn + kn, slots, self.kcache[li], self.vcache[li], self.n_head_local,
                              self.n_kv_local, d, pos, a.rope_base)
                if dense_plan is not None and dense_plan.get("paged"):
                    # chunk continuations and prefix hits: the queries of this step against the paged cache, which
                    # holds the earlier context and (appended above) this step's tokens
                    att = ops.paged_prefill_attention(qkv, self.kcache[li], self.vcache[li], b["block_tables"],
                                                      dense_plan, self.n_head_local, self.n_kv_local, d)
                elif dense_plan is not None:
                    # whole prompts without cached context: causal attention on the tensor cores, straight from the
                    # (already rotated) fused qkv buffer; the cache was filled above for the decode steps to come
                    att = ops.dense_attention(qkv, 0, hn, hn + kn, dense_plan, self.n_head_local, self.n_kv_local, d,
                                              True)
                else:
                    att = ops.paged_attention(qkv, self.kcache[li], self.vcache[li], b["block_tables"], ctx,
                                              self.n_head_local, self.n_kv_local, d, max_ctx, bt_row)
            if li == 0 and on_first_attention is not None:
                on_first_attention()
            x, h = row_parallel(att, L["out"], x, L["ln2"], False, quant_next=L["up"].packed is not None)
            if (h is None or isinstance(h, QuantAct)) and a.mlp != "gelu" and L["up"].packed is not None:
                gu = self._linear(h, L["up"]) if isinstance(h, QuantAct) else self._norm_linear(x, L["ln2"], L["up"])
                if (ops.name == "kernels" and L["down"].packed is not None and gu.is_cuda and (gu.shape[-1] // 2) % 16 == 0
                        and gu.shape[-1] // 2 == L["down"].k and gu.shape[-1] // 2 <= 65536):
                    # SwiGLU and the int8 quantisation in front of the down projection as one kernel
                    from ..ops import bitnet as KB
                    f = QuantAct(*KB.swiglu_quant_int8(gu), gu.dtype)
                else:
                    f = ops.swiglu_fused(gu)
            else:
                if h is None:
                    h = self._norm(x, L["ln2"])
                if a.mlp == "gelu":
                    f = self._linear(h, L["up"], activation="gelu")
                else:
                    f = ops.swiglu_fused(self._linear(h, L["up"]))
            nxt = self.layers[li + 1]["ln1"] if li + 1 < len(self.layers) else (self.lnf if decode else None)
            x, h_next = row_parallel(f, L["down"], x, nxt, True,
                                     quant_next=li + 1 < len(self.layers) and self.layers[li + 1]["qkv"].packed is not None)
        if h_next is not None:
            x = h_next                                   # final norm already applied by the last reduction pass
        else:
            if not decode:
                x = ops.gather_rows(x, b["sample_index_clamped"])
            x = self._norm(x, self.lnf)
        logits = ops.lm_head(x, self.lm_head)
        if want_logits:
            return logits if self.tp == 1 else self.gather_vocab(logits, comm)
        if self.tp == 1:
            return ops.argmax(logits)
        idx, mx = ops.argmax(logits, col_offset=self.vocab_start, return_max=True)
        if local_argmax:
            return idx, mx
        return self.combine_argmax(idx, mx, comm)

    def gather_vocab(self, logits: torch.Tensor, comm=None) -> torch.Tensor:
        """Full-vocabulary fp32 logits on every rank from the vocabulary shards: [rows, world * shard] where column
        r * shard + j is token r * shard + j (columns past the vocabulary hold -inf).  Every rank then samples with the
        same seeds and gets the same tokens, so the replicated schedulers stay in step."""
        comm = comm or self.comm
        rows = logits.shape[0]
        local = torch.full((rows, self.vocab_shard), float("-inf"), dtype=torch.float32, device=logits.device)
        local[:, :self.vocab_local] = logits[:, :self.vocab_local]
        allr = comm.all_gather_small(local)                                   # [world, rows, shard]
        return allr.permute(1, 0, 2).reshape(rows, self.tp * self.vocab_shard)

    def combine_argmax(self, idx, mx, comm=None):
        """Greedy token over the vocabulary shards: gather every rank's (index, max) and keep the largest value."""
        comm = comm or self.comm
        if hasattr(comm, "argmax_combine") and self.ops.name == "kernels":
            return comm.argmax_combine(idx, mx)           # exchange + combine in one kernel over peer memory
        vals = comm.all_gather_small(mx)
        idxs = comm.all_gather_small(idx)
        return self.ops.argmax_combine(vals.contiguous(), idxs.contiguous())

