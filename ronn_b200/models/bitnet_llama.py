"""BitNet b1.58 Llama-style decoder as an ONNX graph over the ``com.ronn`` custom domain.

Architecture per the Llama design notes (docs/new/RONN-Llama-Branch-Prompt.md:425-633: RMSNorm, rotary
embedding theta_i = base^(-2i/d), SwiGLU ``down(silu(gate(x)) * up(x))``) with every projection a
``BitLinear``: ternary weights stored 2-bit packed ``[N, K/4]`` uint8 in the reference's code assignment
(crates/ronn-providers/src/bitnet/quantization.rs:131-153) plus one per-tensor scale, int8 per-token
activations.  Random-init weights are i.i.d. ternary with probability 1/3 each.  The graph runs through
``session.run`` (operator definitions in the registry) and the serving engine reads the same initializers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..core.types import DataType
from ..graph.ir import ModelGraph, TensorInfo
from ..providers.bitnet.quantization import pack_ternary_rows

RONN = "com.ronn"


@dataclass(frozen=True)
class BitNetConfig:
    n_layer: int = 24
    hidden: int = 2560
    n_head: int = 20
    ffn: int = 6912
    vocab_size: int = 32000
    max_pos: int = 4096
    rope_base: float = 10000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_head

    @staticmethod
    def b158_2b() -> "BitNetConfig":
        return BitNetConfig()

    @staticmethod
    def tiny(n_layer=2, hidden=256, n_head=2, ffn=512, vocab_size=512, max_pos=256) -> "BitNetConfig":
        return BitNetConfig(n_layer, hidden, n_head, ffn, vocab_size, max_pos)


def _ternary(n: int, k: int, gen: torch.Generator):
    vals = torch.randint(0, 3, (n, k), generator=gen, dtype=torch.int8) - 1
    scale = 1.0 / math.sqrt(k * 2.0 / 3.0)
    return pack_ternary_rows(vals), torch.tensor(scale, dtype=torch.float32)


def build_bitnet_llama(cfg: BitNetConfig = BitNetConfig(), dtype: torch.dtype = torch.bfloat16, seed: int = 0,
                       with_lm_head: bool = True) -> ModelGraph:
    gen = torch.Generator().manual_seed(seed)
    H, F, d, nh = cfg.hidden, cfg.ffn, cfg.head_dim, cfg.n_head
    dt = DataType.from_torch(dtype)
    g = ModelGraph()
    g.name = "bitnet_llama"
    g.inputs.append(TensorInfo("input_ids", [0, 0], DataType.I64, ["batch", "sequence"]))
    init = g.initializers
    init["embed"] = (torch.randn(cfg.vocab_size, H, generator=gen) * 0.02).to(dtype)
    init["_c.one"] = torch.tensor(1, dtype=torch.int64)
    init["_c.zero"] = torch.tensor(0, dtype=torch.int64)
    init["_c.idx1"] = torch.tensor(1, dtype=torch.int64)
    g.add_node("Shape", ["input_ids"], ["ids_shape"], name="ids_shape")
    g.add_node("Gather", ["ids_shape", "_c.idx1"], ["seq_len"], {"axis": 0}, name="seq_len")
    g.add_node("Range", ["_c.zero", "seq_len", "_c.one"], ["positions"], name="positions")
    g.add_node("Gather", ["embed", "input_ids"], ["x.0"], {"axis": 0}, name="embed_gather")
    x = "x.0"

    def bitlinear(inp, name, n, k, out):
        init[f"{name}.weight"], init[f"{name}.scale"] = _ternary(n, k, gen)
        g.add_node("BitLinear", [inp, f"{name}.weight", f"{name}.scale"], [out],
                   {"k": k, "n": n, "quant": "ternary2", "act_bits": 8}, name=name, domain=RONN)

    for i in range(cfg.n_layer):
        p = f"layers.{i}"
        init[f"{p}.attn_norm.weight"] = torch.ones(H, dtype=dtype)
        init[f"{p}.ffn_norm.weight"] = torch.ones(H, dtype=dtype)
        g.add_node("RMSNorm", [x, f"{p}.attn_norm.weight"], [f"{p}.h1"], {"epsilon": cfg.eps}, name=f"{p}.attn_norm", domain=RONN)
        bitlinear(f"{p}.h1", f"{p}.qkv", 3 * H, H, f"{p}.qkv_out")
        g.add_node("Split", [f"{p}.qkv_out"], [f"{p}.q0", f"{p}.k0", f"{p}.v"], {"axis": -1, "num_outputs": 3}, name=f"{p}.split")
        g.add_node("RotaryEmbedding", [f"{p}.q0", "positions"], [f"{p}.q"], {"num_heads": nh, "base": cfg.rope_base},
                   name=f"{p}.rope_q", domain=RONN)
        g.add_node("RotaryEmbedding", [f"{p}.k0", "positions"], [f"{p}.k"], {"num_heads": nh, "base": cfg.rope_base},
                   name=f"{p}.rope_k", domain=RONN)
        g.add_node("Attention", [f"{p}.q", f"{p}.k", f"{p}.v"], [f"{p}.att"], {"num_heads": nh, "causal": 1}, name=f"{p}.attention")
        bitlinear(f"{p}.att", f"{p}.o", H, H, f"{p}.o_out")
        g.add_node("Add", [x, f"{p}.o_out"], [f"{p}.res1"], name=f"{p}.res1")
        g.add_node("RMSNorm", [f"{p}.res1", f"{p}.ffn_norm.weight"], [f"{p}.h2"], {"epsilon": cfg.eps}, name=f"{p}.ffn_norm", domain=RONN)
        bitlinear(f"{p}.h2", f"{p}.gate_up", 2 * F, H, f"{p}.gu")
        g.add_node("Split", [f"{p}.gu"], [f"{p}.gate", f"{p}.up"], {"axis": -1, "num_outputs": 2}, name=f"{p}.split_gu")
        g.add_node("SwiGLU", [f"{p}.gate", f"{p}.up"], [f"{p}.act"], name=f"{p}.swiglu", domain=RONN)
        bitlinear(f"{p}.act", f"{p}.down", H, F, f"{p}.down_out")
        g.add_node("Add", [f"{p}.res1", f"{p}.down_out"], [f"{p}.out"], name=f"{p}.res2")
        x = f"{p}.out"
    init["norm.weight"] = torch.ones(H, dtype=dtype)
    g.add_node("RMSNorm", [x, "norm.weight"], ["last_hidden_state"], {"epsilon": cfg.eps}, name="final_norm", domain=RONN)
    g.outputs.append(TensorInfo("last_hidden_state", [0, 0, H], dt, ["batch", "sequence", None]))
    if with_lm_head:
        g.add_node("Transpose", ["embed"], ["embed_t"], {"perm": [1, 0]}, name="lm_head_t")
        g.add_node("MatMul", ["last_hidden_state", "embed_t"], ["logits"], name="lm_head")
        g.outputs.append(TensorInfo("logits", [0, 0, cfg.vocab_size], dt, ["batch", "sequence", None]))
    g.metadata.update({"ronn.arch": "bitnet", "ronn.n_layer": str(cfg.n_layer), "ronn.hidden": str(H),
                       "ronn.n_head": str(nh), "ronn.n_kv_head": str(nh), "ronn.head_dim": str(d), "ronn.ffn": str(F),
                       "ronn.vocab_size": str(cfg.vocab_size), "ronn.max_pos": str(cfg.max_pos),
                       "ronn.rope_base": str(cfg.rope_base), "ronn.eps": str(cfg.eps)})
    return g


def load_decoder_weights(runner, init) -> None:
    """Shard the BitNet / Llama initializers for ``DecoderRunner`` (column-parallel qkv and gate|up rows,
    row-parallel o and down along K; packed weights are sliced in their packed form)."""
    from ..serving.model_runner import LinearW
    a, d = runner.arch, runner.arch.head_dim
    dev = runner.device
    hs, hn = runner.h0 * d, runner.n_head_local * d
    H, F = a.hidden, a.ffn
    f0, f1 = runner.rank * runner.ffn_local, (runner.rank + 1) * runner.ffn_local
    runner.wte = runner._dev(init["embed"])
    runner.wpe = None
    runner.lnf = (runner._dev(init["norm.weight"]),)
    runner.lm_head = runner.wte[runner.vocab_start:runner.vocab_start + runner.vocab_local]

    def packed(name, rows=None, kslice=None):
        w = init[f"{name}.weight"]                       # [N, K/4] uint8
        k_full = w.shape[1] * 4
        if rows is not None:
            w = w[rows]
        k = k_full
        if kslice is not None:
            w = w[:, kslice[0] // 4: kslice[1] // 4]
            k = kslice[1] - kslice[0]
        w = w.contiguous().to(dev)
        return LinearW(packed=w, scale=float(init[f"{name}.scale"]), n=w.shape[0], k=k)

    # The packed-weight TMA of the BitLinear kernel wants K shards that are multiples of 64.  A ragged FFN shard (6912 / 8
    # = 864) is widened to the next multiple with weights of zero (code 01): the extra gate | up rows produce
    # silu(0) * 0 = 0 and the extra K columns of the down projection multiply them by zero again.
    fl = f1 - f0
    fpad = (-fl) % 64 if runner.tp > 1 else 0
    zero_code = 0x55                                     # four ternary zeros

    def pad_rows(lw, at, count):
        """`count` all-zero weight rows inserted at each row index of `at` (ascending)."""
        pieces, prev = [], 0
        z = torch.full((count, lw.packed.shape[1]), zero_code, dtype=torch.uint8, device=lw.packed.device)
        for pos in at:
            pieces += [lw.packed[prev:pos], z]
            prev = pos
        pieces.append(lw.packed[prev:])
        w = torch.cat(pieces).contiguous()
        return LinearW(packed=w, scale=lw.scale, n=w.shape[0], k=lw.k)

    def pad_k(lw, count):
        z = torch.full((lw.packed.shape[0], count // 4), zero_code, dtype=torch.uint8, device=lw.packed.device)
        return LinearW(packed=torch.cat([lw.packed, z], dim=1).contiguous(), scale=lw.scale, n=lw.n, k=lw.k + count)

    for i in range(a.n_layer):
        p = f"layers.{i}"
        qrows = torch.cat([torch.arange(hs, hs + hn), H + torch.arange(hs, hs + hn), 2 * H + torch.arange(hs, hs + hn)])
        gurows = torch.cat([torch.arange(f0, f1), F + torch.arange(f0, f1)])
        up, down = packed(f"{p}.gate_up", rows=gurows), packed(f"{p}.down", kslice=(f0, f1))
        if fpad:
            up = pad_rows(up, [fl, 2 * fl], fpad)        # gate rows, pad, up rows, pad
            down = pad_k(down, fpad)
        runner.layers.append({
            "ln1": (runner._dev(init[f"{p}.attn_norm.weight"]),),
            "ln2": (runner._dev(init[f"{p}.ffn_norm.weight"]),),
            "qkv": packed(f"{p}.qkv", rows=qrows),
            "out": packed(f"{p}.o", kslice=(hs, hs + hn)),
            "up": up,
            "down": down,
        })
