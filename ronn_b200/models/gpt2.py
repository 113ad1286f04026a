"""GPT-2 family as an ONNX graph with random-init weights.

Same interface as the reference's export script (models/export_gpt2.py:11-37: input ``input_ids``
[batch, sequence], opset 13+), plus a ``logits`` output through the tied LM head.  The graph uses
standard operators only (Gather, LayerNormalization, MatMul, Add, Split, Attention with
``causal=1``, Gelu), so it runs through ``session.run``; the serving engine reads the same
initializers (HF names: ``wte``, ``wpe``, ``h.N.attn.c_attn.weight`` ...) to build its paged-KV
decoder.  ``metadata_props`` carry the architecture (``ronn.arch=gpt2`` and sizes).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..core.types import DataType
from ..graph.ir import ModelGraph, TensorInfo


@dataclass(frozen=True)
class GPT2Config:
    n_layer: int = 24
    n_embd: int = 1024
    n_head: int = 16
    vocab_size: int = 50257
    n_positions: int = 1024
    layer_norm_epsilon: float = 1e-5

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def small() -> "GPT2Config":
        return GPT2Config(n_layer=12, n_embd=768, n_head=12)

    @staticmethod
    def tiny(n_layer=2, n_embd=128, n_head=2, vocab_size=512, n_positions=256) -> "GPT2Config":
        return GPT2Config(n_layer, n_embd, n_head, vocab_size, n_positions)


def build_gpt2(cfg: GPT2Config = GPT2Config(), dtype: torch.dtype = torch.bfloat16, seed: int = 0,
               with_lm_head: bool = True) -> ModelGraph:
    gen = torch.Generator().manual_seed(seed)
    H, L = cfg.n_embd, cfg.n_layer
    dt = DataType.from_torch(dtype)

    def normal(*shape, std=0.02):
        return (torch.randn(*shape, generator=gen) * std).to(dtype)

    g = ModelGraph()
    g.name = "gpt2"
    g.inputs.append(TensorInfo("input_ids", [0, 0], DataType.I64, ["batch", "sequence"]))
    init = g.initializers
    init["wte"] = normal(cfg.vocab_size, H)
    init["wpe"] = normal(cfg.n_positions, H, std=0.01)
    # positions 0..S-1 from the runtime shape of input_ids
    init["_c.one"] = torch.tensor(1, dtype=torch.int64)
    init["_c.zero"] = torch.tensor(0, dtype=torch.int64)
    init["_c.idx1"] = torch.tensor(1, dtype=torch.int64)
    g.add_node("Shape", ["input_ids"], ["ids_shape"], name="ids_shape")
    g.add_node("Gather", ["ids_shape", "_c.idx1"], ["seq_len"], {"axis": 0}, name="seq_len")
    g.add_node("Range", ["_c.zero", "seq_len", "_c.one"], ["positions"], name="positions")
    g.add_node("Gather", ["wte", "input_ids"], ["tok_emb"], {"axis": 0}, name="wte_gather")
    g.add_node("Gather", ["wpe", "positions"], ["pos_emb"], {"axis": 0}, name="wpe_gather")
    g.add_node("Add", ["tok_emb", "pos_emb"], ["h.in.0"], name="embed_add")
    x = "h.in.0"
    for i in range(L):
        p = f"h.{i}"
        init[f"{p}.ln_1.weight"] = torch.ones(H, dtype=dtype)
        init[f"{p}.ln_1.bias"] = torch.zeros(H, dtype=dtype)
        init[f"{p}.attn.c_attn.weight"] = normal(H, 3 * H)
        init[f"{p}.attn.c_attn.bias"] = torch.zeros(3 * H, dtype=dtype)
        init[f"{p}.attn.c_proj.weight"] = normal(H, H, std=0.02 / (2 * L) ** 0.5)
        init[f"{p}.attn.c_proj.bias"] = torch.zeros(H, dtype=dtype)
        init[f"{p}.ln_2.weight"] = torch.ones(H, dtype=dtype)
        init[f"{p}.ln_2.bias"] = torch.zeros(H, dtype=dtype)
        init[f"{p}.mlp.c_fc.weight"] = normal(H, 4 * H)
        init[f"{p}.mlp.c_fc.bias"] = torch.zeros(4 * H, dtype=dtype)
        init[f"{p}.mlp.c_proj.weight"] = normal(4 * H, H, std=0.02 / (2 * L) ** 0.5)
        init[f"{p}.mlp.c_proj.bias"] = torch.zeros(H, dtype=dtype)
        g.add_node("LayerNormalization", [x, f"{p}.ln_1.weight", f"{p}.ln_1.bias"], [f"{p}.ln1"],
                   {"axis": -1, "epsilon": cfg.layer_norm_epsilon}, name=f"{p}.ln_1")
        g.add_node("MatMul", [f"{p}.ln1", f"{p}.attn.c_attn.weight"], [f"{p}.qkv_mm"], name=f"{p}.c_attn")
        g.add_node("Add", [f"{p}.qkv_mm", f"{p}.attn.c_attn.bias"], [f"{p}.qkv"], name=f"{p}.c_attn_bias")
        g.add_node("Split", [f"{p}.qkv"], [f"{p}.q", f"{p}.k", f"{p}.v"], {"axis": -1, "num_outputs": 3},
                   name=f"{p}.split")
        g.add_node("Attention", [f"{p}.q", f"{p}.k", f"{p}.v"], [f"{p}.attn"],
                   {"num_heads": cfg.n_head, "causal": 1}, name=f"{p}.attention")
        g.add_node("MatMul", [f"{p}.attn", f"{p}.attn.c_proj.weight"], [f"{p}.proj_mm"], name=f"{p}.c_proj")
        g.add_node("Add", [f"{p}.proj_mm", f"{p}.attn.c_proj.bias"], [f"{p}.proj"], name=f"{p}.c_proj_bias")
        g.add_node("Add", [x, f"{p}.proj"], [f"{p}.res1"], name=f"{p}.res1")
        g.add_node("LayerNormalization", [f"{p}.res1", f"{p}.ln_2.weight", f"{p}.ln_2.bias"], [f"{p}.ln2"],
                   {"axis": -1, "epsilon": cfg.layer_norm_epsilon}, name=f"{p}.ln_2")
        g.add_node("MatMul", [f"{p}.ln2", f"{p}.mlp.c_fc.weight"], [f"{p}.fc_mm"], name=f"{p}.c_fc")
        g.add_node("Add", [f"{p}.fc_mm", f"{p}.mlp.c_fc.bias"], [f"{p}.fc"], name=f"{p}.c_fc_bias")
        g.add_node("Gelu", [f"{p}.fc"], [f"{p}.act"], {"approximate": "tanh"}, name=f"{p}.gelu")
        g.add_node("MatMul", [f"{p}.act", f"{p}.mlp.c_proj.weight"], [f"{p}.mlp_mm"], name=f"{p}.mlp_proj")
        g.add_node("Add", [f"{p}.mlp_mm", f"{p}.mlp.c_proj.bias"], [f"{p}.mlp"], name=f"{p}.mlp_proj_bias")
        g.add_node("Add", [f"{p}.res1", f"{p}.mlp"], [f"{p}.out"], name=f"{p}.res2")
        x = f"{p}.out"
    init["ln_f.weight"] = torch.ones(H, dtype=dtype)
    init["ln_f.bias"] = torch.zeros(H, dtype=dtype)
    g.add_node("LayerNormalization", [x, "ln_f.weight", "ln_f.bias"], ["last_hidden_state"],
               {"axis": -1, "epsilon": cfg.layer_norm_epsilon}, name="ln_f")
    g.outputs.append(TensorInfo("last_hidden_state", [0, 0, H], dt, ["batch", "sequence", None]))
    if with_lm_head:
        g.add_node("Transpose", ["wte"], ["wte_t"], {"perm": [1, 0]}, name="lm_head_t")
        g.add_node("MatMul", ["last_hidden_state", "wte_t"], ["logits"], name="lm_head")
        g.outputs.append(TensorInfo("logits", [0, 0, cfg.vocab_size], dt, ["batch", "sequence", None]))
    g.metadata.update({"ronn.arch": "gpt2", "ronn.n_layer": str(L), "ronn.n_embd": str(H),
                       "ronn.n_head": str(cfg.n_head), "ronn.vocab_size": str(cfg.vocab_size),
                       "ronn.n_positions": str(cfg.n_positions), "ronn.eps": str(cfg.layer_norm_epsilon)})
    return g


def config_from_metadata(md) -> GPT2Config:
    return GPT2Config(int(md["ronn.n_layer"]), int(md["ronn.n_embd"]), int(md["ronn.n_head"]),
                      int(md["ronn.vocab_size"]), int(md["ronn.n_positions"]), float(md.get("ronn.eps", 1e-5)))
