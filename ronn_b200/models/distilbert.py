"""DistilBERT-base encoder as a standard-operator ONNX graph with random-init weights.

Interface of the reference's export script (models/export_distilbert.py:11-38: inputs ``input_ids`` and
``attention_mask`` [batch, sequence], output ``last_hidden_state``).  6 layers, hidden 768, 12 heads, FFN 3072,
vocab 30522, post-LayerNorm blocks, weights ~N(0, 0.02).  GELU uses the tanh form, the reference's only
definition (crates/ronn-core/src/ops/arithmetic.rs:281-296).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..core.types import DataType
from ..graph.ir import ModelGraph, TensorInfo


@dataclass(frozen=True)
class DistilBertConfig:
    n_layers: int = 6
    dim: int = 768
    n_heads: int = 12
    hidden_dim: int = 3072
    vocab_size: int = 30522
    max_position_embeddings: int = 512
    eps: float = 1e-12

    @staticmethod
    def base() -> "DistilBertConfig":
        return DistilBertConfig()

    @staticmethod
    def tiny(n_layers=2, dim=128, n_heads=4, hidden_dim=256, vocab_size=512, max_position_embeddings=64):
        return DistilBertConfig(n_layers, dim, n_heads, hidden_dim, vocab_size, max_position_embeddings)


def build_distilbert(cfg: DistilBertConfig = DistilBertConfig(), dtype: torch.dtype = torch.bfloat16, seed: int = 0) -> ModelGraph:
    gen = torch.Generator().manual_seed(seed)
    H = cfg.dim
    dt = DataType.from_torch(dtype)

    def normal(*shape):
        return (torch.randn(*shape, generator=gen) * 0.02).to(dtype)

    g = ModelGraph()
    g.name = "distilbert"
    g.inputs.append(TensorInfo("input_ids", [0, 0], DataType.I64, ["batch", "sequence"]))
    g.inputs.append(TensorInfo("attention_mask", [0, 0], DataType.I64, ["batch", "sequence"]))
    init = g.initializers
    init["embeddings.word_embeddings.weight"] = normal(cfg.vocab_size, H)
    init["embeddings.position_embeddings.weight"] = normal(cfg.max_position_embeddings, H)
    init["embeddings.LayerNorm.weight"] = torch.ones(H, dtype=dtype)
    init["embeddings.LayerNorm.bias"] = torch.zeros(H, dtype=dtype)
    init["_c.one"] = torch.tensor(1, dtype=torch.int64)
    init["_c.zero"] = torch.tensor(0, dtype=torch.int64)
    init["_c.idx1"] = torch.tensor(1, dtype=torch.int64)
    init["_c.onef"] = torch.tensor(1.0, dtype=dtype)
    init["_c.neg"] = torch.tensor(-10000.0, dtype=dtype)
    init["_c.axes12"] = torch.tensor([1, 2], dtype=torch.int64)
    g.add_node("Shape", ["input_ids"], ["ids_shape"], name="ids_shape")
    g.add_node("Gather", ["ids_shape", "_c.idx1"], ["seq_len"], {"axis": 0}, name="seq_len")
    g.add_node("Range", ["_c.zero", "seq_len", "_c.one"], ["positions"], name="positions")
    g.add_node("Gather", ["embeddings.word_embeddings.weight", "input_ids"], ["tok"], {"axis": 0}, name="word_emb")
    g.add_node("Gather", ["embeddings.position_embeddings.weight", "positions"], ["pos"], {"axis": 0}, name="pos_emb")
    g.add_node("Add", ["tok", "pos"], ["emb"], name="emb_add")
    g.add_node("LayerNormalization", ["emb", "embeddings.LayerNorm.weight", "embeddings.LayerNorm.bias"], ["x.0"],
               {"axis": -1, "epsilon": cfg.eps}, name="emb_ln")
    # additive attention mask [B,1,1,S]: 0 where attended, -10000 where padded
    g.add_node("Cast", ["attention_mask"], ["mask_f"], {"to": 16 if dtype == torch.bfloat16 else (10 if dtype == torch.float16 else 1)}, name="mask_cast")
    g.add_node("Sub", ["_c.onef", "mask_f"], ["mask_inv"], name="mask_inv")
    g.add_node("Mul", ["mask_inv", "_c.neg"], ["mask_add"], name="mask_scale")
    g.add_node("Unsqueeze", ["mask_add", "_c.axes12"], ["mask4"], name="mask_unsqueeze")
    x = "x.0"
    for i in range(cfg.n_layers):
        p = f"transformer.layer.{i}"
        for nm, (k, n) in {"attention.q_lin": (H, H), "attention.k_lin": (H, H), "attention.v_lin": (H, H),
                           "attention.out_lin": (H, H), "ffn.lin1": (H, cfg.hidden_dim), "ffn.lin2": (cfg.hidden_dim, H)}.items():
            init[f"{p}.{nm}.weight"] = normal(k, n)          # stored [in, out] as an ONNX MatMul operand
            init[f"{p}.{nm}.bias"] = torch.zeros(n, dtype=dtype)
        for nm in ("sa_layer_norm", "output_layer_norm"):
            init[f"{p}.{nm}.weight"] = torch.ones(H, dtype=dtype)
            init[f"{p}.{nm}.bias"] = torch.zeros(H, dtype=dtype)

        def lin(inp, nm, out):
            g.add_node("MatMul", [inp, f"{p}.{nm}.weight"], [f"{out}_mm"], name=f"{p}.{nm}")
            g.add_node("Add", [f"{out}_mm", f"{p}.{nm}.bias"], [out], name=f"{p}.{nm}.bias_add")

        lin(x, "attention.q_lin", f"{p}.q")
        lin(x, "attention.k_lin", f"{p}.k")
        lin(x, "attention.v_lin", f"{p}.v")
        # mask_type: the additive mask only hides a padded suffix of every row (the contract of `attention_mask` here),
        # which lets a provider pass key lengths to its attention kernel instead of the dense mask
        g.add_node("Attention", [f"{p}.q", f"{p}.k", f"{p}.v", "mask4"], [f"{p}.ctx"],
                   {"num_heads": cfg.n_heads, "mask_type": "key_padding"}, name=f"{p}.attention")
        lin(f"{p}.ctx", "attention.out_lin", f"{p}.sa")
        g.add_node("Add", [f"{p}.sa", x], [f"{p}.sa_res"], name=f"{p}.sa_res")
        g.add_node("LayerNormalization", [f"{p}.sa_res", f"{p}.sa_layer_norm.weight", f"{p}.sa_layer_norm.bias"], [f"{p}.h"],
                   {"axis": -1, "epsilon": cfg.eps}, name=f"{p}.sa_ln")
        lin(f"{p}.h", "ffn.lin1", f"{p}.f1")
        g.add_node("Gelu", [f"{p}.f1"], [f"{p}.act"], {"approximate": "tanh"}, name=f"{p}.gelu")
        lin(f"{p}.act", "ffn.lin2", f"{p}.f2")
        g.add_node("Add", [f"{p}.f2", f"{p}.h"], [f"{p}.ffn_res"], name=f"{p}.ffn_res")
        g.add_node("LayerNormalization", [f"{p}.ffn_res", f"{p}.output_layer_norm.weight", f"{p}.output_layer_norm.bias"],
                   [f"{p}.out"], {"axis": -1, "epsilon": cfg.eps}, name=f"{p}.out_ln")
        x = f"{p}.out"
    g.add_node("Identity", [x], ["last_hidden_state"], name="output")
    g.outputs.append(TensorInfo("last_hidden_state", [0, 0, H], dt, ["batch", "sequence", None]))
    g.metadata.update({"ronn.arch": "distilbert", "ronn.n_layers": str(cfg.n_layers), "ronn.dim": str(H),
                       "ronn.n_heads": str(cfg.n_heads), "ronn.hidden_dim": str(cfg.hidden_dim),
                       "ronn.vocab_size": str(cfg.vocab_size), "ronn.max_pos": str(cfg.max_position_embeddings),
                       "ronn.eps": str(cfg.eps)})
    return g
