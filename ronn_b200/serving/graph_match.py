"""Recognises a GPT-2-style decoder in a standard-operator ONNX graph, so that a model written by an exporter (the
reference's ``models/export_gpt2.py:11-37``: ``torch.onnx.export`` of a Hugging Face GPT-2, opset 13+) can be served by
``LLMEngine`` without the ``ronn.arch`` metadata and initializer names of the in-tree builders.

The match is structural.  In topological order a GPT-2 graph consists of: two embedding Gathers (token ids and
positions), then per layer LayerNorm -> linear [H, 3H] -> causal attention -> linear [H, H] -> residual -> LayerNorm ->
linear [H, F] -> tanh-GELU -> linear [F, H] -> residual, then a final LayerNorm (and optionally the tied LM head).
Exporters rename and re-shape nearly everything around that skeleton (decomposed LayerNorm and GELU, Gemm or MatMul +
Add, Reshape / Transpose / Split plumbing, mask tables), but the order and shapes of the 2-D weights and of the
LayerNorm parameters survive, and that is what is matched; the graph is first normalised with the fusion pass, which
re-assembles decomposed LayerNorm and GELU chains.  The result is the architecture record of the decoder runner plus
the weights under the names the runner expects.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..api.errors import SessionError
from ..graph.ir import ModelGraph


def _linear_layers(graph: ModelGraph):
    """(node, weight [in, out], bias or None) of every linear layer with a constant 2-D weight, in execution order."""
    cons = graph.consumers()
    out = []
    for n in graph.topological_order():
        if n.op_type not in ("MatMul", "Gemm", "FusedGemm") or len(n.inputs) < 2:
            continue
        w = graph.initializers.get(n.inputs[1])
        if w is None or w.dim() != 2 or not w.is_floating_point() or n.inputs[0] in graph.initializers:
            continue
        if n.op_type in ("Gemm", "FusedGemm") and int(n.attr("transB", 0)):
            w = w.t()
        if n.op_type == "Gemm" and (int(n.attr("transA", 0)) or float(n.attr("alpha", 1.0)) != 1.0):
            continue
        bias = graph.initializers.get(n.inputs[2]) if len(n.inputs) > 2 and n.inputs[2] else None
        if bias is None and n.op_type == "MatMul":
            users = cons.get(n.outputs[0], [])
            if len(users) == 1 and users[0].op_type == "Add":
                other = [i for i in users[0].inputs if i != n.outputs[0]]
                cand = graph.initializers.get(other[0]) if other else None
                if cand is not None and cand.dim() == 1 and cand.shape[0] == w.shape[1]:
                    bias = cand
        out.append((n, w, bias))
    return out


def _num_heads(graph: ModelGraph, hidden: int) -> Optional[int]:
    for n in graph.nodes:
        if n.op_type in ("Attention", "MultiHeadAttention") and n.attr("num_heads"):
            return int(n.attr("num_heads"))
    votes: Dict[int, int] = {}
    prod = graph.producers()

    def const_int(name):
        t = graph.initializers.get(name)
        if t is not None and t.numel() == 1 and not t.is_floating_point():
            return int(t.reshape(-1)[0])
        p = prod.get(name)
        if p is not None and p.op_type == "Constant" and isinstance(p.attr("value"), torch.Tensor) and p.attr("value").numel() == 1:
            return int(p.attr("value").reshape(-1)[0])
        return None

    for n in graph.nodes:
        if n.op_type != "Reshape" or len(n.inputs) < 2:
            continue
        shp = graph.initializers.get(n.inputs[1])
        if shp is not None and shp.numel() == 4:
            a, b = int(shp[2]), int(shp[3])
        else:
            # a shape assembled at run time: [batch, sequence, heads, head_dim] with the last two entries constant
            c = prod.get(n.inputs[1])
            if c is None or c.op_type != "Concat" or len(c.inputs) != 4:
                continue
            a, b = const_int(c.inputs[2]), const_int(c.inputs[3])
            if a is None or b is None:
                continue
        if a > 0 and b > 0 and a * b == hidden:
            votes[a] = votes.get(a, 0) + 1
    if votes:
        return max(votes.items(), key=lambda kv: kv[1])[0]
    return None


def match_gpt2(graph: ModelGraph):
    """Returns (architecture fields, canonical initializers) or raises SessionError naming what did not match."""
    from ..graph.passes.constant_folding import ConstantFoldingPass
    from ..graph.passes.fusion import NodeFusionPass
    g = graph.clone()
    ConstantFoldingPass().run(g)               # Constant nodes and constant sub-expressions become initializers
    NodeFusionPass().run(g)                    # decomposed LayerNorm / GELU chains become single nodes again
    g.sort_in_place()
    order = g.topological_order()
    inputs = {i.name for i in g.inputs}

    # ---- embeddings
    gathers = [n for n in order if n.op_type == "Gather" and len(n.inputs) == 2
               and g.initializers.get(n.inputs[0]) is not None and g.initializers[n.inputs[0]].dim() == 2
               and g.initializers[n.inputs[0]].is_floating_point()]
    wte = next((g.initializers[n.inputs[0]] for n in gathers if n.inputs[1] in inputs), None)
    if wte is None:
        raise SessionError("no token-embedding Gather over a graph input found: not a decoder graph")
    wpe = next((g.initializers[n.inputs[0]] for n in gathers
                if n.inputs[1] not in inputs and g.initializers[n.inputs[0]].shape[1] == wte.shape[1]
                and g.initializers[n.inputs[0]] is not wte), None)
    if wpe is None:
        raise SessionError("no learned position-embedding Gather found (only GPT-2-style decoders are recognised)")
    V, H = int(wte.shape[0]), int(wte.shape[1])

    # ---- linear layers: [H,3H] [H,H] [H,F] [F,H] per layer (+ optional LM head [H,V])
    lin = _linear_layers(g)
    shapes = [tuple(w.shape) for _, w, _ in lin]
    if shapes and shapes[-1] == (H, V):
        lin, shapes = lin[:-1], shapes[:-1]
    if not lin or len(lin) % 4:
        raise SessionError(f"expected four linear layers per decoder block, found {len(shapes)} in all: {shapes[:8]}")
    L = len(lin) // 4
    F = shapes[2][1]
    for i in range(L):
        want = [(H, 3 * H), (H, H), (H, F), (F, H)]
        got = shapes[4 * i: 4 * i + 4]
        if got != want:
            raise SessionError(f"block {i}: linear layers have shapes {got}, a GPT-2 block has {want}")

    # ---- LayerNorms: two per block and a final one
    # (the fusion pass may have merged a residual add into the norm: SkipLayerNorm(x, skip, gamma, beta))
    lns = [n for n in order if n.op_type in ("LayerNormalization", "SkipLayerNorm")]
    if len(lns) != 2 * L + 1:
        raise SessionError(f"expected {2 * L + 1} LayerNormalization nodes for {L} blocks, found {len(lns)}")
    eps = float(lns[0].attr("epsilon", 1e-5))

    def ln_params(n):
        return n.inputs[1:3] if n.op_type == "LayerNormalization" else n.inputs[2:4]

    for n in lns:
        if len(ln_params(n)) < 2 or any(g.initializers.get(x) is None for x in ln_params(n)):
            raise SessionError("LayerNormalization with non-constant scale / shift")

    # ---- activation and attention sanity
    ops = [n.op_type for n in order]
    gelu_tanh = sum(1 for n in order if (n.op_type == "Gelu" and n.attr("approximate", "tanh") == "tanh")
                    or (n.op_type == "FusedGemm" and n.attr("activation") == "Gelu")) + ops.count("Tanh")
    if gelu_tanh < L:
        raise SessionError("the MLP activation is not the tanh form of GELU (the decoder runner implements GPT-2's gelu_new)")
    if sum(ops.count(t) for t in ("Softmax", "Attention", "MultiHeadAttention", "ScaledDotProductAttention")) < L:
        raise SessionError(f"expected an attention (Softmax or Attention node) per block, found fewer than {L}")
    heads = _num_heads(g, H)
    if heads is None:
        raise SessionError("cannot determine the number of attention heads (no 4-D Reshape [.., .., heads, head_dim])")

    init: Dict[str, torch.Tensor] = {"wte": wte, "wpe": wpe}
    names = ("attn.c_attn", "attn.c_proj", "mlp.c_fc", "mlp.c_proj")
    for i in range(L):
        for k, nm in enumerate(names):
            _, w, b = lin[4 * i + k]
            init[f"h.{i}.{nm}.weight"] = w
            init[f"h.{i}.{nm}.bias"] = b if b is not None else torch.zeros(w.shape[1], dtype=w.dtype)
        for k, nm in enumerate(("ln_1", "ln_2")):
            ln = lns[2 * i + k]
            init[f"h.{i}.{nm}.weight"] = g.initializers[ln_params(ln)[0]]
            init[f"h.{i}.{nm}.bias"] = g.initializers[ln_params(ln)[1]]
    init["ln_f.weight"] = g.initializers[ln_params(lns[-1])[0]]
    init["ln_f.bias"] = g.initializers[ln_params(lns[-1])[1]]
    fields = {"n_layer": L, "hidden": H, "n_head": heads, "ffn": F, "vocab": V, "max_pos": int(wpe.shape[0]), "eps": eps}
    return fields, init


def decoder_from_graph(graph: ModelGraph):
    """(DecoderArch, initializers) for the serving engine: from the ``ronn.arch`` metadata of the in-tree builders when
    present, otherwise by recognising the decoder in the operator graph."""
    from .model_runner import DecoderArch
    if graph.metadata.get("ronn.arch"):
        return DecoderArch.from_metadata(graph.metadata), graph.initializers
    f, init = match_gpt2(graph)
    arch = DecoderArch("gpt2", f["n_layer"], f["hidden"], f["n_head"], f["n_head"], f["hidden"] // f["n_head"], f["ffn"],
                       f["vocab"], f["max_pos"], eps=f["eps"])
    return arch, init
