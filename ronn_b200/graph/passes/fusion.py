"""Node fusion.

Patterns (the reference names them but never matches, because its graphs have no edges:
crates/ronn-graph/src/passes/fusion.rs:15-83; fusion table in
crates/ronn-providers/src/compiler.rs:267-314):

* Conv -> BatchNormalization            => Conv with folded weights
      W' = W * gamma / sqrt(var + eps),  b' = (b - mean) * gamma / sqrt(var + eps) + beta
* Conv [-> Add(residual)] -> Relu       => com.ronn::FusedConv(activation, optional 4th input)
* MatMul -> Add(constant bias)          => com.ronn::FusedGemm
* Gemm / FusedGemm -> Relu | Gelu(tanh) => FusedGemm(activation)
* FusedGemm -> Add(residual)            => FusedGemm with 4th input
* Add -> LayerNormalization             => com.ronn::SkipLayerNorm(x, skip, gamma, beta) -> (normed, sum): the sum
                                           stays available to its other consumers (the next residual add)
* MatMul(Q, K^T) -> [Div | Mul scalar] -> [Where fill] -> [Add mask] -> Softmax(last axis) -> MatMul(., V)
                                        => com.ronn::ScaledDotProductAttention(Q, K^T, V [, mask]): the attention core
                                           as exporters write it; the GPU provider runs it on the tensor-core kernel
* ReduceMean, Sub, Pow, ReduceMean, Add(eps), Sqrt, Div, Mul(gamma), Add(beta)
                                        => LayerNormalization: the nine-node form exporters write below opset 17
                                           (the reference's own export scripts use opset 13)
* x * 0.5 * (1 + Erf(x / sqrt(2)))      => Gelu(approximate="none"): the five-node chain exporters write for the exact
                                           GELU (either multiplication order)
"""
from __future__ import annotations

import math

import torch

from ..ir import GraphNode, ModelGraph
from .base import OptimizationPass, PassStats

RONN = "com.ronn"


class NodeFusionPass(OptimizationPass):
    name = "NodeFusion"

    def run(self, graph: ModelGraph) -> PassStats:
        stats = PassStats()
        progress = True
        while progress:
            progress = False
            for fn in (self._fold_bn, self._conv_act, self._decomposed_layernorm, self._erf_gelu, self._matmul_bias,
                       self._gemm_act,
                       self._gemm_residual, self._qkv_projection, self._skip_layernorm, self._sdpa):
                n = fn(graph)
                if n:
                    stats.nodes_fused += n
                    progress = True
        return stats

    # -------------------------------------------------------------- helpers
    @staticmethod
    def _single_consumer(graph, cons, name):
        if name in set(graph.output_names()):
            return None
        c = cons.get(name, [])
        return c[0] if len(c) == 1 else None

    # -------------------------------------------------------------- LayerNorm written out in primitives
    def _decomposed_layernorm(self, graph: ModelGraph) -> int:
        cons, prod = graph.consumers(), graph.producers()
        outputs = set(graph.output_names())

        def last_axis_mean(node):
            if node is None or node.op_type != "ReduceMean" or int(node.attr("keepdims", 1)) != 1:
                return False
            axes = node.attr("axes")
            if axes is None and len(node.inputs) > 1:
                t = graph.initializers.get(node.inputs[1])
                axes = None if t is None else [int(v) for v in t.reshape(-1).tolist()]
            return axes is not None and list(axes) == [-1]

        def only(name, *want):
            """the consumers of `name` are exactly `want` nodes (any order) and it is not a graph output"""
            got = cons.get(name, [])
            return name not in outputs and len(got) == len(want) and all(any(g is w for g in got) for w in want)

        for sub in graph.nodes:
            if sub.op_type != "Sub" or len(sub.inputs) != 2:
                continue
            x, mean = sub.inputs[0], prod.get(sub.inputs[1])
            if not last_axis_mean(mean) or mean.inputs[0] != x or not only(mean.outputs[0], sub):
                continue
            users = cons.get(sub.outputs[0], [])
            pw = next((u for u in users if u.op_type == "Pow"), None)
            div = next((u for u in users if u.op_type == "Div" and u.inputs[0] == sub.outputs[0]), None)
            if pw is None or div is None or not only(sub.outputs[0], pw, div):
                continue
            if self._scalar(graph, pw.inputs[1]) != 2.0:
                continue
            var = self._single_consumer(graph, cons, pw.outputs[0])
            if not last_axis_mean(var):
                continue
            add = self._single_consumer(graph, cons, var.outputs[0])
            if add is None or add.op_type != "Add":
                continue
            eps = self._scalar(graph, add.inputs[1] if add.inputs[0] == var.outputs[0] else add.inputs[0])
            sqrt = self._single_consumer(graph, cons, add.outputs[0])
            if eps is None or eps <= 0 or sqrt is None or sqrt.op_type != "Sqrt":
                continue
            if div.inputs[1] != sqrt.outputs[0] or not only(sqrt.outputs[0], div):
                continue
            mul = self._single_consumer(graph, cons, div.outputs[0])
            if mul is None or mul.op_type != "Mul":
                continue
            gname = mul.inputs[1] if mul.inputs[0] == div.outputs[0] else mul.inputs[0]
            gamma = graph.initializers.get(gname)
            addb = self._single_consumer(graph, cons, mul.outputs[0])
            if gamma is None or gamma.dim() != 1 or addb is None or addb.op_type != "Add":
                continue
            bname = addb.inputs[1] if addb.inputs[0] == mul.outputs[0] else addb.inputs[0]
            beta = graph.initializers.get(bname)
            if beta is None or beta.shape != gamma.shape:
                continue
            dead = [mean, sub, pw, var, add, sqrt, div, mul]
            addb.op_type, addb.domain = "LayerNormalization", ""
            addb.inputs = [x, gname, bname]
            addb.attributes = {"axis": -1, "epsilon": float(eps)}
            graph.remove_nodes([n.id for n in dead])
            return len(dead)
        return 0

    # -------------------------------------------------------------- exact GELU written out with Erf
    @staticmethod
    def _scalar(graph, name):
        t = graph.initializers.get(name)
        return float(t.reshape(-1)[0]) if t is not None and t.numel() == 1 and t.is_floating_point() else None

    def _erf_gelu(self, graph: ModelGraph) -> int:
        cons, prod = graph.consumers(), graph.producers()
        close = lambda v, want: v is not None and abs(v - want) < 1e-3 * abs(want)

        def scaled(node, factor_div, factor_mul):
            """node computes x / factor_div or x * factor_mul with a scalar constant: returns x's name."""
            if node is None or len(node.inputs) != 2:
                return None
            a, b = node.inputs
            if node.op_type == "Div" and close(self._scalar(graph, b), factor_div):
                return a
            if node.op_type == "Mul":
                if close(self._scalar(graph, b), factor_mul):
                    return a
                if close(self._scalar(graph, a), factor_mul):
                    return b
            return None

        def other_input(node, name):
            return node.inputs[1] if node.inputs[0] == name else node.inputs[0]

        for erf in graph.nodes:
            if erf.op_type != "Erf":
                continue
            pre = prod.get(erf.inputs[0])
            x = scaled(pre, math.sqrt(2.0), 1.0 / math.sqrt(2.0))
            if x is None or self._single_consumer(graph, cons, pre.outputs[0]) is not erf:
                continue
            add = self._single_consumer(graph, cons, erf.outputs[0])
            if add is None or add.op_type != "Add" or not close(self._scalar(graph, other_input(add, erf.outputs[0])), 1.0):
                continue
            m1 = self._single_consumer(graph, cons, add.outputs[0])
            if m1 is None or m1.op_type != "Mul":
                continue
            partner = other_input(m1, add.outputs[0])
            dead = [pre, erf, add]
            if partner == x:                                   # (x * (1 + erf)) * 0.5
                m2 = self._single_consumer(graph, cons, m1.outputs[0])
                if m2 is None or m2.op_type != "Mul" or not close(self._scalar(graph, other_input(m2, m1.outputs[0])), 0.5):
                    continue
                last = m2
                dead.append(m1)
            else:                                              # (x * 0.5) * (1 + erf)
                half = prod.get(partner)
                if scaled(half, 2.0, 0.5) != x or self._single_consumer(graph, cons, partner) is not m1:
                    continue
                last = m1
                dead.append(half)
            last.op_type, last.domain = "Gelu", ""
            last.inputs = [x]
            last.attributes = {"approximate": "none"}
            graph.remove_nodes([n.id for n in dead])
            return len(dead)
        return 0

    # -------------------------------------------------------------- Conv + BN
    def _fold_bn(self, graph: ModelGraph) -> int:
        cons = graph.consumers()
        for conv in graph.nodes:
            if conv.op_type not in ("Conv", "FusedConv") or conv.attr("activation") or len(conv.inputs) > 3:
                continue
            bn = self._single_consumer(graph, cons, conv.outputs[0])
            if bn is None or bn.op_type != "BatchNormalization" or bn.inputs[0] != conv.outputs[0]:
                continue
            names = [conv.inputs[1]] + bn.inputs[1:5] + ([conv.inputs[2]] if len(conv.inputs) > 2 and conv.inputs[2] else [])
            if any(n not in graph.initializers for n in names):
                continue
            if len(cons.get(conv.inputs[1], [])) != 1:
                continue                # shared weights: folding would change the other user
            w = graph.initializers[conv.inputs[1]]
            gamma, beta, mean, var = (graph.initializers[n].float() for n in bn.inputs[1:5])
            eps = float(bn.attr("epsilon", 1e-5))
            scale = gamma * torch.rsqrt(var + eps)
            b = graph.initializers[conv.inputs[2]].float() if len(conv.inputs) > 2 and conv.inputs[2] else torch.zeros_like(mean)
            w2 = (w.float() * scale.reshape([-1] + [1] * (w.dim() - 1))).to(w.dtype)
            b2 = ((b - mean) * scale + beta).to(w.dtype)
            wn, bn_name = graph.fresh_name(conv.inputs[1] + "_bnfold"), graph.fresh_name(conv.outputs[0] + "_bias")
            graph.initializers[wn] = w2
            graph.initializers[bn_name] = b2
            conv.inputs = [conv.inputs[0], wn, bn_name]
            conv.outputs = [bn.outputs[0]]
            graph.remove_nodes([bn.id])
            return 1
        return 0

    # -------------------------------------------------------------- Conv (+Add) + Relu
    def _conv_act(self, graph: ModelGraph) -> int:
        cons = graph.consumers()
        prod = graph.producers()
        for conv in graph.nodes:
            if conv.op_type not in ("Conv", "FusedConv") or conv.attr("activation"):
                continue
            nxt = self._single_consumer(graph, cons, conv.outputs[0])
            if nxt is None:
                continue
            if nxt.op_type == "Relu":
                self._to_fused_conv(conv)
                conv.attributes["activation"] = "Relu"
                conv.outputs = [nxt.outputs[0]]
                graph.remove_nodes([nxt.id])
                return 1
            if nxt.op_type == "Add" and len(conv.inputs) <= 3 and len(nxt.inputs) == 2:
                other = nxt.inputs[1] if nxt.inputs[0] == conv.outputs[0] else nxt.inputs[0]
                if other == conv.outputs[0] or other in graph.initializers:
                    continue
                # the residual must already exist when the conv runs
                p = prod.get(other)
                order = {n.id: k for k, n in enumerate(graph.nodes)}
                if p is not None and order[p.id] > order[conv.id]:
                    continue
                self._to_fused_conv(conv)
                ins = list(conv.inputs)
                while len(ins) < 3:
                    ins.append("")
                if not ins[2]:
                    zb = graph.fresh_name(conv.outputs[0] + "_zero_bias")
                    w = graph.initializers.get(ins[1])
                    if w is None:
                        continue
                    graph.initializers[zb] = torch.zeros(w.shape[0], dtype=w.dtype)
                    ins[2] = zb
                conv.inputs = ins + [other]
                conv.outputs = [nxt.outputs[0]]
                graph.remove_nodes([nxt.id])
                return 1
        return 0

    @staticmethod
    def _to_fused_conv(conv: GraphNode):
        if conv.op_type == "Conv":
            conv.op_type = "FusedConv"
            conv.domain = RONN

    # -------------------------------------------------------------- MatMul + Add(bias)
    def _matmul_bias(self, graph: ModelGraph) -> int:
        cons = graph.consumers()
        for mm in graph.nodes:
            if mm.op_type != "MatMul" or mm.inputs[1] not in graph.initializers:
                continue
            if graph.initializers[mm.inputs[1]].dim() != 2:
                continue
            add = self._single_consumer(graph, cons, mm.outputs[0])
            if add is None or add.op_type != "Add":
                continue
            other = add.inputs[1] if add.inputs[0] == mm.outputs[0] else add.inputs[0]
            bias = graph.initializers.get(other)
            n = graph.initializers[mm.inputs[1]].shape[1]
            if bias is None or bias.dim() != 1 or bias.shape[0] != n:
                continue
            mm.op_type, mm.domain = "FusedGemm", RONN
            mm.inputs = [mm.inputs[0], mm.inputs[1], other]
            mm.outputs = [add.outputs[0]]
            graph.remove_nodes([add.id])
            return 1
        return 0

    def _qkv_projection(self, graph: ModelGraph) -> int:
        """Q, K and V projections of one Attention node (three linear layers over the same input) become ONE projection
        with the weights side by side, followed by a Split whose outputs are column slices of the fused result: one
        GEMM instead of three, and the attention kernel can read Q and K in place."""
        cons, prod = graph.consumers(), graph.producers()
        outputs = set(graph.output_names())
        for att in graph.nodes:
            if att.op_type not in ("Attention", "MultiHeadAttention") or len(att.inputs) < 3 or att.attr("fused_qkv"):
                continue
            ps = [prod.get(t) for t in att.inputs[:3]]
            if any(p is None or p.op_type not in ("FusedGemm", "MatMul") for p in ps) or len({p.id for p in ps}) != 3:
                continue
            if len({p.inputs[0] for p in ps}) != 1 or len({p.op_type for p in ps}) != 1:
                continue
            ws = [graph.initializers.get(p.inputs[1]) for p in ps]
            if any(w is None or w.dim() != 2 for w in ws) or len({(w.shape[0], w.dtype) for w in ws}) != 1:
                continue
            if any(p.attr("activation") or int(p.attr("transB", 0)) or len(p.inputs) > 3 for p in ps):
                continue
            if any(len(cons.get(p.outputs[0], [])) != 1 or p.outputs[0] in outputs for p in ps):
                continue
            has_bias = [len(p.inputs) > 2 and bool(p.inputs[2]) for p in ps]
            if any(has_bias) and not all(has_bias):
                continue
            biases = [graph.initializers.get(p.inputs[2]) for p in ps] if all(has_bias) else []
            if any(b is None or b.dim() != 1 for b in biases):
                continue
            base = ps[0].name or f"node_{ps[0].id}"
            wname = graph.fresh_name(base + ".qkv_weight")
            graph.initializers[wname] = torch.cat(ws, dim=1).contiguous()
            inputs = [ps[0].inputs[0], wname]
            if biases:
                bname = graph.fresh_name(base + ".qkv_bias")
                graph.initializers[bname] = torch.cat(biases).contiguous()
                inputs.append(bname)
            fused_out = graph.fresh_name(base + ".qkv")
            sizes = graph.fresh_name(base + ".qkv_sizes")
            graph.initializers[sizes] = torch.tensor([int(w.shape[1]) for w in ws], dtype=torch.int64)
            idx = min(graph.nodes.index(p) for p in ps)
            outs = [p.outputs[0] for p in ps]
            op, dom = (("FusedGemm", RONN) if (biases or ps[0].op_type == "FusedGemm") else ("MatMul", ""))
            graph.remove_nodes([p.id for p in ps])
            graph.add_node(op, inputs, [fused_out], {"transB": 0} if op == "FusedGemm" else {}, name=base + ".qkv", domain=dom,
                           index=idx)
            graph.add_node("Split", [fused_out, sizes], outs, {"axis": -1}, name=base + ".qkv_split", index=idx + 1)
            att.attributes["fused_qkv"] = 1
            return 2
        return 0

    def _skip_layernorm(self, graph: ModelGraph) -> int:
        """Add(x, skip) -> LayerNormalization over the last axis: one node that produces the normalised tensor and, as
        a second output, the sum for whoever else reads it."""
        cons, prod = graph.consumers(), graph.producers()
        for add in graph.nodes:
            if add.op_type != "Add" or len(add.inputs) != 2 or any(i in graph.initializers for i in add.inputs):
                continue
            if add.inputs[0] == add.inputs[1]:
                continue
            users = cons.get(add.outputs[0], [])
            lns = [u for u in users if u.op_type == "LayerNormalization" and u.inputs[0] == add.outputs[0]
                   and int(u.attr("axis", -1)) == -1 and len(u.inputs) >= 2 and len(u.outputs) == 1]
            if len(lns) != 1:
                continue
            ln = lns[0]
            ln.op_type, ln.domain = "SkipLayerNorm", RONN
            ln.inputs = [add.inputs[0], add.inputs[1]] + list(ln.inputs[1:3])
            ln.outputs = [ln.outputs[0], add.outputs[0]]
            ln.attributes = {"epsilon": float(ln.attr("epsilon", 1e-5))}
            graph.remove_nodes([add.id])
            return 1
        return 0

    def _sdpa(self, graph: ModelGraph) -> int:
        """The attention core written in primitives becomes one node.  Matched backwards from a Softmax over the last
        axis: an optional additive mask, an optional scalar scale (division or multiplication, before or after the
        mask), and the score MatMul; forwards: the MatMul with V.  Every intermediate must have exactly one reader."""
        cons, prod = graph.consumers(), graph.producers()
        outputs = set(graph.output_names())

        def shape_readers(name):
            return [u for u in cons.get(name, []) if u.op_type == "Shape" and not u.domain]

        def sole(name, but_shapes=False):
            """One reader; with `but_shapes` (the raw score tensor), Shape nodes beside it do not count: exporters
            expand a masked_fill condition to the scores' shape, and that shape can be had from Q and K^T."""
            if name in outputs:
                return False
            users = cons.get(name, [])
            if but_shapes:
                users = [u for u in users if u.op_type != "Shape" or u.domain]
            return len(users) == 1

        def is_scores(name, allow_fill=False):
            """`name` is a MatMul of two non-constant tensors, possibly under one scalar Div / Mul (and, with
            `allow_fill`, under a Where that fills masked scores with a constant)."""
            for _ in range(3):
                n = prod.get(name)
                if n is None or not sole(name, but_shapes=n.op_type == "MatMul"):
                    return False
                if allow_fill and n.op_type == "Where" and len(n.inputs) == 3:
                    allow_fill = False
                    if self._scalar(graph, n.inputs[1]) is not None:
                        name = n.inputs[2]
                    elif self._scalar(graph, n.inputs[2]) is not None:
                        name = n.inputs[1]
                    else:
                        return False
                    continue
                if len(n.inputs) != 2:
                    return False
                if n.op_type == "MatMul":
                    return not any(t in graph.initializers for t in n.inputs)
                if n.op_type not in ("Div", "Mul"):
                    return False
                if self._scalar(graph, n.inputs[1]) is not None:
                    name = n.inputs[0]
                elif n.op_type == "Mul" and self._scalar(graph, n.inputs[0]) is not None:
                    name = n.inputs[1]
                else:
                    return False
            return False

        for sm in graph.nodes:
            if sm.op_type != "Softmax" or sm.domain or sm.attr("legacy_flatten") or int(sm.attr("axis", -1)) != -1:
                continue
            pv = self._single_consumer(graph, cons, sm.outputs[0])
            if pv is None or pv.op_type != "MatMul" or pv.inputs[0] != sm.outputs[0] or pv.inputs[1] in graph.initializers:
                continue
            # walking back from the Softmax: [Add mask] then [scalar scale] then the score MatMul.  (A scale that sits
            # between the mask and the Softmax would scale the mask too: not this pattern.)
            chain, cur, scale, mask, qk = [sm], sm.inputs[0], 1.0, None, None
            fill = None                                    # (condition tensor, value, fill where the condition is true?)
            stage = 0                                      # 0: mask, fill, scale or MatMul may follow; 1: fill, scale or
            while True:                                    # MatMul; 2: scale or MatMul; 3: MatMul
                n = prod.get(cur)
                if n is None or not sole(cur, but_shapes=n.op_type == "MatMul"):
                    break
                if n.op_type == "Where" and len(n.inputs) == 3 and stage <= 1:
                    # masked_fill as exporters write it: Where(cond, value, scores) or Where(cond, scores, value)
                    v1, v2 = self._scalar(graph, n.inputs[1]), self._scalar(graph, n.inputs[2])
                    if v1 is not None and is_scores(n.inputs[2]):
                        fill, cur = (n.inputs[0], v1, 1), n.inputs[2]
                    elif v2 is not None and is_scores(n.inputs[1]):
                        fill, cur = (n.inputs[0], v2, 0), n.inputs[1]
                    else:
                        break
                    stage = 2
                    chain.append(n)
                    continue
                if len(n.inputs) != 2:
                    break
                if n.op_type == "MatMul":
                    qk = n
                    break
                if n.op_type == "Add" and stage == 0:
                    sides = [k for k in (0, 1) if is_scores(n.inputs[k], allow_fill=True)]
                    if len(sides) != 1:
                        break
                    mask, cur, stage = n.inputs[1 - sides[0]], n.inputs[sides[0]], 1
                    chain.append(n)
                    continue
                if n.op_type in ("Div", "Mul") and stage <= 2:
                    c0, c1 = self._scalar(graph, n.inputs[0]), self._scalar(graph, n.inputs[1])
                    if c1 is not None and c1 != 0.0:
                        scale, cur = ((1.0 / c1) if n.op_type == "Div" else c1), n.inputs[0]
                    elif c0 is not None and n.op_type == "Mul":
                        scale, cur = c0, n.inputs[1]
                    else:
                        break
                    stage = 3
                    chain.append(n)
                    continue
                break
            if qk is None:
                continue
            if any(t in graph.initializers for t in qk.inputs):
                continue
            ins = [qk.inputs[0], qk.inputs[1], pv.inputs[1]] + ([mask] if mask is not None else ([""] if fill else []))
            attrs = {"scale": float(scale), "k_transposed": 1}
            if fill:
                ins.append(fill[0])
                attrs["fill_value"], attrs["fill_when"] = float(fill[1]), int(fill[2])
            idx = graph.nodes.index(pv)
            name = (sm.name or f"node_{sm.id}") + ".sdpa"
            out = pv.outputs[0]
            # Shape(scores) readers: shape(Q)[:-1] ++ shape(K^T)[-1:] is the same vector without the scores
            for k, sh in enumerate(shape_readers(qk.outputs[0])):
                lo, hi = int(sh.attr("start", 0)), sh.attr("end")
                if lo != 0 or hi is not None:
                    continue                               # a partial shape: left reading the (still produced) scores
                a_name, b_name = graph.fresh_name(f"{name}.shape_q{k}"), graph.fresh_name(f"{name}.shape_k{k}")
                at = graph.nodes.index(sh)
                res = sh.outputs[0]
                graph.remove_nodes([sh.id])
                graph.add_node("Shape", [qk.inputs[0]], [a_name], {"start": 0, "end": -1}, name=a_name, index=at)
                graph.add_node("Shape", [qk.inputs[1]], [b_name], {"start": -1}, name=b_name, index=at + 1)
                graph.add_node("Concat", [a_name, b_name], [res], {"axis": 0}, name=graph.fresh_name(f"{name}.shape{k}"),
                               index=at + 2)
            if any(u.op_type == "Shape" for u in graph.consumers().get(qk.outputs[0], [])):
                continue                                   # a reader of the scores is left: they must stay
            idx = graph.nodes.index(pv)
            graph.remove_nodes([n.id for n in chain] + [qk.id, pv.id])
            idx = min(idx, len(graph.nodes))
            graph.add_node("ScaledDotProductAttention", ins, [out], attrs, name=name,
                           domain=RONN, index=idx)
            graph.sort_in_place()
            return len(chain) + 1
        return 0

    def _gemm_act(self, graph: ModelGraph) -> int:
        cons = graph.consumers()
        for g in graph.nodes:
            if g.op_type not in ("Gemm", "FusedGemm") or g.attr("activation") or len(g.inputs) > 3:
                continue
            if g.op_type == "Gemm" and (int(g.attr("transA", 0)) or float(g.attr("alpha", 1.0)) != 1.0
                                        or float(g.attr("beta", 1.0)) != 1.0):
                continue
            act = self._single_consumer(graph, cons, g.outputs[0])
            if act is None or act.op_type not in ("Relu", "Gelu"):
                continue
            if act.op_type == "Gelu" and act.attr("approximate", "none") != "tanh":
                continue
            g.op_type, g.domain = "FusedGemm", RONN
            g.attributes = {"transB": int(g.attr("transB", 0)), "activation": act.op_type}
            g.outputs = [act.outputs[0]]
            graph.remove_nodes([act.id])
            return 1
        return 0

    def _gemm_residual(self, graph: ModelGraph) -> int:
        cons = graph.consumers()
        prod = graph.producers()
        order = {n.id: k for k, n in enumerate(graph.nodes)}
        for g in graph.nodes:
            if g.op_type != "FusedGemm" or len(g.inputs) != 3 or not g.inputs[2]:
                continue
            add = self._single_consumer(graph, cons, g.outputs[0])
            if add is None or add.op_type != "Add" or len(add.inputs) != 2:
                continue
            other = add.inputs[1] if add.inputs[0] == g.outputs[0] else add.inputs[0]
            if other == g.outputs[0] or other in graph.initializers:
                continue
            p = prod.get(other)
            if p is not None and order[p.id] > order[g.id]:
                continue
            g.inputs = g.inputs + [other]
            g.outputs = [add.outputs[0]]
            graph.remove_nodes([add.id])
            return 1
        return 0
