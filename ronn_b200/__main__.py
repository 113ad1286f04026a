"""``python -m ronn_b200 <command>`` - command line of the runtime.

    info MODEL.onnx                      inputs, outputs, metadata, operator histogram
    run MODEL.onnx [--level O2] [--provider cpu|gpu|bitnet] [--repeat N]
                                         run the model on random inputs of its declared shapes; shapes and timing
    optimize IN.onnx OUT.onnx [--level O3]
                                         run the graph passes offline and save the rewritten model
    serve ...                            the serving front end (same arguments as ``python -m ronn_b200.serve``)

The reference's command line is the serving one (``ronn serve --model ... --max-batch-size ...``,
docs/new/RONN-Continuous-Batching-Branch-Prompt.md:420-438); the other commands wrap the public API
(crates/ronn-api/src/lib.rs: Model::load, create_session, run) for use from a shell.
"""
from __future__ import annotations

import argparse
import collections
import copy
import json
import sys
import time


def _random_feeds(model):
    import torch
    from .core.types import DataType
    feeds = {}
    for t in model.inputs():
        shape = [int(d) if int(d) > 0 else 1 for d in t.shape]          # symbolic / unknown dimensions run as 1
        if t.data_type in (DataType.F32, DataType.F16, DataType.BF16, DataType.F64):
            feeds[t.name] = torch.rand(shape).to(t.data_type.torch)
        elif t.data_type == DataType.BOOL:
            feeds[t.name] = torch.ones(shape, dtype=torch.bool)
        else:
            feeds[t.name] = torch.zeros(shape, dtype=t.data_type.torch)       # token ids, masks, indices
    return feeds


def cmd_info(a) -> int:
    from . import Model
    m = Model.load(a.model)
    ops = collections.Counter(n.op_type for n in m.graph.nodes)
    print(json.dumps({"inputs": [{"name": t.name, "shape": list(t.shape), "dtype": t.data_type.value} for t in m.inputs()],
                      "outputs": [{"name": t.name, "shape": list(t.shape), "dtype": t.data_type.value} for t in m.outputs()],
                      "metadata": {k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(v))
                                   for k, v in m.metadata().items()},
                      "operators": dict(ops.most_common())}, indent=1))
    return 0


def cmd_run(a) -> int:
    from . import Model, SessionOptions
    m = Model.load(a.model)
    sess = m.create_session(SessionOptions().with_optimization_level(a.level).with_provider(a.provider))
    feeds = _random_feeds(m)
    out = sess.run(feeds)
    t0 = time.perf_counter()
    for _ in range(a.repeat):
        out = sess.run(feeds)
    ms = (time.perf_counter() - t0) * 1e3 / max(a.repeat, 1)
    print(json.dumps({"outputs": {k: {"shape": list(v.shape), "dtype": str(v.dtype).replace("torch.", "")}
                                  for k, v in out.items()},
                      "ms_per_run": round(ms, 4) if a.repeat else None, "level": a.level, "provider": a.provider}))
    return 0


def cmd_optimize(a) -> int:
    from . import Model
    from .graph.optimizer import Optimizer
    m = Model.load(a.model)
    graph = copy.deepcopy(m.graph)
    before = len(graph.nodes)
    opt = Optimizer(a.level)
    stats = opt.optimize(graph)
    Model.from_graph(graph).save(a.out)
    print(json.dumps({"passes": opt.pass_names(), "nodes_before": before, "nodes_after": len(graph.nodes),
                      "nodes_removed": stats.nodes_removed, "nodes_fused": stats.nodes_fused,
                      "nodes_modified": stats.nodes_modified, "iterations": stats.iterations, "saved": a.out}))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "serve":
        from . import serve
        sys.argv = ["ronn_b200.serve"] + argv[1:]
        serve.main()
        return 0
    ap = argparse.ArgumentParser(prog="ronn_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("info")
    p.add_argument("model")
    p = sub.add_parser("run")
    p.add_argument("model")
    p.add_argument("--level", default="O2")
    p.add_argument("--provider", default="cpu")
    p.add_argument("--repeat", type=int, default=10)
    p = sub.add_parser("optimize")
    p.add_argument("model")
    p.add_argument("out")
    p.add_argument("--level", default="O3")
    sub.add_parser("serve", add_help=False)
    a = ap.parse_args(argv)
    return {"info": cmd_info, "run": cmd_run, "optimize": cmd_optimize}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
