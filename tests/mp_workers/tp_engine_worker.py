"""Child process of the tensor-parallel tests: runs the serving engine at the launched world size and
compares its greedy tokens with a single-rank engine built from the same seeded model."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from ronn_b200.api.model import Model  # noqa: E402
from ronn_b200.models.gpt2 import GPT2Config, build_gpt2  # noqa: E402
from ronn_b200.parallel import make_comm  # noqa: E402
from ronn_b200.parallel.group import init_distributed  # noqa: E402
from ronn_b200.serving import EngineConfig, LLMEngine, SamplingParams  # noqa: E402


def main():
    mode = sys.argv[1]            # "cpu" | "nccl" | "fused"
    out_path = sys.argv[2]
    rank, world, local = init_distributed("gloo" if mode == "cpu" else "nccl", timeout_s=120)
    if mode == "cpu":
        dev, dtype, backend = torch.device("cpu"), torch.float32, "torch"
    else:
        dev, dtype, backend = torch.device("cuda", local), torch.bfloat16, "kernels"
    if os.environ.get("RONN_TEST_MODEL") == "bitnet":
        # ternary decoder whose FFN shard (352 / world) is not a multiple of 64: the shards are widened with zero weights
        from ronn_b200.models.bitnet_llama import BitNetConfig, build_bitnet_llama
        bcfg = BitNetConfig.tiny(n_layer=2, hidden=256, n_head=4, ffn=352, vocab_size=1000, max_pos=256)
        model = Model.from_graph(build_bitnet_llama(bcfg, dtype=dtype, seed=7, with_lm_head=False))
    else:
        cfg = GPT2Config.tiny(n_layer=2, n_embd=512, n_head=8, vocab_size=1000, n_positions=256)  # 8 heads: shards up to TP=8
        model = Model.from_graph(build_gpt2(cfg, dtype=dtype, seed=7))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 17, 40, 64, 9, 33)]

    # optional: the tensor-parallel run gets a cache too small for all sequences and swaps preempted ones to the host
    tight = os.environ.get("RONN_TEST_TIGHT_BLOCKS")
    stats = {}
    new_tokens = 8
    if tight:
        prompts = [[3 + i] * 15 for i in range(4)]       # one block each at admission, three each by the end
        new_tokens = 30

    def run(comm, tp_comm):
        extra = {}
        if comm is not None and tight:
            extra = dict(num_blocks=int(tight), preemption="swap", num_cpu_blocks=32)
        ecfg = EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=256,
                            dtype="fp32" if mode == "cpu" else "bf16", backend=backend, tp_size=world if comm else 1,
                            tp_comm=tp_comm, use_cuda_graph=(mode != "cpu"), **{"num_blocks": 64, **extra})
        eng = LLMEngine(model, ecfg, device=dev, comm=comm)
        toks = eng.generate(prompts, SamplingParams(max_new_tokens=new_tokens))
        if comm is not None:
            stats.update(eng.stats())
        return toks

    comm = make_comm("nccl" if mode in ("cpu", "nccl") else "fused", dev)
    tp = run(comm, "nccl" if mode != "fused" else "fused")
    single = run(None, "nccl")
    if mode == "fused":
        comm.check()
    # non-greedy requests (one with its own seed, the others without): the vocabulary shards of the logits are gathered
    # and every rank must draw the same tokens
    sampled_same, sampled_ok = True, True
    if not tight:
        ecfg = EngineConfig(max_num_seqs=8, max_batch_tokens=256, max_model_len=256, dtype="fp32" if mode == "cpu" else "bf16",
                            backend=backend, tp_size=world, tp_comm="nccl" if mode != "fused" else "fused",
                            use_cuda_graph=(mode != "cpu"), num_blocks=64)
        eng = LLMEngine(model, ecfg, device=dev, comm=comm)
        ids = [eng.add_request(pr, SamplingParams(max_new_tokens=6, temperature=0.9, top_k=40, top_p=0.9,
                                                  repeat_penalty=1.1, seed=(11 if k == 0 else None)))
               for k, pr in enumerate(prompts[:4])]
        while eng.has_unfinished():
            eng.step()
        drawn = [eng.requests[i].output_tokens for i in ids]
        allr = [None] * world
        torch.distributed.all_gather_object(allr, drawn)
        sampled_same = all(a == allr[0] for a in allr)
        sampled_ok = all(len(t) == 6 and all(0 <= x < 1000 for x in t) for t in drawn)
    agree = sum(a == b for x, y in zip(tp, single) for a, b in zip(x, y))
    total = sum(len(x) for x in single)
    # every rank must have produced the same tokens (the schedulers run replicated)
    gathered = [None] * world
    torch.distributed.all_gather_object(gathered, tp)
    same_across_ranks = all(g_ == gathered[0] for g_ in gathered)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"agree": agree, "total": total, "same_across_ranks": same_across_ranks, "world": world,
                       "sampled_same_across_ranks": sampled_same, "sampled_in_range": sampled_ok,
                       "fused_calls": getattr(comm, "fused_calls", 0),
                       "swap_preemptions": stats.get("swap_preemptions", 0),
                       "swapped_in_blocks": stats.get("swapped_in_blocks", 0)}, f)
    torch.distributed.barrier()
    if mode != "cpu":
        torch.cuda.synchronize()
        os._exit(0)
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
