"""Engine configuration (docs/new/RONN-Continuous-Batching-Branch-Prompt.md:156-255:
max_batch_size, max_batch_tokens, prefill_chunk_size; KV block size 16 from
docs/new/RONN-KV-Cache-Compression-Branch-Prompt.md:125-195)."""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass
class EngineConfig:
    block_size: int = 16
    num_blocks: int = 0                 # 0 = size from gpu_memory_utilization / max_num_seqs * max_model_len
    max_num_seqs: int = 256
    max_batch_tokens: int = 8192
    max_model_len: int = 1024
    prefill_chunk: int = 0              # 0 = whole prompts
    policy: str = "fcfs"                # "fcfs" | "priority"
    enable_prefix_cache: bool = False
    preemption: str = "recompute"       # "recompute" | "swap" | "auto": what a preempted sequence does with its KV blocks
    num_cpu_blocks: int = 0             # host (pinned) block pool for "swap" / "auto"; 0 = as many as device blocks
    swap_min_tokens: int = 64           # "auto": sequences with fewer cached tokens are recomputed instead
    eos_token_id: int = -1              # -1 = never stop on a token
    use_cuda_graph: bool = True
    dtype: str = "bf16"
    tp_size: int = 1
    backend: str = "kernels"            # "kernels" (hand-written sm_100a) | "torch" (library baseline / CPU)
    tp_comm: str = "fused"              # "fused" (in-kernel NVLink) | "nccl" (library collectives baseline)
    gpu_memory_utilization: float = 0.85
    cluster_norm: bool = False          # TP=1, >= 1024 rows: projection + residual + next norm as one cluster kernel
                                        # (measured slower than GEMM + norm kernel at every size tried; kept optional)
    dense_prefill: bool = True          # whole-prompt prefill steps use the tensor-core attention kernel
    decode_streams: int = 1             # >1: decode batches >= 2*decode_split_min rows run as this many concurrent parts
    decode_split_min: int = 64          # (one stream each, inside the step's CUDA graph): the bandwidth-bound
                                        # attention of one overlaps the latency-bound GEMM chain of the others

    def __post_init__(self):
        if self.block_size != 16:
            raise ValueError("the paged attention kernels are built for 16-token blocks")
        for k in ("max_num_seqs", "max_batch_tokens", "max_model_len", "decode_streams", "cluster_norm"):
            env = os.environ.get("RONN_" + k.upper())
            if env:
                setattr(self, k, int(env))
