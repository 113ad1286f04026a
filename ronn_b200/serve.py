"""``python -m ronn_b200.serve --model MODEL.onnx [--max-batch-size 256] [--port 8000]`` - serve a decoder model.

Command line of the continuous-batching design (``ronn serve --model ... --max-batch-size ...``,
docs/new/RONN-Continuous-Batching-Branch-Prompt.md:420-438).  ``--synthetic gpt2-medium|gpt2-tiny|bitnet-tiny`` serves
a random-init model instead of a file."""
from __future__ import annotations

import argparse


def main():
    ap = argparse.ArgumentParser(prog="ronn_b200.serve")
    ap.add_argument("--model")
    ap.add_argument("--synthetic", choices=["gpt2-medium", "gpt2-tiny", "bitnet-tiny"])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-batch-size", type=int, default=256)
    ap.add_argument("--max-batch-tokens", type=int, default=8192)
    ap.add_argument("--max-model-len", type=int, default=1024)
    ap.add_argument("--prefill-chunk", type=int, default=0)
    ap.add_argument("--policy", default="fcfs", choices=["fcfs", "priority"])
    ap.add_argument("--prefix-cache", action="store_true")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--tokenizer", default="bytes",
                    help="'bytes' (UTF-8 bytes as ids), a SentencePiece .model file, or 'none' (token-id endpoints only)")
    a = ap.parse_args()
    import torch
    import uvicorn
    from . import Model
    from .serving import EngineConfig, LLMEngine
    from .serving.server import create_app
    if a.synthetic:
        if a.synthetic.startswith("gpt2"):
            from .models.gpt2 import GPT2Config, build_gpt2
            cfg = GPT2Config.medium() if a.synthetic == "gpt2-medium" else GPT2Config.tiny()
            model = Model.from_graph(build_gpt2(cfg, dtype=torch.bfloat16))
        else:
            from .models.bitnet_llama import BitNetConfig, build_bitnet_llama
            model = Model.from_graph(build_bitnet_llama(BitNetConfig.tiny(), dtype=torch.bfloat16))
    elif a.model:
        model = Model.load(a.model)
    else:
        ap.error("--model or --synthetic is required")
    engine = LLMEngine(model, EngineConfig(max_num_seqs=a.max_batch_size, max_batch_tokens=a.max_batch_tokens,
                                           max_model_len=a.max_model_len, prefill_chunk=a.prefill_chunk, policy=a.policy,
                                           enable_prefix_cache=a.prefix_cache, dtype=a.dtype))
    from .serving.tokenizer import load_tokenizer
    tok = None if a.tokenizer == "none" else load_tokenizer(a.tokenizer, engine.arch.vocab)
    uvicorn.run(create_app(engine, tok), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
