"""Decode-step time of the installed vLLM on the shapes of ``utils/microbench.py decode`` (library baseline).

    python baseline/vllm_decode_bench.py --model qwen2.5-1.5b --shapes "16,2048;64,2048;128,2048;256,1024"

The engine is created with the reference's arguments (vllm_worker.py:219-232: bf16, prefix caching on, CUDA graphs unless
``--eager``) on a random-init model directory of the named architecture. For every (batch, context) pair ``batch``
requests with ``context`` random prompt tokens are added, the engine is stepped until every request has produced its
first token (prefill done), and then ``--steps`` further engine steps are timed with the host clock around
``torch.cuda.synchronize()`` (each step ends with the sampled tokens on the host, so the host clock sees the device time
of the step plus vLLM's own scheduling). One JSON line per shape. Nothing of ``async_grpo_nccl_b200`` is imported.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--shapes", default="16,2048;64,2048;128,2048;256,1024")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--max-num-seqs", type=int, default=512)
    args = ap.parse_args()

    import numpy as np
    import torch
    from ref_workload import ARCHS, build_model_dir
    from vllm import LLM, SamplingParams, TokensPrompt

    arch = ARCHS[args.model]
    model_dir = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"agrpo_vllm_bench_{args.model}")
    build_model_dir(model_dir, args.model, seed=0)
    kw = dict(model=model_dir, tensor_parallel_size=1, gpu_memory_utilization=0.90, dtype="bfloat16", enable_prefix_caching=True,
              max_num_seqs=args.max_num_seqs, max_model_len=32768, load_format="auto", disable_custom_all_reduce=True,
              disable_log_stats=True, trust_remote_code=True, seed=0)
    if args.eager:
        kw["enforce_eager"] = True
    llm = LLM(**kw)
    engine = llm.llm_engine
    rng = np.random.default_rng(0)
    vocab = int(arch["vocab_size"])
    req = 0
    for shape in args.shapes.split(";"):
        batch, context = (int(x) for x in shape.split(","))
        total = args.steps + 16
        for _ in range(batch):
            ids = [int(t) for t in rng.integers(2, vocab, context)]
            sp = SamplingParams(n=1, temperature=1.0, seed=req, max_tokens=total, min_tokens=total, ignore_eos=True, detokenize=False)
            engine.add_request(f"r{req}", TokensPrompt(prompt_token_ids=ids), sp)
            req += 1
        produced = {}
        # prefill (possibly chunked over several engine steps): until every request has produced at least 4 tokens
        while len(produced) < batch or min(produced.values()) < 4:
            for o in engine.step():
                produced[o.request_id] = len(o.outputs[0].token_ids)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            engine.step()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1000.0 / args.steps
        while engine.has_unfinished_requests():
            engine.step()
        print(json.dumps({"bench": "vllm_decode_step", "model": args.model, "batch": batch, "context": context,
                          "graph": not args.eager, "ms_per_step": ms, "tokens_per_s": batch / ms * 1e3}), flush=True)


if __name__ == "__main__":
    main()
