"""Datasets: JSONL rows in the reference's format and synthetic prompt generators.

A dataset row carries ``input_token_ids`` (final prompt ids, chat template already applied), ``input``
(the decoded prompt, needed by text reward adapters), ``answer`` and optional task fields (``nums``,
``target``, ``end_token``, ``reward``) (Readme.md:209-213, sample-data/create_count_down.py:23-36).
The synthetic generators produce the random-token workloads of the benchmark configurations.
"""
from __future__ import annotations

import json
import math
from typing import Any, Dict, Iterable, List, Optional, Sequence

import numpy as np


def write_jsonl(path: str, rows: Iterable[Dict[str, Any]]) -> None:
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            r = {k: (v.tolist() if isinstance(v, np.ndarray) else v) for k, v in r.items()}
            f.write(json.dumps(r) + "\n")


def synthetic_prompt_rows(num_prompts: int, vocab_size: int, min_len: int, max_len: int, seed: int = 0,
                          samples_per_question: Optional[int] = None, gen_len_range: Optional[Sequence[int]] = None,
                          gen_len_dist: str = "loguniform", reward_p: Optional[float] = None) -> List[Dict[str, Any]]:
    """Uniform-random token prompts with length uniform in [min_len, max_len].

    With ``gen_len_range`` every row also gets ``forced_output_lens`` (one drawn length per sample; the
    engine forces EOS there), so that a random-init model produces a controlled length distribution.
    """
    rng = np.random.default_rng(seed)
    rows = []
    for i in range(num_prompts):
        L = int(rng.integers(min_len, max_len + 1))
        ids = rng.integers(0, vocab_size, L, dtype=np.int64).astype(np.int32)
        row: Dict[str, Any] = {"input_token_ids": ids, "input": "", "answer": "", "__uid__": i}
        if gen_len_range is not None and samples_per_question:
            lo, hi = int(gen_len_range[0]), int(gen_len_range[1])
            if gen_len_dist == "loguniform":
                lens = np.exp(rng.uniform(math.log(lo), math.log(hi), samples_per_question))
            else:
                lens = rng.uniform(lo, hi, samples_per_question)
            row["forced_output_lens"] = [int(max(1, round(float(x)))) for x in lens]
        if reward_p is not None:
            row["reward_p"] = float(reward_p)
        rows.append(row)
    return rows


def countdown_rows(num: int, tokenizer: Any, seed: int = 0, n_numbers: int = 4, max_number: int = 99) -> List[Dict[str, Any]]:
    """Countdown task rows (what the reference's sample-data/create_count_down.py prepares): reach ``target``
    from ``nums`` with + - * /; the prompt ends inside an opened <think> block."""
    rng = np.random.default_rng(seed)
    rows = []
    for i in range(num):
        nums = [int(x) for x in rng.integers(1, max_number + 1, n_numbers)]
        target = int(rng.integers(10, 1000))
        user = (f"Using the numbers {nums}, create an equation that equals {target}. You can use basic arithmetic operations "
                f"(+, -, *, /) and each number can only be used once. Show your work in <think> </think> tags. "
                f"And return the final answer in <answer> </answer> tags, for example <answer> (1 + 2) / 3 </answer>.")
        msgs = [{"role": "system", "content": "You are a helpful assistant. You first think about the reasoning process "
                                              "in your mind and then provide the user with the answer."},
                {"role": "user", "content": user}]
        text = tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True) + "Let me solve this step by step.\n<think>"
        ids = tokenizer.encode(text, add_special_tokens=False)
        rows.append({"input": text, "input_token_ids": ids, "answer": str(target), "nums": nums, "target": target,
                     "end_token": tokenizer.eos_token})
    return rows


MATH_SYSTEM_PROMPT = r"Let's think step by step and output the final answer within \boxed{}."


def math_rows(records: Iterable[Dict[str, Any]], tokenizer: Any, system_prompt: Optional[str] = None,
              skip_indices: Sequence[int] = (), check_round_trip: bool = True) -> List[Dict[str, Any]]:
    """Math-problem rows (what the reference's process_deepscaler.py prepares from the DeepScaleR dump): every record
    has ``problem`` and ``answer`` (``solution`` is carried along when present). The prompt is the chat template applied
    to the problem with the generation prompt appended, tokenised without extra special tokens; records whose ids do
    not decode back to the prompt text are dropped when ``check_round_trip`` is set (the reference's error filter)."""
    skip = set(int(i) for i in skip_indices)
    rows = []
    for i, rec in enumerate(records):
        if i in skip:
            continue
        msgs = []
        if system_prompt:
            msgs.append({"role": "system", "content": system_prompt})
        msgs.append({"role": "user", "content": rec["problem"]})
        text = tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
        ids = list(tokenizer.encode(text, add_special_tokens=False))
        if check_round_trip and tokenizer.decode(ids) != text:
            continue
        row = {"input": text, "input_token_ids": ids, "answer": str(rec["answer"])}
        if "solution" in rec:
            row["solution"] = rec["solution"]
        rows.append(row)
    return rows


def load_jsonl_or_json(path: str) -> List[Dict[str, Any]]:
    with open(path) as f:
        head = f.read(1)
        f.seek(0)
        if head == "[":
            return list(json.load(f))
        return [json.loads(line) for line in f if line.strip()]


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``python -m async_grpo_nccl_b200.data countdown|math|synthetic ...`` writes a training JSONL file."""
    import argparse

    ap = argparse.ArgumentParser(prog="data", description="prepare JSONL datasets in the training format")
    sub = ap.add_subparsers(dest="task", required=True)
    c = sub.add_parser("countdown", help="countdown arithmetic task")
    c.add_argument("--tokenizer", required=True)
    c.add_argument("--num", type=int, default=10000)
    c.add_argument("--seed", type=int, default=0)
    c.add_argument("--out", required=True)
    m = sub.add_parser("math", help="math problems with boxed answers (DeepScaleR-style dump)")
    m.add_argument("--input", required=True, help="JSON list or JSONL with problem / answer / solution")
    m.add_argument("--tokenizer", required=True)
    m.add_argument("--system-prompt", default=None)
    m.add_argument("--skip", type=int, nargs="*", default=[], help="record indices to drop")
    m.add_argument("--out", required=True)
    s = sub.add_parser("synthetic", help="random-token prompts with drawn generation lengths (benchmark workload)")
    s.add_argument("--num", type=int, default=1024)
    s.add_argument("--vocab-size", type=int, default=151936)
    s.add_argument("--prompt-min", type=int, default=64)
    s.add_argument("--prompt-max", type=int, default=512)
    s.add_argument("--samples-per-question", type=int, default=8)
    s.add_argument("--gen-min", type=int, default=256)
    s.add_argument("--gen-max", type=int, default=8192)
    s.add_argument("--reward-p", type=float, default=0.3)
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    if args.task == "synthetic":
        rows = synthetic_prompt_rows(args.num, args.vocab_size, args.prompt_min, args.prompt_max, seed=args.seed,
                                     samples_per_question=args.samples_per_question, gen_len_range=(args.gen_min, args.gen_max),
                                     reward_p=args.reward_p)
        rows = [{**r, "input_token_ids": [int(t) for t in r["input_token_ids"]]} for r in rows]
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
        if args.task == "countdown":
            rows = countdown_rows(args.num, tok, seed=args.seed)
        else:
            rows = math_rows(load_jsonl_or_json(args.input), tok, system_prompt=args.system_prompt, skip_indices=args.skip)
    write_jsonl(args.out, rows)
    print(f"wrote {len(rows)} rows to {args.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
