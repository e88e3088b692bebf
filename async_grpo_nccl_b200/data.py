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
