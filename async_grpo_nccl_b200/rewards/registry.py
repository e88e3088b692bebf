"""Pluggable reward adapters ``sample -> {"reward": float, ...}``.

Same registry surface as the reference (reward_registry.py:104-176): ``RewardType`` with
mathd / sympy / countdown / base / gsm8k, ``REWARD_ADAPTERS`` and ``get_reward_adapter``. Two synthetic
adapters are added for benchmarking and for the CPU plumbing configuration: ``bernoulli`` (reward 1 with
probability p, seeded by a hash of the prompt and the sample index) and ``token_match`` (reward 1 if any
generated token equals the sum of the prompt ids modulo the vocabulary size).
"""
from __future__ import annotations

import hashlib
import re
from enum import Enum
from typing import Any, Callable, Dict

import numpy as np

from .countdown import answer_score, format_score
from .math_grading import extract_answer, grade_answer_mathd, grade_answer_sympy


class RewardType(str, Enum):
    MATHD = "mathd"
    SYMPY = "sympy"
    COUNTDOWN = "countdown"
    BASE = "base"
    GSM8K = "gsm8k"
    BERNOULLI = "bernoulli"
    TOKEN_MATCH = "token_match"


def completion_text(sample: Dict[str, Any]) -> str:
    """Generated text = sample_text with the prompt split off (reward_registry.py:23-24, 68-70)."""
    full = sample.get("sample_text", "") or ""
    prompt = sample.get("input", "") or ""
    if prompt and prompt in full:
        return full.split(prompt, 1)[1]
    return full


def _attempt_and_truth(sample: Dict[str, Any]):
    answer = sample.get("answer", "")
    truth = extract_answer(answer) if isinstance(answer, str) and "\\boxed" in answer else answer
    try:
        attempt = extract_answer(completion_text(sample)) or ""
    except Exception:
        attempt = ""
    sample["parsed_gt_answer"] = truth
    sample["parsed_attempt"] = attempt
    return attempt, (str(truth) if truth is not None else None)


def mathd_adapter(sample: Dict[str, Any], **_: Any) -> Dict[str, Any]:
    attempt, truth = _attempt_and_truth(sample)
    return {"reward": float(grade_answer_mathd(attempt, truth))}


def sympy_adapter(sample: Dict[str, Any], **_: Any) -> Dict[str, Any]:
    attempt, truth = _attempt_and_truth(sample)
    return {"reward": float(grade_answer_sympy(attempt, truth))}


def countdown_adapter(sample: Dict[str, Any], **_: Any) -> Dict[str, Any]:
    response = "<think>" + completion_text(sample)
    f = format_score(response, end_token=sample.get("end_token", ""))
    a = answer_score(response, numbers=sample.get("nums"), target=sample.get("target"))
    return {"reward": 0.1 * f + a, "format_reward": f}


def base_adapter(sample: Dict[str, Any], **_: Any) -> Dict[str, Any]:
    if "reward" not in sample:
        raise ValueError("sample does not contain a 'reward' key")
    return {"reward": float(sample["reward"])}


_FINAL = re.compile(r"<final_answer>\s*([^<]+?)\s*</final_answer>", re.IGNORECASE)


def gsm8k_adapter(sample: Dict[str, Any], **_: Any) -> Dict[str, Any]:
    full = sample.get("sample_text", "") or ""
    prompt = sample.get("input", "") or ""
    completion = full[len(prompt):] if prompt and full.startswith(prompt) else full
    m = _FINAL.search(completion)
    pred = m.group(1).strip() if m else ""
    truth = str(sample.get("answer", "")).strip()
    norm = lambda s: s.replace(",", "").strip()
    return {"reward": float(norm(pred) == norm(truth))}


def bernoulli_adapter(sample: Dict[str, Any], p: float = 0.3, **_: Any) -> Dict[str, Any]:
    ids = np.asarray(sample.get("input_token_ids", sample.get("sample_ids", [])), dtype=np.int64)
    n_in = int(sample.get("input_len", len(ids)))
    h = hashlib.sha256(ids[:n_in].tobytes())
    h.update(np.asarray(sample.get("output_token_ids", []), dtype=np.int64)[:8].tobytes())
    h.update(str(sample.get("sample_index", 0)).encode())
    u = int.from_bytes(h.digest()[:8], "little") / float(1 << 64)
    return {"reward": float(u < float(sample.get("reward_p", p)))}


def token_match_adapter(sample: Dict[str, Any], vocab_size: int = 1024, **_: Any) -> Dict[str, Any]:
    ids = np.asarray(sample.get("sample_ids", []), dtype=np.int64)
    n_in = int(sample.get("input_len", 0))
    v = int(sample.get("vocab_size", vocab_size))
    target = int(ids[:n_in].sum() % v)
    out = np.asarray(sample.get("output_token_ids", ids[n_in:]), dtype=np.int64)
    return {"reward": float(bool((out == target).any()))}


REWARD_ADAPTERS: Dict[RewardType, Callable[..., Dict[str, Any]]] = {
    RewardType.MATHD: mathd_adapter,
    RewardType.SYMPY: sympy_adapter,
    RewardType.COUNTDOWN: countdown_adapter,
    RewardType.BASE: base_adapter,
    RewardType.GSM8K: gsm8k_adapter,
    RewardType.BERNOULLI: bernoulli_adapter,
    RewardType.TOKEN_MATCH: token_match_adapter,
}


def get_reward_adapter(name) -> Callable[..., Dict[str, Any]]:
    try:
        return REWARD_ADAPTERS[RewardType(name)]
    except (KeyError, ValueError) as e:
        raise ValueError(f"unknown reward adapter: {name}") from e


def register_reward(name: str, fn: Callable[..., Dict[str, Any]]) -> None:
    """Adds a user-defined adapter under a new name (looked up by string)."""
    _EXTRA[name] = fn


_EXTRA: Dict[str, Callable[..., Dict[str, Any]]] = {}


def resolve_adapter(name) -> Callable[..., Dict[str, Any]]:
    if isinstance(name, str) and name in _EXTRA:
        return _EXTRA[name]
    return get_reward_adapter(name)
