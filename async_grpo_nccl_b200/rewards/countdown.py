"""Countdown-task reward.

Behaviour of the reference's countdown_reward.py:13-95: a format score (1.0 for
``<think>...</think>\\n<answer>...</answer>`` as the whole response, otherwise 0.1 for a think block plus 0.5
for an answer block) and an answer score (1.0 when the answer expression uses every given number
exactly once, contains only digits / + - * / ( ) / spaces and evaluates to the target); total =
0.1 * format + answer. The expression is evaluated by a small recursive-descent parser instead of
``eval``.
"""
from __future__ import annotations

import re
from typing import Any, Dict, Optional, Sequence

_THINK = re.compile(r"<think>.*?</think>", re.DOTALL)
_ANSWER = re.compile(r"<answer>(.*?)</answer>", re.DOTALL)
_FULL = re.compile(r"^<think>.*?</think>\n<answer>.*?</answer>$", re.DOTALL)
_ALLOWED = re.compile(r"^[0-9+\-*/() ]+$")


def format_score(response: str, end_token: Optional[str] = None) -> float:
    if end_token and response.endswith(end_token):
        response = response[: -len(end_token)]
    if _FULL.match(response):
        return 1.0
    score = 0.0
    if _THINK.search(response):
        score += 0.1
    if _ANSWER.search(response):
        score += 0.5
    return score


class _Parser:
    """expr := term (('+'|'-') term)* ; term := factor (('*'|'/') factor)* ; factor := number | '(' expr ')' | ('+'|'-') factor"""

    def __init__(self, text: str):
        self.toks = re.findall(r"\d+|[+\-*/()]", text)
        self.i = 0

    def peek(self) -> Optional[str]:
        return self.toks[self.i] if self.i < len(self.toks) else None

    def take(self) -> str:
        t = self.toks[self.i]
        self.i += 1
        return t

    def expr(self) -> float:
        v = self.term()
        while self.peek() in ("+", "-"):
            op = self.take()
            r = self.term()
            v = v + r if op == "+" else v - r
        return v

    def term(self) -> float:
        v = self.factor()
        while self.peek() in ("*", "/"):
            op = self.take()
            r = self.factor()
            v = v * r if op == "*" else v / r
        return v

    def factor(self) -> float:
        t = self.peek()
        if t is None:
            raise ValueError("unexpected end")
        if t in ("+", "-"):
            self.take()
            v = self.factor()
            return v if t == "+" else -v
        if t == "(":
            self.take()
            v = self.expr()
            if self.peek() != ")":
                raise ValueError("missing )")
            self.take()
            return v
        if t.isdigit():
            return float(self.take())
        raise ValueError(f"unexpected token {t}")


def evaluate_arithmetic(text: str) -> float:
    p = _Parser(text)
    v = p.expr()
    if p.peek() is not None:
        raise ValueError("trailing tokens")
    return v


def answer_score(response: str, numbers: Optional[Sequence[int]], target: Optional[float]) -> float:
    m = _ANSWER.search(response)
    if not m:
        return 0.0
    content = m.group(1)
    if not content or not _ALLOWED.match(content):
        return 0.0
    used = sorted(int(n) for n in re.findall(r"\d+", content))
    if used != sorted(int(n) for n in (numbers or [])):
        return 0.0
    try:
        if target is not None and abs(evaluate_arithmetic(content) - float(target)) < 1e-5:
            return 1.0
    except (ValueError, ZeroDivisionError, IndexError):
        return 0.0
    return 0.0


def countdown_reward(response: str, numbers: Optional[Sequence[int]] = None, target: Optional[float] = None,
                     end_token: Optional[str] = None) -> Dict[str, Any]:
    f = format_score("<think>" + response, end_token)
    a = answer_score(response, numbers, target)
    return {"reward": 0.1 * f + a, "reward_info": {"format_reward": f, "answer_reward": a}}
