"""Reward adapters (table-driven) and the verifier pool (best-of selection, timeout -> reward 0 + worker replacement)."""
import asyncio
import json
import time

import numpy as np
import pytest

from async_grpo_nccl_b200.ops.reference import normalize_rewards
from async_grpo_nccl_b200.rewards import RewardType, get_reward_adapter, register_reward
from async_grpo_nccl_b200.rewards.countdown import answer_score, countdown_reward, evaluate_arithmetic, format_score
from async_grpo_nccl_b200.rewards.math_grading import extract_answer, grade_answer_mathd, grade_answer_sympy
from async_grpo_nccl_b200.rewards.verifier_pool import VerifierPool, compute_cosine_reward


@pytest.mark.parametrize("resp,want", [
    ("<think>a</think>\n<answer>1+2</answer>", 1.0), ("<think>a</think><answer>1</answer>", 0.6), ("<think>a</think>", 0.1),
    ("<answer>3</answer>", 0.5), ("nothing", 0.0), ("<think>a</think>\n<answer>1+2</answer><|eot|>", 0.6)])
def test_countdown_format(resp, want):
    assert abs(format_score(resp) - want) < 1e-9


def test_countdown_answer_and_total():
    ok = "<think>..</think>\n<answer>(3 + 5) * 2 - 6</answer>"
    assert answer_score(ok, [2, 3, 5, 6], 10) == 1.0
    assert answer_score(ok, [2, 3, 5], 10) == 0.0  # a number is missing from the given list
    assert answer_score(ok, [2, 3, 5, 6], 11) == 0.0
    assert answer_score("<answer>__import__('os')</answer>", [1], 1) == 0.0
    assert answer_score("<answer>4/0</answer>", [0, 4], 1) == 0.0
    assert evaluate_arithmetic("2*(3+4)/7 - -1") == 3.0
    r = countdown_reward("x</think>\n<answer>(3 + 5) * 2 - 6</answer>", [2, 3, 5, 6], 10)
    assert abs(r["reward"] - 1.1) < 1e-9
    out = get_reward_adapter("countdown")({"sample_text": "PROMPT x</think>\n<answer>6+4</answer>", "input": "PROMPT ",
                                           "nums": [4, 6], "target": 10, "end_token": ""})
    assert abs(out["reward"] - 1.1) < 1e-9


@pytest.mark.parametrize("given,truth,mathd,symp", [
    ("\\frac{1}{2}", "\\dfrac{1}{2}", True, True), ("0.5", "\\frac{1}{2}", True, True), ("1/2", "\\frac12", True, True),
    ("x+1", "1+x", False, True), ("10\\%", "10", True, True), ("(1,2)", "(1, 2)", True, True), ("(1,2)", "[1,2]", False, False),
    ("3", "4", False, False), ("\\text{5 cm}", "5", True, True), ("2\\sqrt{2}", "\\sqrt{8}", False, True)])
def test_math_grading(given, truth, mathd, symp):
    assert grade_answer_mathd(given, truth) == mathd
    assert grade_answer_sympy(given, truth) == symp


def test_boxed_extraction_and_math_adapters():
    assert extract_answer("so \\boxed{\\frac{3}{4}} and then \\boxed{7}") == "7"
    assert extract_answer("nested \\boxed{a_{1}+\\frac{1}{2}}") == "a_{1}+\\frac{1}{2}"
    assert extract_answer("none") is None
    s = {"sample_text": "Q: what? A: it is \\boxed{\\frac{1}{2}}", "input": "Q: what?", "answer": "\\boxed{0.5}"}
    assert get_reward_adapter(RewardType.MATHD)(dict(s))["reward"] == 1.0
    assert get_reward_adapter("sympy")(dict(s))["reward"] == 1.0
    g = {"sample_text": "P<final_answer> 1,234 </final_answer>", "input": "P", "answer": "1234"}
    assert get_reward_adapter("gsm8k")(g)["reward"] == 1.0
    assert get_reward_adapter("base")({"reward": 0.25})["reward"] == 0.25
    with pytest.raises(ValueError):
        get_reward_adapter("ksat_math")


def test_synthetic_adapters_and_advantages():
    ids = np.arange(20, dtype=np.int32)
    s = {"sample_ids": ids, "input_len": 5, "output_token_ids": ids[5:], "vocab_size": 1024}
    assert get_reward_adapter("token_match")(s)["reward"] == 1.0  # 0+1+2+3+4 = 10 is among the outputs
    a = get_reward_adapter("bernoulli")({"sample_ids": ids, "input_len": 5, "sample_index": 3})
    b = get_reward_adapter("bernoulli")({"sample_ids": ids, "input_len": 5, "sample_index": 3})
    assert a == b and a["reward"] in (0.0, 1.0)
    adv = normalize_rewards([1.0, 0.0, 0.0, 1.0])
    assert abs(sum(adv)) < 1e-6 and abs(adv[0] - 1.0 / (0.5 + 1e-4) * 0.5) < 1e-6
    assert normalize_rewards([2.0, 2.0]) == [0.0, 0.0]
    assert compute_cosine_reward(100, 100, 1.0, 1.0) == -10
    assert compute_cosine_reward(0, 100, 0.0, 1.0) == 6 and abs(compute_cosine_reward(0, 100, 0.0, 0.0) + 10) < 1e-9


def _slow(sample, **_):
    time.sleep(30)
    return {"reward": 1.0}


def test_verifier_pool_best_of_timeout_and_replacement(tmp_path):
    async def run():
        pool = VerifierPool(2, write_failed=True, reward_fns=["mathd", "sympy"], output_dir=str(tmp_path), timeout_s=20.0)
        s = {"sample_text": "Q A \\boxed{x+1}", "input": "Q", "answer": "\\boxed{1+x}"}
        best = await pool.verify(dict(s))
        assert best["reward"] == 1.0 and best["reward_success"]  # sympy accepts what the string grader rejects
        pool.close()
        # a hung reward function: the worker is killed and replaced, the sample gets reward 0, and it is written out
        hung = VerifierPool(1, write_failed=True, reward_fns=["hang_forever"], output_dir=str(tmp_path), timeout_s=0.5, start_method="fork")
        register_reward("hang_forever", _slow)
        t0 = time.time()
        out = await hung.verify({"sample_text": "x", "input": "", "answer": "1", "arr": np.arange(3)})
        assert time.time() - t0 < 10 and out["reward"] == 0.0 and out["reward_success"] is False
        assert hung.replaced_workers == 1
        again = await hung.verify({"sample_text": "y", "input": "", "answer": "1"}, reward_fns=["base"], )
        assert again["reward_success"] is False  # 'base' needs a reward key: adapter error -> failure, worker survives
        assert hung.replaced_workers == 1
        hung.close()

    asyncio.run(run())
    lines = (tmp_path / "failed_samples_verify.jsonl").read_text().strip().splitlines()
    assert len(lines) == 2 and json.loads(lines[0])["sample_text"] == "x"
