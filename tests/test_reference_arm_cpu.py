"""Host-side pieces of the reference arm of ``bench.py`` (``baseline/``): workload parity with the product's
generator, the restated microbatch planner, the mailbox control plane, the stand-in modules."""
import os
import sys
import threading
from datetime import timedelta

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def test_reference_workload_equals_product_workload():
    from ref_workload import bernoulli_reward, synthetic_rows

    from async_grpo_nccl_b200.data import synthetic_prompt_rows
    from async_grpo_nccl_b200.rewards.registry import bernoulli_adapter

    a = synthetic_rows(24, 151936, 64, 512, 0, 8, (256, 8192), 0.3)
    b = synthetic_prompt_rows(24, 151936, 64, 512, seed=0, samples_per_question=8, gen_len_range=(256, 8192), reward_p=0.3)
    for x, y in zip(a, b):
        assert np.array_equal(x["input_token_ids"], y["input_token_ids"])
        assert x["forced_output_lens"] == y["forced_output_lens"] and x["__uid__"] == y["__uid__"]
    s = {"input_token_ids": a[0]["input_token_ids"], "input_len": len(a[0]["input_token_ids"]),
         "output_token_ids": list(range(20)), "sample_index": 3, "reward_p": 0.3}
    assert bernoulli_reward(s) == bernoulli_adapter(s)["reward"]


def _samples(n, rng):
    out = []
    for i in range(n):
        li, lo = int(rng.integers(10, 50)), int(rng.integers(10, 400))
        out.append({"input_len": li, "output_len": lo, "num_non_masked_output_tokens": lo, "id": i})
    return out


@pytest.mark.parametrize("ranks,budget", [(1, 1000), (2, 600), (4, 450)])
def test_planner_keeps_the_token_budget_and_steps_once_per_minibatch(ranks, budget):
    from reference_arm import plan_microbatches

    rng = np.random.default_rng(ranks)
    samples = _samples(64, rng)
    msgs = plan_microbatches(samples, ranks, budget, minibatch=64)
    counts = [sum(1 for k, _ in q if k == "microbatch") for q in msgs]
    assert len(set(counts)) == 1, "every rank runs the same number of forward/backward passes"
    seen = []
    for q in msgs:
        assert [k for k, _ in q].count("gradient_step") == 1 and q[-1][0] == "batch_done"
        for k, data in q:
            if k == "microbatch" and not data[0].get("dummy"):
                assert sum(s["input_len"] + s["output_len"] for s in data) <= budget or len(data) == 1
                seen.extend(s["id"] for s in data)
    assert sorted(seen) == list(range(64))
    assert all(s["total_non_masked_output_tokens"] == sum(x["output_len"] for x in samples) for s in samples)


def test_mailboxes_deliver_in_order_between_threads():
    import torch.distributed as dist

    from reference_arm import Mail

    port = 29000 + os.getpid() % 500
    store = dist.TCPStore("127.0.0.1", port, world_size=1, is_master=True, timeout=timedelta(seconds=20), wait_for_workers=False)
    a, b = Mail(store), Mail(dist.TCPStore("127.0.0.1", port, world_size=1, is_master=False, timeout=timedelta(seconds=20),
                                           wait_for_workers=False))
    got = []
    t = threading.Thread(target=lambda: [got.append(b.take("box")) for _ in range(5)])
    t.start()
    for i in range(5):
        a.post("box", {"i": i, "payload": list(range(i))})
    t.join(timeout=20)
    assert [g["i"] for g in got] == list(range(5))
    assert not b.ready("box")
    th = [threading.Thread(target=m.barrier, args=("x", 2)) for m in (a, b)]
    [x.start() for x in th]
    [x.join(timeout=20) for x in th]
    assert not any(x.is_alive() for x in th)


def test_stand_in_modules_carry_the_names_the_reference_imports():
    import importlib.util

    import ref_shims

    made = ref_shims.install()
    import ray
    from ray.util.collective import collective

    @ray.remote(num_gpus=1)
    class A:
        pass

    assert isinstance(A, type) and callable(collective.broadcast)
    if "peft" in made:
        ref_shims.retire()
        assert importlib.util.find_spec("peft") is None  # libraries probing for the real package see it as absent


def test_abort_note_first_writer_wins(tmp_path):
    """A failing rank leaves one note; later failures do not overwrite it, and the other ranks read it."""
    from reference_arm import read_abort, write_abort

    p = str(tmp_path / "abort")
    assert read_abort(p) is None
    write_abort(p, "rank 3 failed: boom")
    write_abort(p, "rank 1 failed later")
    assert read_abort(p) == "rank 3 failed: boom"
