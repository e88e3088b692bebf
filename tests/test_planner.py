"""Batching invariants of the microbatch planner (token budget, exact minibatch -> one GRADIENT_STEP, dummy microbatches,
oversize samples) and the ExperienceManager's queue protocol."""
import asyncio

import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from async_grpo_nccl_b200.experience import ExperienceManager, MicrobatchPlanner
from async_grpo_nccl_b200.protocol import MessageType


def _s(n_in, n_out, i=0):
    return {"input_len": n_in, "output_len": n_out, "sample_ids": np.zeros(n_in + n_out, np.int32), "id": i}


def _replay(planner, samples):
    events = []
    for s in samples:
        events += planner.add(s)
    events += planner.finish()
    return events


@settings(max_examples=200, deadline=None)
@given(lens=st.lists(st.tuples(st.integers(1, 60), st.integers(0, 120)), min_size=1, max_size=60),
       ranks=st.integers(1, 4), budget=st.integers(50, 400), minibatch=st.integers(1, 16))
def test_planner_invariants(lens, ranks, budget, minibatch):
    p = MicrobatchPlanner(list(range(ranks)), budget, minibatch)
    samples = [_s(a, b, i) for i, (a, b) in enumerate(lens)]
    events = _replay(p, samples)
    seen, since_step, steps = [], 0, 0
    for kind, payload in events:
        if kind == "microbatch":
            assert set(payload) == set(range(ranks))  # one message per rank, every dispatch
            n_real = 0
            for r, batch in payload.items():
                real = [x for x in batch if not x.get("dummy")]
                if not real:
                    assert len(batch) == 1 and batch[0]["dummy"]  # empty ranks get exactly one dummy
                else:
                    assert all(not x.get("dummy") for x in batch)
                tok = sum(x["input_len"] + x["output_len"] for x in real)
                assert tok <= budget or len(real) == 1  # only a lone oversize sample may exceed the budget
                n_real += len(real)
                seen += [x["id"] for x in real]
            assert n_real > 0  # never an all-dummy dispatch
            since_step += n_real
        else:
            assert since_step > 0
            steps += 1
            since_step = 0
    assert since_step == 0  # everything dispatched got an optimizer step
    assert sorted(seen) == list(range(len(samples)))  # every sample exactly once
    assert steps >= (len(samples) + minibatch - 1) // minibatch - 0 if all(a + b <= budget for a, b in lens) else steps >= 1


def test_exact_minibatch_gives_exactly_one_step():
    p = MicrobatchPlanner([0, 1], 10_000, 8)
    events = _replay(p, [_s(10, 10, i) for i in range(8)])
    assert [k for k, _ in events].count("gradient_step") == 1
    assert events[-1][0] == "gradient_step"  # finish() adds no extra step
    # partial remainder gets its own, smaller step
    p = MicrobatchPlanner([0], 10_000, 8)
    events = _replay(p, [_s(10, 10, i) for i in range(11)])
    assert [k for k, _ in events].count("gradient_step") == 2


def test_least_loaded_rank_and_oversize():
    p = MicrobatchPlanner([0, 1], 100, 100)
    ev = p.add(_s(10, 50, 0)) + p.add(_s(10, 20, 1)) + p.add(_s(5, 5, 2))
    assert ev == []
    assert [x["id"] for x in p.buffers[0]] == [0] and [x["id"] for x in p.buffers[1]] == [1, 2]
    ev = p.add(_s(100, 100, 3))  # oversize: flush, then alone
    kinds = [k for k, _ in ev]
    assert kinds == ["microbatch", "microbatch"]
    alone = ev[1][1]
    assert sum(len([x for x in b if not x.get("dummy")]) for b in alone.values()) == 1


def test_experience_manager_end_to_end_with_fake_controllers():
    class Cfg:
        max_tokens_per_gpu, train_minibatch_sample_size, samples_per_question = 200, 6, 3
        temperature, max_generation_tokens, max_num_seqs, overhead_seqs = 1.0, 16, 8, 2
        prompt_timeout_s, eager_microbatch_dispatch = 30.0, False

    class Gen:
        async def inference(self, q, n, temperature, max_tokens):
            await asyncio.sleep(0.001 * (q["i"] % 3))
            if q["i"] == 2:
                raise RuntimeError("generation failed")  # this prompt is dropped, the batch goes on
            return [dict(_s(5, 7, q["i"] * 10 + c), reward=float(c % 2), num_non_masked_output_tokens=7) for c in range(n)], \
                   {"generation/total_tokens_generated": 7.0 * n, "generation/num_samples_generated": float(n)}

    class Lp:
        async def inference(self, s):
            return dict(s, sample_logprobs=np.zeros(12, np.float32), sample_entropies=np.zeros(12, np.float32))

    async def run():
        em = ExperienceManager(Cfg())
        for r in (0, 1):
            em.register_training_process(r, 200, 6)
        await em.generate_experience([{"i": i} for i in range(5)], [Gen(), Gen()], [Lp()])
        em.start_creating_batches()
        msgs = {0: [], 1: []}
        for r in (0, 1):
            while True:
                m = await asyncio.wait_for(em.get_batch(r), 5)
                msgs[r].append(m)
                if m.type == MessageType.BATCH_DONE:
                    break
        return em, msgs

    em, msgs = asyncio.run(run())
    for r in (0, 1):
        types = [m.type for m in msgs[r]]
        assert types[-1] == MessageType.BATCH_DONE
        assert types.count(MessageType.GRADIENT_STEP) == 2  # 12 samples, minibatch 6
    assert [m.type for m in msgs[0]] == [m.type for m in msgs[1]]  # both ranks see the same message sequence
    done = msgs[0][-1].data
    assert done["batch_metrics"]["total_samples"] == 12 and done["batch_metrics"]["dropped_prompts"] == 1
    real = sum(len([s for s in m.data if not s.get("dummy")]) for r in (0, 1) for m in msgs[r] if m.type == MessageType.MICROBATCH)
    assert real == 12
