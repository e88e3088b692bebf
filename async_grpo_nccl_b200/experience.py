"""ExperienceManager: the asynchronous sample pipeline between rollout, logprob and trainer roles.

Behaviour of the reference's ``ExperienceManager`` actor (orchestrator.py:1464-2034):

* one coroutine per prompt: acquire the least-loaded generation controller (bounded load), generate
  ``samples_per_question`` samples, then send every sample to a least-loaded logprob controller;
* finished prompts are consumed in completion order; as soon as ``train_minibatch_sample_size`` samples
  are ready they are packed by token budget into per-trainer-rank microbatches and dispatched, followed
  by a GRADIENT_STEP; training therefore overlaps with the generation of the rest of the macro-batch;
* every dispatch sends exactly one MICROBATCH to every trainer rank (a dummy for ranks without samples)
  so collectives line up; a sample longer than the budget travels alone;
* at the end of the macro-batch the remainder is flushed (its own, proportionally smaller, optimizer
  step) and BATCH_DONE carries the aggregated generation / reward / timing metrics.

The planning logic is a synchronous, side-effect-free class (``MicrobatchPlanner``) so its invariants
can be property-tested; the manager adds the asyncio plumbing. Controllers are any objects with async
``inference`` methods: in-process role objects or RPC proxies.
"""
from __future__ import annotations

import asyncio
import logging
import math
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

from .protocol import DUMMY_TRAIN_SAMPLE, Message, MessageType, sample_token_count

logger = logging.getLogger(__name__)


_TRAIN_KEYS = ("sample_ids", "input_len", "output_len", "advantage", "sample_logprobs", "sample_entropies", "ref_logprobs",
               "reward", "num_non_masked_output_tokens", "total_non_masked_output_tokens", "truncated_sample",
               "max_reward_in_group", "modified_reward", "delimiter_not_found", "__uid__", "dummy")


def slim_for_training(sample: Dict[str, Any]) -> Dict[str, Any]:
    """What a trainer rank needs from a sample; text, labels and position ids are rebuilt or unused there."""
    return {k: sample[k] for k in _TRAIN_KEYS if k in sample}


class MicrobatchPlanner:
    """Token-budgeted, rank-balanced microbatch planner.

    ``add(sample)`` and ``finish()`` return a list of events:
      ("microbatch", {rank: [samples...]})   one entry per registered rank (dummy list for empty ranks)
      ("gradient_step", None)
    """

    def __init__(self, ranks: Sequence[int], max_tokens_per_gpu: int, minibatch_size: int):
        self.ranks = list(ranks)
        self.max_tokens = int(max_tokens_per_gpu)
        self.minibatch_size = int(minibatch_size)
        self.buffers: Dict[int, List[Dict[str, Any]]] = {r: [] for r in self.ranks}
        self.lengths: Dict[int, int] = {r: 0 for r in self.ranks}
        self.dispatched_since_step = 0

    def _buffered(self) -> int:
        return sum(len(b) for b in self.buffers.values())

    def _dispatch(self, events: List[Tuple[str, Any]]) -> int:
        n_real = self._buffered()
        if n_real == 0:
            return 0
        payload = {r: (list(b) if b else [dict(DUMMY_TRAIN_SAMPLE)]) for r, b in self.buffers.items()}
        events.append(("microbatch", payload))
        for r in self.ranks:
            self.buffers[r] = []
            self.lengths[r] = 0
        self.dispatched_since_step += n_real
        return n_real

    def _maybe_step(self, events: List[Tuple[str, Any]]) -> None:
        if self.dispatched_since_step + self._buffered() >= self.minibatch_size:
            self._dispatch(events)
            events.append(("gradient_step", None))
            self.dispatched_since_step = 0

    def add(self, sample: Dict[str, Any]) -> List[Tuple[str, Any]]:
        events: List[Tuple[str, Any]] = []
        n_tok = sample_token_count(sample)
        rank = min(self.ranks, key=lambda r: self.lengths[r])
        if n_tok > self.max_tokens:
            # oversize sample: send what is buffered, then the sample alone
            self._dispatch(events)
            self.buffers[rank].append(sample)
            self.lengths[rank] += n_tok
            self._dispatch(events)
            self._maybe_step(events)
            return events
        if self.lengths[rank] + n_tok > self.max_tokens:
            self._dispatch(events)  # empty dispatch is a no-op; the sample is accepted either way
            rank = min(self.ranks, key=lambda r: self.lengths[r])
        self.buffers[rank].append(sample)
        self.lengths[rank] += n_tok
        self._maybe_step(events)
        return events

    def finish(self) -> List[Tuple[str, Any]]:
        """End of macro-batch: send the remainder and give it an optimizer step if anything is pending."""
        events: List[Tuple[str, Any]] = []
        self._dispatch(events)
        if self.dispatched_since_step > 0:
            events.append(("gradient_step", None))
            self.dispatched_since_step = 0
        return events


class _LoadBalancer:
    """Least-loaded acquisition with a per-controller cap (orchestrator.py:1611-1677)."""

    def __init__(self, controllers: Sequence[Any], threshold: int):
        self.controllers = list(controllers)
        self.load = {id(c): 0 for c in self.controllers}
        self.threshold = int(threshold)
        self.cond = asyncio.Condition()

    async def acquire(self, n: int = 1) -> Any:
        async with self.cond:
            while True:
                free = [c for c in self.controllers if self.load[id(c)] + n <= self.threshold]
                if free:
                    c = min(free, key=lambda x: self.load[id(x)])
                    self.load[id(c)] += n
                    return c
                await self.cond.wait()

    async def release(self, c: Any, n: int = 1) -> None:
        async with self.cond:
            self.load[id(c)] = max(0, self.load[id(c)] - n)
            self.cond.notify_all()


class ExperienceManager:
    def __init__(self, config: Any):
        self.config = config
        self.queues: Dict[int, asyncio.Queue] = {}
        self.completions: Dict[int, asyncio.Queue] = {}
        self.planner: Optional[MicrobatchPlanner] = None
        self.max_tokens_per_gpu = int(config.max_tokens_per_gpu)
        self.minibatch_size = int(config.train_minibatch_sample_size)
        self.pending_tasks: List[Any] = []
        self.ready: List[Dict[str, Any]] = []
        self._gen_lb: Optional[_LoadBalancer] = None
        self._lp_lb: Optional[_LoadBalancer] = None
        self._batch_task: Optional[asyncio.Task] = None
        self.batch_seq = 0
        self._reset_metrics()

    # ---- registration -----------------------------------------------------------------------
    def register_training_process(self, gpu_rank: int, max_tokens_per_gpu: int, train_minibatch_sample_size: int) -> bool:
        self.max_tokens_per_gpu = int(max_tokens_per_gpu)
        self.minibatch_size = int(train_minibatch_sample_size)
        self.queues[gpu_rank] = asyncio.Queue()
        self.completions[gpu_rank] = asyncio.Queue()
        self.planner = MicrobatchPlanner(sorted(self.queues), self.max_tokens_per_gpu, self.minibatch_size)
        return True

    def _reset_metrics(self) -> None:
        self.gen_metrics = {"total_tokens_generated": 0.0, "inference_duration_sec": 0.0, "num_samples_generated": 0.0}
        self.timing = {"gen_duration": 0.0, "logprob_duration": 0.0, "num_prompts": 0.0}
        self.acc = {"total_samples": 0, "total_reward": 0.0, "total_completion_tokens": 0}
        self.reward_values: List[float] = []
        self.group_std_values: List[float] = []
        self.nonzero_reward = 0
        self.dropped_prompts = 0
        self.batch_start_time: Optional[float] = None
        self.role_failures: List[str] = []  # roles that could not be reached at all (connection lost), this batch

    # ---- generation -------------------------------------------------------------------------
    def _thresholds(self) -> Tuple[int, int]:
        n = int(self.config.samples_per_question)
        per_engine = int(math.ceil(self.config.max_num_seqs / max(1, n))) + int(self.config.overhead_seqs)
        return max(4, n, per_engine), max(8, 2 * n)

    async def generate_experience(self, questions: Sequence[Dict[str, Any]], generation_controllers: Sequence[Any],
                                  logprob_controllers: Sequence[Any]) -> None:
        self._reset_metrics()
        self.batch_start_time = time.time()
        self.batch_seq += 1
        if self._gen_lb is None or self._gen_lb.controllers != list(generation_controllers):
            g, l = self._thresholds()
            self._gen_lb = _LoadBalancer(generation_controllers, g)
            self._lp_lb = _LoadBalancer(logprob_controllers, l)
        timeout = float(getattr(self.config, "prompt_timeout_s", 1200.0))

        async def guarded(q: Dict[str, Any]):
            try:
                return await asyncio.wait_for(self._process_single_prompt(q), timeout)
            except asyncio.TimeoutError:
                logger.warning("prompt pipeline timed out after %.0fs; prompt dropped", timeout)
                return None, None, None

        self.pending_tasks.extend(asyncio.ensure_future(guarded(q)) for q in questions)

    async def _process_single_prompt(self, question: Dict[str, Any]):
        t0 = time.time()
        gen = await self._gen_lb.acquire(1)
        try:
            samples, gen_metrics = await gen.inference(question, n=self.config.samples_per_question,
                                                       temperature=self.config.temperature,
                                                       max_tokens=self.config.max_generation_tokens)
        except Exception as e:  # generation failure: the prompt is skipped
            logger.error("generation failed: %r", e)
            if isinstance(e, (ConnectionError, OSError)):
                self.role_failures.append(f"generation: {e!r}")
            return None, None, None
        finally:
            await self._gen_lb.release(gen, 1)
        gen_duration = time.time() - t0
        if not samples:
            return None, None, None
        t1 = time.time()

        async def one(sample: Dict[str, Any]):
            lp = await self._lp_lb.acquire(1)
            try:
                return await lp.inference(sample)
            finally:
                await self._lp_lb.release(lp, 1)

        async def keep(sample: Dict[str, Any]):
            return sample

        # samples whose old-policy log-probabilities the generation worker already attached (requested when each
        # sample finished) skip this stage
        results = await asyncio.gather(*[keep(s) if s.get("logprobs_attached") else one(s) for s in samples],
                                       return_exceptions=True)
        valid = []
        for r in results:
            if isinstance(r, Exception):
                logger.error("logprob task failed: %r", r)
                if isinstance(r, (ConnectionError, OSError)):
                    self.role_failures.append(f"logprob: {r!r}")
            elif r:
                valid.append(r)
        return valid, gen_metrics, {"gen_duration": gen_duration, "logprob_duration": time.time() - t1}

    # ---- batching ---------------------------------------------------------------------------
    def start_creating_batches(self) -> asyncio.Task:
        self._batch_task = asyncio.ensure_future(self._create_batches())
        return self._batch_task

    async def _emit(self, events: Sequence[Tuple[str, Any]]) -> None:
        for kind, payload in events:
            if kind == "microbatch":
                for rank, samples in payload.items():
                    if rank in self.queues:
                        await self.queues[rank].put(Message(MessageType.MICROBATCH, [slim_for_training(x) for x in samples]))
            else:
                await self.dispatch_signal(MessageType.GRADIENT_STEP)

    async def _flush_ready(self) -> None:
        total = sum(int(s.get("num_non_masked_output_tokens", s.get("output_len", 0))) for s in self.ready)
        for s in self.ready:
            s["total_non_masked_output_tokens"] = total
            await self._emit(self.planner.add(s))
        self.ready.clear()

    def _account(self, samples: Sequence[Dict[str, Any]], gen_metrics: Optional[Dict[str, float]],
                 timing: Optional[Dict[str, float]]) -> None:
        rewards = [float(s.get("reward", 0.0)) for s in samples]
        self.acc["total_samples"] += len(samples)
        self.acc["total_reward"] += sum(rewards)
        self.acc["total_completion_tokens"] += sum(int(s.get("output_len", 0)) for s in samples)
        self.reward_values.extend(rewards)
        self.nonzero_reward += sum(1 for r in rewards if r != 0.0)
        if rewards:
            m = sum(rewards) / len(rewards)
            self.group_std_values.append(math.sqrt(sum((r - m) ** 2 for r in rewards) / len(rewards)))
        if gen_metrics:
            self.gen_metrics["total_tokens_generated"] += float(gen_metrics.get("generation/total_tokens_generated", 0.0))
            self.gen_metrics["inference_duration_sec"] += float(gen_metrics.get("generation/inference_duration_sec", 0.0))
            self.gen_metrics["num_samples_generated"] += float(gen_metrics.get("generation/num_samples_generated", 0.0))
        if timing:
            self.timing["gen_duration"] += float(timing.get("gen_duration", 0.0))
            self.timing["logprob_duration"] += float(timing.get("logprob_duration", 0.0))
            self.timing["num_prompts"] += 1.0

    async def _create_batches(self) -> None:
        assert self.planner is not None, "no trainer rank registered"
        tasks, self.pending_tasks = self.pending_tasks, []
        for fut in asyncio.as_completed(tasks):
            samples, gen_metrics, timing = await fut
            if not samples:
                self.dropped_prompts += 1
                continue
            self._account(samples, gen_metrics, timing)
            self.ready.extend(samples)
            if len(self.ready) >= self.minibatch_size or getattr(self.config, "eager_microbatch_dispatch", False):
                await self._flush_ready()
        if self.ready:
            await self._flush_ready()
        await self._emit(self.planner.finish())
        await self.dispatch_signal_with_data(MessageType.BATCH_DONE, {
            "gen_logprob_metrics": {**{f"generation/{k}": v for k, v in self.gen_metrics.items()}, **self.timing,
                                    "gen_logprob_wall_time": time.time() - self.batch_start_time if self.batch_start_time else 0.0},
            "batch_metrics": self._get_aggregated_batch_metrics()["batch_metrics"],
        })

    def _get_aggregated_batch_metrics(self) -> Dict[str, Any]:
        n = self.acc["total_samples"]
        rv, gv = self.reward_values, self.group_std_values
        mean = sum(rv) / len(rv) if rv else 0.0
        std = math.sqrt(sum((x - mean) ** 2 for x in rv) / len(rv)) if rv else 0.0
        return {
            "gen_metrics": dict(self.gen_metrics),
            "timing_metrics": dict(self.timing),
            "batch_metrics": {
                "avg_reward": self.acc["total_reward"] / n if n else 0.0,
                "total_samples": n,
                "avg_completion_length": self.acc["total_completion_tokens"] / n if n else 0.0,
                "reward_mean": mean, "reward_std": std,
                "reward_min": min(rv) if rv else 0.0, "reward_max": max(rv) if rv else 0.0,
                "group_reward_std_mean": sum(gv) / len(gv) if gv else 0.0,
                "group_reward_std_zero_frac": sum(1 for x in gv if abs(x) < 1e-9) / len(gv) if gv else 0.0,
                "nonzero_reward_frac": self.nonzero_reward / n if n else 0.0,
                "dropped_prompts": self.dropped_prompts,
            },
            "gen_logprob_wall_time": time.time() - self.batch_start_time if self.batch_start_time else 0.0,
        }

    # ---- trainer-facing queues ----------------------------------------------------------------
    async def dispatch_signal(self, signal: MessageType) -> None:
        for q in self.queues.values():
            await q.put(Message(signal))

    async def dispatch_signal_with_data(self, signal: MessageType, data: Any = None) -> None:
        for q in self.queues.values():
            await q.put(Message(signal, data))

    async def get_batch(self, global_rank: int) -> Message:
        return await self.queues[global_rank].get()

    async def get_completion(self, global_rank: int) -> Any:
        return await self.completions[global_rank].get()

    async def put_completion(self, global_rank: int, completion_data: Any) -> None:
        await self.completions[global_rank].put(completion_data)
