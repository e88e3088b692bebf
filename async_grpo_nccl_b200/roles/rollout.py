"""Generation role: owns one rollout engine, builds the per-sample fields, sends every sample through the
verifier pool, and computes group-normalised advantages.

It covers the reference's ``GenerationVLLMWorker`` (vllm_worker.py:128-805): ``inference(sample, n,
temperature, max_tokens)`` -> ``(samples, metrics)``, ``batch_inference_for_evaluation``,
``generate_with_logprobs`` and ``sync_weights``. The engine runs in its own thread; requests from many
concurrent ``inference`` coroutines are batched continuously by the engine's scheduler.
"""
from __future__ import annotations

import asyncio
import logging
import hashlib
import threading
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops.reference import normalize_rewards
from ..protocol import build_sample


logger = logging.getLogger(__name__)

def _uid_seed(uid: Any, base: int) -> int:
    h = hashlib.sha256(repr(uid).encode()).digest()
    return (int.from_bytes(h[:8], "little") ^ (base * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


class GenerationWorker:
    def __init__(self, config: Any, model_cfg: Any, engine: Any, verifier_pool: Any, tokenizer: Any = None,
                 stream: Optional[torch.cuda.Stream] = None, sm_limit: int = 0, mirror: Any = None):
        self.config, self.mcfg, self.engine, self.verifier = config, model_cfg, engine, verifier_pool
        # Leader of a tensor-parallel replica: every engine call is announced to the other members first (they replay it
        # on their own engines, see roles/tp_mirror.py). None for an engine that runs alone.
        self.mirror = mirror
        self.tokenizer = tokenizer
        self.stream = stream
        self.sm_limit = int(sm_limit)  # > 0: the stream runs on an SM group of this size (persistent grids must fit it)
        self._lock = threading.Lock()
        self._incoming: List[Tuple[Any, ...]] = []
        self._futures: Dict[Any, Tuple[Any, ...]] = {}  # request id -> (loop, future, n, finished children, on_child)
        # Optional async callable sample -> {"sample_logprobs", "sample_entropies"} (set by the runtime). When present the
        # old-policy log-probabilities of every sample are requested the moment THAT sample finishes, while its siblings
        # still generate, instead of for the whole group at its end: the logprob role's work spreads over the
        # generation phase instead of piling up behind it. The weights it uses are the same either way (they only
        # change at a weight sync, when generation is paused).
        self.logprob_fn: Optional[Any] = None
        self._want_logprobs = False
        self._req_counter = 0
        self._wake = threading.Event()
        self._stop = False
        self._paused = threading.Event()
        self._idle = threading.Event()
        self._idle.set()
        # One lock orders "the engine thread decides to step" against "a weight sync asks it to stop": the thread
        # re-checks the pause flag and clears the idle flag under it, the sync sets the pause flag under it. Either the
        # sync sees the idle flag cleared and waits for the step to end, or the thread sees the pause flag and stays idle.
        self._gate = threading.Lock()
        self._thread = threading.Thread(target=self._engine_loop, name="rollout-engine", daemon=True)
        self._thread.start()
        self._req_counter = 0
        self.total_tokens = 0
        self.busy_seconds = 0.0

    # ------------------------------------------------------------------ engine thread
    def _engine_loop(self) -> None:
        try:
            self._engine_loop_body()
        except BaseException as e:  # a dead engine thread must not leave requests waiting for their timeout
            logger.exception("rollout engine thread stopped: %r", e)
            self._dead = e
            self._fail_all(e if isinstance(e, Exception) else RuntimeError(repr(e)))

    def _engine_loop_body(self) -> None:
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else _null()
        if self.sm_limit > 0 and hasattr(self.engine, "C"):
            self.engine.C.set_sm_limit(self.sm_limit)  # thread-local: the engine thread only
            self.engine.sm_count = self.sm_limit
        with ctx:
            while not self._stop:
                with self._lock:
                    new, self._incoming = self._incoming, []
                mirror = self.mirror
                if self._want_logprobs and hasattr(self.engine, "enable_logprobs"):
                    if mirror is not None:
                        mirror.send("logprobs")
                    self.engine.enable_logprobs()  # on the engine's own thread, between steps
                    self._want_logprobs = False
                for args in new:
                    if mirror is not None:
                        mirror.send("add", args)
                    self.engine.add_request(*args[0], **args[1])
                with self._gate:
                    go = not self._paused.is_set() and self.engine.has_work()
                    if go:
                        self._idle.clear()
                    else:
                        self._idle.set()
                if not go:
                    self._wake.wait(timeout=0.05)
                    self._wake.clear()
                    continue
                t0 = time.time()
                try:
                    if mirror is not None:
                        mirror.send("step")
                    finished = self.engine.step()
                    # the kernels' status word (bounded waits, index checks): read whenever sequences finish (the step
                    # synchronised anyway), or after every step with kernel_checks
                    if finished or getattr(self.config, "kernel_checks", False):
                        self.engine.check_status()
                except Exception as e:  # fail every waiter instead of hanging them
                    self._fail_all(e)
                    continue
                self.busy_seconds += time.time() - t0
                for f in finished:
                    self._deliver(f)

    def _deliver(self, f: Any) -> None:
        entry = self._futures.get(f.request_id)
        if entry is None:
            return
        loop, fut, n, got, on_child = entry
        got.append(f)
        if on_child is not None:
            loop.call_soon_threadsafe(on_child, f)  # queued before the group's completion below: runs first
        if len(got) == n:
            del self._futures[f.request_id]
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(sorted(got, key=lambda x: x.child)))

    def _fail_all(self, e: Exception) -> None:
        for rid, (loop, fut, *_rest) in list(self._futures.items()):
            loop.call_soon_threadsafe(lambda fut=fut: fut.done() or fut.set_exception(RuntimeError(f"engine failure: {e!r}")))
        self._futures.clear()

    async def _generate(self, prompt_ids: np.ndarray, n: int, max_new: int, temperature: float, seed: int,
                        forced: Optional[Sequence[int]] = None, ignore_eos: bool = False, on_child: Any = None) -> List[Any]:
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        if getattr(self, "_dead", None) is not None:
            raise RuntimeError(f"rollout engine thread has stopped: {self._dead!r}")
        with self._lock:
            self._req_counter += 1
            rid = self._req_counter
            self._futures[rid] = (loop, fut, n, [], on_child)
            self._incoming.append(((rid, prompt_ids), dict(n=n, max_new_tokens=max_new, temperature=temperature, seed=seed,
                                                          forced_new_tokens=forced, ignore_eos=ignore_eos)))
        self._wake.set()
        return await fut

    # ------------------------------------------------------------------ public API
    def get_max_tokens(self, prompt_len: int, max_tokens: Optional[int]) -> int:
        """min(requested, max_model_len) - len(prompt) - 1 (vllm_worker.py:394-401)."""
        cap = int(getattr(self.engine, "max_model_len", self.mcfg.max_position_embeddings))
        req = int(max_tokens) if max_tokens else cap
        return max(1, min(min(req, cap), cap - prompt_len - 1))

    def _decode(self, ids: np.ndarray) -> str:
        if self.tokenizer is None:
            return ""
        return self.tokenizer.decode(ids.tolist(), skip_special_tokens=False)

    async def inference(self, sample: Dict[str, Any], n: int = 1, temperature: float = 1.0,
                        max_tokens: Optional[int] = None) -> Tuple[List[Dict[str, Any]], Dict[str, float]]:
        t0 = time.time()
        prompt = np.asarray(sample["input_token_ids"], dtype=np.int32)
        max_new = self.get_max_tokens(len(prompt), max_tokens)
        forced = sample.get("forced_output_lens")
        seed = _uid_seed(sample.get("__uid__", self._req_counter), int(getattr(self.config, "seed", 0)))
        row = {k: v for k, v in sample.items() if k != "forced_output_lens"}
        eos = int(getattr(self.engine, "eos", self.mcfg.eos_token_id))
        cap = self.get_max_tokens(len(prompt), max_tokens)

        def build(f: Any) -> Dict[str, Any]:
            s = build_sample(row, prompt, f.output_ids, eos)
            s["sample_index"] = f.child
            s["vocab_size"] = self.mcfg.vocab_size
            s["sample_text"] = self._decode(s["sample_ids"])
            return s

        async def finish_child(s: Dict[str, Any]) -> Dict[str, Any]:
            """Reward and old-policy log-probabilities of one finished sample, concurrently."""
            lp_task = asyncio.ensure_future(self.logprob_fn({"sample_ids": s["sample_ids"], "input_len": s["input_len"],
                                                             "output_len": s["output_len"]}))
            v = await self.verifier.verify(s, max_gen_length=cap)
            try:
                lp = await lp_task
                v["sample_logprobs"], v["sample_entropies"] = lp["sample_logprobs"], lp["sample_entropies"]
                v["logprobs_attached"] = True
            except Exception as e:  # the experience manager's own logprob stage picks the sample up instead
                logger.warning("streamed logprob request failed (%r); deferring to the group stage", e)
            return v

        if self.logprob_fn is not None:
            tasks: Dict[int, Any] = {}
            finished = await self._generate(prompt, int(n), max_new, float(temperature), seed, forced,
                                            on_child=lambda f: tasks.__setitem__(f.child, asyncio.ensure_future(finish_child(build(f)))))
            verified = list(await asyncio.gather(*[tasks[f.child] for f in finished]))
        else:
            finished = await self._generate(prompt, int(n), max_new, float(temperature), seed, forced)
            verified = list(await asyncio.gather(*[self.verifier.verify(build(f), max_gen_length=cap) for f in finished]))
        rewards = [float(v.get("reward", 0.0)) for v in verified]
        adv = normalize_rewards(rewards)
        mx = max(rewards) if rewards else 0.0
        for v, a in zip(verified, adv):
            v["advantage"] = float(a)
            v["max_reward_in_group"] = mx
        total_tokens = int(sum(len(f.output_ids) for f in finished))
        self.total_tokens += total_tokens
        metrics = {
            "generation/total_tokens_generated": float(total_tokens),
            "generation/inference_duration_sec": time.time() - t0,
            "generation/num_samples_generated": float(len(finished)),
        }
        return list(verified), metrics

    async def batch_inference_for_evaluation(self, prompts: Sequence[Any], answers: Sequence[Any], max_tokens: int = 1024,
                                             temperature: float = 0.0) -> List[Dict[str, Any]]:
        """Greedy (by default) completions with worker-side reward (vllm_worker.py:525-668). All prompts go to the
        engine at once (it batches continuously); ASYNC_GRPO_EVAL_CONCURRENCY, when set, bounds how many are in flight
        (the reference bounds its evaluation RPCs the same way, orchestrator.py:1291)."""
        import os

        limit = int(os.environ.get("ASYNC_GRPO_EVAL_CONCURRENCY", "0") or 0)
        gate = asyncio.Semaphore(limit) if limit > 0 else None

        async def one(i: int, prompt: Any, answer: Any) -> Dict[str, Any]:
            if gate is None:
                return await run_one(i, prompt, answer)
            async with gate:
                return await run_one(i, prompt, answer)

        async def run_one(i: int, prompt: Any, answer: Any) -> Dict[str, Any]:
            if isinstance(prompt, str):
                if self.tokenizer is None:
                    raise RuntimeError("a tokenizer is required for text prompts")
                ids = np.asarray(self.tokenizer.encode(prompt, add_special_tokens=False), dtype=np.int32)
                text = prompt
            else:
                ids = np.asarray(prompt, dtype=np.int32)
                text = self._decode(ids)
            fin = await self._generate(ids, 1, self.get_max_tokens(len(ids), max_tokens), float(temperature), _uid_seed(("eval", i), 0))
            eos = int(getattr(self.engine, "eos", self.mcfg.eos_token_id))
            s = build_sample({"input": text, "input_token_ids": ids, "answer": answer}, ids, fin[0].output_ids, eos)
            s["sample_text"] = self._decode(s["sample_ids"])
            s["vocab_size"] = self.mcfg.vocab_size
            v = await self.verifier.verify(s)
            return {"prompt": text, "completion": self._decode(fin[0].output_ids), "answer": answer,
                    "reward": float(v.get("reward", 0.0)), "output_len": int(len(fin[0].output_ids))}

        return list(await asyncio.gather(*[one(i, p, a) for i, (p, a) in enumerate(zip(prompts, answers))]))

    async def generate_with_logprobs(self, prompt_ids: Sequence[int], max_tokens: int = 32, temperature: float = 1.0,
                                     seed: int = 0) -> Dict[str, Any]:
        """Probe: sampled token ids with the engine's own log-probability of each (under the sampling temperature), so
        that trainer / logprob-worker values can be compared with the engine's numerics (vllm_worker.py:286-392). The
        first call switches the engine to recording log-probabilities."""
        ids = np.asarray(prompt_ids, dtype=np.int32)
        self._want_logprobs = not getattr(self.engine, "record_logprobs", False)
        fin = await self._generate(ids, 1, self.get_max_tokens(len(ids), max_tokens), float(temperature), int(seed))
        return {"input_token_ids": ids, "output_token_ids": fin[0].output_ids, "output_logprobs": fin[0].output_logprobs,
                "finish_reason": fin[0].finish_reason}

    # ------------------------------------------------------------------ weight sync (receiver side)
    async def pause_for_sync(self) -> bool:
        """Stops stepping after the current step; returns once the engine thread is idle."""
        with self._gate:
            self._paused.set()
        self._wake.set()
        while not self._idle.is_set():
            await asyncio.sleep(0.001)
        if self.mirror is not None:
            self.mirror.send("pause")  # the followers hold here until their own rank's sync has finished
        return True

    async def resume_after_sync(self) -> bool:
        self.engine.update_weights_done()
        self._paused.clear()
        self._wake.set()
        return True

    async def is_ready(self) -> bool:
        return True

    def stats(self) -> Dict[str, float]:
        out = {"total_tokens": float(self.total_tokens), "busy_seconds": self.busy_seconds,
               "launches": float(getattr(self.engine, "launches", 0))}
        if hasattr(self.engine, "timing_stats"):
            out.update(self.engine.timing_stats())
        return out

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        if self.mirror is not None:
            self.mirror.close()


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
