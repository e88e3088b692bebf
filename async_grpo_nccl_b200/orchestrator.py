"""Orchestrator: the single coordinator of a run.

Same public surface as the reference's Ray actor (orchestrator.py:196-1434) without Ray:

    orch = Orchestrator(config_dict=cfg)     # flat config dict, same keys
    orch.run()                               # staged init, epoch / macro-batch loop, eval, checkpoints

plus ``sync_all_weights``, ``run_evaluation`` and ``save_checkpoint``. The roles behind it are created by
:mod:`async_grpo_nccl_b200.launch` either inside this process (one GPU or CPU) or as one process per GPU
reached through RPC proxies; the orchestrator only sees handles with async methods.

Loop per macro-batch (orchestrator.py:708-1251): start the per-prompt pipelines, let the
ExperienceManager cut minibatches while generation is still running, wait for every trainer rank's
completion (with a liveness check on timeout), aggregate and log, push the new weights to the logprob
and rollout ranks, evaluate / checkpoint when due. A failed weight sync raises instead of being skipped
(the reference logs it and keeps generating on stale weights, orchestrator.py:1190-1193).
"""
from __future__ import annotations

import asyncio
import hashlib
import json
import logging
import os
import time
from typing import Any, Dict, List, Optional, Sequence

from . import checkpoint as ckpt
from .config import GRPOConfig, make_config
from .metrics import MetricLogger, aggregate_completions
from .protocol import RoleLostError
from .utils.timing import profile_window

logger = logging.getLogger(__name__)


def configure_logging() -> None:
    """Root INFO (override with GRPO_LOGGING_LEVEL); chatty third-party loggers are lowered
    (gpu_process_worker.py:66-94)."""
    level = os.environ.get("GRPO_LOGGING_LEVEL", "INFO").upper()
    logging.basicConfig(level=getattr(logging, level, logging.INFO),
                        format="%(asctime)s %(name)s %(levelname)s %(message)s")
    for name in ("urllib3", "filelock", "huggingface_hub", "httpx", "h2", "transformers", "asyncio"):
        logging.getLogger(name).setLevel(logging.WARNING)


def load_jsonl(path: str) -> List[Dict[str, Any]]:
    rows = []
    with open(path, "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
    return rows


def stamp_uids(rows: Sequence[Dict[str, Any]], base_index: int = 0) -> List[Dict[str, Any]]:
    """``__uid__`` = dataset index, or a hash of the prompt when no index applies (orchestrator.py:784-789, 881-896)."""
    out = []
    for i, r in enumerate(rows):
        r = dict(r)
        if "__uid__" not in r:
            if "input" in r and base_index < 0:
                r["__uid__"] = hashlib.sha256(str(r["input"]).encode()).hexdigest()[:16]
            else:
                r["__uid__"] = base_index + i
        out.append(r)
    return out


class Orchestrator:
    def __init__(self, config_dict: Optional[Dict[str, Any]] = None, runtime: Any = None, dataset: Optional[Sequence[Dict[str, Any]]] = None,
                 eval_dataset: Optional[Sequence[Dict[str, Any]]] = None, **overrides: Any):
        self.config: GRPOConfig = config_dict if isinstance(config_dict, GRPOConfig) else make_config(config_dict, **overrides)
        self.runtime = runtime
        self.dataset = list(dataset) if dataset is not None else None
        self.eval_dataset = list(eval_dataset) if eval_dataset is not None else None
        self.global_step = 0
        self.total_samples_seen = 0
        self.macro_batch_count = 0
        self.last_eval_samples_seen = 0
        self.last_checkpoint_samples_seen = 0
        self.metrics = MetricLogger(self.config)
        self.step_records: List[Dict[str, Any]] = []
        self.max_macro_batches: Optional[int] = None  # test / bench hook: stop after this many macro-batches

    # ------------------------------------------------------------------ state
    def _load_training_state(self) -> None:
        st = ckpt.load_training_state(self.config.output_dir) if self.config.output_dir else None
        if st:
            self.global_step = int(st.get("global_step", 0))
            self.total_samples_seen = int(st.get("total_samples_seen", 0))
            self.macro_batch_count = int(st.get("macro_batch_count", 0))
            self.last_eval_samples_seen = int(st.get("last_eval_samples_seen", 0))
            self.last_checkpoint_samples_seen = self.total_samples_seen

    def _save_training_state(self) -> None:
        if self.config.output_dir:
            ckpt.save_training_state(self.config.output_dir, {
                "global_step": self.global_step, "total_samples_seen": self.total_samples_seen,
                "macro_batch_count": self.macro_batch_count, "last_eval_samples_seen": self.last_eval_samples_seen})

    # ------------------------------------------------------------------ public entry points
    def run(self) -> Dict[str, Any]:
        """Blocking run. Builds an in-process runtime when none was supplied."""
        configure_logging()
        if self.runtime is None:
            from .launch import build_inprocess_runtime

            self.runtime = build_inprocess_runtime(self.config)
        return asyncio.run(self.run_async())

    async def run_async(self) -> Dict[str, Any]:
        if self.config.resume_state:
            self._load_training_state()
        await self.runtime.initialize(self)
        if self.config.verify_weight_sync_during_init:
            await self._verify_trainer_logprob_sync()
        try:
            return await self._run_training_loop()
        finally:
            await self.runtime.shutdown()

    async def sync_all_weights(self) -> float:
        """Pushes trainer weights to every logprob and rollout rank; returns the wall time in ms."""
        t0 = time.time()
        await self.runtime.sync_weights()
        return (time.time() - t0) * 1000.0

    async def _verify_trainer_logprob_sync(self) -> None:
        """Debug check: trainer and logprob parameters must be identical after a sync (orchestrator.py:642-706)."""
        mismatches = await self.runtime.verify_weight_sync()
        if mismatches:
            raise RuntimeError(f"weight sync verification failed: {mismatches[:20]}")
        logger.info("weight sync verified: trainer and logprob parameters are identical")

    # ------------------------------------------------------------------ main loop
    async def _run_training_loop(self) -> Dict[str, Any]:
        cfg, rt = self.config, self.runtime
        em = rt.experience_manager
        for rank in rt.trainer_ranks:
            await _maybe(em.register_training_process(rank, cfg.max_tokens_per_gpu, cfg.train_minibatch_sample_size))
        await rt.start_trainers()
        rows = self.dataset if self.dataset is not None else load_jsonl(cfg.data_path)
        rows = stamp_uids(rows)
        n_batches = (len(rows) + cfg.batch_size - 1) // cfg.batch_size
        if cfg.eval_at_start and (cfg.test_data_path or self.eval_dataset):
            await self.run_evaluation()
        start_epoch = self.macro_batch_count // max(1, n_batches)
        start_offset = self.macro_batch_count % max(1, n_batches)
        done = False
        for epoch in range(start_epoch, cfg.num_epochs):
            for b in range(n_batches):
                if epoch == start_epoch and b < start_offset:
                    continue  # resume: fast-forward the data order (orchestrator.py:826-866)
                batch = rows[b * cfg.batch_size:(b + 1) * cfg.batch_size]
                # opt-in torch.profiler trace (host + CUDA activity of this process) of one macro-batch
                with profile_window(cfg.profile_trace_path, active=len(self.step_records) == cfg.profile_macro_batch):
                    rec = await self._run_macro_batch(batch, epoch)
                self.step_records.append(rec)
                if self.max_macro_batches is not None and len(self.step_records) >= self.max_macro_batches:
                    done = True
                    break
            if done:
                break
        return {"global_step": self.global_step, "total_samples_seen": self.total_samples_seen, "steps": self.step_records}

    async def _wait_completions(self) -> List[Dict[str, Any]]:
        cfg, rt = self.config, self.runtime
        em = rt.experience_manager
        out = []
        for rank in rt.trainer_ranks:
            while True:
                try:
                    c = await asyncio.wait_for(_maybe(em.get_completion(rank)), cfg.trainer_completion_timeout_s)
                    break
                except asyncio.TimeoutError:
                    alive = await rt.ping_trainers()
                    if not all(alive):
                        self._save_training_state()
                        raise RoleLostError(f"trainer ranks not responding: {[r for r, a in zip(rt.trainer_ranks, alive) if not a]}; "
                                            f"training state saved, restart with resume_state")
                    logger.warning("still waiting for trainer rank %s (all ranks alive)", rank)
            if isinstance(c, dict) and c.get("error"):
                raise RuntimeError(f"trainer rank {c.get('gpu_rank')} failed: {c['error']}")
            out.append(c)
        return out

    async def _run_macro_batch(self, batch: Sequence[Dict[str, Any]], epoch: int) -> Dict[str, Any]:
        cfg, rt = self.config, self.runtime
        em = rt.experience_manager
        t_start = time.time()
        await _maybe(em.generate_experience(list(batch), rt.generation_controllers, rt.logprob_controllers))
        em.start_creating_batches()
        completions = await self._wait_completions()
        lost = list(getattr(em, "role_failures", []))
        if lost:
            # a role process is gone: nothing of this macro-batch is committed (no weight sync with a dead rank, which
            # would block every collective); the counters of the last completed macro-batch are what a restart resumes from
            self._save_training_state()
            raise RoleLostError(f"{len(lost)} request(s) failed because a role process is unreachable ({lost[0]}); "
                                f"training state saved at macro-batch {self.macro_batch_count}, restart with resume_state")
        t_trained = time.time()
        agg = aggregate_completions(completions)
        n_samples = int(agg.get("training/batch_total_samples", 0))
        self.global_step += 1
        self.macro_batch_count += 1
        self.total_samples_seen += n_samples
        sync_ms = 0.0
        if self.macro_batch_count % cfg.weight_sync_every == 0:
            sync_ms = await self.sync_all_weights()
            if cfg.verify_weight_sync_during_init:  # debug flag: re-check after every sync as well
                await self._verify_trainer_logprob_sync()
        total_time = time.time() - t_start
        glm = completions[0].get("gen_logprob_metrics", {}) if completions else {}
        gen_tokens = float(glm.get("generation/total_tokens_generated", 0.0))
        n_prompts = max(1.0, float(glm.get("num_prompts", 1.0)))
        exp = completions[0].get("exp_batch_metrics", {}) if completions else {}
        wall_gen = float(glm.get("gen_logprob_wall_time", 0.0))
        trainer_active = max(0.0, t_trained - t_start - wall_gen) if wall_gen else 0.0
        rec: Dict[str, Any] = dict(agg)
        rec.update({
            "trainer_step": self.global_step, "epoch": epoch,
            "training/samples_per_second": n_samples / total_time if total_time > 0 else 0.0,
            "timing/1_total_batch_time": total_time,
            "timing/2_gen_logprob_wall_time": wall_gen,
            "timing/2a_generation_time": float(glm.get("gen_duration", 0.0)) / n_prompts,
            "timing/2b_logprob_time": float(glm.get("logprob_duration", 0.0)) / n_prompts,
            "timing/3_trainer_active_time": trainer_active,
            "timing/4_total_overhead": max(0.0, total_time - wall_gen - trainer_active),
            "timing/weight_sync_ms": sync_ms,
            # device time of the push itself (CUDA events, max over ranks); the figure above is the host's wall clock
            # around pausing the roles, the RPC fan-out and the push
            "timing/weight_sync_device_ms": float(getattr(rt, "sync_device_ms_max", getattr(rt, "sync_device_ms", 0.0)) or 0.0)
            if sync_ms else 0.0,
            "generation/total_tokens_generated": gen_tokens,
            "generation/inference_duration_sec": float(glm.get("generation/inference_duration_sec", 0.0)),
            "generation/num_samples_generated": float(glm.get("generation/num_samples_generated", 0.0)),
            "generation/inference_throughput_tok_per_sec": gen_tokens / total_time if total_time > 0 else 0.0,
        })
        for k, v in exp.items():
            if isinstance(v, (int, float)):
                rec[f"reward/{k}"] = float(v)
        if cfg.enable_manual_system_metrics:
            from .metrics import system_metrics

            rec.update(system_metrics())
        if cfg.enable_prefix_caching and hasattr(rt, "collect_stats"):
            try:  # share of prompt tokens whose keys / values came from the prefix cache (cumulative over the run)
                st = await rt.collect_stats()
                if st.get("engine_prefix_lookup_tokens", 0.0) > 0:
                    rec["generation/prefix_cache_hit_rate"] = st["engine_prefix_hit_tokens"] / st["engine_prefix_lookup_tokens"]
            except Exception as e:  # statistics never stop a run
                logger.debug("engine statistics unavailable: %r", e)
        self.metrics.log(rec, step=self.global_step)
        for c in completions[:1]:
            for i, s in enumerate(c.get("minibatch_summaries", [])):
                self.metrics.log({"minibatch_step": s.get("optimizer_step", i), **{f"minibatch/{k}": v for k, v in s.items()
                                                                                  if isinstance(v, (int, float))}})
        logger.info("step %d | samples %d | %.2f samples/s | loss %.5f | grad_norm %.4f | reward %.4f | sync %.1f ms",
                    self.global_step, n_samples, rec["training/samples_per_second"], rec.get("training/avg_loss", 0.0),
                    rec.get("training/grad_norm", 0.0), rec.get("training/batch_avg_reward", 0.0), sync_ms)
        if cfg.eval_every_n_macro_batches > 0 and self.macro_batch_count % cfg.eval_every_n_macro_batches == 0 \
                and (cfg.test_data_path or self.eval_dataset):
            await self.run_evaluation()
        if cfg.output_dir and self.total_samples_seen - self.last_checkpoint_samples_seen >= cfg.min_samples_per_checkpoint:
            await self.save_checkpoint()
        return rec

    # ------------------------------------------------------------------ evaluation
    async def run_evaluation(self) -> Dict[str, float]:
        cfg, rt = self.config, self.runtime
        rows = self.eval_dataset if self.eval_dataset is not None else load_jsonl(cfg.test_data_path)
        prompts = [r.get("input_token_ids", r.get("prompt", r.get("input"))) for r in rows]
        answers = [r.get("answer", r.get("label")) for r in rows]
        ctrls = rt.generation_controllers
        shards: List[List[int]] = [[] for _ in ctrls]
        for i in range(len(rows)):
            shards[i % len(ctrls)].append(i)
        results = await asyncio.gather(*[
            _maybe(c.batch_inference_for_evaluation([prompts[i] for i in idx], [answers[i] for i in idx],
                                                    cfg.max_generation_tokens, 0.0))
            for c, idx in zip(ctrls, shards) if idx])
        rewards = [float(r["reward"]) for rs in results for r in rs]
        acc = sum(rewards) / len(rewards) if rewards else 0.0
        out = {"eval/accuracy": acc, "eval/num_samples": float(len(rewards)), "trainer_step": self.global_step}
        self.metrics.log(out, step=self.global_step)
        self.last_eval_samples_seen = self.total_samples_seen
        logger.info("evaluation: accuracy %.4f over %d samples", acc, len(rewards))
        return out

    # ------------------------------------------------------------------ checkpoints
    async def save_checkpoint(self) -> Optional[str]:
        cfg = self.config
        if not cfg.output_dir:
            return None
        path = ckpt.checkpoint_dir(cfg.output_dir, self.global_step, self.total_samples_seen)
        await self.runtime.save_checkpoint(path)
        self.last_checkpoint_samples_seen = self.total_samples_seen
        self._save_training_state()
        ckpt.prune_checkpoints(cfg.output_dir, cfg.keep_last_n_checkpoints)
        logger.info("checkpoint written to %s", path)
        return path


async def _maybe(x: Any) -> Any:
    """Awaits coroutines / futures, passes plain values through (local objects and RPC proxies look the same)."""
    if asyncio.iscoroutine(x) or isinstance(x, asyncio.Future):
        return await x
    return x


def main() -> None:
    """Smoke launch with defaults on the tiny preset and a synthetic dataset (orchestrator.py:1437-1462)."""
    from .data import synthetic_prompt_rows

    cfg = make_config({"model_name_or_path": "tiny", "batch_size": 4, "samples_per_question": 4, "num_epochs": 1,
                       "train_minibatch_sample_size": 8, "max_generation_tokens": 16, "max_tokens_per_gpu": 2048,
                       "reward_fns": ["token_match"], "global_num_verifiers": 0, "num_training_gpu_workers": 1})
    orch = Orchestrator(cfg, dataset=synthetic_prompt_rows(8, 1024, 8, 16, seed=0))
    print(json.dumps(orch.run()["steps"][-1], indent=2, default=float))


if __name__ == "__main__":
    main()
