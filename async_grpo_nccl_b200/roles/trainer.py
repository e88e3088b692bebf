"""Trainer rank: sharded optimizer state, microbatch forward/backward, optimizer step, checkpoints.

Behaviour follows the reference's ``TrainerGPUWorker`` (gpu_process_worker.py:801-1640):
``compute_gradients`` per MICROBATCH with the loss scaled so that the update is the mean over all
samples of the minibatch on all ranks, ``apply_gradients`` per GRADIENT_STEP (global-norm clip 1.0,
AdamW, LR schedule, zero grads), token-weighted metric aggregation per BATCH_DONE, HF-format
checkpoints plus optimizer / scheduler state, and being the source of the weight sync.

B200-first differences:
* parameters live in one flat buffer (see models/layout.py); fp32 master weights and Adam moments are
  sharded over the trainer ranks, the bf16 compute copy is resident on every rank when it fits in HBM
  (ZeRO-2 style: 180 GB per GPU make re-gathering every layer twice per microbatch unnecessary for
  models up to ~30B parameters);
* gradients accumulate locally in fp32 over all microbatches of an optimizer step and are reduced ONCE
  per step (the reference's FSDP2 reduces every microbatch, gpu_process_worker.py:1041);
* the diagnostics are sums produced by the loss kernel and read with one device-to-host copy per
  optimizer step instead of ~15 ``.item()`` syncs per microbatch (grpo_loss.py:410-483);
* the reference's per-step summaries are zeroed before they are aggregated
  (gpu_process_worker.py:1412-1415); here they are aggregated first.
"""
from __future__ import annotations

import math
import os
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..config import GRPOConfig
from ..models.config import ModelConfig
from ..models.decoder import GradSink, LossConfig, NativeDecoder, OracleDecoder
from ..models.layout import ParamLayout
from ..ops import reference as R
from ..packing import pack_samples


def lr_factor(step: int, warmup: int, total: int, kind: str) -> float:
    """Learning-rate factor of optimizer step ``step`` (0-based): the reference's ``LambdaLR`` lambda, term for term
    (gpu_process_worker.py:734-741). Linear warm-up from 0 (its first step has learning rate 0 when warm-up is on), then
    constant, or cosine over ``total`` steps when ``total > 0`` (not clamped past ``total``, as in the reference)."""
    if warmup > 0 and step < warmup:
        return float(step) / float(max(1, warmup))
    if kind == "cosine" and total > 0:
        prog = float(step - warmup) / float(max(1, total - warmup))
        return 0.5 * (1.0 + math.cos(math.pi * prog))
    return 1.0


class TrainerCore:
    def __init__(self, cfg: GRPOConfig, mcfg: ModelConfig, device: torch.device, rank: int = 0, world: int = 1,
                 group: Any = None, init_flat_fp32: Optional[torch.Tensor] = None, seed: int = 0,
                 comm: Any = None):
        self.cfg, self.mcfg = cfg, mcfg
        self.device = torch.device(device)
        self.rank, self.world, self.group = rank, world, group
        self.native = self.device.type == "cuda"
        self.layout = ParamLayout(mcfg, shard_world=world)
        self.compute_dtype = torch.bfloat16 if self.native else torch.float32
        L = self.layout
        if init_flat_fp32 is None:
            init_flat_fp32 = torch.empty(L.total, dtype=torch.float32)
            L.init_random_(init_flat_fp32, seed)
        assert init_flat_fp32.numel() == L.total
        # resident compute copy (bf16 on GPU). With a peer-memory communicator (parallel/symm.py::TrainerComm) the
        # parameter and gradient buffers are symmetric allocations that the other trainer ranks read and write.
        self.comm = comm
        self.zero3 = bool(getattr(comm, "zero3", False))
        if self.zero3:
            self.params = None  # fully sharded: no resident copy, units are gathered on use (parallel/zero3.py)
        elif comm is not None:
            self.params = comm.param_buffer
            self.params.copy_(init_flat_fp32.to(self.compute_dtype))
        else:
            self.params = init_flat_fp32.to(self.device, dtype=self.compute_dtype)
        self.fallback = None
        if world > 1 and comm is None:
            from ..parallel.symm import CollectiveFallback

            self.fallback = CollectiveFallback(group, L, rank, world)
        # sharded fp32 master + moments
        self.shard_map = L.local_to_global_ranges(rank)
        n = L.shard_numel()
        self.master = torch.empty(n, dtype=torch.float32, device=self.device)
        for lo, gs, ln in self.shard_map:
            self.master[lo:lo + ln].copy_(init_flat_fp32[gs:gs + ln])
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        recompute = cfg.activation_recompute == "full"
        if self.zero3:
            assert self.native, "fully sharded mode runs on GPUs"
            self.grad_shard = comm.grad_shard
            self.sink = comm.sink
            comm.shard16.copy_(self.master)  # fp32 -> bf16 slice that the peers gather from
            comm.publish_initial()
        else:
            self.grad_shard = torch.zeros_like(self.master) if world > 1 else None
            self.sink = GradSink(L, self.device, flat=comm.grad_buffer if comm is not None else None)
        if self.zero3:
            self.decoder = NativeDecoder(mcfg, L, None, recompute=recompute, weights=comm.weights)
            self.norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        elif self.native:
            self.decoder = NativeDecoder(mcfg, L, self.params, recompute=recompute)
            self.norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        else:
            self._oracle_params = self.params.clone().requires_grad_(True)
            self.decoder = OracleDecoder(mcfg, L, self._oracle_params)
            self.norm_sq = torch.zeros(1, dtype=torch.float32)
        self.loss_cfg = LossConfig(cfg.clip_low, cfg.clip_high, cfg.clip_ratio_c, cfg.kl_beta, cfg.temperature,
                                   cfg.entropy_coeff, cfg.apply_entropy_bonus)
        self.opt_step = 0
        self.base_lr = cfg.learning_rate
        n_stats = len(R.LOSS_STAT_NAMES)
        self._stats_step = torch.zeros(n_stats, dtype=torch.float32, device=self.device)
        self._stats_mb: List[Tuple[torch.Tensor, Dict[str, float]]] = []
        self._mb_step_buffer: List[Dict[str, float]] = []
        self._reset_batch_accumulators()
        self.last_grad_norm = 0.0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # device-timed phases (CUDA events on this role's stream, NVTX ranges for a profiler), read once per macro-batch
        from ..utils.timing import PhaseTimer

        self.timer = PhaseTimer(cuda=self.native)

    # ------------------------------------------------------------------ metrics plumbing
    def _reset_batch_accumulators(self) -> None:
        self._mb_summaries: List[Dict[str, float]] = []
        self._step_summaries: List[Dict[str, float]] = []
        self._mb_pending: List[Dict[str, Any]] = []
        self._grad_norms: List[float] = []
        self._grad_steps = 0
        self._clipped_steps = 0

    def current_lr(self) -> float:
        return self.base_lr * lr_factor(self.opt_step, self.cfg.lr_warmup_steps, self.cfg.total_steps(), self.cfg.lr_scheduler)

    # ------------------------------------------------------------------ MICROBATCH
    def compute_gradients(self, samples: Sequence[Dict[str, Any]]) -> None:
        """Forward + backward of one microbatch; gradients accumulate locally. No host sync on the native path."""
        real = [s for s in samples if not s.get("dummy", False)]
        n_real = len(real)
        if n_real == 0 and self.world == 1:
            return  # single rank, nothing to do (gpu_process_worker.py:975-985)
        with self.timer.phase("pack_h2d"):
            batch_host = pack_samples(samples if n_real else [{"dummy": True}], pin=self.native)
            self.h2d_bytes += batch_host.h2d_bytes()
            batch = batch_host.to_device(self.device)
        # scale so that the sum over microbatches and ranks is (1/N) * sum_mb n_mb * tokenmean_mb
        loss_scale = float(n_real) / float(self.cfg.train_minibatch_sample_size)
        if self.native:
            with self.timer.phase("forward_backward"):
                stats = self.decoder.forward_backward(batch, self.loss_cfg, loss_scale, self.sink)
            if self.cfg.kernel_checks:
                self.decoder.check_status()  # one synchronisation per microbatch: a failed kernel is named right away
        else:
            loss, stats = self.decoder.loss(batch, self.loss_cfg, loss_scale)
            if n_real > 0 and batch.total_out > 0:
                loss.backward()
                self.sink.flat.add_(self._oracle_params.grad.float())
                self._oracle_params.grad = None
        rewards = [float(s.get("reward", 0.0)) for s in real]
        self._mb_pending.append({"stats": stats, "num_samples": n_real, "total_reward": float(sum(rewards)),
                                 "index": len(self._mb_pending) + len(self._mb_summaries)})

    def _drain_pending(self) -> None:
        """One device-to-host copy for all microbatches since the last drain."""
        if not self._mb_pending:
            return
        stacked = torch.stack([p["stats"].float() for p in self._mb_pending]).cpu().numpy()
        self.d2h_bytes += stacked.nbytes
        for row, p in zip(stacked, self._mb_pending):
            n_tok = float(row[0])
            token_mean = float(row[1]) / max(1.0, n_tok)
            m = R.stats_to_metrics(row, token_mean, p["num_samples"], self.cfg.entropy_coeff)
            # the reference subtracts entropy_coeff * (mean entropy of the output tokens) from the microbatch loss it
            # reports and back-propagates (grpo_loss.py:500-508); its entropy is detached, so only the reported value moves
            bonus = (float(self.cfg.entropy_coeff) * m["entropy"]
                     if (self.cfg.apply_entropy_bonus and float(self.cfg.entropy_coeff) != 0.0 and n_tok > 0) else 0.0)
            summ = {
                "tokens": n_tok, "loss_sum": token_mean * n_tok - bonus, "kl_mean": m["kl_div"], "entropy_mean": m["entropy"],
                "minibatch_index": p["index"], "log_ratio_mean": m["log_ratio_mean"], "log_ratio_std": m["log_ratio_std"],
                "clipfrac_upper": m["clipfrac_upper"], "clipfrac_lower": m["clipfrac_lower"], "adv_mean": m["adv_mean"],
                "adv_std": m["adv_std"], "adv_pos_frac": m["adv_pos_frac"], "adv_zero_frac": m["adv_zero_frac"],
                "old_policy_entropy": m["old_policy_entropy"], "approx_kl": m["approx_kl"], "kl_ref": m["kl_ref"],
                "avg_reward": p["total_reward"] / p["num_samples"] if p["num_samples"] else 0.0,
                "total_reward": p["total_reward"], "total_samples": p["num_samples"],
            }
            self._mb_summaries.append(summ)
            self._mb_step_buffer.append(summ)
        self._mb_pending = []

    # ------------------------------------------------------------------ GRADIENT_STEP
    def apply_gradients(self) -> Dict[str, float]:
        with self.timer.phase("optimizer_step"):
            return self._apply_gradients()

    def _apply_gradients(self) -> Dict[str, float]:
        """Reduce gradients over the trainer ranks, clip by global norm, AdamW on the local shard, publish the bf16
        result into every rank's resident parameter buffer, zero gradients."""
        cfg = self.cfg
        self.opt_step += 1
        lr = self.base_lr * lr_factor(self.opt_step - 1, cfg.lr_warmup_steps, cfg.total_steps(), cfg.lr_scheduler)
        hp = (lr, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, cfg.weight_decay, self.opt_step)
        if self.world == 1:
            g = self.sink.flat
            self.norm_sq.zero_()
            if self.native:
                C = self.decoder.C
                C.sumsq(g, 1.0, self.norm_sq)
                # the master covers the whole buffer: the kernel writes the bf16 compute copy in place and zeroes g
                C.adamw_step(self.master, self.exp_avg, self.exp_avg_sq, g, self.params, *hp, 1.0, self.norm_sq,
                             cfg.max_grad_norm, True)
                self.decoder.launches += 2
            else:
                self.norm_sq.add_(g.pow(2).sum())
                R.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, g, *hp, 1.0, cfg.max_grad_norm, self.norm_sq)
                self.params.copy_(self.master.to(self.compute_dtype))
                self.sink.zero_()
            norm_sq_dev = self.norm_sq
        elif self.zero3:
            # fully sharded path: the gradient shard already holds the sum over ranks and microbatches (GEMM epilogues
            # reduced into it); barrier, norm exchange, AdamW on the shard, barrier
            partials = self.comm.step(self.master, self.exp_avg, self.exp_avg_sq, *hp, cfg.max_grad_norm)
            self.decoder.launches += 6
            norm_sq_dev = partials.sum()
        elif self.comm is not None:
            # peer-memory path: pull-reduce my shard out of every rank's gradient buffer, exchange norm partials,
            # AdamW + store the bf16 shard into every rank's parameter buffer - three fused kernels, no NCCL call
            self.comm.reduce_scatter(self.grad_shard)
            partials = self.comm.adamw_and_publish(self.master, self.exp_avg, self.exp_avg_sq, self.grad_shard, *hp,
                                                   cfg.max_grad_norm)
            self.decoder.launches += 2 * len(self.shard_map) + 4
            norm_sq_dev = partials.sum()
        else:
            fb = self.fallback
            fb.reduce_scatter(self.sink.flat, self.grad_shard)
            self.norm_sq.zero_()
            if self.native:
                C = self.decoder.C
                C.sumsq(self.grad_shard, 1.0, self.norm_sq)
            else:
                self.norm_sq.add_(self.grad_shard.pow(2).sum())
            fb.all_reduce_scalar(self.norm_sq)
            if not hasattr(self, "_shard16") or self._shard16 is None:
                self._shard16 = torch.empty(self.master.numel(), dtype=self.compute_dtype, device=self.device)
            if self.native:
                C.adamw_step(self.master, self.exp_avg, self.exp_avg_sq, self.grad_shard, self._shard16, *hp, 1.0, self.norm_sq,
                             cfg.max_grad_norm, True)
                self.decoder.launches += 2
            else:
                R.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, self.grad_shard, *hp, 1.0, cfg.max_grad_norm, self.norm_sq)
                self._shard16.copy_(self.master.to(self.compute_dtype))
                self.grad_shard.zero_()
            fb.all_gather_params(self._shard16, self.params)
            self.sink.zero_()
            norm_sq_dev = self.norm_sq
        if not self.native:
            with torch.no_grad():
                self._oracle_params.copy_(self.params)
        # one small read per optimizer step: grad norm + the microbatch statistics
        self._mb_step_buffer = []
        self._drain_pending()
        grad_norm = float(norm_sq_dev.sqrt().item())
        self.d2h_bytes += 4
        self.last_grad_norm = grad_norm
        self._grad_norms.append(grad_norm)
        self._grad_steps += 1
        if cfg.max_grad_norm > 0 and grad_norm > cfg.max_grad_norm:
            self._clipped_steps += 1
        step_summary = self._aggregate(self._mb_step_buffer)
        step_summary.update(grad_norm=grad_norm, lr=lr, optimizer_step=self.opt_step)
        self._step_summaries.append(step_summary)
        if self.native:
            self.decoder.check_status()
            if self.comm is not None:
                self.comm.pg.check()
        return step_summary

    # ------------------------------------------------------------------ BATCH_DONE
    @staticmethod
    def _aggregate(summaries: Sequence[Dict[str, float]]) -> Dict[str, float]:
        """Token-weighted means; mean/std pairs are merged through second moments (gpu_process_worker.py:831-900)."""
        denom = sum(s["tokens"] for s in summaries)
        out: Dict[str, float] = {"tokens": float(denom), "num_microbatches": float(len(summaries))}
        if denom <= 0:
            for k in ("loss", "kl_div", "entropy", "log_ratio_mean", "log_ratio_std", "clipfrac_upper", "clipfrac_lower",
                      "adv_mean", "adv_std", "adv_pos_frac", "adv_zero_frac", "old_policy_entropy", "approx_kl", "kl_ref"):
                out[k] = 0.0
            out["total_reward"] = sum(s.get("total_reward", 0.0) for s in summaries)
            out["total_samples"] = sum(s.get("total_samples", 0) for s in summaries)
            out["avg_reward"] = out["total_reward"] / out["total_samples"] if out["total_samples"] else 0.0
            return out

        def wmean(key: str) -> float:
            return sum(s.get(key, 0.0) * s["tokens"] for s in summaries) / denom

        def merged_std(mean_key: str, std_key: str) -> Tuple[float, float]:
            mean = wmean(mean_key)
            second = sum((s.get(std_key, 0.0) ** 2 + s.get(mean_key, 0.0) ** 2) * s["tokens"] for s in summaries) / denom
            return mean, math.sqrt(max(0.0, second - mean * mean))

        out["loss"] = sum(s["loss_sum"] for s in summaries) / denom
        out["kl_div"] = wmean("kl_mean")
        out["entropy"] = wmean("entropy_mean")
        out["log_ratio_mean"], out["log_ratio_std"] = merged_std("log_ratio_mean", "log_ratio_std")
        out["adv_mean"], out["adv_std"] = merged_std("adv_mean", "adv_std")
        for k in ("clipfrac_upper", "clipfrac_lower", "adv_pos_frac", "adv_zero_frac", "old_policy_entropy", "approx_kl", "kl_ref"):
            out[k] = wmean(k)
        out["total_reward"] = sum(s.get("total_reward", 0.0) for s in summaries)
        out["total_samples"] = sum(s.get("total_samples", 0) for s in summaries)
        out["avg_reward"] = out["total_reward"] / out["total_samples"] if out["total_samples"] else 0.0
        return out

    def finish_batch(self, batch_done_data: Optional[Dict[str, Any]], iteration: int) -> Dict[str, Any]:
        """Completion payload for the orchestrator (keys as in gpu_process_worker.py:1521-1534)."""
        self._drain_pending()
        data = batch_done_data or {}
        agg = self._aggregate(self._mb_summaries)
        metrics = {
            "loss": agg["loss"], "loss_per_token": agg["loss"], "kl_div": agg["kl_div"], "entropy": agg["entropy"],
            "token_count": int(agg["tokens"]), "log_ratio_mean": agg["log_ratio_mean"], "log_ratio_std": agg["log_ratio_std"],
            "clipfrac_upper": agg["clipfrac_upper"], "clipfrac_lower": agg["clipfrac_lower"], "adv_mean": agg["adv_mean"],
            "adv_std": agg["adv_std"], "adv_pos_frac": agg["adv_pos_frac"], "adv_zero_frac": agg["adv_zero_frac"],
            "old_policy_entropy": agg["old_policy_entropy"], "approx_kl": agg["approx_kl"], "kl_ref": agg["kl_ref"],
            "grad_norm": sum(self._grad_norms) / len(self._grad_norms) if self._grad_norms else 0.0,
            "lr": self.current_lr(),
        }
        batch_metrics = {"avg_reward": agg["avg_reward"], "total_reward": agg["total_reward"],
                         "total_samples": agg["total_samples"]}
        exp = data.get("batch_metrics", {}) or {}
        for k in ("reward_mean", "reward_std", "reward_min", "reward_max", "group_reward_std_mean",
                  "group_reward_std_zero_frac", "nonzero_reward_frac", "avg_completion_length"):
            if k in exp:
                batch_metrics[k] = exp[k]
        payload = {
            "gpu_rank": self.rank,
            "metrics": metrics,
            "batch_metrics": batch_metrics,
            "gen_logprob_metrics": data.get("gen_logprob_metrics", {}),
            "iteration": iteration,
            "optimizer_steps_in_batch": self._grad_steps,
            "grad_clip_steps_in_batch": self._clipped_steps,
            "grad_clip_ratio_in_batch": self._clipped_steps / self._grad_steps if self._grad_steps else 0.0,
            "exp_batch_metrics": exp,
            "minibatch_summaries": [dict(s) for s in self._step_summaries],
            # device milliseconds of this rank's phases in this macro-batch (CUDA events on the trainer stream)
            "phase_ms": {k: float(v) for k, v in self.timer.summary().items()},
        }
        self._reset_batch_accumulators()
        return payload

    # ------------------------------------------------------------------ weights / checkpoints
    def full_master_fp32(self) -> Optional[torch.Tensor]:
        """Full fp32 parameters on rank 0 (collective when world > 1), None on other ranks."""
        if self.world == 1:
            return self.master
        import torch.distributed as dist

        full = torch.empty(self.layout.total, dtype=torch.float32, device=self.device)
        for u, (lo, gs, ln) in enumerate(self.shard_map):
            s, e = self.layout.unit_ranges[u]
            dist.all_gather_into_tensor(full[s:e], self.master[lo:lo + ln].contiguous(), group=self.group)
        return full if self.rank == 0 else None

    def sync_source(self) -> Tuple[Optional[torch.Tensor], bool]:
        """(bf16 tensor the weight sync reads from, whether it holds only this rank's slices)."""
        if self.zero3:
            return self.comm.shard16, True
        return self.params, False

    def param_checksum(self) -> float:
        if self.zero3:
            return float(self.comm.shard16.double().sum().item())
        return float(self.params.double().sum().item())

    def weights_info(self):
        return self.layout.weights_info()

    def optimizer_state(self) -> Dict[str, Any]:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    def scheduler_state(self) -> Dict[str, Any]:
        return {"opt_step": self.opt_step, "base_lr": self.base_lr, "lr_scheduler": self.cfg.lr_scheduler,
                "lr_warmup_steps": self.cfg.lr_warmup_steps, "total_steps": self.cfg.total_steps()}

    def load_scheduler_state(self, st: Dict[str, Any]) -> None:
        """Restores the position in the schedule. The base learning rate stays the one of the current configuration: a
        run resumed with another ``learning_rate`` uses it from its first step on."""
        self.opt_step = int(st.get("opt_step", 0))

    def _gather_full_master(self) -> torch.Tensor:
        """Full fp32 parameters on EVERY rank (collective over the trainer group when world > 1)."""
        if self.world == 1:
            return self.master
        import torch.distributed as dist

        full = torch.empty(self.layout.total, dtype=torch.float32, device=self.device)
        for u, (lo, gs, ln) in enumerate(self.shard_map):
            s, e = self.layout.unit_ranges[u]
            dist.all_gather_into_tensor(full[s:e], self.master[lo:lo + ln].contiguous(), group=self.group)
        return full

    def load_optimizer_checkpoint(self, path: str) -> bool:
        """Reloads this rank's fp32 master shard, Adam moments and the schedule position from a checkpoint directory
        (re-sharded when it was written by another number of trainer ranks) and rebuilds the compute copy from the
        masters; collective over the trainer group. What the reference does on resume (orchestrator.py:503-509 ->
        gpu_process_worker.py:1160-1223). Returns False when the directory holds no optimizer state."""
        from .. import checkpoint as ckpt

        st = ckpt.load_optimizer_shard(path, self.rank, self.world, self.layout)
        found = st is not None
        if self.world > 1:
            import torch.distributed as dist

            flag = torch.tensor([1 if found else 0], device=self.device if self.native else "cpu")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            found = bool(int(flag.item()))
        if not found:
            return False
        self.master.copy_(st["master"])
        self.exp_avg.copy_(st["exp_avg"])
        self.exp_avg_sq.copy_(st["exp_avg_sq"])
        sched = ckpt.load_scheduler_state(path)
        if sched:
            self.load_scheduler_state(sched)
        if self.zero3:
            self.comm.shard16.copy_(self.master)
            self.comm.publish_initial()
            return True
        full = self._gather_full_master()
        self.params.copy_(full.to(self.device, dtype=self.compute_dtype))
        if not self.native:
            with torch.no_grad():
                self._oracle_params.copy_(self.params)
        return True

    def load_master_from_full(self, full_fp32: torch.Tensor) -> None:
        for lo, gs, ln in self.shard_map:
            self.master[lo:lo + ln].copy_(full_fp32[gs:gs + ln])
        if self.zero3:
            self.comm.shard16.copy_(self.master)
            self.comm.publish_initial()
            return
        self.params.copy_(full_fp32.to(self.device, dtype=self.compute_dtype))
        if not self.native:
            with torch.no_grad():
                self._oracle_params.copy_(self.params)


class TrainerWorker:
    """Message loop of one trainer rank (gpu_process_worker.py:1233-1564): pulls MICROBATCH / GRADIENT_STEP /
    BATCH_DONE messages from the ExperienceManager and pushes the completion payload back. All device work
    runs on one worker thread so the asyncio loop keeps serving RPCs."""

    def __init__(self, core: TrainerCore, stream: Optional[torch.cuda.Stream] = None, sm_limit: int = 0):
        import concurrent.futures

        self.core = core
        self.stream = stream
        self.sm_limit = int(sm_limit)
        self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="trainer")
        self.manager: Any = None
        self.rank_in_manager = core.rank
        self.iteration = 0
        self._loop_task: Any = None
        self.running = False
        self.busy_seconds = 0.0
        self.last_error: Optional[str] = None

    def _run(self, fn, *args):
        t0 = time.time()
        try:
            if self.sm_limit > 0 and self.core.native:
                self.core.decoder.C.set_sm_limit(self.sm_limit)  # thread-local: this worker thread only
            if self.stream is not None:
                with torch.cuda.stream(self.stream):
                    return fn(*args)
            return fn(*args)
        finally:
            self.busy_seconds += time.time() - t0

    async def _exec(self, fn, *args):
        import asyncio

        return await asyncio.get_running_loop().run_in_executor(self._pool, self._run, fn, *args)

    def set_orchestrator(self, manager: Any, rank: int) -> bool:
        self.manager, self.rank_in_manager = manager, rank
        return True

    async def start_training_loop(self) -> bool:
        import asyncio

        if self._loop_task is None or self._loop_task.done():
            self.running = True
            self._loop_task = asyncio.ensure_future(self._training_loop())
        return True

    async def _training_loop(self) -> None:
        from ..protocol import Message, MessageType

        try:
            while self.running:
                msg = await self.manager.get_batch(self.rank_in_manager)
                if isinstance(msg, dict):
                    msg = Message.from_wire(msg)
                if msg.type == MessageType.MICROBATCH:
                    await self._exec(self.core.compute_gradients, msg.data)
                elif msg.type == MessageType.GRADIENT_STEP:
                    await self._exec(self.core.apply_gradients)
                elif msg.type == MessageType.BATCH_DONE:
                    self.iteration += 1
                    payload = await self._exec(self.core.finish_batch, msg.data, self.iteration)
                    await self.manager.put_completion(self.rank_in_manager, payload)
                elif msg.type == MessageType.SHUTDOWN:
                    self.running = False
        except Exception as e:  # surface the failure: the orchestrator's completion wait will see it
            import traceback

            self.last_error = f"{e!r}\n{traceback.format_exc()}"
            self.running = False
            try:
                await self.manager.put_completion(self.rank_in_manager, {"gpu_rank": self.core.rank, "error": self.last_error})
            except Exception:
                pass

    async def stop(self) -> bool:
        self.running = False
        if self._loop_task is not None:
            self._loop_task.cancel()
        return True

    async def is_ready(self) -> bool:
        return self.last_error is None

    async def get_trainer_weights_info(self):
        return self.core.weights_info()

    def stats(self) -> Dict[str, float]:
        return {"busy_seconds": self.busy_seconds, "opt_step": float(self.core.opt_step),
                "launches": float(getattr(self.core.decoder, "launches", 0)), "h2d_bytes": float(self.core.h2d_bytes),
                "d2h_bytes": float(self.core.d2h_bytes)}

    def run_blocking(self, fn, *args):
        return self._pool.submit(self._run, fn, *args).result()
