"""Metric sinks and cross-worker aggregation.

The orchestrator logs the reference's metric names (orchestrator.py:1091-1181: ``training/*``,
``timing/*``, ``generation/*``, ``minibatch/*``, ``eval/*``, ``epoch``). A JSONL sink is always on - the
reference's plotting tools expect ``training_metrics.jsonl`` although nothing in it writes that file
(Readme.md:419-444) - and W&B is attached when the package is importable and a project is configured.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import Any, Dict, List, Optional, Sequence


class JsonlSink:
    def __init__(self, path: Optional[str]):
        self.path = path
        if path:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def log(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        if not self.path:
            return
        rec = {"_time": time.time()}
        if step is not None:
            rec["_step"] = step
        rec.update({k: (float(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else v) for k, v in metrics.items()})
        with open(self.path, "a", encoding="utf-8") as f:
            f.write(json.dumps(rec) + "\n")


class WandbSink:
    def __init__(self, config: Any):
        self.run = None
        if not getattr(config, "wandb_project", None):
            return
        try:
            import wandb  # type: ignore

            self.run = wandb.init(project=config.wandb_project, entity=config.wandb_entity, name=config.wandb_run_name,
                                  id=config.job_id, resume="allow", config=config.to_dict())
            wandb.define_metric("trainer_step")
            wandb.define_metric("minibatch_step")
            wandb.define_metric("training/*", step_metric="trainer_step")
            wandb.define_metric("timing/*", step_metric="trainer_step")
            wandb.define_metric("generation/*", step_metric="trainer_step")
            wandb.define_metric("eval/*", step_metric="trainer_step")
            wandb.define_metric("minibatch/*", step_metric="minibatch_step")
        except Exception:
            self.run = None

    def log(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        if self.run is not None:
            self.run.log(metrics)


class MetricLogger:
    def __init__(self, config: Any):
        self.sinks = [JsonlSink(config.metrics_path()), WandbSink(config)]
        self.history: List[Dict[str, Any]] = []

    def log(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        self.history.append(dict(metrics))
        for s in self.sinks:
            s.log(metrics, step)


def weighted_mean(values: Sequence[float], weights: Sequence[float]) -> float:
    tot = sum(weights)
    return sum(v * w for v, w in zip(values, weights)) / tot if tot > 0 else 0.0


def merge_mean_std(means: Sequence[float], stds: Sequence[float], weights: Sequence[float]):
    """Pooled mean / std from per-worker (mean, std, weight) triples via second moments (orchestrator.py:958-1017)."""
    tot = sum(weights)
    if tot <= 0:
        return 0.0, 0.0
    mean = sum(m * w for m, w in zip(means, weights)) / tot
    second = sum((s * s + m * m) * w for m, s, w in zip(means, stds, weights)) / tot
    return mean, math.sqrt(max(0.0, second - mean * mean))


def aggregate_completions(completions: Sequence[Dict[str, Any]]) -> Dict[str, float]:
    """Token-weighted aggregation of the per-rank completion payloads into ``training/*`` values."""
    ms = [c.get("metrics", {}) for c in completions]
    w = [float(m.get("token_count", 0)) for m in ms]
    out: Dict[str, float] = {}
    for key, name in (("loss", "avg_loss"), ("kl_div", "avg_kl_div"), ("entropy", "avg_entropy"),
                      ("clipfrac_upper", "clipfrac_upper"), ("clipfrac_lower", "clipfrac_lower"),
                      ("adv_pos_frac", "adv_pos_frac"), ("adv_zero_frac", "adv_zero_frac"),
                      ("loss_per_token", "loss_per_token"), ("old_policy_entropy", "old_policy_entropy"),
                      ("approx_kl", "approx_kl"), ("kl_ref", "kl_ref")):
        out[f"training/{name}"] = weighted_mean([float(m.get(key, 0.0)) for m in ms], w)
    lr_m, lr_s = merge_mean_std([float(m.get("log_ratio_mean", 0.0)) for m in ms], [float(m.get("log_ratio_std", 0.0)) for m in ms], w)
    ad_m, ad_s = merge_mean_std([float(m.get("adv_mean", 0.0)) for m in ms], [float(m.get("adv_std", 0.0)) for m in ms], w)
    out.update({"training/log_ratio_mean": lr_m, "training/log_ratio_std": lr_s, "training/adv_mean": ad_m, "training/adv_std": ad_s})
    gn = [float(m.get("grad_norm", 0.0)) for m in ms]
    out["training/grad_norm"] = sum(gn) / len(gn) if gn else 0.0
    out["training/token_count"] = sum(w)
    bm = [c.get("batch_metrics", {}) for c in completions]
    n_s = sum(float(b.get("total_samples", 0)) for b in bm)
    out["training/batch_total_samples"] = n_s
    out["training/batch_avg_reward"] = sum(float(b.get("total_reward", 0.0)) for b in bm) / n_s if n_s else 0.0
    out["training/optimizer_steps_in_batch"] = max([float(c.get("optimizer_steps_in_batch", 0)) for c in completions] or [0.0])
    # device-timed trainer phases: the slowest rank decides (all ranks step together)
    for c in completions:
        for k, v in (c.get("phase_ms") or {}).items():
            out[f"timing/trainer_{k}_ms"] = max(out.get(f"timing/trainer_{k}_ms", 0.0), float(v))
    return out


def system_metrics() -> Dict[str, float]:
    """GPU memory, utilisation, power and SM clock of every visible GPU (read-only NVML queries) as ``system/*`` series.
    Empty when NVML is not available. Stands in for the collector behind the reference's ``enable_manual_system_metrics``
    key (orchestrator.py:168-169)."""
    out: Dict[str, float] = {}
    try:
        import pynvml

        pynvml.nvmlInit()
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            mem = pynvml.nvmlDeviceGetMemoryInfo(h)
            util = pynvml.nvmlDeviceGetUtilizationRates(h)
            out[f"system/gpu{i}_mem_used_gb"] = mem.used / 2 ** 30
            out[f"system/gpu{i}_util_pct"] = float(util.gpu)
            out[f"system/gpu{i}_power_w"] = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
            out[f"system/gpu{i}_sm_mhz"] = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
    except Exception:
        return {}
    return out
