"""Flat config-dict API.

The user passes one flat dict (or a JSON file); keys and defaults follow the reference's
``OrchestratorConfig`` (orchestrator.py:92-193) so an existing config keeps working. Differences:
unknown keys raise, values are validated, and a few keys are new (``kl_beta``,
``weight_sync_every``, ``placement``, ``kernel_checks``, ``activation_recompute``,
``model_config``, ``metrics_jsonl``). Two defaults of the reference that disagree with each other
are resolved the way its code behaves: the LR scheduler that reaches the optimizer is
``constant`` and warm-up comes from ``lr_warmup_steps`` (orchestrator.py:129 vs 186-193).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields, asdict
from typing import Any, Dict, List, Optional


@dataclass
class GRPOConfig:
    # ---- model / data ----
    model_name_or_path: str = "/path/to/model"
    model_config: Optional[Dict[str, Any]] = None  # inline architecture dict (random init) instead of a checkpoint dir
    data_path: Optional[str] = None
    test_data_path: Optional[str] = None
    output_dir: Optional[str] = None
    resume_from_path: Optional[str] = None
    resume_state: bool = False
    # ---- schedule ----
    num_epochs: int = 3
    batch_size: int = 128  # prompts per macro-batch
    learning_rate: float = 1e-6
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler: str = "constant"  # "constant" | "cosine"
    lr_warmup_steps: int = 0
    num_warmup_steps: int = 0  # accepted for compatibility; lr_warmup_steps is what is used
    total_training_steps: int = 0
    estimated_total_optimizer_steps: int = 0
    # ---- GRPO objective ----
    clip_low: float = 0.2
    clip_high: float = 0.28
    clip_ratio_c: float = 3.0
    kl_beta: float = 0.0  # weight of the k3 KL estimator against the supplied reference logprobs
    samples_per_question: int = 32
    temperature: float = 1.0
    apply_entropy_bonus: bool = True
    entropy_coeff: float = 0.0
    loss_chunksize: Optional[int] = None  # accepted; the fused lm_head loss never materialises logits
    use_torch_compile: bool = True  # accepted for compatibility; nothing here is traced
    # ---- rollout ----
    max_generation_tokens: int = 4096
    max_num_seqs: int = 512
    overhead_seqs: int = 8
    enable_prefix_caching: bool = True  # full prompt blocks stay findable by the hash of their token chain until the next weight push
    vllm_engine_preset: str = "eager"  # "eager" | "throughput" (CUDA-graphed decode step)
    kv_block_size: int = 16
    gpu_memory_utilization: float = 0.90
    # ---- verifier / rewards ----
    global_num_verifiers: int = 4
    write_failed_generation_samples: bool = False
    reward_fns: List[str] = field(default_factory=lambda: ["countdown"])
    verifier_timeout_s: float = 30.0
    # ---- placement ----
    num_training_gpu_workers: int = 4
    num_generation_gpu_workers: int = 1
    num_logprob_gpu_workers: int = 1
    generation_tp_size: int = 1
    logprob_fsdp_size: int = 1
    placement: Optional[Dict[str, List[int]]] = None  # {"trainer": [ranks], "logprob": [...], "rollout": [...]}
    # ---- batching ----
    train_minibatch_sample_size: int = 4000
    max_tokens_per_gpu: int = 36000
    infinite_sampler_seed: int = 42  # reference key; no sampler reads it there either (its data order is fixed)
    experience_batcher_name: str = "experience_batcher"
    # ---- logging / eval / checkpoints ----
    wandb_project: Optional[str] = None
    wandb_entity: Optional[str] = None
    wandb_run_name: str = "async-grpo-run"
    job_id: Optional[str] = None
    metrics_jsonl: Optional[str] = None  # default: <output_dir>/training_metrics.jsonl
    eval_every_n_macro_batches: int = 20
    eval_at_start: bool = True
    min_samples_per_checkpoint: int = 30000
    keep_last_n_checkpoints: int = 2
    verify_weight_sync_during_init: bool = False
    # system/* series (GPU memory, utilisation, power, SM clock; read-only NVML queries) once per macro-batch
    # Chrome trace (torch.profiler, host + CUDA activity of the orchestrator's process) of macro-batch number
    # profile_macro_batch of this run, written to profile_trace_path; None = off. The reference only has a stub here
    # (gpu_process_worker.py:49-51).
    profile_trace_path: Optional[str] = None
    profile_macro_batch: int = 1
    enable_manual_system_metrics: bool = False
    system_metrics_interval_sec: float = 10.0  # reference key; sampling here is per macro-batch
    # ---- new: engine behaviour ----
    weight_sync_every: int = 1  # macro-batches between trainer -> rollout/logprob pushes
    # Feed finished samples to the microbatch planner right away instead of waiting for a whole minibatch: the
    # same samples end up in the same optimizer step, but forward/backward overlaps the rest of the generation.
    eager_microbatch_dispatch: bool = False
    comm_backend: str = "auto"  # "auto" (peer-memory kernels when available) | "peer" | "nccl" (library collectives)
    # The kernels always validate indices and report through a status word; with this switch the host reads that word
    # after every microbatch and every engine step (a synchronisation each) instead of once per macro-batch
    kernel_checks: bool = False
    stream_logprobs: bool = True  # request a sample's old-policy logprobs when IT finishes, not when its whole group has
    # > 0: on a GPU that a rollout engine shares with the trainer or the logprob role, the engine gets this many SMs of
    # its own and the other roles the rest (CUDA green contexts, utils/sm_partition.py); 0 = all roles use every SM
    colocated_rollout_sms: int = 0
    colocated_sm_limit: int = 0  # > 0: trainer / logprob GEMMs fill at most this many SMs on a GPU they share with a rollout engine
    # "zero2": resident bf16 copy per trainer rank | "zero3": fully sharded, gathered per layer | "auto": zero3 when the
    # resident form would take more than 60 % of a GPU's memory (launch.resolve_param_sharding)
    param_sharding: str = "auto"
    activation_recompute: str = "auto"  # "none" | "full" | "auto" (by memory estimate)
    trainer_completion_timeout_s: float = 300.0
    prompt_timeout_s: float = 1200.0
    dist_timeout_s: float = 600.0
    seed: int = 0
    # ---- unused by the reference but accepted (LoRA / offload keys exist there and do nothing) ----
    lora_rank: int = 0
    lora_alpha: int = 0
    lora_target_modules: Optional[List[str]] = None
    fsdp_param_offload: bool = False
    fsdp_optimizer_offload: bool = False

    # nested views used by the reference's workers (`model`, `trainer.optim`, `trainer.fsdp`, `rollout`)
    def nested(self) -> Dict[str, Any]:
        return {
            "model": {"path": self.model_name_or_path, "lora_rank": self.lora_rank, "lora_alpha": self.lora_alpha,
                      "target_modules": self.lora_target_modules},
            "trainer": {
                "optim": {"lr": self.learning_rate, "weight_decay": self.weight_decay,
                          "lr_scheduler": self.lr_scheduler, "lr_warmup_steps": self.lr_warmup_steps,
                          "total_training_steps": self.total_steps()},
                "fsdp": {"param_offload": self.fsdp_param_offload, "optimizer_offload": self.fsdp_optimizer_offload,
                         "fsdp_size": self.num_training_gpu_workers},
            },
            "rollout": {"tensor_model_parallel_size": self.generation_tp_size},
        }

    def total_steps(self) -> int:
        return int(self.total_training_steps or self.estimated_total_optimizer_steps or 0)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def metrics_path(self) -> Optional[str]:
        if self.metrics_jsonl:
            return self.metrics_jsonl
        if self.output_dir:
            import os

            return os.path.join(self.output_dir, "training_metrics.jsonl")
        return None

    def resolved_placement(self) -> Dict[str, List[int]]:
        """Ranks per role. Without an explicit placement, ranks are laid out trainer, logprob, rollout."""
        if self.placement is not None:
            return {k: list(v) for k, v in self.placement.items()}
        t, l, r = self.num_training_gpu_workers, self.num_logprob_gpu_workers, self.num_generation_gpu_workers
        return {"trainer": list(range(t)), "logprob": list(range(t, t + l)), "rollout": list(range(t + l, t + l + r))}

    def validate(self) -> "GRPOConfig":
        def need(cond: bool, msg: str) -> None:
            if not cond:
                raise ValueError("config: " + msg)

        need(self.batch_size > 0, "batch_size must be positive")
        need(self.samples_per_question > 0, "samples_per_question must be positive")
        need(self.train_minibatch_sample_size > 0, "train_minibatch_sample_size must be positive")
        need(self.max_tokens_per_gpu > 0, "max_tokens_per_gpu must be positive")
        need(self.num_training_gpu_workers >= 1, "need at least one trainer rank")
        need(self.num_logprob_gpu_workers >= 1, "need at least one logprob rank")
        need(self.num_generation_gpu_workers >= 1, "need at least one generation rank")
        # the reference's two divisibility checks (orchestrator.py:340-341, 369-370)
        need(self.num_logprob_gpu_workers % self.logprob_fsdp_size == 0,
             "num_logprob_gpu_workers must be divisible by logprob_fsdp_size")
        need(self.num_generation_gpu_workers % self.generation_tp_size == 0,
             "num_generation_gpu_workers must be divisible by generation_tp_size")
        need(0.0 <= self.clip_low < 1.0, "clip_low must be in [0, 1)")
        need(self.clip_high >= 0.0, "clip_high must be non-negative")
        need(self.clip_ratio_c > 1.0, "clip_ratio_c must exceed 1")
        need(self.kl_beta >= 0.0, "kl_beta must be non-negative")
        need(self.temperature >= 0.0, "temperature must be non-negative")
        need(self.lr_scheduler in ("constant", "cosine", "constant_with_warmup"), "unknown lr_scheduler")
        need(self.vllm_engine_preset in ("eager", "throughput"), "vllm_engine_preset must be eager or throughput")
        need(self.colocated_sm_limit >= 0, "colocated_sm_limit must be >= 0")
        need(self.colocated_rollout_sms >= 0, "colocated_rollout_sms must be >= 0")
        need(self.param_sharding in ("zero2", "zero3", "auto"), "param_sharding must be zero2/zero3/auto")
        need(self.activation_recompute in ("none", "full", "auto"), "activation_recompute must be none/full/auto")
        need(self.keep_last_n_checkpoints >= 1, "keep_last_n_checkpoints must be >= 1")
        need(self.weight_sync_every >= 1, "weight_sync_every must be >= 1")
        if self.placement is not None:
            for role in ("trainer", "logprob", "rollout"):
                need(role in self.placement and len(self.placement[role]) > 0, f"placement needs ranks for {role}")
        return self


_FIELD_NAMES = {f.name for f in fields(GRPOConfig)}


def make_config(config_dict: Optional[Dict[str, Any]] = None, **overrides: Any) -> GRPOConfig:
    """Build a validated config from a flat dict (plus keyword overrides)."""
    merged: Dict[str, Any] = dict(config_dict or {})
    merged.update(overrides)
    unknown = sorted(k for k in merged if k not in _FIELD_NAMES)
    if unknown:
        raise KeyError(f"unknown config keys: {unknown}")
    return GRPOConfig(**merged).validate()


def load_config(path: str, **overrides: Any) -> GRPOConfig:
    with open(path, "r", encoding="utf-8") as f:
        return make_config(json.load(f), **overrides)
