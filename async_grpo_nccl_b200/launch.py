"""Runtimes: where the roles live and how they are reached.

``InProcessRuntime``   every role in the calling process (one GPU, or CPU with the PyTorch oracle ops);
                       roles overlap through their own worker threads and CUDA streams.
``DistributedRuntime`` one process per GPU (launched by ``torch.distributed.run`` or by ``spawn``), roles
                       placed on ranks by ``config.resolved_placement()``, rank 0 additionally hosts the
                       orchestrator and the ExperienceManager; control plane = :mod:`.rpc`, weight plane =
                       peer-memory push kernels (NCCL broadcast as the measured fallback).

This replaces the reference's Ray placement groups and named actors (ray_utils.py:13-230,
orchestrator.py:302-550).
"""
from __future__ import annotations

import asyncio
import logging
import os
import time
from typing import Any, Dict, List, Optional

import torch

from . import checkpoint as ckpt
from .config import GRPOConfig
from .experience import ExperienceManager
from .models.config import ModelConfig, resolve_model_config
from .models.decoder import NativeDecoder, OracleDecoder
from .models.layout import ParamLayout
from .rewards import get_or_create_verifier_pool
from .roles.logprob import LogProbWorker
from .roles.rollout import GenerationWorker
from .roles.trainer import TrainerCore, TrainerWorker

logger = logging.getLogger(__name__)


def load_tokenizer(config: GRPOConfig) -> Any:
    path = config.model_name_or_path
    if path and os.path.isdir(path) and any(f.startswith("tokenizer") for f in os.listdir(path)):
        try:
            from transformers import AutoTokenizer

            return AutoTokenizer.from_pretrained(path)
        except Exception as e:  # pragma: no cover - depends on local files
            logger.warning("tokenizer could not be loaded from %s: %r", path, e)
    return None


def initial_weights(config: GRPOConfig, mcfg: ModelConfig, layout: ParamLayout, device: Any = None) -> torch.Tensor:
    """Flat fp32 parameters: from an HF checkpoint directory when there is one, else seeded random init."""
    path = config.model_name_or_path
    if path and os.path.isdir(path) and any(f.endswith(".safetensors") for f in os.listdir(path)):
        return ckpt.load_hf_model(path, layout)
    if device is not None and torch.device(device).type == "cuda" and layout.total > (1 << 26):
        flat = torch.empty(layout.total, dtype=torch.float32, device=device)
        layout.init_random_device_(flat, config.seed)
        return flat
    flat = torch.empty(layout.total, dtype=torch.float32)
    layout.init_random_(flat, config.seed)
    return flat


def activation_bytes_per_token(m: ModelConfig) -> int:
    per_layer = 2 * (5 * m.hidden_size + m.qkv_dim + m.q_dim + 3 * m.intermediate_size) + 4 * m.num_attention_heads + 8
    return per_layer * m.num_hidden_layers


def want_recompute(config: GRPOConfig, mcfg: ModelConfig, budget_bytes: float) -> bool:
    if config.activation_recompute != "auto":
        return config.activation_recompute == "full"
    return activation_bytes_per_token(mcfg) * config.max_tokens_per_gpu > budget_bytes


class InProcessRuntime:
    def __init__(self, config: GRPOConfig, device: Optional[str] = None, kv_memory_bytes: Optional[int] = None):
        self.config = config
        self.device = torch.device(device or ("cuda:0" if torch.cuda.is_available() else "cpu"))
        self.native = self.device.type == "cuda"
        self.kv_memory_bytes = kv_memory_bytes
        self.trainer_ranks = [0]
        self.generation_controllers: List[Any] = []
        self.logprob_controllers: List[Any] = []
        self.experience_manager: Optional[ExperienceManager] = None
        self.trainer: Optional[TrainerWorker] = None
        self.sync_ms_history: List[float] = []

    async def initialize(self, orch: Any = None) -> None:
        cfg = self.config
        self.mcfg = resolve_model_config(cfg.model_name_or_path, cfg.model_config)
        mcfg = self.mcfg
        probe_layout = ParamLayout(mcfg, 1)
        flat32 = initial_weights(cfg, mcfg, probe_layout, self.device)
        if self.native:
            torch.cuda.set_device(self.device)
            total = torch.cuda.get_device_properties(self.device).total_memory
            param_bytes = probe_layout.total * 2
            fixed = probe_layout.total * (2 + 12 + 4) + 2 * param_bytes  # trainer + logprob/rollout copies
            free_for_dynamic = max(total * cfg.gpu_memory_utilization - fixed, 8 << 30)
            kv_bytes = self.kv_memory_bytes or int(free_for_dynamic * 0.45)
            act_budget = free_for_dynamic - kv_bytes - (6 << 30)
            cfg_recompute = want_recompute(cfg, mcfg, act_budget)
            if cfg_recompute and cfg.activation_recompute == "auto":
                cfg.activation_recompute = "full"
            self.streams = {k: torch.cuda.Stream(self.device) for k in ("trainer", "logprob", "rollout")}
        else:
            self.streams = {"trainer": None, "logprob": None, "rollout": None}
            kv_bytes = 0
        core = TrainerCore(cfg, mcfg, self.device, 0, 1, None, flat32, cfg.seed)
        self.trainer = TrainerWorker(core, self.streams["trainer"])
        self.layout = core.layout
        # logprob and rollout keep their own copies: they must hold the PREVIOUS policy while the trainer steps
        self.logprob_params = core.params.clone()
        self.rollout_params = core.params.clone()
        if self.native:
            from .engine.engine import RolloutEngine

            lp_dec = NativeDecoder(mcfg, self.layout, self.logprob_params)
            max_len = min(mcfg.max_position_embeddings, cfg.max_generation_tokens + 4096)
            engine = RolloutEngine(mcfg, self.layout, self.rollout_params, max_seqs=cfg.max_num_seqs, max_model_len=max_len,
                                   kv_memory_bytes=kv_bytes, use_cuda_graph=cfg.vllm_engine_preset == "throughput",
                                   block_size=cfg.kv_block_size)
        else:
            from .engine.engine import OracleEngine

            lp_dec = OracleDecoder(mcfg, self.layout, self.logprob_params)
            engine = OracleEngine(mcfg, self.layout, self.rollout_params, max_seqs=cfg.max_num_seqs,
                                  max_model_len=min(mcfg.max_position_embeddings, cfg.max_generation_tokens + 2048))
        self.engine = engine
        self.verifier = get_or_create_verifier_pool(cfg.global_num_verifiers, cfg.write_failed_generation_samples, cfg.reward_fns,
                                                    cfg.output_dir, name=f"verifier_pool_{id(self)}", timeout_s=cfg.verifier_timeout_s)
        self.tokenizer = load_tokenizer(cfg)
        self.logprob = LogProbWorker(cfg, mcfg, lp_dec, self.device, stream=self.streams["logprob"])
        self.generation = GenerationWorker(cfg, mcfg, engine, self.verifier, self.tokenizer, stream=self.streams["rollout"])
        self.generation_controllers = [self.generation]
        self.logprob_controllers = [self.logprob]
        self.experience_manager = ExperienceManager(cfg)
        if cfg.resume_from_path:
            self._load_optimizer(cfg.resume_from_path)

    def _load_optimizer(self, path: str) -> None:
        core = self.trainer.core
        st = ckpt.load_optimizer_shard(path, 0, 1, core.layout)
        if st is not None:
            core.master.copy_(st["master"])
            core.exp_avg.copy_(st["exp_avg"])
            core.exp_avg_sq.copy_(st["exp_avg_sq"])
            core.params.copy_(core.master.to(core.compute_dtype))
            sched = ckpt.load_scheduler_state(path)
            if sched:
                core.load_scheduler_state(sched)
            self.logprob_params.copy_(core.params)
            self.rollout_params.copy_(core.params)

    async def start_trainers(self) -> None:
        self.trainer.set_orchestrator(self.experience_manager, 0)
        await self.trainer.start_training_loop()

    async def ping_trainers(self) -> List[bool]:
        return [await self.trainer.is_ready()]

    async def sync_weights(self) -> None:
        """Same-device sync: stop the engine between steps, then two device copies of the flat buffer."""
        t0 = time.time()
        await self.generation.pause_for_sync()
        core = self.trainer.core
        if self.native:
            torch.cuda.synchronize(self.device)
        self.logprob_params.copy_(core.params)
        self.rollout_params.copy_(core.params)
        if self.native:
            torch.cuda.synchronize(self.device)
        await self.generation.resume_after_sync()
        self.sync_ms_history.append((time.time() - t0) * 1000.0)

    async def verify_weight_sync(self) -> List[str]:
        core = self.trainer.core
        bad = []
        for name in self.layout.segments:
            a = self.layout.view(core.params, name)
            if not torch.equal(a, self.layout.view(self.logprob_params, name)):
                bad.append(f"logprob:{name}")
            if not torch.equal(a, self.layout.view(self.rollout_params, name)):
                bad.append(f"rollout:{name}")
        return bad

    async def save_checkpoint(self, path: str) -> None:
        core = self.trainer.core

        def _save() -> None:
            ckpt.save_hf_model(path, self.mcfg, core.layout, core.master if core.world == 1 else core.full_master_fp32(),
                               tokenizer_src=self.config.model_name_or_path)
            ckpt.save_optimizer_shard(path, 0, 1, core.layout, core.optimizer_state(), core.scheduler_state())

        await asyncio.get_running_loop().run_in_executor(None, self.trainer.run_blocking, _save)

    # ---- measurement hooks used by bench.py ----
    async def barrier_and_sync(self) -> None:
        if self.native:
            torch.cuda.synchronize(self.device)

    async def record_event(self, name: str) -> None:
        if not hasattr(self, "_events"):
            self._events: Dict[str, Any] = {}
            self._walls: Dict[str, float] = {}
        self._walls[name] = time.time()
        if self.native:
            torch.cuda.synchronize(self.device)  # roles run on their own streams: make the default stream see them all
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events[name] = ev

    async def elapsed_ms(self, a: str, b: str) -> float:
        if self.native:
            torch.cuda.synchronize(self.device)
            return float(self._events[a].elapsed_time(self._events[b]))
        return (self._walls[b] - self._walls[a]) * 1000.0

    async def collect_stats(self) -> Dict[str, float]:
        core = self.trainer.core
        eng = self.engine
        return {
            "launches": float(getattr(core.decoder, "launches", 0) + getattr(self.logprob.decoder, "launches", 0) + getattr(eng, "launches", 0)),
            "h2d_bytes": float(core.h2d_bytes + self.logprob.h2d_bytes + getattr(eng, "h2d_bytes", 0)),
            "d2h_bytes": float(core.d2h_bytes + self.logprob.d2h_bytes + getattr(eng, "d2h_bytes", 0)),
        }

    async def shutdown(self) -> None:
        if self.trainer is not None:
            await self.trainer.stop()
        if getattr(self, "generation", None) is not None:
            self.generation.shutdown()
        if getattr(self, "verifier", None) is not None:
            self.verifier.close()


def build_inprocess_runtime(config: GRPOConfig, device: Optional[str] = None, **kw: Any) -> InProcessRuntime:
    return InProcessRuntime(config, device, **kw)
