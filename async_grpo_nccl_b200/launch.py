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
from typing import Any, Dict, List, Optional, Sequence

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


def resolve_param_sharding(mode: str, num_params: int, trainers: int, hbm_bytes: Optional[float], peer: bool) -> str:
    """``auto`` -> ``zero2`` or ``zero3``. With resident parameters (zero2) a trainer rank holds the bf16 copy (2 bytes per
    parameter), a full fp32 gradient buffer (4) and its share of master + moments (12 / trainers); fully sharded (zero3)
    it holds 18 / trainers plus a few layers of staging. zero3 needs the peer-memory backend and more than one trainer
    rank; it is chosen when the resident form would take more than 60 % of the GPU's memory (from about 14B parameters
    on 180 GB parts with 4 trainer ranks), because activations, the logits-free loss scratch and, on shared GPUs, a KV
    cache need the rest."""
    if mode != "auto":
        return mode
    if not peer or trainers <= 1 or not hbm_bytes:
        return "zero2"
    resident = num_params * (6.0 + 12.0 / trainers)
    return "zero3" if resident > 0.6 * hbm_bytes else "zero2"


def want_recompute(config: GRPOConfig, mcfg: ModelConfig, budget_bytes: float) -> bool:
    if config.activation_recompute != "auto":
        return config.activation_recompute == "full"
    return activation_bytes_per_token(mcfg) * config.max_tokens_per_gpu > budget_bytes


def _tune_interpreter_for_role_threads() -> None:
    """The trainer, logprob and rollout roles of one process run on threads that all drive the GPU from Python. With
    the default 5 ms switch interval a decode step (2 ms of device time) can wait several milliseconds for another
    role's launch loop to give up the interpreter lock; 0.2 ms keeps the hand-off below a tenth of a step."""
    import sys

    if sys.getswitchinterval() > 2e-4:
        sys.setswitchinterval(2e-4)


def _role_streams(device: torch.device, rollout_sms: int = 0) -> Dict[str, Any]:
    """One CUDA stream per role. With ``rollout_sms`` > 0 the device's SMs are split into two disjoint groups (green
    contexts): the rollout stream runs on the first, the trainer and logprob streams on the rest; the entries
    ``rollout_sm_count`` / ``other_sm_count`` then give the group sizes that persistent kernels must respect.
    Otherwise: When roles share a GPU the decode step's short, serially dependent kernels must not
    queue behind a trainer kernel that fills every SM, so the rollout stream gets the highest priority (its thread
    blocks are placed first whenever an SM frees up), the old-policy logprob stream the next, the trainer the lowest."""
    import os

    if rollout_sms > 0:
        from .utils import sm_partition

        groups = sm_partition.split(device, rollout_sms)
        if groups is not None:
            g_roll, g_other = groups
            return {"trainer": g_other.stream(0), "logprob": g_other.stream(-1), "rollout": g_roll.stream(-2),
                    "rollout_sm_count": g_roll.sm_count, "other_sm_count": g_other.sm_count, "_groups": groups}
    if os.environ.get("AGRPO_STREAM_PRIORITIES", "1") == "0":
        return {k: torch.cuda.Stream(device) for k in ("trainer", "logprob", "rollout")}
    return {"trainer": torch.cuda.Stream(device, priority=0), "logprob": torch.cuda.Stream(device, priority=-1),
            "rollout": torch.cuda.Stream(device, priority=-2)}


def preflight_placement(place: Dict[str, Sequence[int]], world: int, visible_gpus: Optional[int] = None,
                        free_bytes: Optional[Sequence[int]] = None, need_bytes: int = 0) -> None:
    """Fails fast, with the reason, when a placement cannot be honoured: before any rank allocates or enters a
    collective. Counterpart of the reference's resource check ahead of placement-group creation (ray_utils.py:50-99):
    roles named, ranks inside the job, one GPU per rank on this node, and (when given) enough free memory on each GPU."""
    for role in ("trainer", "logprob", "rollout"):
        ranks = list(place.get(role, []))
        if not ranks:
            raise ValueError(f"placement has no rank for role '{role}'")
        if len(set(ranks)) != len(ranks):
            raise ValueError(f"placement lists a rank twice for role '{role}': {ranks}")
        bad = [r for r in ranks if r < 0 or r >= world]
        if bad:
            raise ValueError(f"placement puts role '{role}' on ranks {bad}, but the job has {world} rank(s) (0..{world - 1}); "
                             f"start {max(max(rs) for rs in place.values()) + 1} processes or change the placement")
    used = sorted({r for rs in place.values() for r in rs})
    if visible_gpus is not None and visible_gpus < len(used):
        raise ValueError(f"the placement needs {len(used)} GPUs (one per rank {used}) but only {visible_gpus} are visible "
                         f"on this node (CUDA_VISIBLE_DEVICES?)")
    if free_bytes is not None and need_bytes > 0:
        short = [(i, f) for i, f in enumerate(free_bytes) if i in used and f < need_bytes]
        if short:
            raise ValueError("not enough free GPU memory for the placement: " +
                             ", ".join(f"GPU {i} has {f / 2 ** 30:.1f} GiB free" for i, f in short) +
                             f"; each rank needs about {need_bytes / 2 ** 30:.1f} GiB (is another job using these GPUs?)")


class InProcessRuntime:
    def __init__(self, config: GRPOConfig, device: Optional[str] = None, kv_memory_bytes: Optional[int] = None):
        self.config = config
        if config.param_sharding == "auto":
            config.param_sharding = "zero2"  # one trainer rank: nothing to shard over
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
            self.streams = _role_streams(self.device, cfg.colocated_rollout_sms)
            _tune_interpreter_for_role_threads()
        else:
            self.streams = {"trainer": None, "logprob": None, "rollout": None}
            kv_bytes = 0
        core = TrainerCore(cfg, mcfg, self.device, 0, 1, None, flat32, cfg.seed)
        # all three roles share this GPU: optionally keep some SMs free for the decode kernels
        lim = cfg.colocated_sm_limit if self.native else 0
        lim = int(self.streams.get("other_sm_count", lim))  # an SM partition decides the count
        self.trainer = TrainerWorker(core, self.streams["trainer"], sm_limit=lim)
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
                                   block_size=cfg.kv_block_size, prefix_caching=cfg.enable_prefix_caching)
        else:
            from .engine.engine import OracleEngine

            lp_dec = OracleDecoder(mcfg, self.layout, self.logprob_params)
            engine = OracleEngine(mcfg, self.layout, self.rollout_params, max_seqs=cfg.max_num_seqs,
                                  max_model_len=min(mcfg.max_position_embeddings, cfg.max_generation_tokens + 2048))
        self.engine = engine
        self.verifier = get_or_create_verifier_pool(cfg.global_num_verifiers, cfg.write_failed_generation_samples, cfg.reward_fns,
                                                    cfg.output_dir, name=f"verifier_pool_{id(self)}", timeout_s=cfg.verifier_timeout_s)
        self.tokenizer = load_tokenizer(cfg)
        self.logprob = LogProbWorker(cfg, mcfg, lp_dec, self.device, stream=self.streams["logprob"], sm_limit=lim)
        self.generation = GenerationWorker(cfg, mcfg, engine, self.verifier, self.tokenizer, stream=self.streams["rollout"],
                                           sm_limit=int(self.streams.get("rollout_sm_count", 0)))
        if cfg.stream_logprobs:
            self.generation.logprob_fn = self.logprob.inference
        self.generation_controllers = [self.generation]
        self.logprob_controllers = [self.logprob]
        self.experience_manager = ExperienceManager(cfg)
        if cfg.resume_from_path:
            self._load_optimizer(cfg.resume_from_path)

    def _load_optimizer(self, path: str) -> None:
        core = self.trainer.core
        if core.load_optimizer_checkpoint(path):
            self.logprob_params.copy_(core.params)
            self.rollout_params.copy_(core.params)
            logger.info("optimizer state and schedule reloaded from %s (optimizer step %d)", path, core.opt_step)
        else:
            logger.warning("resume_from_path %s holds no optimizer state; starting with zero moments", path)

    async def start_trainers(self) -> None:
        self.trainer.set_orchestrator(self.experience_manager, 0)
        await self.trainer.start_training_loop()

    async def ping_trainers(self) -> List[bool]:
        return [await self.trainer.is_ready()]

    async def sync_weights(self) -> None:
        """Same-device sync: stop the engine between steps, then two device copies of the flat buffer."""
        t0 = time.time()
        await self.generation.pause_for_sync()
        await asyncio.get_running_loop().run_in_executor(None, self.logprob.pause)  # no logprob batch in flight either
        core = self.trainer.core
        try:
            if self.native:
                torch.cuda.synchronize(self.device)
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            self.logprob_params.copy_(core.params)
            self.rollout_params.copy_(core.params)
            if self.native:
                ev1.record()
                torch.cuda.synchronize(self.device)
                self.sync_device_ms = float(ev0.elapsed_time(ev1))
        finally:
            self.logprob.resume()
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
        out = {
            "launches": float(getattr(core.decoder, "launches", 0) + getattr(self.logprob.decoder, "launches", 0) + getattr(eng, "launches", 0)),
            "h2d_bytes": float(core.h2d_bytes + self.logprob.h2d_bytes + getattr(eng, "h2d_bytes", 0)),
            "d2h_bytes": float(core.d2h_bytes + self.logprob.d2h_bytes + getattr(eng, "d2h_bytes", 0)),
        }
        if hasattr(eng, "timing_stats"):
            out.update(eng.timing_stats())
            out["engine_busy_s"] = float(self.generation.busy_seconds)
        return out

    async def shutdown(self) -> None:
        if self.trainer is not None:
            await self.trainer.stop()
        if getattr(self, "generation", None) is not None:
            self.generation.shutdown()
        if getattr(self, "verifier", None) is not None:
            self.verifier.close()


def build_inprocess_runtime(config: GRPOConfig, device: Optional[str] = None, **kw: Any) -> InProcessRuntime:
    return InProcessRuntime(config, device, **kw)


# =====================================================================================================
# One process per GPU
# =====================================================================================================
class _RemoteGeneration:
    def __init__(self, proxy: Any):
        self._p = proxy

    async def inference(self, sample, n=1, temperature=1.0, max_tokens=None):
        samples, metrics = await self._p.gen_inference(sample, n, temperature, max_tokens)
        return samples, metrics

    async def batch_inference_for_evaluation(self, prompts, answers, max_tokens=1024, temperature=0.0):
        return await self._p.gen_eval(list(prompts), list(answers), max_tokens, temperature)


class _RemoteLogprob:
    def __init__(self, proxy: Any):
        self._p = proxy

    async def inference(self, sample):
        return await self._p.lp_inference(sample)

    async def compute_batch(self, samples):
        return await self._p.lp_compute_batch(list(samples))


class _RemoteManager:
    """What a trainer rank sees of the ExperienceManager that lives on rank 0."""

    def __init__(self, proxy: Any):
        self._p = proxy

    async def get_batch(self, rank: int):
        return await self._p.em_get_batch(rank)

    async def put_completion(self, rank: int, data: Any):
        return await self._p.em_put_completion(rank, data)


class RoleHost:
    """RPC surface of one rank: thin forwards to the role objects that live in this process."""

    def __init__(self, rt: "DistributedRuntime"):
        self.rt = rt

    async def gen_inference(self, sample, n, temperature, max_tokens):
        return await self.rt.generation.inference(sample, n=n, temperature=temperature, max_tokens=max_tokens)

    async def gen_eval(self, prompts, answers, max_tokens, temperature):
        return await self.rt.generation.batch_inference_for_evaluation(prompts, answers, max_tokens, temperature)

    async def lp_inference(self, sample):
        return await self.rt.logprob.inference(sample)

    async def lp_compute_batch(self, samples):
        return await self.rt.logprob.compute_batch(samples)

    async def trainer_start(self):
        return await self.rt.start_local_trainer()

    async def trainer_ready(self):
        return self.rt.trainer is None or await self.rt.trainer.is_ready()

    async def sync_weights(self):
        return await self.rt.local_sync_weights()

    async def verify_sync(self):
        return await self.rt.local_checksum()

    async def save_checkpoint(self, path):
        return await self.rt.local_save_checkpoint(path)

    async def stats(self):
        return self.rt.local_stats()

    async def barrier_sync(self):
        if self.rt.native:
            torch.cuda.synchronize(self.rt.device)
        return True

    async def record_event(self, name):
        return self.rt.local_record_event(name)

    async def elapsed(self, a, b):
        return self.rt.local_elapsed(a, b)

    async def shutdown(self):
        self.rt.stop_event.set()
        return True

    async def em_get_batch(self, rank):
        return await self.rt.experience_manager.get_batch(rank)

    async def em_put_completion(self, rank, data):
        return await self.rt.experience_manager.put_completion(rank, data)


class DistributedRuntime:
    """Created on EVERY rank (collective construction). Rank 0 then runs the orchestrator against it, the other
    ranks call ``serve_forever``."""

    def __init__(self, config: GRPOConfig, backend: Optional[str] = None):
        import torch.distributed as dist

        self.config = config
        self.dist = dist
        cuda = torch.cuda.is_available()
        if not dist.is_initialized():
            import datetime

            dist.init_process_group(backend or ("nccl" if cuda else "gloo"),
                                    timeout=datetime.timedelta(seconds=float(os.environ.get("TORCH_DIST_TIMEOUT_S", config.dist_timeout_s))))
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.native = cuda
        if cuda:
            self.device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", self.rank % torch.cuda.device_count())))
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        place = config.resolved_placement()
        self.place = place
        free = None
        if cuda:
            f, _ = torch.cuda.mem_get_info(self.device)
            free = [0] * self.world
            free[self.rank] = int(f)
        mcfg0 = resolve_model_config(config.model_name_or_path, config.model_config)
        # parameters in bf16 plus (trainer ranks) fp32 master + moments + gradients of this rank's share: a floor, not a plan
        need = mcfg0.num_parameters() * 2
        preflight_placement(place, self.world, torch.cuda.device_count() if cuda else None,
                            [free[r] if r == self.rank else need for r in range(self.world)] if free else None, need)
        self.trainer_ranks = list(place["trainer"])
        self.logprob_ranks = list(place["logprob"])
        self.rollout_ranks = list(place["rollout"])
        self.infer_ranks = sorted(set(self.logprob_ranks) | set(self.rollout_ranks))
        # generation_tp_size consecutive rollout ranks form one engine replica (vllm_worker.py:219-232,
        # tensor_parallel_size); the orchestrator talks to the first rank of each
        from .roles.tp_mirror import replica_groups

        self.replicas = replica_groups(self.rollout_ranks, max(1, int(config.generation_tp_size)))
        self.my_replica = next((g for g in self.replicas if self.rank in g), None)
        self.rollout_leaders = [g[0] for g in self.replicas]
        self.is_trainer = self.rank in self.trainer_ranks
        self.trainer_index = self.trainer_ranks.index(self.rank) if self.is_trainer else None
        self.mcfg = resolve_model_config(config.model_name_or_path, config.model_config)
        t = len(self.trainer_ranks)
        self.layout = ParamLayout(self.mcfg, shard_world=t)
        self.trainer_group = dist.new_group(self.trainer_ranks)  # every rank must call new_group
        self.world_group = dist.group.WORLD
        # ---- communication plane (collective construction) ----
        self.C = None
        self.trainer_comm = None
        self.weight_sync = None
        use_peer = False
        if self.native:
            from .ops import native as _native
            from .parallel import symm

            self.C = _native()
            use_peer = config.comm_backend in ("auto", "peer") and symm.symmetric_available()
            config.param_sharding = resolve_param_sharding(config.param_sharding, self.mcfg.num_parameters(), t,
                                                           float(torch.cuda.get_device_properties(self.device).total_memory), use_peer)
            if use_peer:
                try:
                    # every rank allocates every symmetric buffer, in the same order, over the WORLD group
                    self.plane = symm.SymmetricPlane(self.device, self.layout, self.C, self.trainer_ranks, self.infer_ranks,
                                                     zero3=config.param_sharding == "zero3")
                    self.trainer_comm = self.plane.trainer_comm()
                    self.weight_sync = self.plane.weight_sync()
                except Exception as e:
                    if config.comm_backend == "peer":
                        raise
                    logger.warning("symmetric memory unavailable (%r): falling back to library collectives", e)
                    self.trainer_comm, self.weight_sync, use_peer = None, None, False
        self.use_peer = use_peer
        if config.param_sharding == "auto":
            config.param_sharding = "zero2"
        if self.rank == 0 and config.param_sharding == "zero3" and not (use_peer and t > 1):
            logger.warning("param_sharding=zero3 needs the peer-memory backend and more than one trainer rank; "
                           "running with resident parameters (zero2) instead")
        self.tp_comm = None
        tp_size = max(1, int(config.generation_tp_size))
        if tp_size > 1 and self.native:
            if not use_peer:
                raise RuntimeError("generation_tp_size > 1 needs the peer-memory backend (comm_backend auto/peer with "
                                   "symmetric memory): the replica's all-reduce runs over peer loads")
            # collective over the world group like every symmetric allocation; ranks outside a replica hold idle buffers
            self.tp_comm = symm.TensorParallelComm(self.my_replica or [], self.rank, min(256, int(config.max_num_seqs)),
                                                   self.mcfg.hidden_size, self.device, self.C)
        # ---- roles of this rank ----
        self.trainer: Optional[TrainerWorker] = None
        self.logprob: Optional[LogProbWorker] = None
        self.generation: Optional[GenerationWorker] = None
        self.engine = None
        self.experience_manager: Optional[ExperienceManager] = ExperienceManager(config) if self.rank == 0 else None
        _tune_interpreter_for_role_threads()
        shares_gpu = self.rank in self.rollout_ranks and (self.is_trainer or self.rank in self.logprob_ranks)
        self.streams = (_role_streams(self.device, config.colocated_rollout_sms if shares_gpu else 0) if self.native
                        else {"trainer": None, "logprob": None, "rollout": None})
        other_lim = int(self.streams.get("other_sm_count", config.colocated_sm_limit if shares_gpu else 0))
        flat32 = initial_weights(config, self.mcfg, self.layout, self.device if self.native else None)
        if self.is_trainer:
            core = TrainerCore(config, self.mcfg, self.device, self.trainer_index, t, self.trainer_group, flat32, config.seed,
                               comm=self.trainer_comm)
            self.trainer = TrainerWorker(core, self.streams["trainer"], sm_limit=other_lim if self.native else 0)
        if self.rank in self.infer_ranks:
            dtype = torch.bfloat16 if self.native else torch.float32
            if self.weight_sync is not None:
                self.infer_params = self.weight_sync.buffer
                self.infer_params.copy_(flat32.to(dtype))
            else:
                self.infer_params = flat32.to(self.device, dtype=dtype).clone()
        else:
            self.infer_params = None
        del flat32
        if self.rank in self.logprob_ranks:
            dec = (NativeDecoder if self.native else OracleDecoder)(self.mcfg, self.layout, self.infer_params)
            self.logprob = LogProbWorker(config, self.mcfg, dec, self.device, stream=self.streams["logprob"],
                                         sm_limit=other_lim if self.native else 0)
        is_rollout = self.rank in self.rollout_ranks
        leader = is_rollout and self.my_replica[0] == self.rank
        followers = [r for r in self.my_replica if r != self.rank] if leader else []
        self.verifier = None
        tp_blocks = None
        if is_rollout and self.native:
            free, _ = torch.cuda.mem_get_info(self.device)
            share = 0.35 if (self.is_trainer or self.rank in self.logprob_ranks) else 0.75
            max_len = min(self.mcfg.max_position_embeddings, config.max_generation_tokens + 4096)
            if self.tp_comm is not None:
                per_block = (self.mcfg.num_hidden_layers * 2 * (self.mcfg.num_key_value_heads // tp_size) * config.kv_block_size
                             * self.mcfg.head_dim * 2)
                tp_blocks = max(64, int(free * share) // per_block)
        if self.tp_comm is not None:
            # the members' schedulers must take identical decisions, so they get the same number of KV blocks: the
            # smallest pool among all tensor-parallel members (a world collective, every rank calls it)
            nb = torch.tensor([tp_blocks or (1 << 40)], dtype=torch.int64, device=self.device)
            dist.all_reduce(nb, op=dist.ReduceOp.MIN)
            tp_blocks = int(nb.item())
        if is_rollout:
            if leader:
                self.verifier = get_or_create_verifier_pool(config.global_num_verifiers, config.write_failed_generation_samples,
                                                            config.reward_fns, config.output_dir, name=f"verifier_pool_{self.rank}",
                                                            timeout_s=config.verifier_timeout_s)
            if self.native:
                from .engine.engine import RolloutEngine

                self.engine = RolloutEngine(self.mcfg, self.layout, self.infer_params, max_seqs=config.max_num_seqs,
                                            max_model_len=max_len, kv_memory_bytes=int(free * share), num_blocks=tp_blocks,
                                            use_cuda_graph=config.vllm_engine_preset == "throughput", block_size=config.kv_block_size,
                                            tp=self.tp_comm, prefix_caching=config.enable_prefix_caching)
            else:
                from .engine.engine import OracleEngine

                self.engine = OracleEngine(self.mcfg, self.layout, self.infer_params, max_seqs=config.max_num_seqs,
                                           max_model_len=min(self.mcfg.max_position_embeddings, config.max_generation_tokens + 2048))
            if leader:
                mirror = None
                if followers:
                    from .roles.tp_mirror import LeaderChannel

                    mirror = LeaderChannel(self._store(), followers)
                self.generation = GenerationWorker(config, self.mcfg, self.engine, self.verifier, load_tokenizer(config),
                                                   stream=self.streams["rollout"], sm_limit=int(self.streams.get("rollout_sm_count", 0)),
                                                   mirror=mirror)
                if config.stream_logprobs:
                    self.generation.logprob_fn = self._stream_logprob
            else:
                # member of a replica that another rank leads: replays the leader's engine calls (on CPU ranks, where
                # the oracle engine has no sharded form, as a full copy of the model)
                from .roles.tp_mirror import FollowerListener, TpFollower

                self.generation = TpFollower(self.engine, FollowerListener(self._store(), self.rank), stream=self.streams["rollout"],
                                             kernel_checks=bool(config.kernel_checks))
        self._lp_next = 0
        import concurrent.futures

        self._comm_pool = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="comm")
        self.host = RoleHost(self)
        self.server: Any = None
        self.clients: Dict[int, Any] = {}
        self.stop_event: Any = None
        self._events: Dict[str, Any] = {}
        self._walls: Dict[str, float] = {}
        self.generation_controllers: List[Any] = []
        self.logprob_controllers: List[Any] = []
        if config.resume_from_path:
            self._resume_optimizer(config.resume_from_path)
        dist.barrier()

    def _resume_optimizer(self, path: str) -> None:
        """Every rank calls this during construction. Trainer ranks reload their optimizer shard (re-sharded when the
        checkpoint was written by another trainer count) and rebuild their parameters from the masters; the first weight
        push then carries them to the inference ranks, which until then take a copy through the trainer group's
        leader so that generation never starts from the initial weights."""
        loaded = False
        if self.is_trainer:
            loaded = self.trainer.core.load_optimizer_checkpoint(path)
            if self.rank == self.trainer_ranks[0]:
                (logger.info if loaded else logger.warning)(
                    "resume_from_path %s: %s", path, "optimizer state and schedule reloaded" if loaded
                    else "no optimizer state found; starting with zero moments")
        flag = torch.tensor([1 if loaded else 0], device=self.device)
        self.dist.broadcast(flag, src=self.trainer_ranks[0])
        if not bool(int(flag.item())):
            return
        # inference copies: one broadcast of the full parameters from the first trainer rank (start-up only)
        core = self.trainer.core if self.is_trainer else None
        dtype = torch.bfloat16 if self.native else torch.float32
        if core is not None and not core.zero3:
            full = core.params.to(dtype)
        elif core is not None:
            full = core._gather_full_master().to(dtype)
        else:
            full = torch.empty(self.layout.total, dtype=dtype, device=self.device)
        self.dist.broadcast(full, src=self.trainer_ranks[0])
        if self.infer_params is not None:
            self.infer_params.copy_(full)

    # ------------------------------------------------------------------ servers / clients
    def _store(self):
        from torch.distributed.distributed_c10d import _get_default_store

        return _get_default_store()

    async def _start_server(self) -> None:
        from .rpc import RpcServer

        self.stop_event = asyncio.Event()
        self.server = RpcServer(self.host, "127.0.0.1", 0)
        port = await self.server.start()
        self._store().set(f"agrpo_rpc_port_{self.rank}", str(port))

    async def _client(self, rank: int) -> Any:
        from .rpc import RpcClient

        if rank not in self.clients:
            loop = asyncio.get_running_loop()
            port = int(await loop.run_in_executor(None, lambda: self._store().get(f"agrpo_rpc_port_{rank}").decode()))
            self.clients[rank] = await RpcClient("127.0.0.1", port, name=f"rank{rank}").connect()
        return self.clients[rank]

    def serve_forever(self) -> None:
        async def _serve() -> None:
            await self._start_server()
            await self.stop_event.wait()
            await self._close()

        asyncio.run(_serve())

    async def _close(self) -> None:
        if self.trainer is not None:
            await self.trainer.stop()
        if self.generation is not None:
            self.generation.shutdown()
        if getattr(self, "verifier", None) is not None:
            self.verifier.close()
        for c in self.clients.values():
            await c.close()
        if self.server is not None:
            await self.server.close()

    # ------------------------------------------------------------------ rank-0 API used by the orchestrator
    async def initialize(self, orch: Any = None) -> None:
        assert self.rank == 0, "the orchestrator runs on rank 0"
        await self._start_server()
        self.generation_controllers = []
        for r in self.rollout_leaders:
            self.generation_controllers.append(self.generation if r == 0 else _RemoteGeneration((await self._client(r)).proxy()))
        self.logprob_controllers = []
        handles = [self.logprob if r == 0 else _RemoteLogprob((await self._client(r)).proxy()) for r in self.logprob_ranks]
        k = max(1, int(self.config.logprob_fsdp_size))
        if k > 1:
            # logprob_fsdp_size ranks form one logprob service: its batches are scattered over the members
            from .roles.logprob import LogProbGroup

            for g in range(0, len(handles), k):
                self.logprob_controllers.append(LogProbGroup(self.config, handles[g:g + k]))
        else:
            self.logprob_controllers = handles
        for r in range(1, self.world):
            await self._client(r)

    async def _all(self, method: str, *args: Any, ranks: Optional[Sequence[int]] = None) -> List[Any]:
        ranks = list(range(self.world)) if ranks is None else list(ranks)
        coros = []
        for r in ranks:
            if r == self.rank:
                coros.append(getattr(self.host, method)(*args))
            else:
                coros.append((await self._client(r)).call(method, *args))
        return list(await asyncio.gather(*coros))

    async def start_trainers(self) -> None:
        await self._all("trainer_start", ranks=self.trainer_ranks)

    async def start_local_trainer(self) -> bool:
        if self.trainer is None:
            return False
        if self.rank == 0:
            mgr: Any = self.experience_manager
        else:
            mgr = _RemoteManager((await self._client(0)).proxy())
        self.trainer.set_orchestrator(mgr, self.rank)
        await self.trainer.start_training_loop()
        return True

    async def ping_trainers(self) -> List[bool]:
        out = []
        for r in self.trainer_ranks:
            try:
                out.append(bool((await self._all("trainer_ready", ranks=[r]))[0]))
            except Exception:
                out.append(False)
        return out

    async def sync_weights(self) -> None:
        """Every rank runs its half; the device time of the push (CUDA events, max over ranks) is kept in
        ``sync_device_ms``."""
        self.sync_device_ms_max = max(float(x or 0.0) for x in await self._all("sync_weights"))

    async def verify_weight_sync(self) -> List[str]:
        sums = await self._all("verify_sync")
        if self.config.param_sharding == "zero3" and len(self.trainer_ranks) > 1 and self.use_peer:
            # fully sharded trainers each hold a slice: their partial sums add up to the checksum of the whole vector
            ref = sum(sums[r]["trainer"] for r in self.trainer_ranks)
            tol = 1e-9 * max(1.0, abs(ref)) + 1e-6
            return [f"rank{r}:infer" for r, s in enumerate(sums) if s["infer"] is not None and abs(s["infer"] - ref) > tol]
        ref = sums[self.trainer_ranks[0]]["trainer"]
        bad = []
        for r, s in enumerate(sums):
            for k, v in s.items():
                if v is not None and abs(v - ref) > 0:
                    bad.append(f"rank{r}:{k}")
        return bad

    async def save_checkpoint(self, path: str) -> None:
        await self._all("save_checkpoint", path, ranks=self.trainer_ranks)

    async def barrier_and_sync(self) -> None:
        await self._all("barrier_sync")

    async def record_event(self, name: str) -> None:
        await self._all("record_event", name)

    async def elapsed_ms(self, a: str, b: str) -> float:
        return max(await self._all("elapsed", a, b))

    async def collect_stats(self) -> Dict[str, float]:
        tot: Dict[str, float] = {}
        for s in await self._all("stats"):
            for k, v in s.items():
                tot[k] = tot.get(k, 0.0) + float(v)
        return tot

    async def shutdown(self) -> None:
        for r in range(1, self.world):
            try:
                await (await self._client(r)).call("shutdown", timeout=10.0)
            except Exception:
                pass
        await self._close()

    async def _stream_logprob(self, sample: Dict[str, Any]) -> Dict[str, Any]:
        """Old-policy log-probabilities of one finished sample, asked of a logprob rank directly by the rollout rank
        that produced it (round robin over the logprob ranks; the local worker when this rank hosts one)."""
        r = self.logprob_ranks[self._lp_next % len(self.logprob_ranks)]
        self._lp_next += 1
        if r == self.rank and self.logprob is not None:
            return await self.logprob.inference(sample)
        return await (await self._client(r)).call("lp_inference", sample)

    # ------------------------------------------------------------------ rank-local halves of collective operations
    def _sync_on_device(self) -> None:
        """Runs on this rank's communication thread; every rank of the world executes it once per sync."""
        if self.native:
            torch.cuda.set_device(self.device)  # the current device is per thread; this thread starts on device 0
        core = self.trainer.core if self.trainer is not None else None
        if self.weight_sync is not None:
            src, sharded = core.sync_source() if core is not None else (None, False)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            self.weight_sync.push(src, self.trainer_index, sharded_src=sharded)
            ev1.record()
            torch.cuda.synchronize(self.device)
            self.sync_device_ms = float(ev0.elapsed_time(ev1))  # barrier + push kernels + barrier, on this rank's GPU
            self.weight_sync.pg.check()
        else:
            from .parallel.symm import broadcast_weights

            if self.world == 1:
                self.infer_params.copy_(core.params)
            else:
                src = core.params if core is not None else None
                if src is None and self.infer_params is None:
                    src = torch.empty(0)
                broadcast_weights(src if src is not None else self.infer_params, self.layout, self.world_group, self.trainer_ranks,
                                  self.trainer_index, self.infer_params)
            if self.native:
                torch.cuda.synchronize(self.device)

    async def local_sync_weights(self) -> float:
        loop = asyncio.get_running_loop()
        if self.generation is not None:
            await self.generation.pause_for_sync()
        if self.logprob is not None:
            await loop.run_in_executor(None, self.logprob.pause)  # the batch in flight finishes, no new one starts
        try:
            if self.native:
                torch.cuda.synchronize(self.device)
            await loop.run_in_executor(self._comm_pool, self._sync_on_device)
        finally:
            if self.logprob is not None:
                self.logprob.resume()
            if self.generation is not None:
                await self.generation.resume_after_sync()
        return float(getattr(self, "sync_device_ms", 0.0))

    async def local_checksum(self) -> Dict[str, Optional[float]]:
        out: Dict[str, Optional[float]] = {"trainer": None, "infer": None}
        if self.trainer is not None:
            out["trainer"] = self.trainer.core.param_checksum()
        if self.infer_params is not None:
            out["infer"] = float(self.infer_params.double().sum().item())
        return out

    async def local_save_checkpoint(self, path: str) -> bool:
        core = self.trainer.core

        def _save() -> None:
            full = core.full_master_fp32()  # collective over the trainer group
            if core.rank == 0:
                ckpt.save_hf_model(path, self.mcfg, core.layout, full, tokenizer_src=self.config.model_name_or_path)
            ckpt.save_optimizer_shard(path, core.rank, core.world, core.layout, core.optimizer_state(), core.scheduler_state())

        await asyncio.get_running_loop().run_in_executor(None, self.trainer.run_blocking, _save)
        return True

    def local_stats(self) -> Dict[str, float]:
        s = {"launches": 0.0, "h2d_bytes": 0.0, "d2h_bytes": 0.0}
        if self.trainer is not None:
            c = self.trainer.core
            s["launches"] += float(getattr(c.decoder, "launches", 0))
            s["h2d_bytes"] += float(c.h2d_bytes)
            s["d2h_bytes"] += float(c.d2h_bytes)
        if self.logprob is not None:
            s["launches"] += float(getattr(self.logprob.decoder, "launches", 0))
            s["h2d_bytes"] += float(self.logprob.h2d_bytes)
            s["d2h_bytes"] += float(self.logprob.d2h_bytes)
        if self.engine is not None:
            s["launches"] += float(getattr(self.engine, "launches", 0))
            s["h2d_bytes"] += float(getattr(self.engine, "h2d_bytes", 0))
            s["d2h_bytes"] += float(getattr(self.engine, "d2h_bytes", 0))
            if hasattr(self.engine, "timing_stats"):
                s.update(self.engine.timing_stats())
                s["engine_busy_s"] = float(self.generation.busy_seconds) if self.generation is not None else 0.0
        return s

    def local_record_event(self, name: str) -> bool:
        self._walls[name] = time.time()
        if self.native:
            torch.cuda.synchronize(self.device)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events[name] = ev
        return True

    def local_elapsed(self, a: str, b: str) -> float:
        if self.native:
            torch.cuda.synchronize(self.device)
            return float(self._events[a].elapsed_time(self._events[b]))
        return (self._walls[b] - self._walls[a]) * 1000.0


def build_distributed_runtime(config: GRPOConfig, backend: Optional[str] = None) -> DistributedRuntime:
    return DistributedRuntime(config, backend)


def _spawn_entry(rank: int, world: int, port: int, cfg_dict: Dict[str, Any], rows: Any, max_batches: Optional[int], out_q: Any) -> None:
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port)})
    from .config import make_config
    from .orchestrator import Orchestrator, configure_logging

    configure_logging()
    cfg = make_config(cfg_dict)
    rt = DistributedRuntime(cfg)
    if rank != 0:
        rt.serve_forever()
        return
    try:
        orch = Orchestrator(cfg, runtime=rt, dataset=rows)
        orch.max_macro_batches = max_batches
        result = asyncio.run(orch.run_async())
    except BaseException as e:  # the parent must not wait for its timeout to learn that the run failed
        import traceback

        out_q.put({"error": f"{e!r}\n{traceback.format_exc()}"})
        raise
    out_q.put({"global_step": result["global_step"], "total_samples_seen": result["total_samples_seen"],
               "last": {k: v for k, v in result["steps"][-1].items() if isinstance(v, (int, float))}})


def spawn(config_dict: Dict[str, Any], rows: Any, world: int, max_macro_batches: Optional[int] = None, port: int = 29640,
          timeout_s: float = 600.0) -> Dict[str, Any]:
    """Starts ``world`` role processes on this node (one per GPU, or CPU ranks over gloo) and runs the orchestrator on
    rank 0. This is the counterpart of the reference's placement-group launch for users who do not use torchrun."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_spawn_entry, args=(r, world, port, config_dict, rows, max_macro_batches, q), daemon=False)
             for r in range(world)]
    for p in procs:
        p.start()
    try:
        result = q.get(timeout=timeout_s)
    finally:
        failed = "result" not in locals() or "error" in result
        for p in procs:
            p.join(timeout=5 if failed else 30)
        for p in procs:
            if p.is_alive():
                p.kill()
    if "error" in result:
        raise RuntimeError("the run failed on rank 0: " + result["error"])
    return result


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``python -m async_grpo_nccl_b200.launch --config run.json [--set key=value ...]``

    Runs the orchestrator on the flat config of a JSON file (the reference takes the same keys as a Python dict,
    orchestrator.py:92-193, and has no command line). Started plainly it runs every role in this process (one GPU or
    CPU); started under ``python -m torch.distributed.run --nproc-per-node N`` every rank builds the multi-process runtime,
    rank 0 drives the orchestrator and the other ranks serve their roles."""
    import argparse
    import json as _json

    from .config import make_config
    from .orchestrator import Orchestrator, configure_logging

    ap = argparse.ArgumentParser(prog="async_grpo_nccl_b200.launch")
    ap.add_argument("--config", required=True, help="JSON file with the flat configuration keys")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE",
                    help="override one key; the value is parsed as JSON when it parses, else taken as a string")
    ap.add_argument("--max-macro-batches", type=int, default=None, help="stop after this many macro-batches")
    args = ap.parse_args(argv)
    with open(args.config) as f:
        cfg_dict = dict(_json.load(f))
    for kv in args.set:
        k, _, v = kv.partition("=")
        try:
            cfg_dict[k] = _json.loads(v)
        except ValueError:
            cfg_dict[k] = v
    configure_logging()
    cfg = make_config(cfg_dict)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        rt = DistributedRuntime(cfg)
        if rt.rank != 0:
            rt.serve_forever()
            return 0
        orch = Orchestrator(cfg, runtime=rt)
        orch.max_macro_batches = args.max_macro_batches
        result = asyncio.run(orch.run_async())
    else:
        orch = Orchestrator(cfg)
        orch.max_macro_batches = args.max_macro_batches
        result = orch.run()
    last = result["steps"][-1] if result["steps"] else {}
    print(_json.dumps({"global_step": result["global_step"], "total_samples_seen": result["total_samples_seen"],
                       "last": {k: v for k, v in last.items() if isinstance(v, (int, float))}}, default=float))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
