"""Stand-ins for the libraries the reference imports that this image does not have.

The reference's modules import ``ray``, ``omegaconf``, ``peft`` and three vLLM v0 worker classes at module
level (gpu_process_worker.py:8, 20-21, 35-37, 46). None of them can be installed offline here. Only names
are needed to let ``gpu_process_worker.py`` load and its worker methods run unmodified:

* ``ray.remote`` decorates the worker classes; the stand-in returns the class itself, so a "remote actor"
  is a plain object in the calling process.
* ``ray.util.collective.collective.broadcast`` is what every worker's ``sync_weights`` calls once per
  parameter tensor (gpu_process_worker.py:1634, 1734, 1906). The stand-in performs the same NCCL broadcast
  over a communicator that spans one member per process (``SyncGroup``); workers that share a process (and
  therefore a GPU, which NCCL refuses to list twice) exchange the tensor through ``SyncGroup.stash``.
* ``omegaconf.DictConfig`` and ``peft.*`` are annotations / unused imports.
* The vLLM v0 classes are only used by ``RolloutGPUWorker``, which this harness replaces by vLLM 0.22's own
  in-process worker.

This file imports nothing from ``async_grpo_nccl_b200``.
"""
from __future__ import annotations

import sys
import types
from typing import Any, Dict, List, Optional


class SyncGroup:
    """The reference's ``sync_group`` communicator: rank order trainer + logprob + rollout, source = rank 0
    (orchestrator.py:552-579, 596-625). One NCCL member per process."""

    def __init__(self) -> None:
        self.comm = None            # PyNcclCommunicator or None (single member)
        self.rank = 0
        self.world = 1
        self.stash: List[Any] = []  # tensors the first worker of this process sent / received, in call order
        self.replay: Optional[int] = None  # index into stash while a colocated second worker "receives"
        self.calls = 0
        self.bytes = 0

    def broadcast(self, tensor, src_rank: int = 0, group_name: str = "default") -> None:
        if self.replay is not None:
            # second worker of this process: same bytes, device-to-device
            tensor.copy_(self.stash[self.replay])
            self.replay += 1
            return
        if self.comm is not None:
            self.comm.broadcast(tensor, src=src_rank)
        self.calls += 1
        self.bytes += tensor.numel() * tensor.element_size()
        if self.keep_stash:
            self.stash.append(tensor)

    keep_stash = False

    def begin_primary(self, keep_stash: bool) -> None:
        self.stash = []
        self.replay = None
        self.keep_stash = keep_stash

    def begin_secondary(self) -> None:
        self.replay = 0

    def end(self) -> None:
        self.stash = []
        self.replay = None
        self.keep_stash = False


SYNC_GROUP = SyncGroup()


STUBS: List[str] = []


def _module(name: str, **attrs: Any) -> types.ModuleType:
    import importlib.machinery

    m = types.ModuleType(name)
    m.__spec__ = importlib.machinery.ModuleSpec(name, None)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    STUBS.append(name)
    return m


def retire(names=("peft", "omegaconf")) -> None:
    """Takes stand-ins out of ``sys.modules`` once the reference's modules hold the names they imported, so that
    libraries probing for the real package (``transformers`` asks for ``peft``) see it as absent."""
    for n in names:
        if n in STUBS and n in sys.modules:
            del sys.modules[n]


def transformers_compat() -> str:
    """The reference reads ``model._no_split_modules[0]`` (gpu_process_worker.py:402, its FSDP wrapping for more than one
    trainer rank). The installed transformers 5 keeps that attribute as a set; older versions kept the class's list. This
    makes the set indexable (sorted order; Qwen2 has a single entry) without touching the reference or the set semantics
    that transformers itself relies on. Returns a description for the JSON record."""
    from transformers import PreTrainedModel

    class IndexableSet(set):
        def __getitem__(self, i):
            return sorted(self)[i]

    orig = PreTrainedModel.post_init
    if not getattr(orig, "_agrpo_compat", False):
        def post_init(self, *a: Any, **k: Any):
            out = orig(self, *a, **k)
            ns = getattr(self, "_no_split_modules", None)
            if isinstance(ns, set) and not isinstance(ns, IndexableSet):
                self._no_split_modules = IndexableSet(ns)
            return out

        post_init._agrpo_compat = True  # type: ignore[attr-defined]
        PreTrainedModel.post_init = post_init
    return "transformers.PreTrainedModel._no_split_modules made indexable (a set since transformers 5)"


def install() -> Dict[str, str]:
    """Registers the stand-in modules. Returns {module name: what it stands for} for the JSON record."""
    made: Dict[str, str] = {}

    def remote(*args: Any, **kwargs: Any):
        if len(args) == 1 and not kwargs and isinstance(args[0], type):
            return args[0]
        return lambda cls: cls

    if "ray" not in sys.modules:
        class _Collective:
            @staticmethod
            def broadcast(tensor, src_rank: int = 0, group_name: str = "default"):
                SYNC_GROUP.broadcast(tensor, src_rank, group_name)

            @staticmethod
            def barrier(group_name: str = "default"):
                return None

        ray = _module("ray", remote=remote, get=lambda x: x, kill=lambda *a, **k: None)
        util = _module("ray.util")
        coll_pkg = _module("ray.util.collective", collective=_Collective, broadcast=_Collective.broadcast)
        _module("ray.util.collective.collective", broadcast=_Collective.broadcast, barrier=_Collective.barrier)
        ray.util = util
        util.collective = coll_pkg
        ray.actor = _module("ray.actor", ActorHandle=object)
        pg = _module("ray.util.placement_group", placement_group=None, PlacementGroup=object, remove_placement_group=None,
                     placement_group_table=None)
        util.placement_group = pg
        ss = _module("ray.util.scheduling_strategies", PlacementGroupSchedulingStrategy=object,
                     NodeAffinitySchedulingStrategy=object)
        util.scheduling_strategies = ss
        util.get_node_ip_address = lambda: "127.0.0.1"
        _module("ray.exceptions", RayActorError=Exception, GetTimeoutError=TimeoutError, RayTaskError=Exception)
        made["ray"] = "decorator + NCCL broadcast stand-in"
    try:
        import omegaconf  # noqa: F401
    except Exception:
        _module("omegaconf", DictConfig=dict)
        made["omegaconf"] = "DictConfig annotation"
    try:
        import peft  # noqa: F401
    except Exception:
        _module("peft", LoraConfig=object, TaskType=object, get_peft_model=lambda m, *a, **k: m)
        made["peft"] = "unused imports"
    for name, attrs in (("vllm.worker", {}), ("vllm.worker.worker", {"Worker": object}),
                        ("vllm.worker.worker_base", {"WorkerWrapperBase": object}),
                        ("vllm.model_executor.sampling_metadata", {"SamplingMetadata": object})):
        try:
            __import__(name)
        except Exception:
            _module(name, **attrs)
            made[name] = "vLLM v0 class name (RolloutGPUWorker only)"
    return made
