"""Spatial partition of one GPU's SMs between roles that share it (CUDA green contexts).

When the rollout engine shares a GPU with the trainer and the logprob role (one-GPU runs, or a placement that puts a
rollout rank on a trainer's GPU) the roles' kernels compete for the same SMs. A decode step is a chain of short,
latency-bound kernels; a trainer GEMM is a persistent kernel that holds every SM for milliseconds and cannot be
pre-empted. Stream priorities only decide which thread block is placed next, so without a partition every decode step
queues behind whatever trainer blocks are resident, and the trainer in turn starves while a persistent decode kernel
holds all SMs. With the SMs split into two disjoint sets both run at the same time: the decode chain keeps its latency,
and the trainer's work (a few seconds per macro-batch) hides behind the much longer generation phase.

The reference gives every role its own GPU (Ray ``num_gpus=1`` actors, ray_utils.py:158-197) and has no counterpart.

``split(device, first)`` returns two ``SmGroup``s (``first`` SMs rounded to the hardware's granularity, and the
rest), each with a factory for ``torch`` streams that run only on that group's SMs. Memory is shared (green contexts
belong to the device's primary context). Kernels that size a persistent grid by the SM count must be told the group's
count (``ops.native().set_sm_limit``): a cooperative launch larger than the group cannot become resident.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

import torch

logger = logging.getLogger(__name__)


@dataclass
class SmGroup:
    sm_count: int
    green_ctx: Any
    device: torch.device
    _streams: List[Any]

    def stream(self, priority: int = 0) -> torch.cuda.Stream:
        from cuda.bindings import driver as drv

        err, s = drv.cuGreenCtxStreamCreate(self.green_ctx, drv.CUstream_flags.CU_STREAM_NON_BLOCKING, priority)
        _check(err, "cuGreenCtxStreamCreate")
        self._streams.append(s)
        return torch.cuda.ExternalStream(int(s), device=self.device)


def _check(err: Any, what: str) -> None:
    from cuda.bindings import driver as drv

    if err != drv.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"{what} failed: {err}")


def split(device: torch.device, first: int) -> Optional[Tuple[SmGroup, SmGroup]]:
    """Two disjoint SM groups of ``device``: about ``first`` SMs and the remainder. None when the driver or the device
    does not offer green contexts (the caller then runs all roles on the whole device, as before)."""
    try:
        from cuda.bindings import driver as drv
    except Exception as e:  # pragma: no cover - depends on the image
        logger.warning("SM partition unavailable (cuda-python missing: %r)", e)
        return None
    try:
        device = torch.device(device)
        torch.cuda.init()
        with torch.cuda.device(device):
            torch.cuda.current_stream().synchronize()  # the primary context exists
            err, dev = drv.cuDeviceGet(device.index or 0)
            _check(err, "cuDeviceGet")
            err, sm_res = drv.cuDeviceGetDevResource(dev, drv.CUdevResourceType.CU_DEV_RESOURCE_TYPE_SM)
            _check(err, "cuDeviceGetDevResource")
            total = int(sm_res.sm.smCount)
            if first < 8 or first > total - 8:
                raise ValueError(f"cannot split {total} SMs into {first} + rest")
            err, groups, n_groups, remaining = drv.cuDevSmResourceSplitByCount(1, sm_res, 0, int(first))
            _check(err, "cuDevSmResourceSplitByCount")
            if n_groups < 1 or int(remaining.sm.smCount) < 8:
                raise RuntimeError("split returned no usable groups")
            out = []
            for res in (groups[0], remaining):
                err, desc = drv.cuDevResourceGenerateDesc([res], 1)
                _check(err, "cuDevResourceGenerateDesc")
                err, gctx = drv.cuGreenCtxCreate(desc, dev, drv.CUgreenCtxCreate_flags.CU_GREEN_CTX_DEFAULT_STREAM)
                _check(err, "cuGreenCtxCreate")
                out.append(SmGroup(int(res.sm.smCount), gctx, device, []))
            logger.info("GPU %s split into %d + %d SMs", device, out[0].sm_count, out[1].sm_count)
            return out[0], out[1]
    except Exception as e:
        logger.warning("SM partition unavailable on %s: %r", device, e)
        return None
