"""Symmetric (peer-mapped) device buffers and the collectives built on them.

Every rank of a group allocates the same buffers through ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations whose handles are exchanged between the processes), so each rank holds a device pointer to every
peer's copy. The kernels in ``csrc/kernels/symm.cu`` then move data themselves:

* ``TrainerComm.reduce_scatter``  owner pulls its shard out of every peer's fp32 gradient buffer (+ norm partial)
* ``TrainerComm.adamw_and_publish`` AdamW on the shard, bf16 result stored into every trainer rank's resident
  parameter buffer (this IS the parameter all-gather)
* ``WeightSync.push``             trainer shard -> every rollout / logprob rank's parameter buffer
* ``barrier``                     epoch flags with bounded waits

They replace the NCCL calls of the reference: FSDP2's reduce-scatter / all-gather and ``clip_grad_norm_``'s
all-reduce (gpu_process_worker.py:696-713, 1052-1079) and the per-tensor broadcast of the weight sync
(gpu_process_worker.py:1609-1637). ``CollectiveFallback`` implements the same operations with
``torch.distributed`` collectives (NCCL on GPUs, gloo on CPU ranks); it is the measured baseline and the path
taken when symmetric memory is unavailable.
"""
from __future__ import annotations

import logging
from typing import Any, List, Optional, Sequence

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)

WAIT_BUDGET_S = 20.0  # a barrier partner may legitimately be busy for seconds (long backward); bounded all the same


class SymmetricBuffer:
    def __init__(self, local: torch.Tensor, peer_ptrs: List[int], handle: Any):
        self.local, self.peer_ptrs, self.handle = local, peer_ptrs, handle
        # NVSwitch multicast address of the buffer (0 when the fabric or the driver offers none): one store to it
        # lands in every rank's copy, one ld_reduce from it sums every rank's copy inside the switch
        try:
            self.mc_ptr = int(getattr(handle, "multicast_ptr", 0) or 0)
        except Exception:
            self.mc_ptr = 0


def _trace(op: str, **kw: Any) -> None:
    """AGRPO_TRACE_COLLECTIVES=1 logs every collective / barrier this rank enqueues, with its epoch: a mismatched
    sequence between ranks (the usual cause of a barrier that runs out) shows up by diffing the ranks' logs. The
    reference has the same aid for torch.distributed calls (gpu_process_worker.py:557-592), also off by default."""
    import os

    if os.environ.get("AGRPO_TRACE_COLLECTIVES", "0") == "1":
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        logger.info("[collective rank %d] %s %s", rank, op, " ".join(f"{k}={v}" for k, v in kw.items()))


def multicast_enabled() -> bool:
    """NVLS (multimem) variants of the weight push and the gradient reduce-scatter are used when the symmetric
    allocation comes with a multicast address, unless AGRPO_MULTICAST=0."""
    import os

    return os.environ.get("AGRPO_MULTICAST", "1") != "0"


def symmetric_available() -> bool:
    try:
        import torch.distributed._symmetric_memory as sm  # noqa: F401

        return torch.cuda.is_available()
    except Exception:
        return False


def alloc_symmetric(numel: int, dtype: torch.dtype, device: torch.device, group: Any) -> SymmetricBuffer:
    """Collective over ``group``: every rank gets its local tensor and the device addresses of all peers' tensors."""
    import torch.distributed._symmetric_memory as sm

    name = group.group_name if hasattr(group, "group_name") else group
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            sm.enable_symm_mem_for_group(name)  # needed by older torch releases, a no-op on newer ones
        except Exception:
            pass
    t = sm.empty(numel, dtype=dtype, device=device)
    try:
        hdl = sm.rendezvous(t, group=name)
    except TypeError:
        hdl = sm.rendezvous(t, name)
    t.zero_()
    return SymmetricBuffer(t, [int(p) for p in hdl.buffer_ptrs], hdl)


class PeerGroup:
    """Epoch flags + device-side barrier among ``members`` (global ranks). The flag words live in a symmetric buffer
    allocated over the WORLD group: symmetric allocations are always made by every rank of the job, in the same
    order, so that no rank waits in a rendezvous that others never enter; sub-groups are index subsets of it."""

    def __init__(self, flags: SymmetricBuffer, members: Sequence[int], my_global_rank: int, device: torch.device, C: Any,
                 slot_base: int = 0):
        self.members = list(members)
        self.is_member = my_global_rank in self.members
        self.rank = self.members.index(my_global_rank) if self.is_member else -1
        self.world = len(self.members)
        self.C, self.device = C, device
        # every member's flag block starts slot_base words into its flag buffer (8 bytes per word)
        self.ptrs = [flags.peer_ptrs[r] + 8 * slot_base for r in self.members]
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def barrier(self) -> None:
        """Enqueues a device-side barrier on the current stream (no host synchronisation)."""
        if not self.is_member:
            return
        self.epoch += 1
        _trace("barrier", members=self.members, epoch=self.epoch)
        self.C.flag_barrier(self.ptrs, self.rank, self.epoch, WAIT_BUDGET_S, self.status)

    def check(self) -> None:
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer barrier / flag wait ran out (status {code}): a rank of the group did not arrive")


class SymmetricPlane:
    """All symmetric buffers of a job, allocated collectively over the WORLD group by every rank in a fixed order."""

    def __init__(self, device: torch.device, layout: Any, C: Any, trainer_ranks: Sequence[int], infer_ranks: Sequence[int],
                 world_group: Any = None, zero3: bool = False):
        self.device, self.layout, self.C = device, layout, C
        self.group = world_group if world_group is not None else dist.group.WORLD
        self.my_rank = dist.get_rank()
        self.trainer_ranks, self.infer_ranks = list(trainer_ranks), list(infer_ranks)
        need_train = len(self.trainer_ranks) > 1
        self.flags = alloc_symmetric(128, torch.int64, device, self.group)          # [0,64): trainer barrier, [64,128): world
        self.norm_tab = alloc_symmetric(64, torch.float32, device, self.group)
        self.infer_params = alloc_symmetric(layout.total, torch.bfloat16, device, self.group)
        self.zero3 = bool(zero3) and need_train
        self.train_params = self.grads = self.shard16 = self.grad_shard = None
        if self.zero3:
            # fully sharded: every rank holds 1/W of the bf16 parameters and of the fp32 gradients, nothing else
            n = layout.shard_numel()
            self.shard16 = alloc_symmetric(n, torch.bfloat16, device, self.group)
            self.grad_shard = alloc_symmetric(n, torch.float32, device, self.group)
        elif need_train:
            self.train_params = alloc_symmetric(layout.total, torch.bfloat16, device, self.group)
            self.grads = alloc_symmetric(layout.total, torch.float32, device, self.group)

    def trainer_comm(self) -> Optional[Any]:
        if self.my_rank not in self.trainer_ranks:
            return None
        if self.zero3:
            from .zero3 import Zero3Comm

            return Zero3Comm(self)
        if self.grads is None:
            return None
        return TrainerComm(self)

    def weight_sync(self) -> "WeightSync":
        return WeightSync(self)


class TrainerComm:
    """Peer-memory gradient reduce-scatter, norm exchange and AdamW + parameter publish for the trainer ranks."""

    def __init__(self, plane: SymmetricPlane):
        self.plane = plane
        self.layout, self.C, self.device = plane.layout, plane.C, plane.device
        self.pg = PeerGroup(plane.flags, plane.trainer_ranks, plane.my_rank, plane.device, plane.C, slot_base=0)
        self.rank, self.world = self.pg.rank, self.pg.world
        tr = plane.trainer_ranks
        self.grad_ptrs = [plane.grads.peer_ptrs[r] for r in tr]
        self.param_ptrs = [plane.train_params.peer_ptrs[r] for r in tr]
        self.norm_ptrs = [plane.norm_tab.peer_ptrs[r] for r in tr]
        self.norm_local = torch.zeros(1, dtype=torch.float32, device=plane.device)
        # in-switch reduction: valid because every rank of the job holds a gradient buffer of the same shape and the
        # ranks that do not train never write theirs (it stays zero)
        self.grads_mc = plane.grads.mc_ptr if multicast_enabled() else 0

    @property
    def param_buffer(self) -> torch.Tensor:
        return self.plane.train_params.local

    @property
    def grad_buffer(self) -> torch.Tensor:
        return self.plane.grads.local

    @property
    def norm_partials(self) -> torch.Tensor:
        return self.plane.norm_tab.local[: self.world]

    def reduce_scatter(self, grad_shard: torch.Tensor) -> None:
        """grad_shard <- sum over ranks of this rank's slice of every unit; norm partial published to all peers."""
        C, L = self.C, self.layout
        _trace("reduce_scatter", multicast=bool(self.grads_mc))
        C.set_comm_guard(self.pg.status)  # kernels behind a barrier that timed out return without touching anything
        self.pg.barrier()  # every rank's backward has finished and its gradients are visible
        self.norm_local.zero_()
        for u, (lo, gs, ln) in enumerate(L.local_to_global_ranges(self.rank)):
            if self.grads_mc:
                C.rs_pull_sumsq_mc(self.grads_mc, gs, lo, ln, grad_shard, self.norm_local)
            else:
                C.rs_pull_sumsq(self.grad_ptrs, self.rank, gs, lo, ln, grad_shard, self.norm_local)
        C.publish_norm(self.norm_local, self.norm_ptrs, self.rank)
        self.pg.barrier()  # all partials have landed; all peers are done reading my gradient buffer
        self.grad_buffer.zero_()

    def adamw_and_publish(self, master, exp_avg, exp_avg_sq, grad_shard, lr, beta1, beta2, eps, wd, step, max_norm,
                          extra_dst_ptrs: Sequence[int] = ()) -> torch.Tensor:
        """Returns the device tensor holding the per-rank squared-norm partials (sum = global squared norm)."""
        C, L = self.C, self.layout
        _trace("adamw_and_publish", step=step)
        C.set_comm_guard(self.pg.status)
        dsts = list(self.param_ptrs) + list(extra_dst_ptrs)
        partials = self.norm_partials
        for u, (lo, gs, ln) in enumerate(L.local_to_global_ranges(self.rank)):
            C.adamw_push(master, exp_avg, exp_avg_sq, grad_shard, lo, gs, ln, lr, beta1, beta2, eps, wd, step, 1.0, partials,
                         max_norm, dsts)
        self.pg.barrier()  # every rank's bf16 shard is in my parameter buffer before the next forward reads it
        return partials


class WeightSync:
    """Trainer shards -> inference parameter buffers; barriers span every rank of the job."""

    def __init__(self, plane: SymmetricPlane):
        self.plane = plane
        self.layout, self.C = plane.layout, plane.C
        self.trainer_ranks, self.infer_ranks = plane.trainer_ranks, plane.infer_ranks
        world = list(range(dist.get_world_size()))
        self.pg = PeerGroup(plane.flags, world, plane.my_rank, plane.device, plane.C, slot_base=64)
        self.dst_ptrs = [plane.infer_params.peer_ptrs[r] for r in self.infer_ranks]
        # multicast push: the switch replicates every store into all ranks' buffers (also into the unused copies of
        # ranks that host no inference role), so a trainer's egress does not grow with the number of receivers
        self.dst_mc = plane.infer_params.mc_ptr if (multicast_enabled() and len(self.infer_ranks) > 1) else 0

    @property
    def buffer(self) -> torch.Tensor:
        return self.plane.infer_params.local

    def push(self, src_params: Optional[torch.Tensor], trainer_index: Optional[int], sharded_src: bool = False) -> None:
        """Collective over all ranks. Trainer ranks pass their bf16 parameters (the resident flat buffer, or with
        ``sharded_src`` just their own slices back to back) and their index among the trainers; the others pass None
        and only take part in the barriers."""
        _trace("weight_push", source=trainer_index, sharded=sharded_src, multicast=bool(self.dst_mc))
        self.C.set_comm_guard(self.pg.status)
        self.pg.barrier()  # inference ranks are idle (paused by the orchestrator) and trainers finished their step
        if src_params is not None and trainer_index is not None:
            t = len(self.trainer_ranks)
            lo = 0
            for u in range(len(self.layout.unit_ranges)):
                s, e = self.layout.unit_ranges[u]
                n = (e - s) // t
                a = s + trainer_index * n
                if self.dst_mc:
                    self.C.weight_push_mc(src_params, lo if sharded_src else a, a, n, self.dst_mc)
                else:
                    self.C.weight_push(src_params, lo if sharded_src else a, a, n, self.dst_ptrs)
                lo += n
        self.pg.barrier()  # all shards have landed everywhere


class TensorParallelComm:
    """What a tensor-parallel rollout rank needs from peer memory (the reference gets it from vLLM's NCCL all-reduce,
    vllm_worker.py:219-232): two symmetric [rows, H] bf16 buffers that receive this rank's partial products of the
    row-parallel projections (o and down), a barrier whose epoch lives on the device (so the step can be replayed from a
    CUDA graph), and the all-reduce + residual + row-statistic kernel that reads every member's partial with peer loads.

    Every rank of the job allocates the buffers (symmetric allocations are collective over the world group); ``members``
    are the global ranks of ONE engine replica, in tensor-parallel order."""

    def __init__(self, members: Sequence[int], my_global_rank: int, rows: int, hidden: int, device: torch.device, C: Any,
                 group: Any = None):
        grp = group if group is not None else dist.group.WORLD
        self.members = list(members)
        self.size = len(self.members)
        self.rank = self.members.index(my_global_rank) if my_global_rank in self.members else -1
        self.C, self.device, self.rows, self.hidden = C, device, rows, hidden
        self.flags = alloc_symmetric(64, torch.int64, device, grp)
        self.bufs = [alloc_symmetric(rows * hidden, torch.bfloat16, device, grp) for _ in range(2)]
        self.flags.local.zero_()
        self.flag_ptrs = [self.flags.peer_ptrs[r] for r in self.members]
        self.partial_ptrs = [[b.peer_ptrs[r] for r in self.members] for b in self.bufs]
        self.epoch = torch.zeros(1, dtype=torch.int64, device=device)
        self.arrive = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def partial(self, which: int, rows: int) -> torch.Tensor:
        """This rank's partial-product buffer ``which`` (0: o projection, 1: down projection) as [rows, H]."""
        return self.bufs[which].local[: rows * self.hidden].view(rows, self.hidden)

    def allreduce_residual(self, which: int, residual: torch.Tensor, out: torch.Tensor, ss: Optional[torch.Tensor]) -> None:
        """out = residual + sum over members of their partial ``which``; ss += row sums of squares of out."""
        self.C.tp_allreduce_residual(self.partial_ptrs[which], self.flag_ptrs, self.rank, self.epoch, self.arrive, residual, out,
                                     ss, WAIT_BUDGET_S, self.status)

    def check(self) -> None:
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"tensor-parallel barrier ran out (status {code}): a member of the engine replica did not arrive")


class CollectiveFallback:
    """The same three operations on ``torch.distributed`` collectives (NCCL / gloo)."""

    def __init__(self, group: Any, layout: Any, rank: int, world: int):
        self.group, self.layout, self.rank, self.world = group, layout, rank, world
        self.backend = dist.get_backend(group)

    def reduce_scatter(self, full_grad: torch.Tensor, grad_shard: torch.Tensor) -> None:
        for u, (lo, gs, ln) in enumerate(self.layout.local_to_global_ranges(self.rank)):
            s, e = self.layout.unit_ranges[u]
            if self.backend == "gloo":
                buf = full_grad[s:e].clone()
                dist.all_reduce(buf, group=self.group)
                grad_shard[lo:lo + ln].copy_(buf[gs - s: gs - s + ln])
            else:
                dist.reduce_scatter_tensor(grad_shard[lo:lo + ln], full_grad[s:e], op=dist.ReduceOp.SUM, group=self.group)

    def all_gather_params(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        for u, (lo, gs, ln) in enumerate(self.layout.local_to_global_ranges(self.rank)):
            s, e = self.layout.unit_ranges[u]
            if self.backend == "gloo":
                parts = [torch.empty(ln, dtype=shard.dtype) for _ in range(self.world)]
                dist.all_gather(parts, shard[lo:lo + ln].contiguous(), group=self.group)
                full[s:e].copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(full[s:e], shard[lo:lo + ln].contiguous(), group=self.group)

    def all_reduce_scalar(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, group=self.group)


def broadcast_weights(params: torch.Tensor, layout: Any, world_group: Any, trainer_global_ranks: Sequence[int],
                      is_trainer_index: Optional[int], dst: Optional[torch.Tensor]) -> None:
    """NCCL / gloo weight sync: every trainer rank broadcasts its shard of every unit to the whole world group.
    Ranks that hold inference parameters copy the received ranges into ``dst``. This mirrors the reference's
    broadcast-based sync (one broadcast per shard range instead of one per tensor)."""
    t = len(trainer_global_ranks)
    for u in range(len(layout.unit_ranges)):
        s, e = layout.unit_ranges[u]
        n = (e - s) // t
        for ti, gr in enumerate(trainer_global_ranks):
            a, b = s + ti * n, s + (ti + 1) * n
            if is_trainer_index == ti:
                buf = params[a:b]
            else:
                buf = dst[a:b] if dst is not None else torch.empty(b - a, dtype=params.dtype if params is not None else torch.bfloat16,
                                                                  device=(dst.device if dst is not None else params.device))
            dist.broadcast(buf, src=gr, group=world_group)
            if is_trainer_index == ti and dst is not None:
                dst[a:b].copy_(buf)
