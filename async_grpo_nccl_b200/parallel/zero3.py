"""Fully sharded parameters and gradients (ZeRO-3 / FSDP style) on peer memory.

The reference shards every transformer block with FSDP2 (``fully_shard`` per block and on the root,
gpu_process_worker.py:408-418): before a block runs NCCL all-gathers its parameters, after its backward NCCL
reduce-scatters its gradients. Here the same two collectives are fused with the GEMMs next to them:

* ``ShardedWeights``  Each rank keeps only its 1/W slice of every layout unit (bf16, symmetric memory). A unit is
  staged into one of two local buffers by copier CTAs that pull the slices out of the owners' memory over NVLink.
  Those CTAs ride in the grid of a GEMM of the previous unit (``ag_gemm``): the gather of layer l+1 overlaps the
  math of layer l inside one kernel, no second stream, no NCCL. When the GEMM consumes the unit being gathered, its
  TMA producer waits (bounded) on per-chunk ready flags, tile by tile.
* ``ScatterSink``     Weight-gradient GEMMs do not store dW: the epilogue adds every fp32 tile with vector ``red``
  straight into the gradient shard of the rank that owns it (``gemm_rs``). Reductions from every rank and every
  microbatch meet in the owner's shard; one barrier before the optimizer step is the only synchronisation. The
  gradients that no GEMM produces (norm weights, biases, the embedding group) go through ``scatter_add_f32``.

Per-rank memory for P parameters over W ranks: 2P/W (bf16 slice) + 16P/W (fp32 master, two moments, gradient shard)
+ two staged layers + the embedding group (bf16 staging and fp32 gradients), instead of 2P + 4P + 12P/W.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

SMALL_LAYER_PARAMS = ("ln1", "ln2", "bqkv")


class ShardedWeights:
    """Just-in-time all-gather of layout units into local staging buffers."""

    def __init__(self, layout: Any, C: Any, device: torch.device, my_rank: int, shard_ptrs: Sequence[int],
                 n_copy: int = 8, chunk_elems: int = 1 << 18):
        self.layout, self.C, self.device = layout, C, torch.device(device)
        self.rank, self.world = int(my_rank), len(shard_ptrs)
        assert self.world == layout.shard_world, "the layout must be padded for this many owners"
        self.shard_ptrs = [int(p) for p in shard_ptrs]
        self.n_copy, self.chunk = int(n_copy), int(chunk_elems)
        self.unit_start = [s for s, _ in layout.unit_ranges]
        self.unit_n = [e - s for s, e in layout.unit_ranges]
        self.local_off = [lo for lo, _, _ in layout.local_to_global_ranges(self.rank)]
        layer_max = max(self.unit_n[1:]) if len(self.unit_n) > 1 else 128
        bf16 = torch.bfloat16
        # slot 0: the embedding group, resident for a whole step; slots 1 and 2: alternating layers
        self.staging = [torch.empty(self.unit_n[0], dtype=bf16, device=self.device),
                        torch.empty(layer_max, dtype=bf16, device=self.device),
                        torch.empty(layer_max, dtype=bf16, device=self.device)]
        self.flags = [torch.zeros((t.numel() + self.chunk - 1) // self.chunk, dtype=torch.int64, device=self.device)
                      for t in self.staging]
        self.resident: List[Optional[Tuple[int, int]]] = [None, None, None]  # (unit, version) per slot
        self.version = 0
        self.epoch = 0
        self.pending: Optional[int] = None
        self.status: Optional[torch.Tensor] = None  # error word of the decoder that uses these weights
        self.gathers_standalone = 0
        self.gathers_fused = 0

    # ---- bookkeeping ----
    def slot_of(self, unit: int) -> int:
        return 0 if unit == 0 else 1 + (unit % 2)

    def is_resident(self, unit: int) -> bool:
        return self.resident[self.slot_of(unit)] == (unit, self.version)

    def invalidate(self) -> None:
        """The owners' slices changed (optimizer step): everything staged is stale."""
        self.version += 1
        self.pending = None

    def _src_ptrs(self, unit: int) -> List[int]:
        return [p + 2 * self.local_off[unit] for p in self.shard_ptrs]

    def _job(self, unit: int) -> Dict[str, Any]:
        slot = self.slot_of(unit)
        self.epoch += 1
        self.resident[slot] = (unit, self.version)
        return dict(src_ptrs=self._src_ptrs(unit), my_rank=self.rank, staging=self.staging[slot],
                    n_per_owner=self.unit_n[unit] // self.world, flags=self.flags[slot], epoch=self.epoch,
                    chunk_elems=self.chunk)

    # ---- used by the decoder ----
    def enter(self, unit: int, then: Optional[int]) -> int:
        """``unit`` is about to be used: stage it now unless it already is. ``then`` is gathered by the next large GEMM
        launch. Returns the number of kernels launched."""
        n = 0
        if self.pending == unit:
            self.pending = None
        if not self.is_resident(unit):
            j = self._job(unit)
            self.C.unit_gather(j["src_ptrs"], j["my_rank"], j["staging"], j["n_per_owner"], j["flags"], j["epoch"],
                               j["chunk_elems"], 64, self.status)
            self.gathers_standalone += 1
            n = 1
        self.pending = then if (then is not None and not self.is_resident(then)) else None
        return n

    def wants_ride(self, a: torch.Tensor, b: torch.Tensor) -> bool:
        """A pending gather rides on the largest GEMM of a block (the gate/up projection or its input-gradient GEMM):
        the launch lasts as long as the slower of its math and the copy, so a small GEMM would be stretched."""
        if self.pending is None or a.shape[0] < 1024:
            return False
        return b.numel() * 5 >= 2 * self.unit_n[self.pending]

    def gemm_with_prefetch(self, a, b, out, a_mn, b_mn, bias, accumulate, status, residual) -> None:
        unit = self.pending
        assert unit is not None
        self.pending = None
        j = self._job(unit)
        self.C.ag_gemm(a, b, out, a_mn, b_mn, bias, accumulate, status, residual, n_copy=self.n_copy, **j)
        self.gathers_fused += 1

    def view(self, name: str) -> torch.Tensor:
        seg = self.layout.segments[name]
        if not self.is_resident(seg.unit):
            raise RuntimeError(f"parameter {name} used before its unit {seg.unit} was gathered")
        off = seg.offset - self.unit_start[seg.unit]
        return self.staging[self.slot_of(seg.unit)][off: off + seg.numel].view(seg.shape)

    def gather_full(self, out: torch.Tensor) -> None:
        """Materialises the whole flat parameter vector (checkpointing, tests)."""
        for u in range(len(self.unit_n)):
            if not self.is_resident(u):
                self.enter(u, None)
            s = self.unit_start[u]
            out[s: s + self.unit_n[u]].copy_(self.staging[self.slot_of(u)][: self.unit_n[u]])


class ScatterSink:
    """Gradient sink whose large weight gradients never exist locally (see module docstring). Implements the interface
    of ``models.decoder.GradSink``."""

    scatter = True

    def __init__(self, layout: Any, C: Any, device: torch.device, my_rank: int, grad_shard_ptrs: Sequence[int]):
        self.layout, self.C, self.device = layout, C, torch.device(device)
        self.rank, self.world = int(my_rank), len(grad_shard_ptrs)
        assert self.world == layout.shard_world
        self.ptrs = [int(p) for p in grad_shard_ptrs]
        self.unit_start = [s for s, _ in layout.unit_ranges]
        self.unit_n = [e - s for s, e in layout.unit_ranges]
        self.local_off = [lo for lo, _, _ in layout.local_to_global_ranges(self.rank)]
        self.unit0 = torch.zeros(self.unit_n[0], dtype=torch.float32, device=self.device)
        # the small per-layer vectors share one scratch area that every layer reuses
        self.small_off: Dict[str, int] = {}
        off = 0
        for short in SMALL_LAYER_PARAMS:
            seg = layout.segments.get(f"layers.0.{short}")
            if seg is not None:
                self.small_off[short] = off
                off += (seg.numel + 127) // 128 * 128
        self.small = torch.zeros(max(off, 128), dtype=torch.float32, device=self.device)
        self.launches = 0

    @property
    def flat(self) -> torch.Tensor:
        raise RuntimeError("a scatter sink has no flat local gradient buffer")

    def _dst(self, unit: int) -> List[int]:
        return [p + 4 * self.local_off[unit] for p in self.ptrs]

    def view(self, name: str) -> torch.Tensor:
        seg = self.layout.segments[name]
        if seg.unit == 0:
            off = seg.offset - self.unit_start[0]
            return self.unit0[off: off + seg.numel].view(seg.shape)
        short = name.rsplit(".", 1)[-1]
        if short in self.small_off:
            o = self.small_off[short]
            return self.small[o: o + seg.numel].view(seg.shape)
        raise RuntimeError(f"gradient of {name} is produced by gemm_rs, it has no local buffer")

    def wgrad(self, dy: torch.Tensor, x: torch.Tensor, name: str, status: Optional[torch.Tensor]) -> None:
        seg = self.layout.segments[name]
        u = seg.unit
        if u == 0:  # embedding group accumulates locally (it also receives sparse row updates)
            self.C.gemm_bf16(dy, x, self.view(name), True, True, None, 1.0, True, status, None)
            return
        self.C.gemm_rs(dy, x, True, True, 1.0, self._dst(u), self.unit_n[u] // self.world,
                       seg.offset - self.unit_start[u], seg.shape[1], status)

    def unit_done(self, unit: int) -> None:
        """Backward of ``unit`` has finished on this rank for this microbatch: send what was accumulated locally."""
        if unit == 0:
            self.C.scatter_add_f32(self.unit0, 0, self._dst(0), self.unit_n[0] // self.world, True)
            self.launches += 1
            return
        i = unit - 1
        for short, o in self.small_off.items():
            seg = self.layout.segments[f"layers.{i}.{short}"]
            self.C.scatter_add_f32(self.small[o: o + seg.numel], seg.offset - self.unit_start[unit], self._dst(unit),
                                   self.unit_n[unit] // self.world, True)
            self.launches += 1

    def zero_(self) -> None:
        self.unit0.zero_()
        self.small.zero_()


class Zero3Comm:
    """What the trainer needs in fully sharded mode: the weight provider, the gradient sink and the optimizer-step
    collectives (barrier, global norm, AdamW on the shard). Built from the job's symmetric plane."""

    zero3 = True

    def __init__(self, plane: Any):
        from .symm import PeerGroup

        self.plane = plane
        self.layout, self.C, self.device = plane.layout, plane.C, plane.device
        tr = plane.trainer_ranks
        self.pg = PeerGroup(plane.flags, tr, plane.my_rank, plane.device, plane.C, slot_base=0)
        self.rank, self.world = self.pg.rank, self.pg.world
        self.shard16 = plane.shard16.local
        self.grad_shard = plane.grad_shard.local
        self.norm_ptrs = [plane.norm_tab.peer_ptrs[r] for r in tr]
        self.norm_local = torch.zeros(1, dtype=torch.float32, device=plane.device)
        self.weights = ShardedWeights(self.layout, self.C, self.device, self.rank, [plane.shard16.peer_ptrs[r] for r in tr])
        self.sink = ScatterSink(self.layout, self.C, self.device, self.rank, [plane.grad_shard.peer_ptrs[r] for r in tr])

    @property
    def norm_partials(self) -> torch.Tensor:
        return self.plane.norm_tab.local[: self.world]

    def publish_initial(self) -> None:
        """Call after every rank has written its initial slices: nobody gathers before all slices exist."""
        self.pg.barrier()
        self.weights.invalidate()

    def step(self, master, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, wd, step, max_norm) -> torch.Tensor:
        """Optimizer step on this rank's shard; returns the device tensor of per-rank squared-norm partials."""
        C = self.C
        C.set_comm_guard(self.pg.status)  # a timed-out barrier turns the update below into a no-op (the host then raises)
        self.pg.barrier()  # every rank's backward has finished: all reductions into my gradient shard have landed
        self.norm_local.zero_()
        C.sumsq(self.grad_shard, 1.0, self.norm_local)
        C.publish_norm(self.norm_local, self.norm_ptrs, self.rank)
        self.pg.barrier()  # all norm partials are in my table
        partials = self.norm_partials
        n = master.numel()
        # the kernel clips by the global norm, updates master and moments, stores the bf16 slice and zeroes the gradients
        C.adamw_push(master, exp_avg, exp_avg_sq, self.grad_shard, 0, 0, n, lr, beta1, beta2, eps, wd, step, 1.0, partials,
                     max_norm, [self.shard16.data_ptr()])
        self.pg.barrier()  # every slice is updated and every gradient shard is zero before the next forward
        self.weights.invalidate()
        return partials
