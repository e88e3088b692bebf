"""Old-policy logprob role with dynamic token-budget batching.

Behaviour of the reference's ``LogProbFSDPWorker`` + ``LogProbGPUWorker`` (logprob_worker.py:136-216,
gpu_process_worker.py:1663-1709): requests queue up; a centralizer takes one request and keeps adding
while the packed token count stays below ``max_tokens_per_gpu``, waiting up to 10 ms for each further
request and carrying over the one that did not fit; the batch is packed 1 x T, the eval-mode forward
returns per-token logprob and entropy on the logit-position grid, which are attached to each sample as
``sample_logprobs`` / ``sample_entropies``. Results are matched to requests by position, not by the
token tuple (the reference's keying collapses identical samples, logprob_worker.py:127-131).
"""
from __future__ import annotations

import asyncio
import concurrent.futures
import time
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..packing import pack_for_logprob


class LogProbWorker:
    def __init__(self, config: Any, model_cfg: Any, decoder: Any, device: torch.device, temperature: Optional[float] = None,
                 fill_window_s: float = 0.010, stream: Optional[torch.cuda.Stream] = None, sm_limit: int = 0):
        self.config, self.mcfg, self.decoder, self.device = config, model_cfg, decoder, torch.device(device)
        self.temperature = float(config.temperature if temperature is None else temperature) or 1.0
        self.max_tokens = int(config.max_tokens_per_gpu)
        self.fill_window_s = fill_window_s
        self.stream = stream
        self.sm_limit = int(sm_limit)
        self._queue: Optional[asyncio.Queue] = None
        self._task: Optional[asyncio.Task] = None
        self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="logprob")
        self._carry: Optional[Tuple[asyncio.Future, Dict[str, Any]]] = None
        self.tokens_processed = 0
        self.batches = 0
        self.busy_seconds = 0.0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _ensure_started(self) -> None:
        if self._queue is None:
            self._queue = asyncio.Queue()
            self._task = asyncio.ensure_future(self._centralize())

    async def inference(self, sample: Dict[str, Any]) -> Dict[str, Any]:
        self._ensure_started()
        fut: asyncio.Future = asyncio.get_running_loop().create_future()
        await self._queue.put((fut, sample))
        return await fut

    # ---- batching loop ----
    async def _centralize(self) -> None:
        loop = asyncio.get_running_loop()
        while True:
            first = self._carry or await self._queue.get()
            self._carry = None
            batch = [first]
            tokens = len(first[1]["sample_ids"])
            while tokens < self.max_tokens:
                try:
                    nxt = await asyncio.wait_for(self._queue.get(), self.fill_window_s)
                except asyncio.TimeoutError:
                    break
                n = len(nxt[1]["sample_ids"])
                if tokens + n > self.max_tokens:
                    self._carry = nxt  # goes first in the next batch
                    break
                batch.append(nxt)
                tokens += n
            samples = [s for _, s in batch]
            try:
                results = await self._run_batch(samples)
                for (fut, s), (lp, ent) in zip(batch, results):
                    if not fut.done():
                        out = dict(s)
                        out["sample_logprobs"] = lp
                        out["sample_entropies"] = ent
                        fut.set_result(out)
            except Exception as e:
                for fut, _ in batch:
                    if not fut.done():
                        fut.set_exception(e)
                await asyncio.sleep(1.0)

    async def _run_batch(self, samples: List[Dict[str, Any]]) -> List[Tuple[np.ndarray, np.ndarray]]:
        return await asyncio.get_running_loop().run_in_executor(self._pool, self._compute, samples)

    async def compute_batch(self, samples: List[Dict[str, Any]]) -> List[Tuple[np.ndarray, np.ndarray]]:
        """One already formed batch (a group controller's share for this rank), ordered with this rank's other work."""
        return await self._run_batch(samples)

    # ---- compute (worker thread) ----
    def _compute(self, samples: List[Dict[str, Any]]) -> List[Tuple[np.ndarray, np.ndarray]]:
        t0 = time.time()
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else _null()
        if self.sm_limit > 0 and self.device.type == "cuda":
            self.decoder.C.set_sm_limit(self.sm_limit)  # thread-local: this worker thread only
        with ctx, torch.no_grad():
            host = pack_for_logprob(samples, pin=self.device.type == "cuda")
            self.h2d_bytes += host.h2d_bytes()
            batch = host.to_device(self.device)
            logp, ent = self.decoder.logprobs(batch, self.temperature)
            both = torch.stack([logp.float(), ent.float()]).cpu().numpy()  # one device-to-host copy per batch
            self.d2h_bytes += both.nbytes
        out = []
        off = 0
        for s in samples:
            L = len(s["sample_ids"])
            out.append((both[0, off:off + L].copy(), both[1, off:off + L].copy()))
            off += L
        self.tokens_processed += off
        self.batches += 1
        self.busy_seconds += time.time() - t0
        return out

    async def is_ready(self) -> bool:
        return True

    def stats(self) -> Dict[str, float]:
        return {"tokens": float(self.tokens_processed), "batches": float(self.batches), "busy_seconds": self.busy_seconds,
                "launches": float(getattr(self.decoder, "launches", 0))}

    def pause(self) -> None:
        """Blocks until the batch in flight (if any) has finished and keeps the compute thread from starting another
        one until :meth:`resume`. The weight sync brackets its device half with the pair, so that no forward pass runs on
        parameters that are being overwritten. Call it from a thread that may block."""
        import threading

        self._hold = threading.Event()
        started = threading.Event()

        def holder() -> None:
            started.set()
            self._hold.wait(timeout=600.0)

        self._pool.submit(holder)
        started.wait()

    def resume(self) -> None:
        hold = getattr(self, "_hold", None)
        if hold is not None:
            hold.set()

    def run_blocking(self, fn, *args):
        """Runs ``fn`` on the compute thread: it starts after the batch that is being computed and before the next one
        (the pool has one thread). The weight sync runs its device half through here, so that no forward pass reads
        parameters that are half written."""
        return self._pool.submit(fn, *args).result()


class LogProbGroup(LogProbWorker):
    """Controller of ``logprob_fsdp_size`` logprob ranks that act as one logprob service (the reference's
    ``LogProbFSDPWorker`` over its FSDP ranks, logprob_worker.py:57-134): requests are batched by the same token budget
    and every batch is scattered round-robin over the member ranks, which compute their shares concurrently; results go
    back to the requests by position. Every member holds the whole model here (a B200 has room for every preset), so an
    empty share needs no dummy sample: there is no collective that all members would have to enter together."""

    def __init__(self, config: Any, members: List[Any], fill_window_s: float = 0.010):
        # members: objects with ``async compute_batch(samples)`` - the local LogProbWorker and / or RPC proxies of others
        self.config = config
        self.members = list(members)
        self.temperature = float(config.temperature) or 1.0
        self.max_tokens = int(config.max_tokens_per_gpu)
        self.fill_window_s = fill_window_s
        self._queue = None
        self._task = None
        self._carry = None
        self.tokens_processed = 0
        self.batches = 0
        self.busy_seconds = 0.0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.shares: List[int] = [0] * len(self.members)  # samples sent to each member so far

    async def _run_batch(self, samples: List[Dict[str, Any]]) -> List[Tuple[np.ndarray, np.ndarray]]:
        k = len(self.members)
        chunks: List[List[int]] = [[] for _ in range(k)]
        for i in range(len(samples)):
            chunks[i % k].append(i)
        live = [(m, idx) for m, idx in enumerate(chunks) if idx]
        parts = await asyncio.gather(*[self.members[m].compute_batch([samples[i] for i in idx]) for m, idx in live])
        out: List[Any] = [None] * len(samples)
        for (m, idx), res in zip(live, parts):
            self.shares[m] += len(idx)
            for i, r in zip(idx, res):
                out[i] = (np.asarray(r[0], dtype=np.float32), np.asarray(r[1], dtype=np.float32))
        self.batches += 1
        self.tokens_processed += sum(len(s["sample_ids"]) for s in samples)
        return out

    def pause(self) -> None:  # members are paused by their own ranks' weight sync
        return

    def resume(self) -> None:
        return


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
