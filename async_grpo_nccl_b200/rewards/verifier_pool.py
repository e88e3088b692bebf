"""Built-in verifier pool.

A pool of N CPU worker processes. ``verify(sample)`` runs one task per configured reward function in
parallel, each with a timeout; a worker that times out or dies is killed and replaced and that task
yields reward 0 with ``reward_success=False``; the best result by ``(reward, reward_success)`` is
returned; samples for which no reward function succeeded can be appended to a JSONL file under a file
lock. This is the behaviour of the reference's Ray-actor pool (verifier_pool.py:57-171) on plain
processes and pipes. ``num_workers=0`` evaluates inline in the caller (no isolation, no timeout).
"""
from __future__ import annotations

import asyncio
import copy
import json
import math
import multiprocessing as mp
import os
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

from .registry import resolve_adapter


def compute_cosine_reward(gen_length: int, max_length: int, format_quality: float, is_correct: float,
                          r_c_0: float = 6, r_c_L: float = 5, r_w_0: float = -10, r_w_L: float = 0,
                          r_f_0: float = 1.0, r_f_L: float = 0.5, exceed_penalty: float = -10) -> float:
    """Length-aware reward: cosine interpolation between a value at length 0 and a value at the maximum length,
    chosen by correctness, plus a format term; a response that hits the length cap gets ``exceed_penalty``
    (verifier_pool.py:21-55; unused by the reference's own pipeline)."""
    if gen_length >= max_length:
        return float(exceed_penalty)
    if is_correct >= 1.0:
        lo, hi = r_c_0, r_c_L
    else:
        lo, hi = r_w_0, r_w_L
    t = 0.5 * (1.0 + math.cos(math.pi * gen_length / max_length))
    base = hi + (lo - hi) * t
    fmt = r_f_L + (r_f_0 - r_f_L) * t
    return float(base + format_quality * fmt)


def _apply(sample: Dict[str, Any], fn_name: str, kwargs: Dict[str, Any]) -> Dict[str, Any]:
    out = resolve_adapter(fn_name)(sample, **kwargs)
    if "debug_logs" in out:
        sample["debug_logs"] = out.pop("debug_logs")
    sample.update(out)
    sample["reward_success"] = True
    return sample


def _worker_main(conn) -> None:
    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            return
        if msg is None:
            return
        sample, fn_name, kwargs = msg
        try:
            conn.send(("ok", _apply(sample, fn_name, kwargs)))
        except Exception as e:  # adapter failure is reported, the worker stays alive
            try:
                conn.send(("err", repr(e)))
            except Exception:
                return


class _Worker:
    def __init__(self, ctx) -> None:
        self.parent, child = ctx.Pipe()
        self.proc = ctx.Process(target=_worker_main, args=(child,), daemon=True)
        self.proc.start()
        child.close()

    def kill(self) -> None:
        try:
            self.proc.kill()
            self.proc.join(timeout=2)
        except Exception:
            pass
        try:
            self.parent.close()
        except Exception:
            pass


class VerifierPool:
    def __init__(self, global_num_verifiers: int = 4, write_failed: bool = False, reward_fns: Optional[Sequence[str]] = None,
                 output_dir: Optional[str] = None, timeout_s: float = 30.0, start_method: str = "spawn"):
        self.num_workers = int(global_num_verifiers)
        self.write_failed = bool(write_failed)
        self.reward_fns: List[str] = [str(getattr(f, "value", f)) for f in (reward_fns or ["mathd", "sympy"])]
        self.timeout_s = float(timeout_s)
        self.outfile = Path(output_dir or ".") / "failed_samples_verify.jsonl"
        if self.write_failed:
            self.outfile.parent.mkdir(parents=True, exist_ok=True)
            self.outfile.unlink(missing_ok=True)
        self._ctx = mp.get_context(start_method) if self.num_workers > 0 else None
        self._idle: Optional[asyncio.Queue] = None
        self._workers: List[_Worker] = []
        self.replaced_workers = 0
        self.verified = 0

    # -- lifecycle
    def _ensure_started(self) -> None:
        if self._idle is not None or self.num_workers == 0:
            return
        self._idle = asyncio.Queue()
        for _ in range(self.num_workers):
            w = _Worker(self._ctx)
            self._workers.append(w)
            self._idle.put_nowait(w)

    def close(self) -> None:
        for w in self._workers:
            try:
                w.parent.send(None)
            except Exception:
                pass
            w.kill()
        self._workers = []
        self._idle = None

    # -- one task on one worker
    async def _verify_single(self, sample: Dict[str, Any], fn_name: str, kwargs: Dict[str, Any]) -> Dict[str, Any]:
        if self.num_workers == 0:
            try:
                return _apply(sample, fn_name, kwargs)
            except Exception:
                sample["reward"] = 0.0
                sample["reward_success"] = False
                return sample
        self._ensure_started()
        worker: _Worker = await self._idle.get()
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        fd = worker.parent.fileno()

        def _ready() -> None:
            if not fut.done():
                fut.set_result(True)

        try:
            worker.parent.send((sample, fn_name, kwargs))
            loop.add_reader(fd, _ready)
            try:
                await asyncio.wait_for(fut, self.timeout_s)
            finally:
                loop.remove_reader(fd)
            status, payload = worker.parent.recv()
            self._idle.put_nowait(worker)
            if status == "ok":
                return payload
            raise RuntimeError(payload)
        except (asyncio.TimeoutError, EOFError, OSError, BrokenPipeError):
            # hung or dead worker: kill, replace, reward 0
            worker.kill()
            if worker in self._workers:
                self._workers.remove(worker)
            nw = _Worker(self._ctx)
            self._workers.append(nw)
            self._idle.put_nowait(nw)
            self.replaced_workers += 1
        except RuntimeError:
            pass
        sample["reward"] = 0.0
        sample["reward_success"] = False
        return sample

    @staticmethod
    def pick_verified_sample(results: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
        return max(results, key=lambda r: (r.get("reward", 0) or 0, bool(r.get("reward_success", False))))

    def _write_failed_sample(self, sample: Dict[str, Any]) -> None:
        if not self.write_failed:
            return
        lock = str(self.outfile) + ".lock"
        deadline = time.time() + 20.0
        while True:
            try:
                fd = os.open(lock, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
                break
            except FileExistsError:
                if time.time() > deadline:
                    return
                time.sleep(0.01)
        try:
            with open(self.outfile, "a", encoding="utf-8") as f:
                f.write(json.dumps(_jsonable(sample)) + "\n")
        finally:
            os.close(fd)
            try:
                os.unlink(lock)
            except OSError:
                pass

    async def verify(self, sample: Dict[str, Any], **kwargs: Any) -> Dict[str, Any]:
        fns = [str(getattr(f, "value", f)) for f in kwargs.pop("reward_fns", self.reward_fns)]
        results = await asyncio.gather(*[self._verify_single(copy.deepcopy(sample), fn, kwargs) for fn in fns])
        self.verified += 1
        if not any(r.get("reward_success", False) for r in results):
            self._write_failed_sample(sample)
        return self.pick_verified_sample(results)


def _jsonable(obj: Any) -> Any:
    import numpy as np

    if isinstance(obj, dict):
        return {str(k): _jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_jsonable(v) for v in obj]
    if isinstance(obj, np.ndarray):
        return obj.tolist()
    if isinstance(obj, (np.integer,)):
        return int(obj)
    if isinstance(obj, (np.floating,)):
        return float(obj)
    return obj


_POOLS: Dict[str, VerifierPool] = {}


def get_or_create_verifier_pool(global_num_verifiers: int, write_failed: bool = False,
                                reward_fns: Optional[Sequence[str]] = None, output_dir: Optional[str] = None,
                                name: str = "verifier_pool", timeout_s: float = 30.0) -> VerifierPool:
    """One pool per name per process; a second caller gets the existing pool (the reference relies on a failing
    named-actor creation for this, verifier_pool.py:164-169)."""
    pool = _POOLS.get(name)
    if pool is None:
        pool = VerifierPool(global_num_verifiers, write_failed, reward_fns, output_dir, timeout_s)
        _POOLS[name] = pool
    return pool
