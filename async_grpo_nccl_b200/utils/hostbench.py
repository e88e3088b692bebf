"""Host-side component benchmarks (no GPU needed): the C++ packer against its NumPy restatement, the microbatch planner,
the verifier pool, checkpoint save / load.

    python -m async_grpo_nccl_b200.utils.hostbench [packer] [planner] [verifier] [checkpoint] [rpc]

Each line of output is a JSON record. Wall-clock timings on the host (median of repeats after a warm-up call).
"""
from __future__ import annotations

import asyncio
import json
import os
import sys
import tempfile
import time
from typing import Any, Callable, Dict, List

import numpy as np


def _median_time(fn: Callable[[], Any], repeats: int = 7) -> float:
    fn()
    ts = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[len(ts) // 2]


def _out(rec: Dict[str, Any]) -> None:
    print(json.dumps(rec), flush=True)


def _samples(n_tokens: int, rng: np.random.Generator, vocab: int = 151936) -> List[Dict[str, Any]]:
    out, tot = [], 0
    while tot < n_tokens:
        li, lo = int(rng.integers(64, 512)), int(rng.integers(256, 4096))
        L = li + lo
        if tot + L > n_tokens and out:
            break
        out.append(dict(sample_ids=rng.integers(0, vocab, L).astype(np.int32), input_len=li, output_len=lo,
                        advantage=float(rng.normal()), sample_logprobs=rng.random(L).astype(np.float32),
                        sample_entropies=rng.random(L).astype(np.float32), reward=1.0))
        tot += L
    return out


def bench_packer() -> None:
    """One 32k-token microbatch: C++ packer (one pass into one buffer) against the NumPy restatement of the same layout
    (which itself replaces the reference's numba helpers + per-field torch tensors, sample_processing_utils.py:29-223)."""
    from ..ops import have_native
    from ..packing import pack_samples

    rng = np.random.default_rng(0)
    samples = _samples(32768, rng)
    tokens = sum(len(s["sample_ids"]) for s in samples)
    t_np = _median_time(lambda: pack_samples(samples, pin=False, use_native=False))
    rec = {"bench": "packer", "samples": len(samples), "tokens": tokens, "numpy_us": t_np * 1e6}
    if have_native():
        t_cc = _median_time(lambda: pack_samples(samples, pin=False, use_native=True))
        rec.update(cpp_us=t_cc * 1e6, speedup=t_np / t_cc, cpp_ns_per_token=t_cc * 1e9 / tokens)
    _out(rec)


def bench_planner() -> None:
    """Token-budget planning of one 1024-sample macro-batch over 4 trainer ranks: host microseconds per sample."""
    from ..experience import MicrobatchPlanner

    rng = np.random.default_rng(1)
    lens = [(int(rng.integers(64, 512)), int(np.exp(rng.uniform(np.log(256), np.log(8192))))) for _ in range(1024)]
    samples = [dict(sample_ids=np.zeros(a + b, np.int32), input_len=a, output_len=b, advantage=0.0) for a, b in lens]

    def run() -> int:
        p = MicrobatchPlanner([0, 1, 2, 3], 32768, 1024)
        n = 0
        for s in samples:
            n += len(p.add(s))
        n += len(p.finish())
        return n

    t = _median_time(run, repeats=5)
    _out({"bench": "planner", "samples": len(samples), "ranks": 4, "events": run(), "total_ms": t * 1e3,
          "us_per_sample": t * 1e6 / len(samples)})


def bench_verifier() -> None:
    """Verifications per second through the process pool (countdown and boxed-math adapters)."""
    from ..rewards.verifier_pool import VerifierPool

    async def run(fns: List[str], samples: List[Dict[str, Any]], workers: int) -> float:
        pool = VerifierPool(workers, False, fns, None, timeout_s=30.0)
        try:
            await asyncio.gather(*[pool.verify(dict(s)) for s in samples[:8]])  # start the workers
            t0 = time.perf_counter()
            await asyncio.gather(*[pool.verify(dict(s)) for s in samples])
            return time.perf_counter() - t0
        finally:
            pool.close()

    cd = [{"sample_text": f"<think>t</think>\n<answer>({i % 7 + 1} + 3) * 2</answer>", "nums": [i % 7 + 1, 3, 2],
           "target": (i % 7 + 4) * 2, "answer": str((i % 7 + 4) * 2), "input": "q", "end_token": ""} for i in range(512)]
    mt = [{"sample_text": "so the result is \\boxed{\\frac{%d}{2}}" % (2 * i), "answer": str(i), "input": "q"} for i in range(256)]
    for name, fns, data in (("countdown", ["countdown"], cd), ("mathd+sympy", ["mathd", "sympy"], mt)):
        for workers in (0, 4):
            t = asyncio.run(run(fns, data, workers))
            _out({"bench": "verifier", "adapters": name, "workers": workers, "samples": len(data),
                  "verifications_per_s": len(data) / t})


def bench_checkpoint(model: str = "qwen2.5-1.5b") -> None:
    """HF-format save and load of the model plus one optimizer shard, to local disk."""
    import torch

    from .. import checkpoint as ckpt
    from ..models.config import PRESETS
    from ..models.layout import ParamLayout

    cfg = PRESETS[model]
    layout = ParamLayout(cfg)
    flat = torch.empty(layout.total, dtype=torch.float32).normal_(0, 0.02)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ckpt")
        t0 = time.perf_counter()
        ckpt.save_hf_model(path, cfg, layout, flat)
        t_save = time.perf_counter() - t0
        size = sum(os.path.getsize(os.path.join(path, f)) for f in os.listdir(path))
        t0 = time.perf_counter()
        back = ckpt.load_hf_model(path, layout)
        t_load = time.perf_counter() - t0
        same = bool(torch.equal(back.to(torch.bfloat16), flat.to(torch.bfloat16)))
        state = {"master": flat, "exp_avg": torch.zeros_like(flat), "exp_avg_sq": torch.zeros_like(flat)}
        t0 = time.perf_counter()
        ckpt.save_optimizer_shard(path, 0, 1, layout, state, {"opt_step": 1})
        t_opt = time.perf_counter() - t0
    _out({"bench": "checkpoint", "model": model, "params_b": layout.total / 1e9, "model_files_gb": size / 1e9,
          "save_model_s": t_save, "load_model_s": t_load, "round_trip_exact_in_bf16": same, "save_optimizer_shard_s": t_opt})


def bench_rpc() -> None:
    """Control-plane round trips: a 2048-token sample (ids + logprobs as numpy) through the msgpack RPC on loopback."""
    from ..rpc import RpcClient, RpcServer

    class Echo:
        async def echo(self, x: Any) -> Any:
            return x

    async def run() -> Dict[str, float]:
        srv = RpcServer(Echo(), "127.0.0.1", 0)
        port = await srv.start()
        cli = await RpcClient("127.0.0.1", port, name="bench").connect()
        payload = {"sample_ids": np.arange(2048, dtype=np.int32), "sample_logprobs": np.zeros(2048, np.float32), "reward": 1.0}
        for _ in range(50):
            await cli.call("echo", payload)
        t0 = time.perf_counter()
        n = 500
        for _ in range(n):
            await cli.call("echo", payload)
        seq = (time.perf_counter() - t0) / n
        t0 = time.perf_counter()
        await asyncio.gather(*[cli.call("echo", payload) for _ in range(n)])
        par = (time.perf_counter() - t0) / n
        await cli.close()
        await srv.close()
        return {"round_trip_us": seq * 1e6, "pipelined_us_per_call": par * 1e6}

    _out({"bench": "rpc", "payload_bytes": 2048 * 8, **asyncio.run(run())})


class _FileStore:
    """The two calls of the job's key-value store that the replica channel uses, on files (for two local processes)."""

    def __init__(self, root: str):
        self.root = root

    def set(self, k: str, v: str) -> None:
        tmp = os.path.join(self.root, k + ".tmp")
        with open(tmp, "w") as f:
            f.write(v)
        os.replace(tmp, os.path.join(self.root, k))

    def get(self, k: str) -> bytes:
        path = os.path.join(self.root, k)
        for _ in range(2000):
            if os.path.exists(path):
                with open(path, "rb") as f:
                    return f.read()
            time.sleep(0.005)
        raise TimeoutError(k)


class _CountingEngine:
    """Replays nothing; drops a file when it has seen ``warm`` steps and another at ``warm + want``."""

    def __init__(self, warm: int, want: int, root: str):
        self.n, self.marks, self.root = 0, {warm: "warm", warm + want: "done"}, root

    def step(self) -> list:
        self.n += 1
        name = self.marks.get(self.n)
        if name:
            with open(os.path.join(self.root, name), "w") as f:
                f.write(name)
        return []

    def add_request(self, *a: Any, **k: Any) -> None:
        pass

    def check_status(self) -> None:
        pass


def _replica_follower_process(root: str, warm: int, want: int) -> None:
    from ..roles.tp_mirror import FollowerListener, TpFollower

    fol = TpFollower(_CountingEngine(warm, want, root), FollowerListener(_FileStore(root), 1))
    fol._thread.join()


def bench_replica() -> None:
    """Host cost of a tensor-parallel replica per decode step: the leader's ``step`` commands reaching a follower in another
    process over the loopback connection (one-way stream: commands per second until the follower has replayed all of
    them), and the prefix-cache hashing of one 512-token prompt."""
    import hashlib
    import multiprocessing as mp
    import tempfile

    from ..roles.tp_mirror import LeaderChannel

    warm, n = 100, 20000
    with tempfile.TemporaryDirectory() as root:
        proc = mp.get_context("spawn").Process(target=_replica_follower_process, args=(root, warm, n), daemon=True)
        proc.start()
        lead = LeaderChannel(_FileStore(root), [1])

        def wait_for(name: str) -> None:
            t = time.perf_counter()
            while not os.path.exists(os.path.join(root, name)) and time.perf_counter() - t < 120:
                time.sleep(0.0002)

        for _ in range(warm):  # the follower imports its libraries while these wait in the socket
            lead.send("step")
        wait_for("warm")
        t0 = time.perf_counter()
        for _ in range(n):
            lead.send("step")
        wait_for("done")
        per = (time.perf_counter() - t0) / n
        lead.close()
        proc.join(timeout=10)
    prompt = np.arange(512, dtype=np.int32)

    def hashes() -> None:
        prev = b"agrpo-prefix"
        for b in range(512 // 16):
            prev = hashlib.blake2b(prev + prompt[b * 16:(b + 1) * 16].tobytes(), digest_size=8).digest()

    _out({"bench": "replica_host", "step_command_us": per * 1e6, "prefix_hash_512_tokens_us": _median_time(hashes) * 1e6})


def main() -> int:
    which = sys.argv[1:] or ["packer", "planner", "verifier", "checkpoint", "rpc", "replica"]
    table = {"packer": bench_packer, "planner": bench_planner, "verifier": bench_verifier, "checkpoint": bench_checkpoint,
             "rpc": bench_rpc, "replica": bench_replica}
    for w in which:
        if w not in table:
            raise SystemExit(f"unknown benchmark {w}; choose from {sorted(table)}")
        table[w]()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
