"""Host side of a tensor-parallel rollout replica: the leader's engine commands, mirrored to the other members.

The reference leaves tensor parallelism to vLLM (``tensor_parallel_size``, vllm_worker.py:219-232), whose executor
broadcasts the scheduler's output to the workers of a replica every step. Here every member of a replica runs a complete
engine (scheduler, sampler, KV block tables) on its share of the heads and MLP columns. The engines are deterministic
state machines: given the same sequence of ``add_request`` / ``step`` calls they take the same scheduling decisions and,
because the all-reduce sums in rank order on every member, sample the same tokens. So the only thing that has to cross
between the processes on the host is that call sequence. The leader (first rank of the replica) owns the request queue
and the results; before each engine call it writes one small message to a TCP connection per follower. The followers
replay the calls on their own engine thread and drop the results. On the device the members meet in the all-reduce
barrier of every layer, so a follower that runs late only delays the step; one that never arrives lets the barrier's
budget run out, which the leader reports as an engine failure.

Weight synchronisation: the leader sends ``pause`` once its engine is idle. A follower that reads ``pause`` has replayed
everything before it, reports idle to its own rank's weight-sync code and stops reading until that code resumes it (its
folded weights are recomputed by then). Commands that the leader sends in the meantime wait in the socket.
"""
from __future__ import annotations

import logging
import pickle
import socket
import struct
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

logger = logging.getLogger(__name__)

_HDR = struct.Struct("<I")


def _send_msg(sock: socket.socket, obj: Any) -> None:
    data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    sock.sendall(_HDR.pack(len(data)) + data)


def _recv_exact(sock: socket.socket, n: int) -> Optional[bytes]:
    chunks, got = [], 0
    while got < n:
        b = sock.recv(n - got)
        if not b:
            return None
        chunks.append(b)
        got += len(b)
    return b"".join(chunks)


def _recv_msg(sock: socket.socket) -> Any:
    hdr = _recv_exact(sock, _HDR.size)
    if hdr is None:
        return None
    body = _recv_exact(sock, _HDR.unpack(hdr)[0])
    return None if body is None else pickle.loads(body)


class LeaderChannel:
    """Leader side: one connection per follower; ``send`` writes the same message to all of them, in order."""

    def __init__(self, store: Any, follower_ranks: Sequence[int], host: str = "127.0.0.1", key: str = "agrpo_tp_port"):
        self.socks: List[socket.socket] = []
        self._lock = threading.Lock()
        for r in follower_ranks:
            port = int(store.get(f"{key}_{r}").decode())  # blocks until the follower has published it
            s = socket.create_connection((host, port), timeout=120.0)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(None)
            self.socks.append(s)

    def send(self, *cmd: Any) -> None:
        with self._lock:
            for s in self.socks:
                _send_msg(s, cmd)

    def close(self) -> None:
        with self._lock:
            for s in self.socks:
                try:
                    _send_msg(s, ("stop",))
                except OSError:
                    pass
                try:
                    s.close()
                except OSError:
                    pass
            self.socks = []


class FollowerListener:
    """Follower side: listens on an ephemeral port, publishes it in the job's store, accepts the leader once."""

    def __init__(self, store: Any, rank: int, host: str = "127.0.0.1", key: str = "agrpo_tp_port"):
        self.srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.srv.bind((host, 0))
        self.srv.listen(1)
        store.set(f"{key}_{rank}", str(self.srv.getsockname()[1]))
        self.conn: Optional[socket.socket] = None

    def accept(self, timeout_s: float = 600.0) -> socket.socket:
        self.srv.settimeout(timeout_s)
        conn, _ = self.srv.accept()
        conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        conn.settimeout(None)
        self.conn = conn
        self.srv.close()
        return conn


class TpFollower:
    """Stands where a GenerationWorker stands on the non-leader ranks of a replica: same pause / resume / shutdown
    surface towards the runtime, but its engine is driven by the leader's command stream."""

    def __init__(self, engine: Any, listener: FollowerListener, stream: Any = None, kernel_checks: bool = False):
        self.engine, self.listener, self.stream = engine, listener, stream
        self.kernel_checks = kernel_checks
        self.busy_seconds = 0.0
        self.steps = 0
        self._idle = threading.Event()      # set while the thread sits on a ``pause`` command
        self._resume = threading.Event()
        self._stop = False
        self._dead: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._run, name="tp-follower", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        try:
            self._loop()
        except BaseException as e:
            logger.exception("tensor-parallel follower stopped: %r", e)
            self._dead = e
            # the leader must learn of it: with the connection closed its next command raises instead of piling up
            try:
                if self.listener.conn is not None:
                    self.listener.conn.close()
            except OSError:
                pass

    def _loop(self) -> None:
        import torch

        conn = self.listener.accept()
        ctx = torch.cuda.stream(self.stream) if (self.stream is not None and torch.cuda.is_available()) else _null()
        with ctx:
            while not self._stop:
                cmd = _recv_msg(conn)
                if cmd is None or cmd[0] == "stop":
                    break
                op = cmd[0]
                if op == "add":
                    args, kw = cmd[1]
                    self.engine.add_request(*args, **kw)
                elif op == "step":
                    t0 = time.time()
                    finished = self.engine.step()
                    if finished or self.kernel_checks:
                        self.engine.check_status()
                    self.busy_seconds += time.time() - t0
                    self.steps += 1
                elif op == "logprobs":
                    if hasattr(self.engine, "enable_logprobs"):
                        self.engine.enable_logprobs()
                elif op == "pause":
                    self._resume.clear()
                    self._idle.set()
                    while not self._stop and not self._resume.wait(timeout=0.1):
                        pass
                else:
                    raise RuntimeError(f"unknown replica command {op!r}")
        self._dead = self._dead or RuntimeError("the leader closed the command stream")

    # ---- the runtime's view (same names as GenerationWorker) ----
    async def pause_for_sync(self) -> bool:
        import asyncio

        while not self._idle.is_set():
            if self._dead is not None:
                raise RuntimeError(f"tensor-parallel follower has stopped: {self._dead!r}")
            await asyncio.sleep(0.001)
        if self._dead is not None:
            raise RuntimeError(f"tensor-parallel follower has stopped: {self._dead!r}")
        return True

    async def resume_after_sync(self) -> bool:
        if hasattr(self.engine, "update_weights_done"):
            self.engine.update_weights_done()
        self._idle.clear()   # before the thread can run on: a later pause must wait for the leader's next ``pause``
        self._resume.set()
        return True

    async def is_ready(self) -> bool:
        return self._dead is None

    def stats(self) -> Dict[str, float]:
        return {"busy_seconds": self.busy_seconds, "steps": float(self.steps)}

    def shutdown(self) -> None:
        self._stop = True
        self._resume.set()
        try:
            if self.listener.conn is not None:
                self.listener.conn.shutdown(socket.SHUT_RDWR)
        except OSError:
            pass
        self._thread.join(timeout=5.0)


class _null:
    def __enter__(self) -> None:
        return None

    def __exit__(self, *a: Any) -> None:
        return None


def replica_groups(rollout_ranks: Sequence[int], tp: int) -> List[List[int]]:
    """Consecutive runs of ``tp`` rollout ranks form one replica; the first of each run leads it."""
    ranks = list(rollout_ranks)
    if tp <= 1:
        return [[r] for r in ranks]
    if len(ranks) % tp:
        raise ValueError(f"{len(ranks)} rollout ranks cannot form replicas of {tp}")
    return [ranks[i:i + tp] for i in range(0, len(ranks), tp)]
