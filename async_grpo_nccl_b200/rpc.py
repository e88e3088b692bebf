"""Control plane: asyncio RPC over TCP (127.0.0.1 within a node) with msgpack framing.

It replaces the Ray actor calls and object store of the reference (orchestrator.py, ray_utils.py): every
role process hosts an ``RpcServer`` around its role object, the orchestrator and the trainer ranks hold
``RpcClient`` proxies. Token arrays travel as raw NumPy buffers (an msgpack extension type), not as
Python lists. ``ping`` doubles as the liveness probe (the reference's ``is_ready`` / ``ping_all``,
trainer_worker.py:191-206).
"""
from __future__ import annotations

import asyncio
import itertools
import struct
import traceback
from typing import Any, Awaitable, Callable, Dict, Optional

import msgpack
import numpy as np

_EXT_NDARRAY = 1
_EXT_TUPLE = 2
_MAX_FRAME = 1 << 31


def _default(obj: Any) -> Any:
    if isinstance(obj, np.ndarray):
        a = np.ascontiguousarray(obj)
        head = msgpack.packb((a.dtype.str, list(a.shape)), use_bin_type=True)
        return msgpack.ExtType(_EXT_NDARRAY, struct.pack("<I", len(head)) + head + a.tobytes())
    if isinstance(obj, (np.integer,)):
        return int(obj)
    if isinstance(obj, (np.floating,)):
        return float(obj)
    if isinstance(obj, (np.bool_,)):
        return bool(obj)
    if isinstance(obj, tuple):
        return msgpack.ExtType(_EXT_TUPLE, msgpack.packb(list(obj), default=_default, use_bin_type=True))
    if hasattr(obj, "to_wire"):
        return {"__wire__": type(obj).__name__, **obj.to_wire()}
    raise TypeError(f"cannot serialise {type(obj)!r}")


def _ext_hook(code: int, data: bytes) -> Any:
    if code == _EXT_NDARRAY:
        (n,) = struct.unpack("<I", data[:4])
        dtype, shape = msgpack.unpackb(data[4:4 + n], raw=False)
        return np.frombuffer(data[4 + n:], dtype=np.dtype(dtype)).reshape(shape).copy()
    if code == _EXT_TUPLE:
        return tuple(msgpack.unpackb(data, ext_hook=_ext_hook, raw=False, strict_map_key=False))
    return msgpack.ExtType(code, data)


def dumps(obj: Any) -> bytes:
    return msgpack.packb(obj, default=_default, use_bin_type=True, strict_types=True)


def loads(data: bytes) -> Any:
    out = msgpack.unpackb(data, ext_hook=_ext_hook, raw=False, strict_map_key=False)
    return _revive(out)


def _revive(obj: Any) -> Any:
    if isinstance(obj, dict):
        if obj.get("__wire__") == "Message":
            from .protocol import Message

            return Message.from_wire({"type": obj["type"], "data": _revive(obj.get("data"))})
        return {k: _revive(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_revive(v) for v in obj]
    return obj


async def _read_frame(reader: asyncio.StreamReader) -> bytes:
    head = await reader.readexactly(4)
    (n,) = struct.unpack("<I", head)
    if n >= _MAX_FRAME:
        raise ValueError("frame too large")
    return await reader.readexactly(n)


def _write_frame(writer: asyncio.StreamWriter, payload: bytes) -> None:
    writer.write(struct.pack("<I", len(payload)) + payload)


class RpcServer:
    """Serves the public (non-underscore) methods of ``target``; coroutine methods are awaited."""

    def __init__(self, target: Any, host: str = "127.0.0.1", port: int = 0):
        self.target, self.host, self.port = target, host, port
        self._server: Optional[asyncio.AbstractServer] = None
        self.drop_filter: Optional[Callable[[str], bool]] = None  # test hook: return True to drop a request

    async def start(self) -> int:
        self._server = await asyncio.start_server(self._handle, self.host, self.port, limit=1 << 26)
        self.port = self._server.sockets[0].getsockname()[1]
        return self.port

    async def close(self) -> None:
        if self._server is not None:
            self._server.close()
            await self._server.wait_closed()
            self._server = None

    async def _handle(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
        lock = asyncio.Lock()

        async def serve_one(req: Dict[str, Any]) -> None:
            rid, method = req.get("id"), req.get("method", "")
            try:
                if method == "ping":
                    result: Any = True
                else:
                    if method.startswith("_") or not hasattr(self.target, method):
                        raise AttributeError(f"no such method: {method}")
                    out = getattr(self.target, method)(*req.get("args", []), **req.get("kwargs", {}))
                    result = await out if asyncio.iscoroutine(out) or isinstance(out, Awaitable) else out
                resp = {"id": rid, "ok": True, "result": result}
            except Exception as e:
                resp = {"id": rid, "ok": False, "error": f"{type(e).__name__}: {e}", "trace": traceback.format_exc()}
            try:
                data = dumps(resp)
            except Exception as e:
                data = dumps({"id": rid, "ok": False, "error": f"serialisation failed: {e}", "trace": ""})
            async with lock:
                _write_frame(writer, data)
                await writer.drain()

        try:
            while True:
                req = loads(await _read_frame(reader))
                if self.drop_filter is not None and self.drop_filter(req.get("method", "")):
                    continue
                asyncio.ensure_future(serve_one(req))
        except (asyncio.IncompleteReadError, ConnectionResetError, BrokenPipeError):
            pass
        finally:
            try:
                writer.close()
            except Exception:
                pass


class RpcError(RuntimeError):
    pass


class RpcClient:
    def __init__(self, host: str, port: int, name: str = ""):
        self.host, self.port, self.name = host, port, name or f"{host}:{port}"
        self._reader: Optional[asyncio.StreamReader] = None
        self._writer: Optional[asyncio.StreamWriter] = None
        self._pending: Dict[int, asyncio.Future] = {}
        self._ids = itertools.count(1)
        self._recv_task: Optional[asyncio.Task] = None
        self._wlock: Optional[asyncio.Lock] = None

    async def connect(self, retries: int = 200, delay: float = 0.1) -> "RpcClient":
        last: Optional[Exception] = None
        for _ in range(retries):
            try:
                self._reader, self._writer = await asyncio.open_connection(self.host, self.port, limit=1 << 26)
                break
            except OSError as e:
                last = e
                await asyncio.sleep(delay)
        else:
            raise ConnectionError(f"cannot connect to {self.name}: {last}")
        self._wlock = asyncio.Lock()
        self._recv_task = asyncio.ensure_future(self._recv_loop())
        return self

    async def _recv_loop(self) -> None:
        try:
            while True:
                resp = loads(await _read_frame(self._reader))
                fut = self._pending.pop(resp.get("id"), None)
                if fut is not None and not fut.done():
                    if resp.get("ok"):
                        fut.set_result(resp.get("result"))
                    else:
                        fut.set_exception(RpcError(f"{self.name}: {resp.get('error')}\n{resp.get('trace', '')}"))
        except (asyncio.IncompleteReadError, ConnectionResetError, BrokenPipeError, asyncio.CancelledError):
            pass
        finally:
            for fut in self._pending.values():
                if not fut.done():
                    fut.set_exception(ConnectionError(f"connection to {self.name} lost"))
            self._pending.clear()

    async def call(self, method: str, *args: Any, timeout: Optional[float] = None, **kwargs: Any) -> Any:
        if self._writer is None:
            await self.connect()
        rid = next(self._ids)
        fut: asyncio.Future = asyncio.get_running_loop().create_future()
        self._pending[rid] = fut
        data = dumps({"id": rid, "method": method, "args": list(args), "kwargs": kwargs})
        async with self._wlock:
            _write_frame(self._writer, data)
            await self._writer.drain()
        if timeout is None:
            return await fut
        try:
            return await asyncio.wait_for(fut, timeout)
        finally:
            self._pending.pop(rid, None)

    async def ping(self, timeout: float = 5.0) -> bool:
        try:
            return bool(await self.call("ping", timeout=timeout))
        except Exception:
            return False

    async def close(self) -> None:
        if self._recv_task is not None:
            self._recv_task.cancel()
        if self._writer is not None:
            try:
                self._writer.close()
            except Exception:
                pass
        self._writer = None

    def proxy(self) -> "RpcProxy":
        return RpcProxy(self)


class RpcProxy:
    """``await proxy.method(*args)`` forwards to the remote object."""

    def __init__(self, client: RpcClient):
        self._client = client

    def __getattr__(self, name: str) -> Callable[..., Awaitable[Any]]:
        if name.startswith("_"):
            raise AttributeError(name)

        async def _call(*args: Any, **kwargs: Any) -> Any:
            return await self._client.call(name, *args, **kwargs)

        return _call
