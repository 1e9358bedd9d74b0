"""One worker object per process, driven from a single controller — the role
Ray actors play in the reference (one ``ParaWorker`` actor per GPU,
distserve/worker.py:24; methods run one at a time in submission order,
distserve/worker.py:77-81; the engines fan a call out to all workers and wait
on the returned futures, distserve/single_stage_engine.py:224-233).

``ActorPool.spawn(factory, *args)`` starts a process (``spawn`` start method,
so CUDA is initialised in the child only), builds ``factory(*args)`` there and
returns a proxy.  ``proxy.method(*args)`` sends the call and returns a
``concurrent.futures.Future``; calls to one actor execute strictly in order.
An exception raised by the method travels back and is raised by
``Future.result()``, which is how a native failure reaches the engine in the
reference as well.

Arguments and results are pickled, exactly like Ray's: block lists, parallel
configs and the pool handles (plain integer lists) all travel this way.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import threading
import traceback
from concurrent.futures import Future
from typing import Callable, Dict, List, Optional

_CTX = mp.get_context("spawn")


def _actor_main(conn, factory: Callable, args, kwargs, env: Dict[str, str]) -> None:
    os.environ.update(env)
    try:
        obj = factory(*args, **kwargs)
        conn.send(("ready", None))
    except BaseException as e:   # construction failed: report and leave
        conn.send(("failed", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            return
        if msg is None:
            return
        call_id, method, m_args, m_kwargs = msg
        try:
            result = getattr(obj, method)(*m_args, **m_kwargs)
            conn.send((call_id, True, result))
        except BaseException as e:
            conn.send((call_id, False, f"{type(e).__name__}: {e}"))


class ActorError(RuntimeError):
    """A method raised inside the actor process."""


class ActorHandle:
    """Proxy of an object living in another process."""

    def __init__(self, process, conn) -> None:
        self._process = process
        self._conn = conn
        self._pending: Dict[int, Future] = {}
        self._next_id = 0
        self._lock = threading.Lock()
        self._reader = threading.Thread(target=self._read_loop, daemon=True)
        self._reader.start()

    def _read_loop(self) -> None:
        while True:
            try:
                call_id, ok, payload = self._conn.recv()
            except (EOFError, OSError):
                with self._lock:
                    pending, self._pending = self._pending, {}
                for fut in pending.values():
                    fut.set_exception(ActorError("the actor process ended before answering"))
                return
            with self._lock:
                fut = self._pending.pop(call_id, None)
            if fut is None:
                continue
            if ok:
                fut.set_result(payload)
            else:
                fut.set_exception(ActorError(payload))

    def call(self, method: str, *args, **kwargs) -> Future:
        fut: Future = Future()
        with self._lock:
            call_id = self._next_id
            self._next_id += 1
            self._pending[call_id] = fut
            try:
                self._conn.send((call_id, method, args, kwargs))
            except (OSError, ValueError) as e:
                self._pending.pop(call_id, None)
                fut.set_exception(ActorError(f"the actor process is gone: {e}"))
        return fut

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *args, **kwargs: self.call(name, *args, **kwargs)

    def stop(self, timeout: float = 30.0) -> None:
        try:
            self._conn.send(None)
        except (OSError, ValueError):
            pass
        self._process.join(timeout)
        if self._process.is_alive():
            self._process.kill()      # the exact process this handle started
            self._process.join(5)

    @property
    def pid(self) -> int:
        return self._process.pid

    def is_alive(self) -> bool:
        return self._process.is_alive()


class ActorPool:
    """Starts actors and stops them together."""

    def __init__(self) -> None:
        self.actors: List[ActorHandle] = []

    def spawn(self, factory: Callable, *args, env: Optional[Dict[str, str]] = None, start_timeout: float = 300.0,
              **kwargs) -> ActorHandle:
        parent, child = _CTX.Pipe()
        proc = _CTX.Process(target=_actor_main, args=(child, factory, args, kwargs, dict(env or {})), daemon=True)
        proc.start()
        child.close()
        if not parent.poll(start_timeout):
            proc.kill()
            raise ActorError("the actor did not come up in time")
        state, detail = parent.recv()
        if state != "ready":
            proc.join(5)
            raise ActorError(f"the actor could not be constructed: {detail}")
        handle = ActorHandle(proc, parent)
        self.actors.append(handle)
        return handle

    def stop(self, timeout: float = 30.0) -> None:
        """Ask every actor to leave, give each `timeout` seconds, then end the ones still there."""
        for a in self.actors:
            a.stop(timeout)
        self.actors = []

    def __enter__(self) -> "ActorPool":
        return self

    def __exit__(self, *exc) -> None:
        self.stop()
