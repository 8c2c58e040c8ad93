"""Worker groups: the controller-side handle on a set of worker processes.

``WorkerGroup`` turns every ``@register``-decorated method of the worker class into a controller-side
callable that dispatches arguments, executes on the workers and collects results
(reference: axon/controller/worker_group.py, axon/controller/ray/worker_group.py:101-385). The
reference backs this with Ray actors; here a single box needs no cluster manager:

  ``LocalWorkerGroup(backend="process")``  one spawned process per rank (env RANK / WORLD_SIZE /
        LOCAL_RANK / MASTER_ADDR / MASTER_PORT set before the worker is built), pickled RPC over
        pipes, one dispatcher thread per worker so calls to different workers overlap, bounded RPC
        timeouts, and an aliveness monitor that aborts the controller when a worker dies.
  ``LocalWorkerGroup(backend="inline")``   workers are plain objects in the controller process
        (single GPU, CPU tests).
"""
from __future__ import annotations

import multiprocessing as mp
import os
import signal
import socket
import threading
import time
import traceback
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Callable

from .decorator import MAGIC_ATTR, Dispatch, get_predefined_dispatch_fn, get_predefined_execute_fn


class ClassWithInitArgs:
    """A worker class plus the arguments to build it with, instantiated lazily inside the worker process."""

    def __init__(self, cls, *args, **kwargs):
        self.cls, self.args, self.kwargs = cls, args, kwargs

    def __call__(self):
        return self.cls(*self.args, **self.kwargs)

    # A class assembled at run time (``synthesize_class``) cannot be pickled by reference; its recipe
    # (name, base, mixins) travels instead and the worker process assembles it again.
    def __getstate__(self):
        state = dict(self.__dict__)
        spec = getattr(self.cls, "_synth_spec", None)
        if spec is not None:
            state["cls"] = None
            state["_spec"] = spec
        fused = getattr(self.cls, "_fused_spec", None)       # a colocated multi-role worker: its roles' recipes travel
        if fused is not None:
            state["cls"] = None
            state["_fused"] = fused
        return state

    def __setstate__(self, state):
        spec = state.pop("_spec", None)
        fused = state.pop("_fused", None)
        self.__dict__.update(state)
        if spec is not None:
            self.cls = synthesize_class(*spec)
        if fused is not None:
            from .fused_worker_group import fuse_worker_cls
            self.cls = fuse_worker_cls(fused).cls


def synthesize_class(name: str, base: type, mixins: tuple = ()) -> type:
    """``type(name, (*mixins, base), {})`` that remembers its recipe (see ``ClassWithInitArgs``)."""
    if not mixins:
        return base
    cls = type(name, (*mixins, base), {})
    cls._synth_spec = (name, base, tuple(mixins))
    return cls


class WorkerDiedError(RuntimeError):
    pass


class RPCTimeoutError(TimeoutError):
    pass


def func_generator(self, method_name, dispatch_fn, collect_fn, execute_fn, blocking):
    def call(*args, **kwargs):
        args, kwargs = dispatch_fn(self, *args, **kwargs)
        out = execute_fn(method_name, *args, **kwargs)
        if blocking:
            out = [o.result(self.rpc_timeout) if isinstance(o, Future) else o for o in out] \
                if isinstance(out, list) else (out.result(self.rpc_timeout) if isinstance(out, Future) else out)
        return collect_fn(self, out)
    call.__name__ = method_name
    return call


class WorkerGroup:
    def __init__(self):
        self._workers: list = []
        self._dispatch_info: dict[str, list[int]] = {}
        self._collect_info: dict[str, list[bool]] = {}
        self._monitor: threading.Thread | None = None
        self._monitor_stop = threading.Event()
        self.rpc_timeout: float | None = None

    @property
    def world_size(self) -> int:
        return len(self._workers)

    @property
    def workers(self):
        return self._workers

    def _is_worker_alive(self, worker) -> bool:
        raise NotImplementedError

    def start_worker_aliveness_check(self, every_n_seconds: float = 1.0, on_failure: Callable | None = None) -> None:
        """Poll every worker; when one is gone call ``on_failure(rank)`` (default: SIGABRT this process,
        which is how the controller learns that a step cannot complete)."""
        def default_failure(rank):
            os.kill(os.getpid(), signal.SIGABRT)

        handler = on_failure or default_failure

        def loop():
            while not self._monitor_stop.wait(every_n_seconds):
                for rank, w in enumerate(self._workers):
                    if not self._is_worker_alive(w):
                        handler(rank)
                        return
        self._monitor_stop.clear()
        self._monitor = threading.Thread(target=loop, daemon=True, name="worker-aliveness")
        self._monitor.start()

    def stop_worker_aliveness_check(self) -> None:
        self._monitor_stop.set()
        if self._monitor is not None:
            self._monitor.join(timeout=5)
            self._monitor = None

    def _bind_worker_method(self, user_defined_cls, generator=func_generator, prefix: str = "") -> list[str]:
        """Create one controller-side callable per registered worker method. Returns the bound names."""
        bound = []
        for name in dir(user_defined_cls):
            try:
                method = getattr(user_defined_cls, name)
            except Exception:  # noqa: BLE001
                continue
            info = getattr(method, MAGIC_ATTR, None)
            if not callable(method) or info is None:
                continue
            mode = info["dispatch_mode"]
            fns = mode if isinstance(mode, dict) else get_predefined_dispatch_fn(mode)
            execute_fn = getattr(self, get_predefined_execute_fn(info["execute_mode"])["execute_fn_name"])
            fn = generator(self, name, fns["dispatch_fn"], fns["collect_fn"], execute_fn, info["blocking"])
            bind_as = prefix + name
            if hasattr(type(self), bind_as):
                # the group has a method of its own under this name (``shutdown`` tears the worker processes down): the
                # workers' method of the same name stays reachable as ``worker_<name>`` and never shadows the group's
                bind_as = "worker_" + bind_as
            setattr(self, bind_as, fn)
            bound.append(bind_as)
        return bound

    def _query_dispatch_info(self, mesh_name: str) -> list[int]:
        return self.execute_all_sync("_query_dispatch_info", *[[mesh_name] * self.world_size])

    def _query_collect_info(self, mesh_name: str) -> list[bool]:
        return self.execute_all_sync("_query_collect_info", *[[mesh_name] * self.world_size])

    # subclasses implement execute_all / execute_rank_zero returning futures or values
    def execute_all_sync(self, method_name: str, *args, **kwargs) -> list:
        out = self.execute_all(method_name, *args, **kwargs)
        return [o.result(self.rpc_timeout) if isinstance(o, Future) else o for o in out]


# ------------------------------------------------------------------------------------------------
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_main(conn, factory: ClassWithInitArgs, env: dict, max_concurrency: int = 4) -> None:
    """Worker process body. Calls run on a small thread pool so that a long call (a rollout) does not
    block a short one that must overlap with it (pause, weight receive); replies carry the call id."""
    os.environ.update(env)
    try:
        obj = factory()
        conn.send(("ready", None, None))
    except BaseException:  # noqa: BLE001
        conn.send(("error", None, traceback.format_exc()))
        return
    send_lock = threading.Lock()
    pool = ThreadPoolExecutor(max_workers=max(1, max_concurrency), thread_name_prefix="rpc-exec")

    def bind_device():
        """The current CUDA device is a per-thread setting: the worker chose its GPU on the main thread, every pool
        thread has to choose it again or its allocations and collectives land on GPU 0."""
        dev = getattr(obj, "device", None)
        if dev is None:
            for role in getattr(obj, "role_objects", {}).values():
                dev = getattr(role, "device", None)
                if dev is not None:
                    break
        if dev is not None and getattr(dev, "type", None) == "cuda":
            import torch
            torch.cuda.set_device(dev)

    def execute(call_id, name, args, kwargs):
        try:
            bind_device()
            res = getattr(obj, name)(*args, **kwargs)
            if hasattr(res, "__await__"):
                import asyncio
                res = asyncio.run(res)
            reply = ("ok", call_id, res)
        except BaseException:  # noqa: BLE001
            reply = ("error", call_id, traceback.format_exc())
        with send_lock:
            try:
                conn.send(reply)
            except Exception:  # noqa: BLE001 - result not picklable
                conn.send(("error", call_id, "result could not be pickled:\n" + traceback.format_exc()))

    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            break
        if msg is None:
            break
        call_id, name, args, kwargs = msg
        pool.submit(execute, call_id, name, args, kwargs)
    pool.shutdown(wait=False, cancel_futures=True)
    os._exit(0)


class _ProcessWorker:
    def __init__(self, rank: int, factory: ClassWithInitArgs, env: dict, ctx, max_concurrency: int = 4):
        self.rank = rank
        self.conn, child = ctx.Pipe()
        self.proc = ctx.Process(target=_worker_main, args=(child, factory, env, max_concurrency), daemon=True)
        self.proc.start()
        child.close()
        self._send_lock = threading.Lock()
        self._pending: dict[int, Future] = {}
        self._pending_lock = threading.Lock()
        self._next_id = 0
        self._reader: threading.Thread | None = None

    def wait_ready(self, timeout: float) -> None:
        if not self.conn.poll(timeout):
            raise RPCTimeoutError(f"worker {self.rank} did not start within {timeout}s")
        tag, _, payload = self.conn.recv()
        if tag != "ready":
            raise RuntimeError(f"worker {self.rank} failed to start:\n{payload}")
        self._reader = threading.Thread(target=self._read_loop, daemon=True, name=f"rpc-read-{self.rank}")
        self._reader.start()

    def _fail_all(self, exc: BaseException) -> None:
        with self._pending_lock:
            pend, self._pending = self._pending, {}
        for fut in pend.values():
            if not fut.done():
                fut.set_exception(exc)

    def _read_loop(self) -> None:
        while True:
            try:
                if not self.conn.poll(0.2):
                    if not self.proc.is_alive():
                        self._fail_all(WorkerDiedError(f"worker {self.rank} died"))
                        return
                    continue
                tag, call_id, payload = self.conn.recv()
            except (EOFError, OSError):
                self._fail_all(WorkerDiedError(f"worker {self.rank} is gone"))
                return
            with self._pending_lock:
                fut = self._pending.pop(call_id, None)
            if fut is None or fut.done():
                continue
            if tag == "ok":
                fut.set_result(payload)
            else:
                fut.set_exception(RuntimeError(f"worker {self.rank} raised:\n{payload}"))

    def call(self, name, args, kwargs, timeout) -> Future:
        fut: Future = Future()
        with self._pending_lock:
            call_id = self._next_id
            self._next_id += 1
            self._pending[call_id] = fut
        try:
            with self._send_lock:
                self.conn.send((call_id, name, args, kwargs))
        except (BrokenPipeError, OSError) as e:
            with self._pending_lock:
                self._pending.pop(call_id, None)
            fut.set_exception(WorkerDiedError(f"worker {self.rank} is gone"))
            fut.__cause__ = e
            return fut
        if timeout is not None:
            def expire():
                with self._pending_lock:
                    f = self._pending.pop(call_id, None)
                if f is not None and not f.done():
                    f.set_exception(RPCTimeoutError(f"worker {self.rank}: '{name}' exceeded {timeout}s"))
            t = threading.Timer(timeout, expire)
            t.daemon = True
            t.start()
            fut.add_done_callback(lambda _f: t.cancel())
        return fut

    def shutdown(self) -> None:
        try:
            with self._send_lock:
                self.conn.send(None)
        except (BrokenPipeError, OSError):
            pass
        self.proc.join(timeout=5)
        if self.proc.is_alive():
            self.proc.terminate()
        self._fail_all(WorkerDiedError(f"worker {self.rank} was shut down"))


class LocalWorkerGroup(WorkerGroup):
    def __init__(self, resource_pool=None, cls_with_init: ClassWithInitArgs | None = None, backend: str = "process",
                 world_size: int | None = None, env: dict | None = None, rpc_timeout: float | None = 600.0,
                 start_timeout: float = 300.0, bind: bool = True, max_concurrency: int = 4):
        super().__init__()
        assert backend in ("process", "inline")
        self.backend = backend
        self.rpc_timeout = rpc_timeout
        self.cls_with_init = cls_with_init
        n = world_size if world_size is not None else (resource_pool.world_size if resource_pool is not None else 1)
        offset = getattr(resource_pool, "device_offset", 0) if resource_pool is not None else 0
        addr, port = "127.0.0.1", str(_free_port())
        base_env = dict(env or {})
        for rank in range(n):
            wenv = {"WORLD_SIZE": str(n), "RANK": str(rank), "LOCAL_RANK": str(rank + offset),
                    "LOCAL_WORLD_SIZE": str(n), "MASTER_ADDR": addr, "MASTER_PORT": port, **base_env}
            if backend == "inline":
                saved = {k: os.environ.get(k) for k in wenv}
                os.environ.update(wenv)
                try:
                    self._workers.append(cls_with_init())
                finally:
                    for k, v in saved.items():
                        if v is None:
                            os.environ.pop(k, None)
                        else:
                            os.environ[k] = v
            else:
                self._workers.append(_ProcessWorker(rank, cls_with_init, wenv, mp.get_context("spawn"), max_concurrency))
        if backend == "process":
            for w in self._workers:
                w.wait_ready(start_timeout)
        if bind and cls_with_init is not None:
            self._bind_worker_method(cls_with_init.cls)

    def _is_worker_alive(self, worker) -> bool:
        return True if self.backend == "inline" else worker.proc.is_alive()

    def _call(self, rank: int, name: str, args, kwargs):
        w = self._workers[rank]
        if self.backend == "inline":
            res = getattr(w, name)(*args, **kwargs)
            if hasattr(res, "__await__"):
                import asyncio
                res = asyncio.run(res)
            return res
        return w.call(name, args, kwargs, self.rpc_timeout)

    def execute_all(self, method_name: str, *args, **kwargs) -> list:
        """Per-worker argument lists (length == world_size) are scattered; anything else is replicated."""
        n = self.world_size
        per_worker = all(isinstance(a, list) and len(a) == n for a in args) and \
            all(isinstance(v, list) and len(v) == n for v in kwargs.values()) and (args or kwargs)
        out = []
        for i in range(n):
            a = tuple(x[i] for x in args) if per_worker else args
            k = {key: v[i] for key, v in kwargs.items()} if per_worker else kwargs
            out.append(self._call(i, method_name, a, k))
        return out

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        n = self.world_size
        scattered = (args or kwargs) and all(isinstance(a, list) and len(a) == n for a in args) and \
            all(isinstance(v, list) and len(v) == n for v in kwargs.values())
        if scattered:      # a replicating dispatch produced per-worker lists: rank 0 takes its own share
            args = tuple(a[0] for a in args)
            kwargs = {k: v[0] for k, v in kwargs.items()}
        return self._call(0, method_name, args, kwargs)

    def execute(self, method_name: str, *args, ranks: list[int] | None = None, **kwargs) -> list:
        return [self._call(r, method_name, args, kwargs) for r in (ranks if ranks is not None else range(self.world_size))]

    def shutdown(self) -> None:
        """Tell the workers to wind down (their own ``shutdown``, where they have one: servers, threads), then end the
        worker processes."""
        self.stop_worker_aliveness_check()
        stop = getattr(self, "worker_shutdown", None)
        if stop is not None and self._workers:
            try:
                stop()
            except Exception:  # noqa: BLE001 - a worker that is already gone cannot wind down
                pass
        if self.backend == "process":
            for w in self._workers:
                w.shutdown()
        self._workers = []


def init_worker_group(class_dict: dict[str, ClassWithInitArgs], resource_pool, backend: str = "process", **kw):
    """One role: a plain group. Several roles on the same pool: a fused (colocated) group whose workers
    host every role in one process; per-role views come from ``RoleProxy``."""
    if len(class_dict) == 1:
        (role, cwi), = class_dict.items()
        return {role: LocalWorkerGroup(resource_pool, cwi, backend=backend, **kw)}
    from .fused_worker_group import RoleProxy, fuse_worker_cls
    fused = fuse_worker_cls(class_dict)
    wg = LocalWorkerGroup(resource_pool, fused, backend=backend, **kw)
    return {role: RoleProxy(wg, role, class_dict[role].cls) for role in class_dict}
