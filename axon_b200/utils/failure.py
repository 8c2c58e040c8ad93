"""Failure detection that keeps every wait bounded and every failure on the host.

* ``Heartbeat``: each rank of a job publishes a counter in a key-value store from a background
  thread; ``check()`` tells which peers stopped beating. Workers call it between steps, before they
  launch a collective, so a rank that died is noticed on the host instead of inside a kernel that
  would wait for it. (The reference has only the controller-side liveness thread,
  axon/controller/worker_group.py:54-95, and NCCL timeouts, axon/trainer/megatron_trainer.py:231-244.)
* ``guarded_collective``: runs a collective under a deadline and turns a timeout into
  ``CollectiveTimeout`` (used with short process-group timeouts in tests and at shutdown).
* Device side: kernels that wait on other ranks (``parallel/symm.PeerBarrier``, the fused ZeRO-1 and
  P2P kernels) give up after about two seconds and record ``AXB_ERR_WAIT_PEER`` in the per-device
  status word, which ``ops._common.check_status`` raises as ``NativeKernelError``; the CUDA context
  stays usable.
"""
from __future__ import annotations

import threading
import time


class PeerLostError(RuntimeError):
    def __init__(self, ranks: list[int], age: dict[int, float]):
        self.ranks, self.age = ranks, age
        super().__init__("no heartbeat from rank(s) " + ", ".join(f"{r} ({age[r]:.1f}s)" for r in ranks))


class CollectiveTimeout(TimeoutError):
    pass


class Heartbeat:
    """``store`` is any object with ``set(key, value)`` and ``get(key)`` (``torch.distributed.TCPStore``,
    ``FileStore``, a dict-backed fake in tests)."""

    def __init__(self, store, rank: int, world_size: int, interval: float = 0.5, timeout: float = 5.0, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._seen: dict[int, tuple[int, float]] = {}       # rank -> (last counter, time it changed)
        self._count = 0

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def start(self) -> "Heartbeat":
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:         # noqa: BLE001 - the store went away: the job is ending
                    return
        self._thread = threading.Thread(target=loop, daemon=True, name=f"heartbeat-{self.rank}")
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def _read(self, r: int) -> int | None:
        try:
            v = self.store.get(self._key(r))
        except Exception:                 # noqa: BLE001 - key missing / store timeout
            return None
        if isinstance(v, bytes):
            v = v.decode()
        try:
            return int(v)
        except (TypeError, ValueError):
            return None

    def lost_peers(self) -> dict[int, float]:
        now = time.monotonic()
        lost = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            c = self._read(r)
            last = self._seen.get(r)
            if c is not None and (last is None or c != last[0]):
                self._seen[r] = (c, now)
                continue
            since = now - (last[1] if last is not None else self._seen.setdefault(r, (-1, now))[1])
            if since > self.timeout:
                lost[r] = since
        return lost

    def check(self) -> None:
        lost = self.lost_peers()
        if lost:
            raise PeerLostError(sorted(lost), lost)


def guarded_collective(fn, timeout_s: float, what: str = "collective"):
    """Run ``fn()`` (a blocking collective) in a helper thread; raise ``CollectiveTimeout`` if it is not
    back after ``timeout_s``. The helper thread is a daemon: a stuck call does not keep the process."""
    box: dict = {}

    def run():
        try:
            box["v"] = fn()
        except BaseException as e:       # noqa: BLE001
            box["e"] = e
    t = threading.Thread(target=run, daemon=True, name=f"guarded-{what}")
    t.start()
    t.join(timeout_s)
    if t.is_alive():
        raise CollectiveTimeout(f"{what} did not finish within {timeout_s}s")
    if "e" in box:
        raise box["e"]
    return box.get("v")
