"""Host-side failure detection: heartbeats through the rendezvous store.

The reference has no failure detection beyond the 1800 s store timeout (``bmtrain/init.py:59-65``): a rank that dies
or hangs leaves the others blocked in their next collective.  Here every rank can run a small daemon thread that
publishes a counter under its own key of the job's TCP store and reads the counters of the others.  A rank whose counter
has not moved for ``timeout`` seconds is reported as lost: :func:`check` raises on the caller's thread (call it between
steps, before the next collective is launched) and an optional callback fires from the daemon thread.

Nothing here touches a GPU; the device-side counterpart is the bounded waits of the peer-memory kernels
(``parallel/symm.py``: ``PeerRuntime.check``).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional

from .global_var import config

_state: Dict[str, object] = {"thread": None}


class Heartbeat:
    """Publishes this rank's liveness and watches the others.

    ``store`` is any object with ``set(key, value)`` / ``get(key)`` (a ``torch.distributed`` store); ``get`` of a key
    that does not exist yet may block or raise, both are handled by publishing the own key before reading.
    """

    def __init__(self, store, rank: int, world_size: int, interval: float = 1.0, timeout: float = 30.0,
                 on_failure: Optional[Callable[[List[int]], None]] = None, prefix: str = "bmt_hb"):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.interval, self.timeout, self.on_failure, self.prefix = interval, timeout, on_failure, prefix
        self._beat = 0
        self._seen: Dict[int, tuple] = {}      # rank -> (last counter value, local time it changed)
        self._lost: List[int] = []
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None

    # ------------------------------------------------------------------ control
    def start(self) -> "Heartbeat":
        self._publish()
        now = time.monotonic()
        for r in range(self.world_size):
            self._seen[r] = (-1, now)
        self._thread = threading.Thread(target=self._run, name="bmt-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5 * self.interval + 1)
            self._thread = None

    def pause(self) -> None:
        """Stop publishing (the watcher keeps running): what a hung rank looks like to the others.  For tests."""
        self._paused.set()

    def resume(self) -> None:
        self._paused.clear()

    # ------------------------------------------------------------------ queries
    def lost_ranks(self) -> List[int]:
        with self._lock:
            return list(self._lost)

    def check(self) -> None:
        """Raise ``RuntimeError`` naming the ranks whose heartbeat stopped."""
        lost = self.lost_ranks()
        if lost:
            raise RuntimeError(f"rank {self.rank}: no heartbeat from rank(s) {lost} for more than {self.timeout:.1f} s")

    # ----------------------------------------------------------------- internals
    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def _publish(self) -> None:
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))

    def _read(self, r: int) -> Optional[int]:
        try:
            key = self._key(r)
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None  # not published yet (a plain get would block until the store's own timeout)
            return int(bytes(self.store.get(key)).decode())
        except Exception:  # key not there yet, or the store itself is gone
            return None

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                if not self._paused.is_set():
                    self._publish()
            except Exception:
                pass  # a dead store shows up as everybody's heartbeat stopping
            now = time.monotonic()
            newly = []
            for r in range(self.world_size):
                if r == self.rank:
                    continue
                value = self._read(r)
                last_value, last_time = self._seen[r]
                if value is not None and value != last_value:
                    self._seen[r] = (value, now)
                    with self._lock:
                        if r in self._lost:
                            self._lost.remove(r)  # it came back (e.g. a long garbage-collection pause)
                elif now - last_time > self.timeout:
                    with self._lock:
                        if r not in self._lost:
                            self._lost.append(r)
                            newly.append(r)
            if newly and self.on_failure is not None:
                try:
                    self.on_failure(newly)
                except Exception:
                    pass


def _default_store():
    import torch.distributed as dist

    return dist.distributed_c10d._get_default_store()


def start(interval: float = 1.0, timeout: float = 30.0, on_failure: Optional[Callable[[List[int]], None]] = None) -> Heartbeat:
    """Start the heartbeat of this process (after ``init_distributed``); returns the running :class:`Heartbeat`."""
    if _state["thread"] is not None:
        return _state["thread"]  # type: ignore[return-value]
    hb = Heartbeat(_default_store(), config["rank"], config["world_size"], interval, timeout, on_failure).start()
    _state["thread"] = hb
    return hb


def check() -> None:
    """Raise if a rank stopped answering (no-op when the heartbeat is not running)."""
    hb = _state["thread"]
    if hb is not None:
        hb.check()  # type: ignore[union-attr]


def stop() -> None:
    hb = _state["thread"]
    if hb is not None:
        hb.stop()  # type: ignore[union-attr]
        _state["thread"] = None
