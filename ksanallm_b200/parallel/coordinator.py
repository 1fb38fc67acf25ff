"""Liveness of a multi-rank engine: the host control channel (csrc/engine/control_channel.cpp) wired to the service.

Rank 0 runs the ``ControlMaster``, every other rank a ``ControlWorker`` (TCP, heartbeats both ways). A monitor thread
on every rank watches ``alive()``: when a peer's connection closes or its heartbeats stop, the rank ends the service -
requests in flight are answered with RET_RUNTIME, the event is logged and the process exits - instead of sitting
forever in a collective that can no longer complete. This is the behaviour of the reference's control channel and
service lifetime (src/ksana_llm/distributed/control_channel.cpp:63-111 heartbeat loss -> ShutdownService,
src/ksana_llm/service/service_lifetime.cpp:9), with the difference that one process per GPU means the channel is
also used between the ranks of one node. Nothing here touches a device: failure handling is host-only.

Environment: ``KSANA_CONTROL_PLANE=0`` disables it; ``KSANA_CONTROL_PORT`` (default MASTER_PORT + 17);
``KSANA_HEARTBEAT_INTERVAL_MS`` / ``KSANA_HEARTBEAT_TIMEOUT_MS`` (defaults 5000 / 20000).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, List, Optional

from ..utils import logger
from ..utils import native_engine as ne

_stop_hooks: List[Callable[[str], None]] = []
_exit_fn: Callable[[int], None] = os._exit          # tests replace it


def register_stop_hook(fn: Callable[[str], None]) -> None:
    """``fn(reason)`` runs before the process leaves because the service can no longer run (engines register the
    hook that answers their in-flight requests)."""
    _stop_hooks.append(fn)


def shutdown_service(reason: str, code: int = 1) -> None:
    """Ends this rank's service: hooks, log record, process exit (a rank blocked in a collective cannot be stopped in
    any gentler way). Counterpart of the reference's ShutdownService."""
    logger.error(f"service shutdown: {reason}")
    for fn in list(_stop_hooks):
        try:
            fn(reason)
        except Exception as e:  # noqa: BLE001 - a failing hook must not keep the process alive
            logger.error(f"stop hook failed: {e!r}")
    _exit_fn(code)


class DistributedCoordinator:
    """One per rank. ``start()`` connects the ranks (collective), ``close()`` tells the workers to leave in an orderly
    way (rank 0) and stops the threads."""

    def __init__(self, rank: int, world: int, host: str, port: int, interval_ms: int = 5000, timeout_ms: int = 20000,
                 on_lost: Optional[Callable[[str], None]] = None):
        self.rank, self.world, self.host, self.port = rank, world, host, port
        self.interval_ms, self.timeout_ms = interval_ms, timeout_ms
        self.on_lost = on_lost or (lambda reason: shutdown_service(reason, 1))
        self.master = None
        self.worker = None
        self._monitor: Optional[threading.Thread] = None
        self._closing = False

    @staticmethod
    def from_env(rank: int, world: int) -> Optional["DistributedCoordinator"]:
        if world <= 1 or os.environ.get("KSANA_CONTROL_PLANE", "1") == "0":
            return None
        host = os.environ.get("MASTER_ADDR") or os.environ.get("MASTER_HOST") or "127.0.0.1"
        port = int(os.environ.get("KSANA_CONTROL_PORT", int(os.environ.get("MASTER_PORT", "29511")) + 17))
        return DistributedCoordinator(rank, world, host, port,
                                      int(os.environ.get("KSANA_HEARTBEAT_INTERVAL_MS", "5000")),
                                      int(os.environ.get("KSANA_HEARTBEAT_TIMEOUT_MS", "20000")))

    def start(self, timeout_ms: int = 120000) -> None:
        if self.rank == 0:
            self.master = ne.ControlMaster(self.host, self.port, self.world, self.interval_ms, self.timeout_ms)
            if not self.master.wait_for_nodes(timeout_ms):
                raise RuntimeError(f"control channel: not all of the {self.world - 1} worker ranks registered")
        else:
            self.worker = ne.ControlWorker(self.host, self.port, self.rank, self.interval_ms, self.timeout_ms)
            if not self.worker.connect(timeout_ms):
                raise RuntimeError(f"control channel: rank {self.rank} cannot reach the master at {self.host}:{self.port}")
        logger.info(f"control channel up: rank {self.rank} of {self.world} at {self.host}:{self.port}")
        self._monitor = threading.Thread(target=self._watch, name="ksana-liveness", daemon=True)
        self._monitor.start()

    def alive(self) -> bool:
        if self.master is not None:
            return bool(self.master.alive())
        return self.worker is not None and bool(self.worker.alive())

    def _watch(self) -> None:
        while not self._closing:
            time.sleep(0.1)
            if self._closing:
                return
            if self.master is not None and not self.master.alive():
                self.on_lost(f"worker rank(s) {self.master.failed_nodes()} lost (connection closed or heartbeats stopped)")
                return
            if self.worker is not None and not self.worker.alive():
                if self.worker.shutdown_requested():
                    logger.info(f"rank {self.rank}: rank 0 closed the control channel (orderly shutdown)")
                else:
                    self.on_lost("the master rank is gone (connection closed or heartbeats stopped)")
                return

    def close(self, wait_s: float = 5.0) -> None:
        """Orderly end, called by every rank when the job is over. Rank 0 tells the workers (shutdown packet) before
        it closes its sockets; a worker keeps its connection until that packet arrives (bounded), so that rank 0 never
        sees a worker's normal exit as a lost peer."""
        self._closing = True
        if self.master is not None:
            self.master.shutdown_cluster()
            self.master.stop()
        if self.worker is not None:
            deadline = time.time() + wait_s
            while time.time() < deadline and self.worker.alive() and not self.worker.shutdown_requested():
                time.sleep(0.02)
            self.worker.stop()
