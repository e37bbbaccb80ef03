"""Host-side failure detection for multi-rank runs: heartbeats through the rendezvous store, a failure flag that a
rank raises before it stops, and a communicator wrapper that turns a lost peer into one well-defined error.

What the reference does (``cpp/runtime/multiDevice/runtimeCoordinator.cpp:625-662``): a worker that fails records the
failure and aborts the communicators so that peers blocked in a collective return.  Here every rank runs in its own
process, so the same guarantees come from three pieces:

* a **heartbeat** thread per rank that bumps a counter in a ``torch.distributed`` TCP store; a peer whose counter has not
  moved for ``timeout`` seconds is reported lost *before* the next collective is entered (checks happen between steps,
  when no kernel or collective of this rank is in flight);
* a **failure flag**: a rank that catches an exception publishes ``failed = "<rank>: <reason>"`` and every other rank
  stops at its next check instead of waiting for a collective to time out;
* the process group's own **timeout** as the backstop for a peer that dies inside a collective: the wrapper converts the
  backend's error into :class:`RankLostError` and publishes the flag.

Device-side waits in the fused kernels are bounded separately and report through a status word
(``ops/cuda.py: Workspace.check_status``); nothing here touches a GPU."""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Tuple


class RankLostError(RuntimeError):
    """A peer stopped answering or reported a failure; the step that was about to run must not be launched."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} is lost: {reason}")
        self.rank, self.reason = rank, reason


class HealthMonitor:
    def __init__(self, store, rank: int, world_size: int, interval_s: float = 0.2, timeout_s: float = 2.0):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout = interval_s, timeout_s
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, Tuple[str, float]] = {}          # peer → (last counter value, local time it changed)
        self._beats = 0

    # ---- this rank's side ------------------------------------------------------------------------
    def _beat(self):
        while not self._stop.is_set():
            self._beats += 1
            try:
                self.store.set(f"hb/{self.rank}", str(self._beats))
                self._observe()        # note when each peer's counter last moved, so that check() can judge staleness
            except Exception:          # the store's host went away: peers will see this rank go stale
                return
            self._stop.wait(self.interval)

    def _observe(self) -> None:
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._get(f"hb/{r}")
            if v is None:
                continue                                   # not started yet: the rendezvous barrier covers start-up
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)

    def start(self) -> "HealthMonitor":
        self.store.set(f"hb/{self.rank}", "0")
        self._thread = threading.Thread(target=self._beat, name=f"telb-heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def leave(self) -> None:
        """Orderly departure between steps: peers see ``left/<rank>`` and report it at their next check."""
        try:
            self.store.set(f"left/{self.rank}", "1")
        finally:
            self.stop()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 0.5)
            self._thread = None

    def report_failure(self, reason: str) -> None:
        try:
            self.store.set("failed", f"{self.rank}: {reason}")
        except Exception:
            pass

    # ---- looking at the peers --------------------------------------------------------------------
    def _get(self, key: str) -> Optional[str]:
        try:
            if not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except RankLostError:
            raise
        except Exception as e:       # the store's host process is gone: whoever held it has stopped
            raise RankLostError(-1, f"rendezvous store unreachable ({type(e).__name__})") from e

    def check(self) -> None:
        """Raise :class:`RankLostError` if a peer failed, left, or went silent.  Cheap; call it between steps."""
        failed = self._get("failed")
        if failed is not None:
            r, _, why = failed.partition(": ")
            if int(r) != self.rank:
                raise RankLostError(int(r), why or "reported a failure")
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self._get(f"left/{r}") is not None:
                raise RankLostError(r, "left the job")
        self._observe()
        for r, (_, changed) in list(self._seen.items()):
            if now - changed > self.timeout:
                raise RankLostError(r, f"no heartbeat for {now - changed:.1f} s")

    def wait_for_loss(self, max_wait_s: float) -> None:
        """Poll :meth:`check` for up to ``max_wait_s`` (used when a collective is about to be entered and a peer looked
        slow): returns quietly if everyone keeps beating."""
        end = time.monotonic() + max_wait_s
        while time.monotonic() < end:
            self.check()
            time.sleep(self.interval)


class GuardedComm:
    """Wraps a communicator (``parallel/comm.py`` interface): peers are checked before every collective and a backend
    error inside one becomes :class:`RankLostError` after the failure flag is published."""

    _COLLECTIVES = ("all_reduce", "all_gather_cols", "all_gather_rows", "reduce_scatter_rows", "broadcast_tokens", "all_to_all",
                    "add_rmsnorm", "barrier")

    def __init__(self, comm, monitor: HealthMonitor):
        self._comm, self.monitor = comm, monitor

    def __getattr__(self, name):
        attr = getattr(self._comm, name)
        if name not in self._COLLECTIVES:
            return attr

        def guarded(*a, **kw):
            self.monitor.check()
            try:
                return attr(*a, **kw)
            except RankLostError:
                raise
            except Exception as e:       # the backend timed out or lost its connection inside the collective
                try:                     # whose fault?  give the heartbeats one timeout to name the silent peer
                    self.monitor.wait_for_loss(self.monitor.timeout + 3 * self.monitor.interval)
                except RankLostError as lost:
                    raise lost from e
                self.monitor.report_failure(f"{name} failed: {type(e).__name__}")
                raise RankLostError(-1, f"{name} failed: {e}") from e
        return guarded
