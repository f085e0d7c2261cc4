"""Failure detection for multi-rank jobs, on the host.

The reference's only failure handling lives in its HTTP cooperative modes (stale-round 409, poisoned-blob 400, gossip
timeouts that are logged and ignored: bin/coop_coordinator.dart:210-246, bin/coop_peer.dart:313-329); it has no
heartbeat or membership protocol.  Synchronous data / tensor / expert parallelism needs one: a rank that dies between
steps must be noticed *before* the others launch kernels that would wait for it.

``Heartbeat`` keeps a few keys per rank in the job's ``torch.distributed`` store (TCPStore, FileStore, HashStore):

* liveness: a counter bumped by ``beat()`` (and by the optional background thread, so a rank blocked inside a
  collective still looks alive);
* progress: the number of steps entered (``guard()`` bumps it);
* failure: a reason published by ``report_failure()`` (``guard()`` publishes local exceptions before they propagate).

``check()`` raises ``PeerFailure`` for a peer that reported a failure, whose liveness counter stood still for
``timeout`` seconds, or that never appeared.  ``check_progress()`` additionally flags a live peer that is behind this
rank's step and has not moved for ``timeout`` seconds (alive but stuck).  ``wait_collective(work, hb)`` polls an
asynchronous collective while checking, so a rank never blocks forever on a vanished or stuck peer.  On the device
every wait is bounded and reports through the status word (``_native.raise_on_device_error``).
"""
from __future__ import annotations

import contextlib
import threading
import time
from typing import Dict, Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, timeout: float = 30.0, prefix: str = "dptb/health",
                 background_interval: Optional[float] = None):
        self.store, self.rank, self.world, self.timeout, self.prefix = store, rank, world_size, timeout, prefix
        self._live = 0
        self._step = 0
        self._seen_live: Dict[int, tuple] = {}
        self._seen_step: Dict[int, tuple] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = None
        self.beat()
        self.store.set(self._key("step", rank), "0")
        if background_interval:
            self._thread = threading.Thread(target=self._run, args=(background_interval,), daemon=True)
            self._thread.start()

    def _run(self, interval: float) -> None:
        while not self._stop.wait(interval):
            try:
                self.beat()
            except Exception:
                return

    def close(self) -> None:
        self._stop.set()

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self) -> None:
        with self._lock:
            self._live += 1
            self.store.set(self._key("live", self.rank), str(self._live))

    def enter_step(self) -> int:
        self._step += 1
        self.store.set(self._key("step", self.rank), str(self._step))
        return self._step

    def report_failure(self, reason: str) -> None:
        self.store.set(self._key("fail", self.rank), reason[:500])

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode("utf-8")
        except Exception:
            return None

    def _stale(self, table: Dict[int, tuple], r: int, value, now: float) -> float:
        """Seconds since ``value`` of rank ``r`` last changed, as observed locally (no cross-host clock comparison)."""
        prev = table.get(r)
        if prev is None or prev[0] != value:
            table[r] = (value, now)
            return 0.0
        return now - prev[1]

    def failed_peers(self, progress: bool = False) -> Dict[int, str]:
        out = {}
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            why = self._get(self._key("fail", r))
            if why is not None:
                out[r] = why
                continue
            live = self._get(self._key("live", r))
            age = self._stale(self._seen_live, r, live, now)
            if age > self.timeout:
                out[r] = (f"no heartbeat for {age:.1f}s" if live is not None
                          else f"never joined (no heartbeat for {age:.1f}s)")
                continue
            if progress and live is not None:
                step = int(self._get(self._key("step", r)) or 0)
                lag = self._stale(self._seen_step, r, step, now)
                if step < self._step and lag > self.timeout:
                    out[r] = f"stuck at step {step} for {lag:.1f}s (this rank is at step {self._step})"
        return out

    def check(self, progress: bool = False) -> None:
        bad = self.failed_peers(progress)
        if bad:
            r = min(bad)
            raise PeerFailure(r, bad[r])

    def check_progress(self) -> None:
        self.check(progress=True)

    @contextlib.contextmanager
    def guard(self):
        """``with hb.guard(): step()`` -- checks the peers first, publishes a local failure, beats after."""
        self.check()
        self.enter_step()
        try:
            yield
        except PeerFailure:
            raise
        except BaseException as e:  # noqa: BLE001 - the reason is published, then the exception continues
            self.report_failure(f"{type(e).__name__}: {e}")
            raise
        self.beat()


def wait_collective(work, hb: Heartbeat, poll_s: float = 0.05) -> None:
    """Wait for an asynchronous collective (``async_op=True``) while watching the peers: raises ``PeerFailure`` instead
    of blocking when a peer failed, died or stopped making progress."""
    while not work.is_completed():
        hb.check_progress()
        time.sleep(poll_s)
    work.wait()


def wait_for_peers(hb: Heartbeat, deadline_s: float = 30.0, poll_s: float = 0.05) -> None:
    """Block until every rank has beaten at least once, or raise ``PeerFailure`` for the first one that has not by
    the deadline (a rank that never joins)."""
    t0 = time.time()
    while True:
        for r in range(hb.world):
            why = hb._get(hb._key("fail", r)) if r != hb.rank else None
            if why is not None:
                raise PeerFailure(r, why)
        missing = [r for r in range(hb.world) if r != hb.rank and hb._get(hb._key("live", r)) is None]
        if not missing:
            return
        if time.time() - t0 > deadline_s:
            raise PeerFailure(missing[0], f"never joined within {deadline_s:.1f}s")
        time.sleep(poll_s)
