"""Host-side rank liveness: heartbeats and failure notices through the rendezvous store.

Device-side waits in this package are bounded, so a peer that disappears costs the others a
time-out instead of a hang.  This module lets them learn about it *before* their next launch:

* every rank runs a small thread that writes ``<prefix>/beat/<rank> = "<unix time>:<step>"``
  into the process group's key-value store every ``interval_s`` seconds;
* a rank whose training step raises calls :meth:`announce_failure` (the trainer does this in its
  exception path), which writes ``<prefix>/failed/<rank>`` with the reason;
* :meth:`check` — called by the trainer between steps, with nothing of its own in flight — reads
  the peers' keys and raises :class:`RankFailure` when a peer announced a failure or when its
  last heartbeat is older than ``deadline_s``.

Nothing here touches a GPU.  The reference has no liveness mechanism at all (its Ray actors are
killed with ``no_restart=True``, ``vrl/distributed/ray/rollout/runtime.py:64``); the recovery it
relies on — restart from the last ``checkpoint.pt`` — is what a :class:`RankFailure` leads to here
as well: the job ends cleanly on every rank and is relaunched with ``trainer.resume_from``.
"""

from __future__ import annotations

import threading
import time
from typing import Any


class RankFailure(RuntimeError):
    """A peer rank announced a failure or stopped sending heartbeats."""

    def __init__(self, rank: int, reason: str) -> None:
        super().__init__(f"rank {rank} is gone: {reason}")
        self.rank = rank
        self.reason = reason


class InjectedFault(RuntimeError):
    """Raised on the host by :func:`maybe_inject_fault`; never reaches a device."""


def maybe_inject_fault(rank: int, step: int) -> None:
    """Host-side fault injection for recovery drills and tests: with
    ``VRL_FAULT_INJECT="rank=<r>,step=<s>[,attempt=<a>]"`` in the environment, rank ``r`` raises
    :class:`InjectedFault` at the start of its step ``s`` (0-based count of completed steps),
    before anything is launched.  ``attempt`` (default 0) is compared with ``VRL_RESTART_ATTEMPT``
    (set by the in-place restart loop) or else the launcher's ``TORCHELASTIC_RESTART_COUNT``, so
    that the restarted run is left alone."""
    import os

    plan = os.environ.get("VRL_FAULT_INJECT", "").strip()
    if not plan:
        return
    fields = dict(part.split("=", 1) for part in plan.replace(" ", "").split(",") if "=" in part)
    try:
        want_rank, want_step = int(fields["rank"]), int(fields["step"])
        want_attempt = int(fields.get("attempt", 0))
    except (KeyError, ValueError) as exc:
        raise ValueError(f"VRL_FAULT_INJECT={plan!r}: expected rank=<int>,step=<int>[,attempt=<int>]") from exc
    attempt = int(os.environ.get("VRL_RESTART_ATTEMPT") or os.environ.get("TORCHELASTIC_RESTART_COUNT") or 0)
    if (rank, step, attempt) == (want_rank, want_step, want_attempt):
        raise InjectedFault(f"injected failure on rank {rank} at step {step} (attempt {attempt})")


def default_store() -> Any:
    """The key-value store of the default process group (``None`` when not initialised)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return None
    return dist.distributed_c10d._get_default_store()


class RankLiveness:
    def __init__(self, store: Any, rank: int, world: int, *, interval_s: float = 1.0,
                 deadline_s: float = 15.0, prefix: str = "vrl/liveness",
                 clock: Any = time.time) -> None:
        if deadline_s <= interval_s:
            raise ValueError("deadline_s must be larger than interval_s")
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.interval_s, self.deadline_s = float(interval_s), float(deadline_s)
        self.prefix = prefix
        self._clock = clock
        self._step = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._started_at = clock()

    # -- keys ------------------------------------------------------------------------------------
    def _beat_key(self, rank: int) -> str:
        return f"{self.prefix}/beat/{rank}"

    def _fail_key(self, rank: int) -> str:
        return f"{self.prefix}/failed/{rank}"

    # -- this rank ---------------------------------------------------------------------------------
    def beat(self, step: int | None = None) -> None:
        if step is not None:
            self._step = int(step)
        self.store.set(self._beat_key(self.rank), f"{self._clock():.3f}:{self._step}")

    def start(self) -> "RankLiveness":
        """Send heartbeats from a daemon thread until :meth:`stop`."""
        if self._thread is not None:
            return self
        self.beat()
        self._stop.clear()

        def loop() -> None:
            while not self._stop.wait(self.interval_s):
                try:
                    self.beat()
                except Exception:  # noqa: BLE001 - the store went away with the job
                    return

        self._thread = threading.Thread(target=loop, name="vrl-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval_s + 1.0)
            self._thread = None

    def announce_failure(self, reason: str) -> None:
        try:
            self.store.set(self._fail_key(self.rank), str(reason)[:500] or "unknown")
        except Exception:  # noqa: BLE001
            pass

    # -- the peers ---------------------------------------------------------------------------------
    def _read(self, key: str) -> str | None:
        # `get` blocks until the key exists; `check` answers at once
        if not self.store.check([key]):
            return None
        value = self.store.get(key)
        return value.decode() if isinstance(value, (bytes, bytearray)) else str(value)

    def peer_age_s(self, rank: int) -> float | None:
        """Seconds since ``rank``'s last heartbeat (``None`` before its first one)."""
        raw = self._read(self._beat_key(rank))
        if raw is None:
            return None
        try:
            stamp = float(raw.split(":", 1)[0])
        except ValueError:
            return None
        return max(0.0, self._clock() - stamp)

    def failed_peers(self) -> dict[int, str]:
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            reason = self._read(self._fail_key(r))
            if reason is not None:
                out[r] = reason
        return out

    def check(self) -> None:
        """Raise :class:`RankFailure` for the first peer that failed or fell silent."""
        failed = self.failed_peers()
        if failed:
            rank = min(failed)
            raise RankFailure(rank, f"it reported: {failed[rank]}")
        for r in range(self.world):
            if r == self.rank:
                continue
            age = self.peer_age_s(r)
            if age is None:
                # never heard from: allowed only while the job is starting up
                if self._clock() - self._started_at > self.deadline_s:
                    raise RankFailure(r, f"no heartbeat within {self.deadline_s:.0f} s of start-up")
            elif age > self.deadline_s:
                raise RankFailure(r, f"last heartbeat {age:.1f} s ago (deadline {self.deadline_s:.0f} s)")


def build_liveness(mesh: Any, *, interval_s: float = 1.0, deadline_s: float = 15.0) -> RankLiveness | None:
    """Heartbeats for a multi-rank job; ``None`` for a single rank."""
    store = default_store()
    if store is None or getattr(mesh, "world_size", 1) <= 1:
        return None
    return RankLiveness(store, mesh.rank, mesh.world_size, interval_s=interval_s,
                        deadline_s=deadline_s, prefix=f"vrl/liveness/{incarnation()}").start()


def incarnation() -> str:
    """Names this start of the job.  A launcher that restarts its workers keeps one store for all
    of them, so the failure notice that ended one incarnation must not be read by the next."""
    import os

    return (f"{os.environ.get('TORCHELASTIC_RESTART_COUNT') or 0}."
            f"{os.environ.get('VRL_RESTART_ATTEMPT') or 0}")


__all__ = ["InjectedFault", "RankFailure", "RankLiveness", "build_liveness", "default_store", "incarnation",
           "maybe_inject_fault"]
