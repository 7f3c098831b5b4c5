"""Failure detection for the N-partitioned path, on the host.

The exchange step of the path (all-gather of output column slices) is the only place where one rank waits
for another, so it is the only place a lost peer can hang the others.  Two guards keep a rank from ever
entering that step with a dead peer or a broken communicator:

  Heartbeat      liveness through the process group's key-value store.  Before a step, a rank publishes the
                 step number and waits (bounded) until every peer has published the same step.  A peer that
                 said goodbye (`leave()`), or that stays silent past the deadline, raises PeerLost in all the
                 others BEFORE they launch — no kernel or collective is in flight when a rank is declared lost.
  CommWatchdog   polls an error source on a background thread — for NCCL the communicator's asynchronous
                 error state (ProcessGroupNCCL.get_error(), i.e. ncclCommGetAsyncError) — and, at the first
                 error, runs an abort action once (ProcessGroupNCCL.abort(), i.e. ncclCommAbort) so that
                 blocked collectives return; `check()` re-raises the error in the caller's thread before its
                 next launch.

The communicator itself belongs to torch.distributed (one per process, created by init_process_group); the
library's C ABI does not link NCCL.  Both guards are plain Python over the store / an injected error source,
so they are tested on CPU ranks (gloo) and with a fake communicator; nothing here touches a GPU.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Iterable


class PeerLost(RuntimeError):
    """A peer rank left or stopped answering.  `ranks` lists them, `reason` maps rank -> text."""

    def __init__(self, reason: dict[int, str]):
        self.ranks = sorted(reason)
        self.reason = dict(reason)
        super().__init__("lost peer rank(s) " + ", ".join(f"{r} ({reason[r]})" for r in self.ranks))


class CommError(RuntimeError):
    """The communicator reported an asynchronous error (or its watchdog timed out)."""


class Heartbeat:
    """Step-granular liveness over a torch.distributed store (TCPStore, FileStore, HashStore ...)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "tb200/hb", poll_s: float = 0.01):
        self.store, self.rank, self.world, self.prefix, self.poll_s = store, int(rank), int(world), prefix, poll_s

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _read(self, rank: int) -> str | None:
        key = self._key(rank)
        if not self.store.check([key]):            # non-blocking: get() would wait for a missing key
            return None
        return self.store.get(key).decode()

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self, why: str = "left") -> None:
        """Say goodbye between steps, with none of this rank's kernels or collectives in flight."""
        self.store.set(self._key(self.rank), f"left:{why}")

    def begin_step(self, step: int, timeout_s: float = 5.0) -> None:
        """Publish `step`, then wait until every peer has reached it.  Raises PeerLost for peers that left or
        stayed silent for `timeout_s`; returns only when the whole group is known to be alive at `step`."""
        self.beat(step)
        deadline = time.monotonic() + timeout_s
        pending = {r for r in range(self.world) if r != self.rank}
        lost: dict[int, str] = {}
        while pending:
            for r in sorted(pending):
                v = self._read(r)
                if v is None:
                    continue
                if v.startswith("left:"):
                    lost[r] = v[5:] or "left"
                    pending.discard(r)
                elif int(v) >= step:
                    pending.discard(r)
            if not pending:
                break
            if time.monotonic() > deadline:
                for r in pending:
                    v = self._read(r)
                    lost[r] = f"silent for {timeout_s:g} s at step {step} (last seen: {'never' if v is None else 'step ' + v})"
                break
            time.sleep(self.poll_s)
        if lost:
            raise PeerLost(lost)


class CommWatchdog:
    """Background poller of a communicator's asynchronous error state.

    error_source() returns None (healthy) or a description of the error; abort() is called once, from the
    watchdog thread, at the first error — it must unblock collectives that wait on the broken communicator.
    `heartbeat_timeout_s`: if the poller itself cannot complete a poll within that time (a hung driver
    call), `check()` reports it too."""

    def __init__(self, error_source: Callable[[], str | None], abort: Callable[[], None] | None = None,
                 period_s: float = 0.05, heartbeat_timeout_s: float = 10.0):
        self._source, self._abort, self._period = error_source, abort, period_s
        self._hb_timeout = heartbeat_timeout_s
        self._stop = threading.Event()
        self._error: str | None = None
        self._aborted = False
        self._last_poll = time.monotonic()
        self._thread: threading.Thread | None = None
        self.polls = 0

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                err = self._source()
            except Exception as e:                     # the source itself failing is an error of the communicator
                err = f"error source raised {type(e).__name__}: {e}"
            self._last_poll = time.monotonic()
            self.polls += 1
            if err is not None and self._error is None:
                self._error = str(err)
                if self._abort is not None and not self._aborted:
                    self._aborted = True
                    try:
                        self._abort()
                    except Exception as e:
                        self._error += f" (abort failed: {type(e).__name__}: {e})"
                return
            self._stop.wait(self._period)

    def start(self) -> "CommWatchdog":
        if self._thread is None:
            self._last_poll = time.monotonic()
            self._thread = threading.Thread(target=self._loop, name="tb200-comm-watchdog", daemon=True)
            self._thread.start()
        return self

    @property
    def error(self) -> str | None:
        return self._error

    @property
    def aborted(self) -> bool:
        return self._aborted

    def check(self) -> None:
        """Call before every launch that involves the communicator; raises CommError once an error was seen."""
        if self._error is not None:
            raise CommError(self._error)
        if self._thread is not None and self._thread.is_alive() and time.monotonic() - self._last_poll > self._hb_timeout:
            raise CommError(f"communicator watchdog made no progress for {self._hb_timeout:g} s")

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)


def nccl_error_source(group=None) -> Callable[[], str | None]:
    """Error source over torch's NCCL process group: its get_error() reads ncclCommGetAsyncError."""
    import torch
    import torch.distributed as dist
    backend = (group or dist.group.WORLD)._get_backend(torch.device("cuda"))
    ok = {"SUCCESS"}

    def source() -> str | None:
        err = backend.get_error()
        name = getattr(err, "name", str(err))
        return None if name in ok else f"NCCL communicator error: {name}"
    return source


def nccl_abort(group=None) -> Callable[[], None]:
    """Abort action over torch's NCCL process group (ncclCommAbort on its communicators)."""
    import torch
    import torch.distributed as dist
    backend = (group or dist.group.WORLD)._get_backend(torch.device("cuda"))
    return backend.abort


def guarded_steps(heartbeat: Heartbeat, steps: Iterable[int], watchdog: CommWatchdog | None = None, timeout_s: float = 5.0):
    """Yields each step number after the guards have passed for it: `for step in guarded_steps(hb, range(n)): launch(step)`."""
    for step in steps:
        if watchdog is not None:
            watchdog.check()
        heartbeat.begin_step(step, timeout_s)
        yield step
