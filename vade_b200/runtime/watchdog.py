"""Deadlines for every host-side wait on the GPU, and a bounded teardown.

Each place where the host blocks on the device (a token read-back, a stream synchronize, a graph replay
that is read afterwards) runs inside ``watchdog.wait(label)``: the wait registers a deadline
(``VADE_GPU_WAIT_TIMEOUT_SECS``, default 120 s).  One daemon thread looks at the open waits; when one is
past its deadline it records the event, marks the engine failed (``/health`` reports it) and ends the
process ``grace`` seconds later (4.5 s), so a stuck driver can never hold a rank for ever.  A stalled GPU
is never provoked to test this: tests use a manual clock and an ``on_expire`` callback instead of an exit.
Parity: engine/crates/gpu/src/teardown.rs:1-60 (deadline registry, 4.5 s bound, signal-safe arm).
"""
from __future__ import annotations

import contextlib
import os
import sys
import threading
import time

from ..utils import events
from ..utils.env import integer

GRACE_SECONDS = 4.5


class Watchdog:
    def __init__(self, timeout_s: float | None = None, clock=time.monotonic, on_expire=None, poll_s: float = 0.25,
                 grace_s: float = GRACE_SECONDS, start_thread: bool = True):
        self.timeout = float(timeout_s if timeout_s is not None else integer("VADE_GPU_WAIT_TIMEOUT_SECS", 120, 1, 86400))
        self.clock = clock
        self.on_expire = on_expire or self._exit
        self.poll = poll_s
        self.grace = grace_s
        self.lock = threading.Lock()
        self.open: dict = {}                 # id -> (label, deadline)
        self.next_id = 0
        self.expired: tuple | None = None    # (label, overdue seconds) of the first expiry
        self.armed_at: float | None = None
        self._thread = None
        if start_thread:
            self._thread = threading.Thread(target=self._run, name="vade-watchdog", daemon=True)
            self._thread.start()

    # ---- registry
    @contextlib.contextmanager
    def wait(self, label: str, timeout_s: float | None = None):
        with self.lock:
            wid = self.next_id
            self.next_id += 1
            self.open[wid] = (label, self.clock() + (timeout_s if timeout_s is not None else self.timeout))
        try:
            yield
        finally:
            with self.lock:
                self.open.pop(wid, None)

    @property
    def failed(self) -> bool:
        return self.expired is not None

    def check(self) -> bool:
        """One look at the open waits (the thread calls this; tests call it with a manual clock).
        Returns True when the process should end now."""
        now = self.clock()
        with self.lock:
            if self.expired is None:
                for label, deadline in self.open.values():
                    if now > deadline:
                        self.expired = (label, now - deadline)
                        self.armed_at = now
                        events.note("gpu_wait_expired", f"gpu_wait_expired label={label} overdue_s={now - deadline:.1f}")
                        break
            armed = self.armed_at
        if armed is not None and now - armed >= self.grace:
            return True
        return False

    def arm(self) -> None:
        """Ends the process after the grace period even if nothing else happens (fatal error paths)."""
        with self.lock:
            if self.armed_at is None:
                self.armed_at = self.clock()
                if self.expired is None:
                    self.expired = ("armed", 0.0)

    def _run(self) -> None:
        while True:
            time.sleep(self.poll)
            if self.check():
                self.on_expire(self.expired)
                return

    @staticmethod
    def _exit(expired) -> None:
        label, over = expired if expired else ("?", 0.0)
        try:
            print(f"watchdog: GPU wait '{label}' is {over:.1f} s past its deadline; ending the process", file=sys.stderr, flush=True)
        finally:
            os._exit(70)


_global: Watchdog | None = None


def get() -> Watchdog:
    global _global
    if _global is None:
        _global = Watchdog()
    return _global


def wait(label: str, timeout_s: float | None = None):
    return get().wait(label, timeout_s)
