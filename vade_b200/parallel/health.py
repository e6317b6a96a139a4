"""Host-side failure detection between ranks: heartbeats, a sticky failure word, peer admission.

Failure handling is deliberately minimal, as in the reference: a lost rank is DETECTED quickly and the
group stops; nothing is retried and no conversation is recovered ("If a rank fails, the launcher stops
the group", engine/docs/multi-spark.md:211-213).

* ``Heartbeat``  every rank publishes a counter in a shared key/value store (``torch.distributed``'s
  TCPStore, or any object with ``set``/``get``) at most every ``period`` seconds
  (``min(limit / 4, 0.5 s)``); before its next launch a rank calls ``check()``, which raises
  ``PeerLost`` when a peer has been silent for ``limit`` seconds or has published a failure.  A rank
  therefore leaves a group only BETWEEN steps, with none of its kernels or collectives in flight, and the
  others learn of it on the host before they launch.  ``fail(reason)`` is sticky: once set, every
  later ``check()`` on every rank raises (a poisoned group refuses further collectives).
  Parity: engine/crates/engine/src/flash/next_pp_heartbeat.rs:129-170 (STATUS_WORKING every
  min(limit/4, 500 ms), link failed after ``limit`` of silence), seqpar/src/transport.rs:1478 (poisoned ring).
* ``admit`` / ``Challenge``  HMAC-SHA256 challenge/response bound to both nonces and both roles for
  any non-loopback control connection (gateway <-> replica, launcher <-> rank); secrets shorter than 16
  bytes are refused.  Parity: engine/crates/seqpar/src/control.rs:22-140.
"""
from __future__ import annotations

import hashlib
import hmac
import secrets
import time


class PeerLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process groups)."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, limit_s: float = 10.0, clock=time.monotonic, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.limit = float(limit_s)
        self.period = min(self.limit / 4.0, 0.5)
        self.clock = clock
        self.prefix = prefix
        self.count = 0
        self.last_sent = None
        self.seen = {r: (None, clock()) for r in range(world) if r != rank}   # rank -> (last counter, when it changed)
        self.failed: PeerLost | None = None

    def _key(self, what: str, rank: int) -> str:
        return f"{self.prefix}/{what}/{rank}"

    def beat(self, force: bool = False) -> bool:
        """Publishes this rank's counter if ``period`` has passed; returns whether it wrote."""
        now = self.clock()
        if not force and self.last_sent is not None and now - self.last_sent < self.period:
            return False
        self.count += 1
        self.store.set(self._key("beat", self.rank), str(self.count))
        self.last_sent = now
        return True

    def fail(self, reason: str) -> None:
        self.store.set(self._key("fail", self.rank), reason[:200])
        self.failed = PeerLost(self.rank, reason)

    def _read(self, key: str):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key)
        except (KeyError, RuntimeError):
            return None

    def check(self) -> None:
        """Call between steps, before the next launch or collective.  Raises PeerLost (sticky)."""
        if self.failed is not None:
            raise self.failed
        self.beat()
        now = self.clock()
        for r in list(self.seen):
            why = self._read(self._key("fail", r))
            if why is not None:
                self.failed = PeerLost(r, "reported failure: " + (why.decode() if isinstance(why, bytes) else str(why)))
                raise self.failed
            v = self._read(self._key("beat", r))
            last, when = self.seen[r]
            if v is not None and v != last:
                self.seen[r] = (v, now)
            elif now - when > self.limit:
                self.failed = PeerLost(r, f"silent for {now - when:.1f} s (limit {self.limit:.1f} s)")
                raise self.failed


    def step_barrier(self, step: int, poll_s: float = 0.01, sleep=time.sleep) -> None:
        """Host-side rendezvous before a step's first launch or collective: publishes "ready for `step`" and
        polls until every peer has done so, checking heartbeats meanwhile.  A peer that left or died never
        becomes ready, so this raises PeerLost after ``limit`` instead of entering a collective that cannot finish."""
        self.store.set(self._key(f"ready{step}", self.rank), "1")
        waiting = [r for r in self.seen]
        while waiting:
            self.check()
            waiting = [r for r in waiting if self._read(self._key(f"ready{step}", r)) is None]
            if waiting:
                sleep(poll_s)


# ------------------------------------------------------------------ peer admission
MIN_SECRET = 16


def _mac(secret: bytes, *parts: bytes) -> bytes:
    h = hmac.new(secret, digestmod=hashlib.sha256)
    for p in parts:
        h.update(len(p).to_bytes(4, "big"))
        h.update(p)
    return h.digest()


class Challenge:
    """One side of the handshake.  A -> B: nonce_a;  B -> A: nonce_b, mac(B's role);  A -> B: mac(A's role).
    Each MAC covers both nonces and both role names, so a reply cannot be replayed to another role or session."""

    def __init__(self, secret: bytes, role: str, peer_role: str):
        if len(secret) < MIN_SECRET:
            raise ValueError(f"control secret must be at least {MIN_SECRET} bytes")
        self.secret, self.role, self.peer_role = secret, role.encode(), peer_role.encode()
        self.nonce = secrets.token_bytes(32)

    def respond(self, peer_nonce: bytes) -> bytes:
        first, second = sorted([self.nonce, peer_nonce])
        return _mac(self.secret, b"vade-control-1", first, second, self.role, self.peer_role)

    def verify(self, peer_nonce: bytes, peer_mac: bytes) -> bool:
        first, second = sorted([self.nonce, peer_nonce])
        want = _mac(self.secret, b"vade-control-1", first, second, self.peer_role, self.role)
        return hmac.compare_digest(want, peer_mac)


def admit(secret: bytes, a_role: str = "controller", b_role: str = "rank") -> bool:
    """Runs both sides in one process (self-test and documentation of the message order)."""
    a, b = Challenge(secret, a_role, b_role), Challenge(secret, b_role, a_role)
    return a.verify(b.nonce, b.respond(a.nonce)) and b.verify(a.nonce, a.respond(b.nonce))
