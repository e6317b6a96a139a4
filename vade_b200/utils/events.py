"""Best-effort event counters and the last 64 log lines, exposed at ``GET /v1/events`` and inside
``/health``.  Fixed memory, lock-protected, never raises into the caller.
Parity: engine/crates/base/src/events.rs:1-80 (note, counts_json)."""
from __future__ import annotations

import json
import sys
import threading
import time
from collections import deque

_lock = threading.Lock()
_counts: dict = {}
_lines: deque = deque(maxlen=64)
_t0 = time.time()


def note(name: str, detail: str | None = None) -> None:
    with _lock:
        _counts[name] = _counts.get(name, 0) + 1
        if detail is not None:
            _lines.append(f"{time.time() - _t0:.3f} {name} {detail}")


def log(first_word: str, **fields) -> None:
    """Structured ``key=value`` stderr line with a stable first word."""
    line = first_word + "".join(f" {k}={v}" for k, v in fields.items())
    with _lock:
        _lines.append(f"{time.time() - _t0:.3f} {line}")
    print(line, file=sys.stderr, flush=True)


def counts() -> dict:
    with _lock:
        return dict(_counts)


def lines() -> list:
    with _lock:
        return list(_lines)


def counts_json() -> str:
    return json.dumps({"uptime_s": round(time.time() - _t0, 3), "counts": counts(), "lines": lines()})


def reset() -> None:
    with _lock:
        _counts.clear()
        _lines.clear()
