"""Switch-gated profiling: device time per kernel and per kernel class, fixed-storage collective histograms.

Nothing here changes arithmetic and nothing runs unless a switch asks for it:

``VADE_PROFILE=1``             per-pass CUDA-event timing lines (``pass_profile`` context manager)
``VADE_DECODE_PROFILE=gpu``    per-kernel device time of decode steps, classified by kernel NAME into
                               dense / gdn / attention / experts / head / norm / other (``step_profile``)
``VADE_PROFILE_COLLECTIVES=1`` per (kind x path) count, bytes and p50/p99 upper bounds from 256 log
                               buckets, fixed memory, no allocation per sample (``CollectiveProfiler``)

Parity: gpu/src/next_profile.rs:5-40 (kernel-name -> class map), gpu/src/decode_profile.rs:1-30 (event
attribution), fabric/src/profile.rs:20-57,115-264 (bounded collective profiler).
"""
from __future__ import annotations

import collections
import contextlib
import math
import sys
import time

from .env import flag, choice

#: first match wins; a kernel's class is a pure function of its name
KERNEL_CLASSES = (
    ("experts", ("route", "router_rows", "combine_add_norm", "swiglu", "gather_rows")),
    ("gdn", ("gdn_",)),
    ("attention", ("attn_",)),
    ("head", ("argmax", "embed_kernel")),
    ("norm", ("fold_add_norm", "rmsnorm")),
    ("dense", ("umma_gemm", "rows_mma")),
)


def kernel_class(name: str, grouped: bool = False) -> str:
    low = name.lower()
    for cls, keys in KERNEL_CLASSES:
        if any(k in low for k in keys):
            return cls
    return "other_gpu"


def profile_enabled() -> bool:
    return flag("VADE_PROFILE", False)


def decode_profile_enabled() -> bool:
    return choice("VADE_DECODE_PROFILE", ("off", "gpu"), "off") == "gpu"


def collectives_enabled() -> bool:
    return flag("VADE_PROFILE_COLLECTIVES", False)


@contextlib.contextmanager
def pass_profile(label: str, rows: int, stream=None, out=sys.stderr):
    """CUDA-event time of one pass, printed as a key=value line, only when VADE_PROFILE=1."""
    if not profile_enabled():
        yield
        return
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record(stream)
    try:
        yield
    finally:
        e1.record(stream)
        e1.synchronize()
        print(f"pass_profile label={label} rows={rows} device_ms={e0.elapsed_time(e1):.3f} "
              f"host_ms={(time.perf_counter() - t0) * 1e3:.3f}", file=out)


def device_profile(fn, repeats: int = 1) -> dict:
    """Runs fn() `repeats` times under the CUDA activity profiler and returns
    {"total_us", "kernels": [(name, calls, total_us)], "classes": {class: us}} per repeat."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(repeats):
            fn()
        torch.cuda.synchronize()
    agg = collections.OrderedDict()
    for ev in prof.events():
        if "cuda" not in str(ev.device_type).lower():
            continue
        a = agg.setdefault(ev.name, [0, 0.0])
        a[0] += 1
        a[1] += ev.device_time
    kernels = sorted(((n, c / repeats, t / repeats) for n, (c, t) in agg.items()), key=lambda r: -r[2])
    classes = collections.OrderedDict()
    for n, _, t in kernels:
        classes[kernel_class(n)] = classes.get(kernel_class(n), 0.0) + t
    return {"total_us": sum(t for _, _, t in kernels), "kernels": kernels, "classes": classes}


def format_profile(title: str, p: dict, top: int = 24) -> str:
    lines = [f"{title}: {p['total_us']:.1f} us of device time in {sum(c for _, c, _ in p['kernels']):.0f} launches"]
    lines.append("  by class: " + ", ".join(f"{k} {v:.1f} us ({100 * v / max(p['total_us'], 1e-9):.0f}%)" for k, v in
                                            sorted(p["classes"].items(), key=lambda kv: -kv[1])))
    for n, c, t in p["kernels"][:top]:
        lines.append(f"  {t:10.1f} us  {c:6.0f} x {t / max(c, 1e-9):9.2f} us  [{kernel_class(n)}] {n[:110]}")
    return "\n".join(lines)


class CollectiveProfiler:
    """Fixed-storage latency histograms per (kind, path): 256 log2/8 buckets of nanoseconds, counts and bytes.
    ``note`` never allocates; ``report`` gives upper bounds of the p50/p99 buckets."""

    BUCKETS = 256

    def __init__(self, kinds=("gather", "reduce", "send", "recv", "broadcast", "exchange"), paths=("nccl", "gloo", "peer")):
        self.keys = [(k, p) for k in kinds for p in paths]
        self.index = {kp: i for i, kp in enumerate(self.keys)}
        n = len(self.keys)
        self.hist = [[0] * self.BUCKETS for _ in range(n)]
        self.count = [0] * n
        self.bytes = [0] * n
        self.wait_ns = [0] * n

    @staticmethod
    def bucket(ns: int) -> int:
        if ns < 1:
            return 0
        return min(CollectiveProfiler.BUCKETS - 1, int(math.log2(ns) * 8))

    @staticmethod
    def upper_ns(bucket: int) -> float:
        return 2.0 ** ((bucket + 1) / 8.0)

    def note(self, kind: str, path: str, ns: int, nbytes: int, wait_ns: int = 0) -> None:
        i = self.index.get((kind, path))
        if i is None:
            return
        self.hist[i][self.bucket(ns)] += 1
        self.count[i] += 1
        self.bytes[i] += nbytes
        self.wait_ns[i] += wait_ns

    def _pct(self, i: int, q: float) -> float:
        want, seen = q * self.count[i], 0
        for b, c in enumerate(self.hist[i]):
            seen += c
            if seen >= want and c:
                return self.upper_ns(b)
        return 0.0

    def report(self) -> list:
        out = []
        for i, (k, p) in enumerate(self.keys):
            if self.count[i]:
                out.append({"kind": k, "path": p, "count": self.count[i], "bytes": self.bytes[i],
                            "p50_us_upper": self._pct(i, 0.50) / 1e3, "p99_us_upper": self._pct(i, 0.99) / 1e3,
                            "wait_ms": self.wait_ns[i] / 1e6})
        return out

    def lines(self) -> list:
        return [f"collective_profile kind={r['kind']} path={r['path']} count={r['count']} bytes={r['bytes']} "
                f"p50_us<={r['p50_us_upper']:.1f} p99_us<={r['p99_us_upper']:.1f} wait_ms={r['wait_ms']:.2f}" for r in self.report()]


_collectives = None


def collectives() -> CollectiveProfiler | None:
    """The process-wide profiler when VADE_PROFILE_COLLECTIVES=1, else None (callers skip all work)."""
    global _collectives
    if _collectives is None and collectives_enabled():
        _collectives = CollectiveProfiler()
    return _collectives
