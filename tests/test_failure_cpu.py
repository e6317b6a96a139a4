"""Failure detection without a GPU fault: every failure is made on the host (a rank that stops beating, a
reported error, a wait past its deadline on a manual clock)."""
import os
import socket

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from vade_b200.parallel.health import Challenge, DictStore, Heartbeat, PeerLost, admit
from vade_b200.runtime.watchdog import Watchdog
from vade_b200.utils import events
from vade_b200.utils.profile import CollectiveProfiler, kernel_class


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_watchdog_expires_on_a_manual_clock_and_ends_after_the_grace_period():
    clk, fired = Clock(), []
    wd = Watchdog(timeout_s=10, clock=clk, on_expire=fired.append, start_thread=False)
    with wd.wait("token read-back"):
        clk.t = 9.0
        assert not wd.check() and not wd.failed
        clk.t = 11.0
        assert not wd.check()                  # expired now, process ends only after the grace period
        assert wd.failed and wd.expired[0] == "token read-back"
        clk.t = 11.0 + 4.4
        assert not wd.check()
        clk.t = 11.0 + 4.6
        assert wd.check()
    assert events.counts().get("gpu_wait_expired", 0) >= 1


def test_watchdog_closed_waits_never_expire():
    clk = Clock()
    wd = Watchdog(timeout_s=1, clock=clk, on_expire=lambda e: None, start_thread=False)
    with wd.wait("short"):
        clk.t = 0.5
    clk.t = 100.0
    assert not wd.check() and not wd.failed


def test_heartbeat_silent_peer_and_sticky_failure():
    store, clk = DictStore(), Clock()
    a = Heartbeat(store, 0, 2, limit_s=2.0, clock=clk)
    b = Heartbeat(store, 1, 2, limit_s=2.0, clock=clk)
    assert a.period == 0.5
    for step in range(8):                      # both alive: no error however long it runs
        clk.t += 0.6
        a.check()
        b.check()
    for step in range(4):                      # b stops between steps; a keeps checking (last change seen at +0.6)
        clk.t += 0.6
        a.check()
    clk.t += 0.6
    with pytest.raises(PeerLost) as e:
        a.check()
    assert e.value.rank == 1 and "silent" in e.value.reason
    with pytest.raises(PeerLost):              # sticky: the group stays refused
        a.check()


def test_heartbeat_reported_failure_reaches_every_rank():
    store, clk = DictStore(), Clock()
    hs = [Heartbeat(store, r, 3, limit_s=5.0, clock=clk) for r in range(3)]
    for h in hs:
        h.check()
    hs[2].fail("routing rejected a row")
    for r in (0, 1):
        with pytest.raises(PeerLost) as e:
            hs[r].check()
        assert e.value.rank == 2 and "routing rejected" in e.value.reason


def test_peer_admission_binds_roles_and_nonces():
    secret = b"0123456789abcdef-secret"
    assert admit(secret)
    a, b = Challenge(secret, "controller", "rank"), Challenge(secret, "rank", "controller")
    mac_b = b.respond(a.nonce)
    assert a.verify(b.nonce, mac_b)
    assert not a.verify(b.nonce, mac_b[:-1] + bytes([mac_b[-1] ^ 1]))
    other = Challenge(secret, "controller", "rank")          # a reply cannot be replayed into another session
    assert not other.verify(b.nonce, mac_b)
    wrong_role = Challenge(secret, "gateway", "controller")  # nor does a different role pass
    assert not a.verify(wrong_role.nonce, wrong_role.respond(a.nonce))
    assert not Challenge(b"another-secret-of-16B", "rank", "controller").verify(a.nonce, a.respond(b.nonce))
    with pytest.raises(ValueError):
        Challenge(b"short", "a", "b")


def test_collective_profiler_buckets_and_kernel_classes():
    p = CollectiveProfiler()
    for ns in [1000] * 98 + [1_000_000] * 2:
        p.note("gather", "nccl", ns, 4096)
    (r,) = p.report()
    assert r["count"] == 100 and r["bytes"] == 409600
    assert 1.0 <= r["p50_us_upper"] <= 1.1 and 1000.0 <= r["p99_us_upper"] <= 1100.0
    p.note("nonsense", "nccl", 5, 1)                          # unknown kinds are ignored, never an error
    assert kernel_class("void vade::rows_mma_kernel<1, 1, false>(...)") == "dense"
    assert kernel_class("vade::gdn_scan_kernel<2, true>") == "gdn"
    assert kernel_class("vade::router_rows_kernel<1, 16>") == "experts"
    assert kernel_class("vade::attn_split_kernel") == "attention"
    assert kernel_class("memcpy32_post") == "other_gpu"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _report(q, msg, code):
    q.put(msg)
    q.close()
    q.join_thread()          # the feeder thread must flush before the process ends
    os._exit(code)


def _rank(rank, world, port, q):
    """Two gloo ranks step together; rank 1 leaves BETWEEN steps (no collective in flight).  Rank 0 learns of it
    from the store before its next collective and stops instead of hanging in it."""
    import time
    import torch
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.TCPStore("127.0.0.1", port + 1, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, limit_s=1.0)
    steps = 0
    try:
        for step in range(50):
            if rank == 1 and step == 3:
                _report(q, (rank, "left", steps), 0)          # between steps: nothing in flight
            hb.step_barrier(step)                             # host rendezvous: never enter a collective a peer will not join
            t = torch.ones(4)
            dist.all_reduce(t)
            assert float(t[0]) == world
            steps += 1
        _report(q, (rank, "never noticed", steps), 1)
    except PeerLost as e:
        _report(q, (rank, f"lost rank {e.rank}", steps), 0)


def test_rank_leaving_between_steps_is_detected_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        r, what, steps = q.get(timeout=60)
        got[r] = (what, steps)
    for p in procs:
        p.join(20)
    assert got[1] == ("left", 3)
    assert got[0] == ("lost rank 1", 3), got               # three full steps, then a clean stop on the host
