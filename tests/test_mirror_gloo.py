"""Serving with tensor parallelism: the scheduler runs replicated on both ranks (gloo on CPU); the leader takes the
requests, the follower applies the leader's per-turn intake, and every chat gets its single-process ids."""
import os
import socket
import threading
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vade_b200.config import tiny_config
from vade_b200.runtime.build import build_engine
from vade_b200.runtime.sampler import Sampling
from vade_b200.runtime.scheduler import Request, Scheduler, SchedulerConfig


def _ids(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 4000, (n,), generator=g).tolist()


def _requests():
    return [Request(prompt=_ids(40, 1), max_tokens=8, ignore_eos=True),
            Request(prompt=_ids(130, 2), max_tokens=6, ignore_eos=True, sampling=Sampling(temperature=0.8, top_p=0.9, top_k=20, seed=7)),
            Request(prompt=_ids(75, 3), max_tokens=40, ignore_eos=True),                       # cancelled while it runs
            Request(prompt=_ids(66, 4), max_tokens=5, ignore_eos=True, cache=True),
            Request(prompt=_ids(66, 4) + _ids(20, 5), max_tokens=5, ignore_eos=True, cache=True)]   # resumes from the prefix above


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vade_b200.parallel.groups import make_parallel
    from vade_b200.runtime.mirror import Mirror
    par = make_parallel(tp=world, pp=1)
    eng = build_engine(tiny_config(), seed=0, tp=world, tp_rank=par.tp_rank, comm=par.comm, slots=4, max_seq=512, prefill_chunk=64)
    mirror = Mirror(keepalive_s=0.2)
    from vade_b200.runtime.mirror import AgreementError, startup_agreement
    agreed = startup_agreement(mirror.group, same={"config": "tiny", "draft_block": True}, least={"slots": 3 + rank, "pages": 100 - rank})
    assert agreed == {"slots": 3, "pages": 99}
    try:
        startup_agreement(mirror.group, same={"checkpoint": f"sha-{rank}"})
        raise SystemExit("ranks with different checkpoints were allowed to start")
    except AgreementError as e:
        assert "checkpoint" in str(e) and "rank 1" in str(e)
    sched = Scheduler(eng, SchedulerConfig(reserve_foreground=0, max_active=3, prefix_cache_entries=4), mirror=mirror)
    if rank != 0:
        sched.run_forever()                                  # returns when the leader publishes stop
        q.put((rank, sched.ticks, None))
    else:
        loop = threading.Thread(target=sched.run_forever, daemon=True)
        loop.start()
        reqs = _requests()
        for r in reqs[:4]:
            sched.submit(r)
        time.sleep(0.5)                                      # an idle stretch: keepalive messages only
        while reqs[2].state != "decode" or len(reqs[2].output) < 3:
            time.sleep(0.01)
        sched.cancel(reqs[2].id)
        while reqs[3].state != "done":
            time.sleep(0.01)
        sched.submit(reqs[4])
        while any(r.state != "done" for r in reqs):
            time.sleep(0.01)
        sched.stop()
        loop.join(60)
        q.put((rank, sched.ticks, [(list(r.output), r.finish_reason, r.cached_tokens) for r in reqs]))
    dist.barrier()
    dist.destroy_process_group()


def test_mirrored_scheduler_on_two_tensor_parallel_ranks_gives_single_process_ids():
    eng = build_engine(tiny_config(), seed=0, slots=4, max_seq=512, prefill_chunk=64)
    solo = []
    for r in _requests():
        s = Scheduler(eng, SchedulerConfig(reserve_foreground=0))
        s.submit(r)
        while r.state != "done":
            if not s.tick():
                s._reap()
        solo.append(list(r.output))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    outs = {r: (ticks, res) for r, ticks, res in (q.get(timeout=300) for _ in range(2))}
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    res = outs[0][1]
    assert outs[0][0] == outs[1][0], "the follower ran a different number of turns than the leader"
    for i in (0, 1, 3, 4):
        assert res[i][0] == solo[i] and res[i][1] == "length"
    assert res[2][1] == "cancelled" and res[2][0] == solo[2][:len(res[2][0])] and len(res[2][0]) < 40
    assert res[4][2] == 64, "the second chat did not resume from the retained prefix"
