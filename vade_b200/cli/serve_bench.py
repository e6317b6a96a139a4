"""Continuous-batching serving load on one engine: N concurrent requests through the scheduler, seeded sampling,
aggregate output tokens per second, TTFT percentiles, and a check that sampled requests reproduce their solo run.

    python -m vade_b200.cli.serve_bench [--config qwen3-next-80b-a3b] [--requests 64] [--min-prompt 512] [--max-prompt 4096]
                                        [--output 256] [--temperature 0.7] [--top-p 0.95] [--top-k 0] [--check 4] [--max-active 16]
    python -m vade_b200.cli.serve_bench --step-times          # device time of the pooled decode step at widths 1..16

Prompt lengths are uniform on [min, max] from seed 2, token ids uniform-random, every request carries its own sampler
seed.  All requests are submitted at time zero; TTFT is measured from submission to the first emitted token, so it
includes the time a request waits in the queue behind earlier prompts.  ``--check K`` re-runs the first K requests
alone afterwards and compares ids (the batch-invariance of the sampler and of the decode class under load).
Parity: the reference's outside-in serving benchmark (engine/tools/bench/README.md:24-70: TTFT, decode rate, cohorts).
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def run(engine, n_requests: int, min_prompt: int, max_prompt: int, n_out: int, temperature: float, top_p: float, check: int,
        max_active: int, out=print, top_k: int = 0) -> dict:
    from ..runtime.sampler import Sampling
    from ..runtime.scheduler import Request, Scheduler, SchedulerConfig
    V = engine.model.cfg.vocab_size
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(min_prompt, max_prompt + 1, (n_requests,), generator=g).tolist()
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]

    def make(i):
        samp = Sampling(temperature=temperature, top_p=top_p, top_k=top_k, seed=1000 + i) if temperature > 0 else Sampling()
        return Request(prompt=list(prompts[i]), max_tokens=n_out, ignore_eos=True, sampling=samp)

    sched = Scheduler(engine, SchedulerConfig(reserve_foreground=0, max_active=max_active, max_queue=max(256, n_requests)))
    if engine.device.type == "cuda":
        torch.cuda.synchronize()
    t0 = time.monotonic()
    reqs = [sched.submit(make(i)) for i in range(n_requests)]
    while any(r.state != "done" for r in reqs):
        if not sched.tick():
            sched._reap()
    if engine.device.type == "cuda":
        torch.cuda.synchronize()
    wall = time.monotonic() - t0
    bad = [r for r in reqs if r.finish_reason != "length" or len(r.output) != n_out]
    ttft = sorted((r.first_token_at - r.created) for r in reqs if r.first_token_at is not None)
    pct = lambda q: ttft[min(len(ttft) - 1, int(q * len(ttft)))] if ttft else float("nan")
    total_out = sum(len(r.output) for r in reqs)
    res = {"requests": n_requests, "prompt_tokens": sum(lens), "output_tokens": total_out, "wall_s": round(wall, 3),
           "output_tok_s": round(total_out / wall, 1), "total_tok_s": round((total_out + sum(lens)) / wall, 1),
           "ttft_p50_s": round(pct(0.50), 3), "ttft_p99_s": round(pct(0.99), 3), "incomplete": len(bad),
           "max_active": max_active, "captured_steps": getattr(sched.pool, "replays", 0) if sched.pool is not None else 0,
           "sampling": {"temperature": temperature, "top_p": top_p, "top_k": top_k}}
    same = 0
    for i in range(min(check, n_requests)):
        solo = Scheduler(engine, SchedulerConfig(reserve_foreground=0))
        r = solo.submit(make(i))
        while r.state != "done":
            if not solo.tick():
                solo._reap()
        same += int(list(r.output) == list(reqs[i].output))
    res["solo_checked"] = min(check, n_requests)
    res["solo_identical"] = same
    out(json.dumps(res))
    return res


def step_times(engine, out=print, rows: int = 16, prompt: int = 1024) -> dict:
    """Device time of the pooled decode step at every captured width (CUDA events over 20 replays after 3 warm-up
    replays), on ``rows`` sequences prefilled with prompts of ``prompt`` + 64 i tokens."""
    from ..runtime.engine import Sequence
    V = engine.model.cfg.vocab_size
    g = torch.Generator().manual_seed(3)
    seqs = [Sequence(engine.cache.new_slot()) for _ in range(rows)]
    items = [(s, torch.randint(0, V, (prompt + 64 * i,), generator=g).tolist(), False) for i, s in enumerate(seqs)]
    for k in range(0, rows, 4):
        engine.prefill_many(items[k:k + 4])
    pool = engine.decode_pool()
    res = {}
    for w in pool.WIDTHS:
        if w > rows:
            break
        sl, pos, tok = [s.slot for s in seqs[:w]], [len(s.tokens) for s in seqs[:w]], [5 + i for i in range(w)]
        for _ in range(3):
            pool.step(sl, tok, pos)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(20):
            pool.step(sl, tok, [p + i + 1 for p in pos])
        e1.record()
        torch.cuda.synchronize()
        res[w] = round(e0.elapsed_time(e1) / 20, 3)
    for s in seqs:
        engine.cache.free_slot(s.slot)
    out(json.dumps({"decode_step_ms_by_width": res}))
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", default="qwen3-next-80b-a3b")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--min-prompt", type=int, default=512)
    ap.add_argument("--max-prompt", type=int, default=4096)
    ap.add_argument("--output", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--top-k", type=int, default=0, help="1..64 takes the compact device top-k path; 0 reads the whole logits row per sampled token")
    ap.add_argument("--check", type=int, default=4)
    ap.add_argument("--max-active", type=int, default=16)
    ap.add_argument("--step-times", action="store_true", help="GPU: only time the pooled decode step at every captured width")
    a = ap.parse_args(argv)
    from ..config import NAMED_CONFIGS
    from ..runtime.build import build_engine
    cfg = NAMED_CONFIGS[a.config]("nvfp4") if a.config in ("qwen3-next-80b-a3b", "hybrid-200b") else NAMED_CONFIGS[a.config]()
    on_gpu = a.device.startswith("cuda")
    eng = build_engine(cfg, device=a.device, slots=a.max_active + 2, max_seq=a.max_prompt + a.output + 64, synth_on_device=on_gpu,
                       with_mtp=False, prefill_chunk=2048 if on_gpu else 64)
    if a.step_times:
        step_times(eng, rows=a.max_active)
        eng.model.ops.check_status()
        return 0
    res = run(eng, a.requests, a.min_prompt, a.max_prompt, a.output, a.temperature, a.top_p, a.check, a.max_active, top_k=a.top_k)
    if on_gpu:
        eng.model.ops.check_status()
    return 0 if res["incomplete"] == 0 and res["solo_identical"] == res["solo_checked"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
