"""Per-kernel micro-benchmark with a correctness gate and a roofline score.

    python -m vade_b200.cli.kernel_bench [--case NAME ...] [--iters N] [--json]

Each case builds the operands of one hot kernel at the shapes of the 80B-A3B configuration,
refuses to time it unless its output agrees with the plain PyTorch statement of the op, then times
it with CUDA events (warm-up, L2 flushed between iterations by writing a 256 MB buffer) and reports
the compulsory bytes / FLOPs, the achieved rate and the fraction of the measured peaks in
``MEASURED_PEAKS.json`` (6.65 TB/s and 1.59 PFLOP/s when that file is absent).
Parity: the reference's paired ``kernel-bench`` with its byte-equality precheck and as-stored
floor model (engine/tools/bench/src/kernel_floor.rs:7-60).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..config import qwen3_next_80b_config
from ..models import weights as W
from ..ops import reference as R

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> dict:
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Timer:
    def __init__(self, device):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def time(self, fn, iters: int, warmup: int = 3) -> float:
        """Median milliseconds of fn() with the L2 flushed before every timed call."""
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]


def _rand_q(n, k, dev, e=0):
    gen = torch.Generator(device=dev).manual_seed(7)
    lead = (e,) if e else ()
    packed = torch.randint(0, 256, (*lead, n, k // 2), dtype=torch.uint8, device=dev, generator=gen)
    scale = torch.randint(0x28, 0x38, (*lead, n, k // 16), dtype=torch.uint8, device=dev, generator=gen)
    rs = torch.full((*lead, n), 0.01, dtype=torch.float32, device=dev)
    return W.QLinear(n, k, "nvfp4", packed=packed, scale=scale, row_scale=rs, tiles=W.pack_tiles(packed, scale), e=e)


def case_gemm(ops, name, n, k, T, ranges=1, plain=False):
    dev = ops.device
    if plain:
        w = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)
        q = W.QLinear(n, k, "plain", w=w, row_scale=torch.ones(n, device=dev))
        wbytes = n * k * 2
    else:
        q = _rand_q(n, k, dev)
        wbytes = n * k // 2 + n * k // 16
    x = torch.randn(T, k, device=dev).to(torch.bfloat16)
    if ranges > 1:
        fn = lambda: ops.linear_ranges(x, q, ranges)
        got = fn().sum(0)
    else:
        fn = lambda: ops.linear(x, q, out_fp32=True)
        got = fn()
    rows = min(n, 512)
    ref = R.dot_rows(x.float(), q.dense()[:rows]) * q.row_scale[:rows]
    ok = torch.allclose(got[:, :rows], ref, rtol=2e-3, atol=2e-3 * float(ref.abs().max()))
    nbytes = wbytes + T * k * 2 + T * n * 4 * ranges
    return name, fn, ok, nbytes, 2.0 * n * k * T


CASES = {
    "gemm_gdn_in_proj_decode": lambda ops: case_gemm(ops, "NVFP4 12352x2048, 1 row", 12352, 2048, 1),
    "gemm_qkv_decode": lambda ops: case_gemm(ops, "NVFP4 9216x2048, 1 row", 9216, 2048, 1),
    "gemm_out_proj_decode": lambda ops: case_gemm(ops, "NVFP4 2048x4096, 8 ranges, 1 row", 2048, 4096, 1, ranges=8),
    "gemm_lm_head_decode": lambda ops: case_gemm(ops, "bf16 151936x2048, 1 row", 151936, 2048, 1, plain=True),
    "gemm_gdn_in_proj_prefill": lambda ops: case_gemm(ops, "NVFP4 12352x2048, 2048 rows", 12352, 2048, 2048),
    "gemm_out_proj_prefill": lambda ops: case_gemm(ops, "NVFP4 2048x4096, 8 ranges, 2048 rows", 2048, 4096, 2048, ranges=8),
}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--case", action="append", help="case name (default: all); see --list")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    if args.list:
        print("\n".join(CASES))
        return
    from ..ops.cuda import CudaOps
    dev = torch.device("cuda:0")
    ops = CudaOps(qwen3_next_80b_config(), dev)
    pk = peaks()
    timer = Timer(dev)
    results = []
    for key in (args.case or list(CASES)):
        name, fn, ok, nbytes, flops = CASES[key](ops)
        ops.check_status()
        if not ok:
            results.append({"case": key, "error": "output differs from the PyTorch statement; not timed"})
            print(f"{key:32s} MISMATCH (not timed)")
            continue
        ms = timer.time(fn, args.iters)
        gbs = nbytes / ms / 1e6
        tfl = flops / ms / 1e9
        frac = max(gbs / pk["hbm_gbs"], tfl / pk["bf16_tflops"])
        results.append({"case": key, "what": name, "ms": round(ms, 4), "gb_s": round(gbs, 1), "tflops": round(tfl, 2),
                        "fraction_of_peak": round(frac, 4), "peaks": pk["source"]})
        print(f"{key:32s} {ms * 1e3:9.1f} us  {gbs:8.1f} GB/s  {tfl:8.2f} TFLOP/s  {100 * frac:5.1f}% of {pk['source']} peak  [{name}]")
    if args.json:
        print(json.dumps(results))


if __name__ == "__main__":
    main()
