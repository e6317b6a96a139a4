"""Pipeline-parallel hand-over between layer stages over torch.distributed point-to-point.

A stage owns a contiguous interval of layers (parallel/plan.py).  fp32 residual rows
``[rows, hidden]`` cross each boundary unchanged; the last stage owns sampling and drafting
and tells every other stage what it decided (token rows, accept counts) so all stages run the
same passes.  On GPUs the sends are NCCL p2p on the current stream; on CPU they are gloo.
Parity: the reference's layer chain and its framed residual messages
(engine/crates/engine/src/flash/next_pp.rs:1-5,54-140).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class PipelineComm:
    def __init__(self, stage: int, stages: int, prev_rank: int | None, next_rank: int | None, last_rank: int,
                 group=None, int_device="cpu", first_rank: int = 0):
        self.stage, self.stages = stage, stages
        self.prev, self.next, self.last = prev_rank, next_rank, last_rank
        self.first = first_rank
        self.group = group
        self.int_device = int_device
        self.sent_bytes = 0

    def send_rows(self, x: torch.Tensor) -> None:
        x = x.contiguous()
        self.sent_bytes += x.numel() * x.element_size()
        dist.send(x, self.next)

    def recv_rows(self, rows: int, hidden: int, device) -> torch.Tensor:
        buf = torch.empty(rows, hidden, dtype=torch.float32, device=device)
        dist.recv(buf, self.prev)
        return buf

    def feed_back(self, tokens: torch.Tensor) -> None:
        """The last stage's chosen token rows reach the first stage (which embeds them next step) on the device,
        with no host round trip: capturable inside a CUDA graph."""
        if self.stages == 1:
            return
        if self.stage == self.stages - 1:
            dist.send(tokens, self.first)
        elif self.stage == 0:
            dist.recv(tokens, self.last)

    def broadcast_ints(self, values: list) -> list:
        """The last stage's list reaches every stage of this pipeline (length first, then values)."""
        n = torch.tensor([len(values)], dtype=torch.int64, device=self.int_device)
        dist.broadcast(n, self.last, group=self.group)
        buf = torch.tensor(list(values) if self.stage == self.stages - 1 else [0] * int(n), dtype=torch.int64,
                           device=self.int_device)
        dist.broadcast(buf, self.last, group=self.group)
        return [int(v) for v in buf.tolist()]
