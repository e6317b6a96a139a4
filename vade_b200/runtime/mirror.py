"""Serving on several GPUs: every rank runs the same scheduler on the same inputs.

With tensor + expert parallelism every rank must run the same passes over the same rows.  Instead of a command
protocol per engine call, the whole scheduler is replicated: rank 0 (the leader) owns the HTTP front end and, at the
start of every scheduler turn, publishes what changed since the last one (new requests, cancellations, expired
deadlines, cache releases, stop); the followers apply the same message and then run the same turn.  Everything else
the scheduler decides from is identical on every rank by construction: the token ids (the exchanges give every rank
the same bits), the page ledger, the prefix cache, the adaptive draft depth (a function of the request's own
acceptance history).  Nothing time-dependent is decided on a follower.

The message travels as one pickled object over a host-side (gloo) group, so the device streams carry model traffic
only.  An idle leader publishes an empty message every few seconds, so a follower's blocking receive never meets the
group's timeout, and a follower that stops hearing from the leader fails there instead of hanging for good.
Parity: the reference's rank-0 scheduler with mirroring workers (engine/crates/tp/src/flash/next_batched_service.rs:
13-200 `run_back`, engine/crates/tp/src/flash/service.rs worker loop, tp/src/transport.rs:4-25 commands).
"""
from __future__ import annotations

import time

import torch.distributed as dist


class Mirror:
    def __init__(self, group=None, leader_rank: int = 0, keepalive_s: float = 5.0):
        """``group``: a host-side process group of all serving ranks (gloo); None = a new gloo group over all ranks."""
        self.group = group if group is not None else dist.new_group(backend="gloo")
        self.leader_rank = leader_rank
        self.leader = dist.get_rank() == leader_rank
        self.keepalive_s = keepalive_s
        self.last = time.monotonic()
        self.published = 0

    def keepalive_due(self) -> bool:
        return time.monotonic() - self.last >= self.keepalive_s

    def publish(self, msg: dict) -> None:
        dist.broadcast_object_list([msg], src=self.leader_rank, group=self.group)
        self.last = time.monotonic()
        self.published += 1

    def receive(self) -> dict:
        box = [None]
        dist.broadcast_object_list(box, src=self.leader_rank, group=self.group)
        return box[0]


class AgreementError(RuntimeError):
    pass


def startup_agreement(group, same: dict, least: dict | None = None) -> dict:
    """Every serving rank publishes what it loaded before the first pass; the job starts only if they agree.

    ``same``: values that must be equal on every rank (checkpoint fingerprint, model dimensions, weight format, draft
    block present, kernel build stamp, switches that change arithmetic).  ``least``: capacities of which the job takes
    the minimum over ranks (sequence slots, KV pages, context), so that every rank admits exactly the same requests.
    Returns the agreed capacities.  A mismatch raises the same error on every rank, naming the key and the ranks.
    Parity: engine/crates/tp/src/bin/flash-serve.rs:385-390,416-424,460-477 (precision / MTP bytes, residency flags
    and limits gathered at start-up), engine/crates/tp/src/startup_pool.rs (`agree`: least session count and pool)."""
    least = least or {}
    box = [None] * dist.get_world_size(group)
    dist.all_gather_object(box, {"same": same, "least": least}, group=group)
    for key in sorted(box[0]["same"]):
        vals = [b["same"].get(key) for b in box]
        if any(v != vals[0] for v in vals):
            raise AgreementError(f"ranks disagree on {key}: " + ", ".join(f"rank {i}: {v!r}" for i, v in enumerate(vals)))
    if any(set(b["same"]) != set(box[0]["same"]) or set(b["least"]) != set(box[0]["least"]) for b in box):
        raise AgreementError("ranks published different sets of start-up keys")
    return {key: min(b["least"][key] for b in box) for key in box[0]["least"]}
