"""Batch-invariant seeded sampler.

A draw is a pure function of (logits row, sampling options, seed, absolute position): no RNG
state is consumed, so replaying, batching or re-ordering requests never changes a token.
Pipeline: penalties -> greedy shortcut (ties to the lowest id) -> top-k -> weights
exp((logit - best) / T) in float64 -> top-p over the canonical order (descending weight, then
ascending id) -> min-p -> inverse-CDF draw with u = uniform(seed, position), a SplitMix64
finaliser over the position mixed with the seed.
Parity: engine/crates/engine/src/sample.rs:4-16 (options), 83-94 (uniform), 96-157 (order,
nucleus, min-p); docs/sampling.md:27-79.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict

import torch

_M64 = (1 << 64) - 1


def _mix(x: int) -> int:
    x &= _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform(seed: int, position: int) -> float:
    """Position-keyed draw in [0, 1): the top 53 bits of mix(seed ^ mix(position + golden))."""
    return (_mix((seed & _M64) ^ _mix((position + 0x9E3779B97F4A7C15) & _M64)) >> 11) * (1.0 / 9007199254740992.0)


@dataclass
class Sampling:
    temperature: float = 0.0
    top_k: int = 0                  # 0 disables
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = 0

    def validate(self) -> None:
        import math
        ok = (math.isfinite(self.temperature) and self.temperature >= 0.0
              and math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0
              and 0.0 <= self.min_p <= 1.0 and self.top_k >= 0
              and math.isfinite(self.repetition_penalty) and self.repetition_penalty > 0.0
              and -2.0 <= self.presence_penalty <= 2.0 and -2.0 <= self.frequency_penalty <= 2.0)
        if not ok:
            raise ValueError("invalid sampling parameters")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def plain_greedy(self) -> bool:
        """Greedy with no history-dependent penalty: the device argmax path is exact."""
        return (self.greedy and self.repetition_penalty == 1.0 and self.presence_penalty == 0.0
                and self.frequency_penalty == 0.0)

    def echo(self) -> dict:
        return asdict(self)


def apply_penalties(logits: torch.Tensor, history: list, s: Sampling) -> torch.Tensor:
    if (s.repetition_penalty == 1.0 and s.presence_penalty == 0.0 and s.frequency_penalty == 0.0) or not history:
        return logits
    out = logits.clone()
    ids, counts = torch.unique(torch.tensor(history, dtype=torch.int64), return_counts=True)
    v = out[ids]
    if s.repetition_penalty != 1.0:
        v = torch.where(v > 0, v / s.repetition_penalty, v * s.repetition_penalty)
    v = v - s.presence_penalty - s.frequency_penalty * counts.to(v.dtype)
    out[ids] = v
    return out


def candidates(logits: torch.Tensor, s: Sampling):
    """Filtered support in canonical order with unnormalised float64 weights: (ids, weights)."""
    l64 = logits.to(torch.float64)
    n = l64.numel()
    idx = torch.arange(n, dtype=torch.int64)
    # canonical order: descending logit, ascending id among equals (stable sort of a descending key)
    order = torch.sort(l64, descending=True, stable=True).indices
    if s.top_k and s.top_k < n:
        order = order[:s.top_k]
    w = torch.exp((l64[order] - l64[order[0]]) / s.temperature)
    if s.top_p < 1.0:
        total = float(w.sum())
        c = torch.cumsum(w, 0)
        keep = int(torch.searchsorted(c, torch.tensor(s.top_p * total, dtype=torch.float64), right=False)) + 1
        keep = max(1, min(keep, w.numel()))
        order, w = order[:keep], w[:keep]
    if s.min_p > 0.0:
        m = w >= s.min_p
        order, w = order[m], w[m]
    return idx[order], w


def candidates_from_topk(vals: torch.Tensor, ids: torch.Tensor, s: Sampling):
    """The same filtered support as ``candidates`` when the row's top_k best logits are already known in
    canonical order (vals descending, ids ascending among equals): identical float64 arithmetic on k values."""
    l64 = vals.detach().cpu().to(torch.float64)
    ids = ids.detach().cpu().to(torch.int64)
    w = torch.exp((l64 - l64[0]) / s.temperature)
    if s.top_p < 1.0:
        total = float(w.sum())
        c = torch.cumsum(w, 0)
        keep = int(torch.searchsorted(c, torch.tensor(s.top_p * total, dtype=torch.float64), right=False)) + 1
        keep = max(1, min(keep, w.numel()))
        ids, w = ids[:keep], w[:keep]
    if s.min_p > 0.0:
        m = w >= s.min_p
        ids, w = ids[m], w[m]
    return ids, w


def compact_ok(s: Sampling, vocab: int) -> bool:
    """The compact device top-k path gives exactly the full path's draw: top_k in 1..64 and no penalty that
    could reorder the candidates."""
    return (not s.greedy and 0 < s.top_k <= 64 and s.top_k < vocab and s.repetition_penalty == 1.0
            and s.presence_penalty == 0.0 and s.frequency_penalty == 0.0)


def sample_compact(vals: torch.Tensor, ids: torch.Tensor, s: Sampling, position: int) -> int:
    cid, w = candidates_from_topk(vals, ids, s)
    return draw(cid, w, uniform(s.seed, position))


def draw(ids: torch.Tensor, w: torch.Tensor, u: float) -> int:
    mass = float(w.sum())
    if not (mass > 0.0) or mass != mass or mass == float("inf"):
        raise ValueError("empty sampling distribution")
    target = u * mass
    c = 0.0
    for i, wi in zip(ids.tolist(), w.tolist()):
        c += wi
        if target < c:
            return i
    return int(ids[-1])


def sample(logits: torch.Tensor, s: Sampling, position: int, history: list | None = None) -> int:
    """One token for one row of fp32 logits at absolute ``position``."""
    logits = apply_penalties(logits.detach().float().cpu(), history or [], s)
    if s.greedy:
        m = logits.max()
        return int(torch.nonzero(logits == m)[0, 0])
    ids, w = candidates(logits, s)
    return draw(ids, w, uniform(s.seed, position))
