"""Plain PyTorch fp32 statements of every op of the hybrid model.

These functions are the oracle of the CUDA kernels (GPU tests compare each kernel with the
function of the same name here) and the execution path of CPU runs.  They are written from
the model math of the reference's fp32 CPU decoder (engine/crates/model/src/flash/refcpu.rs:
72-94 rms_group, 283-300 rope, 338-418 full attention, 453-529 gdn_token, 719-841 MoE) but in
batch form over ragged rows; every reduction that a kernel must reproduce bit for bit
(ordered expert fold, range tree fold) is spelled out in its fixed order.

Rounding: ``act`` is the storage type of activations between ops (torch.bfloat16 on GPU
configurations, torch.float32 for the fp32 CPU configuration).  Sums are fp32.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _round(x: torch.Tensor, act: torch.dtype) -> torch.Tensor:
    return x.to(act).to(torch.float32) if act != torch.float32 else x


# ------------------------------------------------------------------ dot products
def dot_rows(x: torch.Tensor, w: torch.Tensor, block: int = 512) -> torch.Tensor:
    """y[t, n] = sum_k x[t, k] * w[n, k] in fp32.  On CPU each output is one inner-dimension
    reduction whose order depends on K only, never on how many rows or columns are computed
    beside it, so a rank that owns a slice of the rows of ``w`` gets the bits of the unsplit
    product.  On GPU this is the fp32 comparison value for tensor-core kernels."""
    x = x.to(torch.float32)
    w = w.to(torch.float32)
    if x.is_cuda:
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            return x @ w.t()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
    t, k = x.shape
    n = w.shape[0]
    out = torch.empty(t, n, dtype=torch.float32)
    step = max(1, min(n, (1 << 24) // max(1, t * k)))
    step = min(step, block)
    for n0 in range(0, n, step):
        out[:, n0:n0 + step] = (x.unsqueeze(1) * w[n0:n0 + step].unsqueeze(0)).sum(-1)
    return out


def fold_tree(parts: torch.Tensor) -> torch.Tensor:
    """Fixed balanced pair tree over the leading dimension: ((p0+p1)+(p2+p3))+((p4+p5)+(p6+p7)).
    The leading size must be a power of two.  Same tree as the reference's rank fold
    (engine/crates/seqpar/src/transport.rs:272-283) widened to eight canonical ranges."""
    n = parts.shape[0]
    assert n & (n - 1) == 0, "fold_tree needs a power-of-two number of parts"
    while n > 1:
        parts = parts[0::2] + parts[1::2]
        n //= 2
    return parts[0]


def fp8_dot(x: torch.Tensor, w8: torch.Tensor, wscale: torch.Tensor, ranges: int = 1) -> torch.Tensor:
    """Block-scaled W8A8 product: x (fp32 [T, K]) is quantised per token and 128-column group
    (scale = max|x|/448), each K block's e4m3 x e4m3 dot is accumulated in fp32, multiplied by
    (token scale * weight scale) and added in ascending block order.  ``ranges`` > 1 returns the
    partial sums of equal runs of K blocks, fp32 [ranges, T, N]; else fp32 [T, N].
    w8: e4m3 bytes [N, K]; wscale: fp32 [N, K/128] (engine/docs/flash-fp8-math.md:36-45)."""
    from ..quant import codecs
    T, K = x.shape
    kb = K // 128
    q, s = codecs.fp8_quantize_activation(x.float().cpu())
    xa = codecs.e4m3_decode(q).view(T, kb, 128).to(x.device)
    s = s.to(x.device)
    wa = codecs.e4m3_decode(w8.cpu()).view(w8.shape[0], kb, 128).to(x.device)
    per = kb // ranges
    outs = []
    for r in range(ranges):
        acc = torch.zeros(T, w8.shape[0], dtype=torch.float32, device=x.device)
        for b in range(r * per, (r + 1) * per):
            acc = acc + dot_rows(xa[:, b], wa[:, b]) * (s[:, b, None] * wscale[None, :, b].float())
        outs.append(acc)
    return outs[0] if ranges == 1 else torch.stack(outs)


def qdot(x: torch.Tensor, q, idx: int | None = None) -> torch.Tensor:
    """x [T, K] times the rows of a stored matrix, WITHOUT its row scale, in that storage's arithmetic."""
    if q.kind == "fp8":
        return fp8_dot(x, q.packed if idx is None else q.packed[idx], q.scale if idx is None else q.scale[idx])
    return dot_rows(x.float(), q.dense(idx))


def linear_ranges(x: torch.Tensor, w: torch.Tensor, ranges: int, r0: int = 0, r1: int | None = None) -> torch.Tensor:
    """Row-parallel product as ``ranges`` partial sums over equal K slices.
    Returns fp32 [r1-r0, T, N]; ``w`` and ``x`` hold only the K columns of ranges [r0, r1)."""
    r1 = ranges if r1 is None else r1
    k_local = x.shape[1]
    per = k_local // (r1 - r0)
    return torch.stack([dot_rows(x[:, i * per:(i + 1) * per], w[:, i * per:(i + 1) * per])
                        for i in range(r1 - r0)])


# ------------------------------------------------------------------ norms / elementwise
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, one_plus: bool, act: torch.dtype) -> torch.Tensor:
    x = x.to(torch.float32)
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    y = x * torch.rsqrt(ms + eps) * ((1.0 + w.float()) if one_plus else w.float())
    return _round(y, act)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20.0, x, torch.log1p(torch.exp(x)))


def l2norm(x: torch.Tensor) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


# ------------------------------------------------------------------ rotary
def rope_tables(positions: torch.Tensor, rot: int, theta: float):
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64),
                    -torch.arange(0, rot, 2, dtype=torch.float64) / rot)
    ang = positions.to(torch.float64).unsqueeze(-1) * inv.to(positions.device)
    return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot: int) -> torch.Tensor:
    """Rotate-half on the first ``rot`` dims of [T, heads, hd]; cos/sin are [T, rot/2]."""
    half = rot // 2
    x1, x2, rest = x[..., :half], x[..., half:rot], x[..., rot:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


# ------------------------------------------------------------------ gated delta net
def gdn_conv(raw: torch.Tensor, conv_w: torch.Tensor, hist: torch.Tensor, seq_slots, seq_start,
             act: torch.dtype) -> torch.Tensor:
    """Depthwise causal conv (kernel 4) + SiLU over [hist(3), rows] per sequence.
    raw fp32 [T, C]; conv_w [C, 4]; hist fp32 [slots, 3, C] is updated to the last 3 raw rows."""
    out = torch.empty_like(raw)
    w = conv_w.float()
    for b, slot in enumerate(seq_slots):
        s, e = seq_start[b], seq_start[b + 1]
        ext = torch.cat([hist[slot], raw[s:e]], 0)            # [3 + n, C]
        n = e - s
        acc = torch.zeros(n, raw.shape[1], dtype=torch.float32, device=raw.device)
        for tap in range(4):
            acc = acc + ext[tap:tap + n] * w[:, tap]
        out[s:e] = silu(acc)
        hist[slot] = ext[-3:]
    return _round(out, act)


def gdn_gates(a: torch.Tensor, b: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor):
    """beta = sigmoid(b); g = -exp(A_log) * softplus(a + dt_bias)  (log decay per value head)."""
    beta = torch.sigmoid(b.float())
    g = -torch.exp(a_log.float()) * softplus(a.float() + dt_bias.float())
    return beta, g


def gdn_recurrent(q, k, v, beta, g, state, seq_slots, seq_start):
    """Token recurrence per value head: S *= e^g; delta = (v - S^T k) beta; S += k (x) delta; o = S^T q.
    q,k fp32 [T, kh, kd] (already l2-normalised, q scaled); v [T, vh, vd]; beta,g [T, vh];
    state fp32 [slots, vh, kd, vd] updated in place.  Returns o fp32 [T, vh, vd]."""
    T, vh, vd = v.shape
    kh = q.shape[1]
    rep = vh // kh
    o = torch.empty(T, vh, vd, dtype=torch.float32, device=v.device)
    for bi, slot in enumerate(seq_slots):
        S = state[slot]                                        # [vh, kd, vd]
        for t in range(seq_start[bi], seq_start[bi + 1]):
            qt = q[t].repeat_interleave(rep, 0)                # [vh, kd]
            kt = k[t].repeat_interleave(rep, 0)
            S = S * torch.exp(g[t]).view(vh, 1, 1)
            mem = (S * kt.unsqueeze(-1)).sum(1)                # [vh, vd]
            delta = (v[t] - mem) * beta[t].unsqueeze(-1)
            S = S + kt.unsqueeze(-1) * delta.unsqueeze(1)
            o[t] = (S * qt.unsqueeze(-1)).sum(1)
        state[slot] = S
    return o


def gdn_chunked(q, k, v, beta, g, state, seq_slots, seq_start, seq_pos0, chunk: int = 64):
    """Chunk form of the same recurrence (WY representation), chunks cut at ABSOLUTE positions
    that are multiples of ``chunk`` so any split of a prompt into calls visits the same chunks.
    Mathematically equal to gdn_recurrent; this is the algebra of the prefill kernel."""
    T, vh, vd = v.shape
    kh, kd = q.shape[1], q.shape[2]
    rep = vh // kh
    o = torch.empty(T, vh, vd, dtype=torch.float32, device=v.device)
    for bi, slot in enumerate(seq_slots):
        S = state[slot]
        s, e = seq_start[bi], seq_start[bi + 1]
        pos = seq_pos0[bi]
        t = s
        while t < e:
            n = min(e - t, chunk - (pos % chunk))
            Q = q[t:t + n].repeat_interleave(rep, 1).transpose(0, 1)      # [vh, n, kd]
            K = k[t:t + n].repeat_interleave(rep, 1).transpose(0, 1)
            V = v[t:t + n].transpose(0, 1)                                # [vh, n, vd]
            B = beta[t:t + n].transpose(0, 1)                             # [vh, n]
            G = torch.cumsum(g[t:t + n].transpose(0, 1), -1)              # [vh, n] inclusive log decay
            # u_i = beta_i (v_i - e^{G_i} S0^T k_i - sum_{j<i} e^{G_i-G_j} (k_j.k_i) u_j)
            KK = torch.einsum("hik,hjk->hij", K, K)
            decay = torch.exp(torch.tril(G.unsqueeze(-1) - G.unsqueeze(-2)))   # [vh, i, j]; upper part unused
            A = torch.tril(KK * decay, -1) * B.unsqueeze(-1)              # strictly lower
            rhs = (V - torch.exp(G).unsqueeze(-1) * torch.einsum("hkd,hik->hid", S, K)) * B.unsqueeze(-1)
            U = torch.empty_like(rhs)
            for i in range(n):
                U[:, i] = rhs[:, i] - torch.einsum("hj,hjd->hd", A[:, i, :i], U[:, :i])
            QK = torch.tril(torch.einsum("hik,hjk->hij", Q, K) * decay)   # j <= i
            o[t:t + n] = (torch.exp(G).unsqueeze(-1) * torch.einsum("hkd,hik->hid", S, Q)
                          + torch.einsum("hij,hjd->hid", QK, U)).transpose(0, 1)
            tail = torch.exp(G[:, -1:] - G)                               # e^{G_n - G_j}
            S = S * torch.exp(G[:, -1]).view(vh, 1, 1) + torch.einsum("hjk,hjd->hkd", K * tail.unsqueeze(-1), U)
            t += n
            pos += n
        state[slot] = S
    return o


def gdn_gated_norm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, act: torch.dtype,
                   gate: str = "sigmoid") -> torch.Tensor:
    """RMSNorm(o) * w (*) gate(z) per value head; o fp32 [T, vh, vd], z [T, vh, vd]."""
    ms = (o * o).sum(-1, keepdim=True) / o.shape[-1]
    y = o * torch.rsqrt(ms + eps) * w.float()
    zf = z.float()
    y = y * (torch.sigmoid(zf) if gate == "sigmoid" else silu(zf))
    return _round(y.reshape(o.shape[0], -1), act)


# ------------------------------------------------------------------ attention
def attention_paged(q, k_pages, v_pages, block_table, seq_slots, seq_start, seq_pos0, scale: float):
    """Causal GQA over a paged KV cache.  q fp32 [T, nh, hd]; pages [P, page, kvh, hd];
    block_table [slots, max_pages] int; token i of sequence b sits at position seq_pos0[b]+i and
    sees cache positions 0..its own.  Returns fp32 [T, nh, hd]."""
    T, nh, hd = q.shape
    page, kvh = k_pages.shape[1], k_pages.shape[2]
    rep = nh // kvh
    out = torch.empty(T, nh, hd, dtype=torch.float32, device=q.device)
    for bi, slot in enumerate(seq_slots):
        s, e = seq_start[bi], seq_start[bi + 1]
        n = e - s
        total = seq_pos0[bi] + n
        npages = -(-total // page)
        ids = block_table[slot, :npages].long()
        K = k_pages[ids].reshape(npages * page, kvh, hd)[:total].float()
        V = v_pages[ids].reshape(npages * page, kvh, hd)[:total].float()
        K = K.repeat_interleave(rep, 1)                                   # [L, nh, hd]
        V = V.repeat_interleave(rep, 1)
        sc = torch.einsum("ihd,jhd->hij", q[s:e], K) * scale             # [nh, n, L]
        qpos = torch.arange(n, device=q.device) + seq_pos0[bi]
        mask = torch.arange(total, device=q.device).unsqueeze(0) > qpos.unsqueeze(1)
        sc = sc.masked_fill(mask.unsqueeze(0), float("-inf"))
        p = torch.softmax(sc, -1)
        out[s:e] = torch.einsum("hij,jhd->ihd", p, V)
    return out


def kv_append(k, v, k_pages, v_pages, block_table, slots_per_row, positions):
    """Write row t's K,V ([kvh, hd]) to page block_table[slot, pos // page], offset pos % page."""
    page = k_pages.shape[1]
    pg = block_table[slots_per_row.long(), (positions // page).long()].long()
    off = (positions % page).long()
    k_pages[pg, off] = k.to(k_pages.dtype)
    v_pages[pg, off] = v.to(v_pages.dtype)


# ------------------------------------------------------------------ MoE
def route_topk(logits: torch.Tensor, k: int, renorm: bool):
    """softmax (fp32) -> top-k by probability, ties to the lower expert id -> renormalise.
    Returns ids int32 [T, k] sorted by DESCENDING probability and weights fp32 [T, k]."""
    p = torch.softmax(logits.float(), -1)
    # stable descending sort keeps the lower id first among equal probabilities
    order = torch.sort(p, dim=-1, descending=True, stable=True)
    ids = order.indices[:, :k]
    w = order.values[:, :k]
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w


def swiglu(gate: torch.Tensor, up: torch.Tensor, act: torch.dtype) -> torch.Tensor:
    return _round(silu(gate.float()) * up.float(), act)


def moe_combine(pair_out: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[t] = sum over the token's experts in ASCENDING expert id of w * y, as one fp32 chain
    from +0 (engine/crates/model/src/flash/refcpu.rs:809-840).  pair_out fp32 [T, k, H]."""
    order = torch.argsort(ids.long(), dim=-1, stable=True)
    T, k, H = pair_out.shape
    acc = torch.zeros(T, H, dtype=torch.float32, device=pair_out.device)
    for j in range(k):
        sel = order[:, j]
        y = pair_out[torch.arange(T, device=ids.device), sel]
        acc = acc + w[torch.arange(T, device=ids.device), sel].unsqueeze(-1) * y
    return acc


# ------------------------------------------------------------------ head
def argmax_lowest(logits: torch.Tensor) -> torch.Tensor:
    """Greedy token: the largest logit, ties to the lowest id (engine/crates/engine/src/lib.rs:84-87)."""
    m = logits.max(-1, keepdim=True).values
    idx = torch.arange(logits.shape[-1], device=logits.device).expand_as(logits)
    big = torch.full_like(idx, logits.shape[-1])
    return torch.where(logits == m, idx, big).min(-1).values
