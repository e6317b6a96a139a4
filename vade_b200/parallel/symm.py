"""Peer-mapped exchange buffers for the fused compute + collective kernels.

Every rank of a tensor/expert-parallel group allocates the same arena with ``cudaMalloc`` and maps
every other rank's arena through CUDA IPC, so a kernel on any rank can store straight into any
rank's copy of a buffer over NVLink (plain peer stores; no TMA and no library kernel ever touches a
peer pointer).  Three exchange kinds live in the arena, each double-buffered and each with a flag
word per source rank:

* ``parts``  fp32 canonical-range partial sums of o_proj / GDN out_proj: the GEMM epilogue writes
             this rank's ranges into every rank's ``[8, T, H]`` block (GEMM -> all-gather), the
             fold kernel waits for all ranks and adds the eight ranges in the fixed tree;
* ``pairs``  bf16 expert outputs in the global row layout of the routing kernels: the down-projection
             epilogue writes the rows of this rank's experts everywhere, the combine kernel waits
             and adds each token's experts in ascending expert id;
* ``head``   (value, id) candidates of the vocabulary-parallel greedy head.

The protocol (sequence numbers, parity, bounded waits) is documented beside ``PeerExchange`` in
csrc/common/ptx.cuh.  Parity: the reference's in-stream mailbox with sequence words and a bounded
take (engine/crates/gpu/kernels/src/tp_mailbox.rs:56-108), mapped from RDMA slots to NVLink peers.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _ext


@dataclass
class Exchange:
    """Kernel-facing description of one exchange kind."""
    out: list               # device address of each rank's buffer (index = rank)
    flags: list             # device address of each rank's flag array [ranks] for this kind
    local: int              # device address of this rank's two sequence words
    half_stride: int        # elements between the two halves
    ranks: int
    self_rank: int
    buffer: torch.Tensor    # this rank's buffer (both halves), typed


class SymmArena:
    def __init__(self, group, device, hidden: int, max_rows: int, slots_per_row: int, head_rows: int = 64,
                 head_chunks: int = 64):
        self.group = group
        self.device = torch.device(device)
        self.ranks = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        ext = _ext.load()
        self.ext = ext
        al = lambda n: (n + 255) // 256 * 256
        self.parts_half = 8 * max_rows * hidden                    # fp32 elements
        self.pairs_half = max_rows * slots_per_row * hidden        # bf16 elements
        self.head_half = self.ranks * head_rows * head_chunks      # 8-byte pairs
        self.head_rows, self.head_chunks = head_rows, head_chunks
        sizes = {"parts": al(2 * self.parts_half * 4), "pairs": al(2 * self.pairs_half * 2),
                 "head": al(2 * self.head_half * 8), "flags": 4096}
        self.offsets, off = {}, 0
        for k, v in sizes.items():
            self.offsets[k] = off
            off += v
        self.nbytes = off
        self.arena = ext.symm_alloc(off, self.device.index or 0)
        handle = bytes(ext.symm_handle(self.arena))
        handles = [None] * self.ranks
        dist.all_gather_object(handles, handle, group=group)
        self.base = []
        for r, h in enumerate(handles):
            self.base.append(self.arena.data_ptr() if r == self.rank else ext.symm_open(h, self.device.index or 0))
        # sequence words are private to the rank: [kind][2] uint32
        self.local = torch.zeros(3, 2, dtype=torch.int32, device=self.device)
        kinds = ["parts", "pairs", "head"]
        self.ex = {}
        for i, kind in enumerate(kinds):
            dtype = {"parts": torch.float32, "pairs": torch.bfloat16, "head": torch.int64}[kind]
            half = {"parts": self.parts_half, "pairs": self.pairs_half, "head": self.head_half}[kind]
            item = {"parts": 4, "pairs": 2, "head": 8}[kind]
            buf = self.arena[self.offsets[kind]:self.offsets[kind] + 2 * half * item].view(dtype)
            self.ex[kind] = Exchange(
                out=[b + self.offsets[kind] for b in self.base],
                flags=[b + self.offsets["flags"] + i * 64 for b in self.base],
                local=self.local.data_ptr() + i * 8, half_stride=half, ranks=self.ranks, self_rank=self.rank, buffer=buf)
        dist.barrier(group=group)

    def close(self) -> None:
        for r, b in enumerate(self.base):
            if r != self.rank:
                self.ext.symm_close(b)
        self.base = []
