"""Whole-matrix sharding across ranks and the all-gather of packed NVFP4 weights.

The reference is single-GPU; this is the multi-GPU form the path takes here: every rank owns a
subset of whole matrices (greedy by Newton-Schulz FLOPs), runs their updates locally and
all-gathers packed codes + block scales + tensor scales from equally sized per-rank arenas.
`torch.distributed` supplies the rendezvous (and the gloo path for CPU tests); on GPUs the
collective itself is NCCL, either through torch or through the library's own communicator.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from . import _ffi


def shard_plan(shapes: Sequence[tuple[int, int]], world: int):
    """-> (owner rank per slot, FLOPs per rank).  b2_shard_plan in the C ABI."""
    n = len(shapes)
    rows = (C.c_uint32 * n)(*[int(r) for r, _ in shapes])
    cols = (C.c_uint32 * n)(*[int(c) for _, c in shapes])
    owner = (C.c_uint32 * n)()
    load = (C.c_double * world)()
    _ffi.check(_ffi.lib().b2_shard_plan(rows, cols, n, world, owner, load), "shard_plan")
    return list(owner), list(load)


@dataclass
class ArenaEntry:
    slot: int
    rank: int
    codes_off: int      # byte offsets inside the owner's arena slice
    scales_off: int
    gscale_off: int
    codes_bytes: int
    scales_bytes: int


class Nvfp4Arena:
    """Layout of the all-gather buffer: `world` equal slices; rank r's matrices packed back to
    back (codes, scales, 4-byte tensor scale; 16-byte aligned) inside slice r."""

    def __init__(self, shapes: Sequence[tuple[int, int]], owner: Sequence[int], world: int, scales_bytes_fn):
        self.world = world
        self.entries: list[ArenaEntry] = []
        used = [0] * world
        for s, ((rows, cols), r) in enumerate(zip(shapes, owner)):
            n = rows * cols
            cb, sb = n // 2, int(scales_bytes_fn(rows, cols))
            off = used[r]
            co = off
            so = _align(co + cb, 16)
            go = _align(so + sb, 16)
            used[r] = _align(go + 4, 16)
            self.entries.append(ArenaEntry(s, r, co, so, go, cb, sb))
        self.bytes_per_rank = _align(max(used) if used else 0, 256)
        self.total_bytes = self.bytes_per_rank * world
        self.payload_bytes = sum(e.codes_bytes + e.scales_bytes + 4 for e in self.entries)

    def offsets(self, slot: int):
        e = self.entries[slot]
        base = e.rank * self.bytes_per_rank
        return base + e.codes_off, base + e.scales_off, base + e.gscale_off


def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def all_gather_arena(arena_tensor, arena: Nvfp4Arena, group=None):
    """In-place all-gather of the per-rank slices with torch.distributed (NCCL on GPUs, gloo on
    CPU ranks).  `arena_tensor` is a uint8 tensor of arena.total_bytes."""
    import torch.distributed as dist

    rank = dist.get_rank(group)
    n = arena.bytes_per_rank
    mine = arena_tensor[rank * n:(rank + 1) * n]
    if arena_tensor.is_cuda:
        dist.all_gather_into_tensor(arena_tensor, mine, group=group)
    else:
        parts = [arena_tensor[r * n:(r + 1) * n] for r in range(arena.world)]
        gathered = [p.clone() for p in parts]
        dist.all_gather(gathered, mine.clone(), group=group)
        for p, g in zip(parts, gathered):
            p.copy_(g)


def arena_slice_checksums(arena_tensor, arena: Nvfp4Arena, piece: int = 32 << 20):
    """Two checksums per rank slice of a gathered arena (a plain byte sum and a position-weighted one), as an
    int64 tensor [2, world] on the arena's device.  Ranks that hold the same arena get the same numbers."""
    import torch

    n, w = arena.bytes_per_rank, arena.world
    dev = arena_tensor.device
    sums = torch.zeros(2, w, dtype=torch.int64, device=dev)
    for r in range(w):
        for a in range(0, n, piece):
            v = arena_tensor[r * n + a:r * n + min(a + piece, n)].to(torch.int64)
            weight = ((torch.arange(v.numel(), device=dev, dtype=torch.int64) + a) % 251) + 1
            sums[0, r] += v.sum()
            sums[1, r] += (v * weight).sum()
    return sums


def gathered_arena_consistent(arena_tensor, arena: Nvfp4Arena, group=None) -> bool:
    """After the all-gather every rank must hold the same arena: the per-slice checksums are reduced with MIN
    and MAX over the ranks and must agree, and every slice that carries payload must be non-zero (a rank whose
    slice never arrived would otherwise agree with everybody on zeros only if all were empty).  Collective:
    every rank of `group` calls it."""
    import torch
    import torch.distributed as dist

    sums = arena_slice_checksums(arena_tensor, arena)
    lo, hi = sums.clone(), sums.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    used = torch.zeros(arena.world, dtype=torch.bool, device=arena_tensor.device)
    for e in arena.entries:
        if e.codes_bytes:
            used[e.rank] = True
    filled = bool(((sums[0] != 0) | ~used).all().item())
    return bool(torch.equal(lo, hi)) and filled


class Communicator:
    """The library's own NCCL communicator (b2_comm_*), bootstrapped over torch.distributed."""

    def __init__(self, rank: int, world: int, broadcast_bytes):
        L = _ffi.lib()
        uid = (C.c_uint8 * 128)()
        if rank == 0:
            _ffi.check(L.b2_comm_unique_id(uid), "comm_unique_id")
        data = broadcast_bytes(bytes(uid))
        uid = (C.c_uint8 * 128)(*data)
        self._h = C.c_void_p()
        _ffi.check(L.b2_comm_create(C.byref(self._h), uid, rank, world), "comm_create")

    def all_gather(self, arena_ptr: int, bytes_per_rank: int, stream: int) -> None:
        _ffi.check(_ffi.lib().b2_allgather_nvfp4(self._h, arena_ptr, bytes_per_rank, stream), "allgather_nvfp4")

    def close(self):
        if self._h.value:
            _ffi.lib().b2_comm_destroy(self._h)
            self._h = C.c_void_p()
