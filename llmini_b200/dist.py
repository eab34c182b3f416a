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


def bucket_plan(shapes: Sequence[tuple[int, int]], world: int, buckets: int):
    """-> (bucket per slot, owner rank per slot).  The matrices, in their given order, are cut into `buckets`
    contiguous runs of about equal Newton-Schulz FLOPs, and every run is spread over the ranks (one bucket:
    shard_plan; more: see below).  A rank then works through the buckets one after the other, and the all-gather of a bucket's
    packed weights runs while the next bucket is computed: only the last bucket's gather is left uncovered."""
    n = len(shapes)
    buckets = max(1, min(int(buckets), max(1, sum(1 for r, c in shapes if r * c))))
    flops = []
    for r, c in shapes:
        lo, hi = float(min(r, c)), float(max(r, c))
        flops.append(4.0 * lo * lo * hi + 2.0 * lo * lo * lo)
    total = sum(flops)
    bucket, acc, b = [0] * n, 0.0, 0
    for i in range(n):
        # a matrix goes to the bucket in which its midpoint falls
        mid = acc + 0.5 * flops[i]
        b = max(b, min(buckets - 1, int(mid * buckets / total))) if total > 0 else 0
        bucket[i] = b
        acc += flops[i]
    if buckets == 1:
        return bucket, shard_plan(shapes, world)[0]
    # Bucket after bucket, largest matrix first, each to the rank with the least work SO FAR (over all buckets up
    # to here; ties to the lowest rank): every bucket is spread over the ranks, and what a bucket leaves uneven the
    # next one evens out, so the ranks' totals (one Newton-Schulz pass over everything) stay balanced.
    owner, load = [0] * n, [0.0] * world
    for b in range(buckets):
        ids = sorted((i for i in range(n) if bucket[i] == b), key=lambda i: (-flops[i], i))
        for i in ids:
            r = min(range(world), key=lambda k: (load[k], k))
            owner[i] = r
            load[r] += flops[i]
    return bucket, owner


@dataclass
class ArenaEntry:
    slot: int
    rank: int
    bucket: int
    codes_off: int      # byte offsets inside the owner's arena slice
    scales_off: int
    gscale_off: int
    codes_bytes: int
    scales_bytes: int


class Nvfp4Arena:
    """Layout of the all-gather buffer.  One region per bucket (one bucket unless `bucket` is given); a region is
    `world` equal slices, rank r's matrices of that bucket packed back to back (codes, scales, 4-byte tensor
    scale; 16-byte aligned) inside slice r.  Every region is gathered by one all-gather."""

    def __init__(self, shapes: Sequence[tuple[int, int]], owner: Sequence[int], world: int, scales_bytes_fn,
                 bucket: Sequence[int] | None = None):
        self.world = world
        bucket = list(bucket) if bucket is not None else [0] * len(shapes)
        self.buckets = (max(bucket) + 1) if bucket else 1
        self.entries: list[ArenaEntry] = []
        used = [[0] * world for _ in range(self.buckets)]
        for s, ((rows, cols), r, b) in enumerate(zip(shapes, owner, bucket)):
            n = rows * cols
            cb, sb = n // 2, int(scales_bytes_fn(rows, cols))
            off = used[b][r]
            co = off
            so = _align(co + cb, 16)
            go = _align(so + sb, 16)
            used[b][r] = _align(go + 4, 16)
            self.entries.append(ArenaEntry(s, r, b, co, so, go, cb, sb))
        self.bucket_bytes_per_rank = [_align(max(u) if u else 0, 256) for u in used]
        self.bucket_base = [0] * self.buckets
        for b in range(1, self.buckets):
            self.bucket_base[b] = self.bucket_base[b - 1] + self.bucket_bytes_per_rank[b - 1] * world
        self.bytes_per_rank = sum(self.bucket_bytes_per_rank)   # (one slice per bucket: see rank_slices)
        self.total_bytes = self.bytes_per_rank * world
        self.payload_bytes = sum(e.codes_bytes + e.scales_bytes + 4 for e in self.entries)

    def offsets(self, slot: int):
        e = self.entries[slot]
        base = self.bucket_base[e.bucket] + e.rank * self.bucket_bytes_per_rank[e.bucket]
        return base + e.codes_off, base + e.scales_off, base + e.gscale_off

    def region(self, bucket: int):
        """(byte offset, bytes) of a bucket's region = `world` slices of bucket_bytes_per_rank[bucket]."""
        return self.bucket_base[bucket], self.bucket_bytes_per_rank[bucket] * self.world

    def rank_slices(self, rank: int):
        """[(byte offset, bytes)] of the slices rank `rank` fills, one per bucket."""
        return [(self.bucket_base[b] + rank * n, n) for b, n in enumerate(self.bucket_bytes_per_rank)]


def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def all_gather_bucket(arena_tensor, arena: Nvfp4Arena, bucket: int, group=None):
    """In-place all-gather of one bucket's region (NCCL on GPUs, gloo on CPU ranks)."""
    import torch.distributed as dist

    rank = dist.get_rank(group)
    base, size = arena.region(bucket)
    n = arena.bucket_bytes_per_rank[bucket]
    if n == 0:
        return
    region = arena_tensor[base:base + size]
    mine = region[rank * n:(rank + 1) * n]
    if arena_tensor.is_cuda:
        dist.all_gather_into_tensor(region, mine, group=group)
    else:
        parts = [region[r * n:(r + 1) * n] for r in range(arena.world)]
        gathered = [p.clone() for p in parts]
        dist.all_gather(gathered, mine.clone(), group=group)
        for p, g in zip(parts, gathered):
            p.copy_(g)


def all_gather_arena(arena_tensor, arena: Nvfp4Arena, group=None):
    """In-place all-gather of every bucket's region.  `arena_tensor` is a uint8 tensor of arena.total_bytes."""
    for b in range(arena.buckets):
        all_gather_bucket(arena_tensor, arena, b, group)


def arena_slice_checksums(arena_tensor, arena: Nvfp4Arena, piece: int = 32 << 20):
    """Two checksums per rank (a plain byte sum and a position-weighted one over the rank's slices of all
    buckets), as an int64 tensor [2, world] on the arena's device.  Ranks that hold the same arena get the same
    numbers."""
    import torch

    w = arena.world
    dev = arena_tensor.device
    sums = torch.zeros(2, w, dtype=torch.int64, device=dev)
    for r in range(w):
        for start, n in arena.rank_slices(r):
            for a in range(0, n, piece):
                v = arena_tensor[start + a:start + min(a + piece, n)].to(torch.int64)
                weight = ((torch.arange(v.numel(), device=dev, dtype=torch.int64) + start + a) % 251) + 1
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


class _DeviceBytes:
    """A raw device allocation seen by torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerArena:
    """The gathered arena in memory that the other ranks map (b2_peer_*): `tensor` is this rank's copy of the whole
    arena (a uint8 torch view of the library's allocation); `push(offset, bytes)` copies a piece of it to the same
    place in every peer's copy with one small kernel; `wait()` makes the stream wait until every copy that any
    rank enqueued before its own wait has arrived here.  One process per GPU; `exchange(obj) -> list` gathers one
    picklable object from every rank (torch.distributed.all_gather_object does)."""

    def __init__(self, arena_bytes: int, rank: int, world: int, exchange, device):
        import torch

        if world > _ffi.MAX_PEERS:
            raise ValueError(f"at most {_ffi.MAX_PEERS} ranks")
        L = _ffi.lib()
        self._lib, self.rank, self.world, self.arena_bytes = L, rank, world, int(arena_bytes)
        self._own, self._opened, self.tensor = C.c_void_p(), [], None
        handle = (C.c_uint8 * 64)()
        # Every rank goes through both exchanges whatever happens to it, so that all of them succeed or all of them
        # raise: a rank that left early would leave the others waiting.
        with torch.cuda.device(device):
            rc = L.b2_peer_buffer_alloc(self.arena_bytes, C.byref(self._own), handle)
            handles = exchange(bytes(handle) if rc == 0 else None)
            problem = None
            if any(h is None for h in handles):
                problem = "a rank could not allocate its buffer"
            else:
                self.group = _ffi.PeerGroup()
                self.group.world, self.group.rank, self.group.arena_bytes = world, rank, self.arena_bytes
                for r in range(world):
                    if r == rank:
                        self.group.base[r] = self._own.value
                        continue
                    p = C.c_void_p()
                    rc = L.b2_peer_buffer_open((C.c_uint8 * 64)(*handles[r]), C.byref(p))
                    if rc != 0:
                        problem = f"rank {rank} could not map rank {r}'s buffer (error {rc})"
                        break
                    self._opened.append(p)
                    self.group.base[r] = p.value
            problems = [q for q in exchange(problem) if q]
            if problems:
                self.close()
                raise RuntimeError(problems[0])
        self.tensor = torch.as_tensor(_DeviceBytes(self._own.value, max(self.arena_bytes, 1)), device=device)[:self.arena_bytes]

    def push(self, offset: int, nbytes: int, stream: int, ctas: int = 0) -> None:
        _ffi.check(self._lib.b2_peer_push(C.byref(self.group), offset, nbytes, ctas, stream), "peer_push")

    def wait(self, stream: int, wait_ns: int = 0) -> None:
        _ffi.check(self._lib.b2_peer_wait(C.byref(self.group), wait_ns, stream), "peer_wait")

    def status(self, stream: int) -> int:
        return int(self._lib.b2_peer_status(C.byref(self.group), stream))

    def close(self) -> None:
        """Every rank must have finished with the others' buffers (a barrier) before any rank frees its own."""
        for p in self._opened:
            self._lib.b2_peer_buffer_close(p)
        self._opened = []
        if self._own.value:
            self.tensor = None
            self._lib.b2_peer_buffer_free(self._own)
            self._own = C.c_void_p()


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
