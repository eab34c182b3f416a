"""Multi-rank host logic on CPU ranks (gloo, world size 2): shard plan agreement, arena layout,
and the all-gather of packed codes + scales + tensor scales.  No GPU is involved; the NVFP4
payloads are produced by the oracle so that what is gathered is real quantiser output."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llmini_b200.dist import Nvfp4Arena, all_gather_arena, shard_plan

SHAPES = [(256, 128), (128, 128), (384, 128), (128, 512), (0, 0), (64, 256)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scales_bytes(rows, cols):
    return rows * cols // 16


def _payload(slot, rows, cols):
    from oracle import oracle as o

    rng = np.random.default_rng(100 + slot)
    x = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
    codes, raw, gs, _ = o.nvfp4_quantize(x)
    return codes, raw, np.float32(gs)


def _worker(rank, world, port, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        owner, load = shard_plan(SHAPES, world)
        # every rank derives the same plan without communicating
        gathered = [None] * world
        dist.all_gather_object(gathered, owner)
        assert all(g == owner for g in gathered)
        arena = Nvfp4Arena(SHAPES, owner, world, _scales_bytes)
        buf = torch.zeros(arena.total_bytes, dtype=torch.uint8)
        for slot, (rows, cols) in enumerate(SHAPES):
            if owner[slot] != rank or rows * cols == 0:
                continue
            codes, raw, gs = _payload(slot, rows, cols)
            co, so, go = arena.offsets(slot)
            buf[co:co + codes.size] = torch.from_numpy(codes)
            buf[so:so + raw.size] = torch.from_numpy(raw)
            buf[go:go + 4] = torch.from_numpy(np.frombuffer(gs.tobytes(), np.uint8).copy())
        all_gather_arena(buf, arena)
        ok = True
        for slot, (rows, cols) in enumerate(SHAPES):
            if rows * cols == 0:
                continue
            codes, raw, gs = _payload(slot, rows, cols)
            co, so, go = arena.offsets(slot)
            ok &= np.array_equal(buf[co:co + codes.size].numpy(), codes)
            ok &= np.array_equal(buf[so:so + raw.size].numpy(), raw)
            ok &= buf[go:go + 4].numpy().tobytes() == gs.tobytes()
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def _checksum_worker(rank, world, port, corrupt, out):
    from llmini_b200.dist import gathered_arena_consistent

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        owner, _ = shard_plan(SHAPES, world)
        arena = Nvfp4Arena(SHAPES, owner, world, _scales_bytes)
        buf = torch.zeros(arena.total_bytes, dtype=torch.uint8)
        for slot, (rows, cols) in enumerate(SHAPES):
            if owner[slot] != rank or rows * cols == 0:
                continue
            codes, raw, gs = _payload(slot, rows, cols)
            co, so, go = arena.offsets(slot)
            buf[co:co + codes.size] = torch.from_numpy(codes)
            buf[so:so + raw.size] = torch.from_numpy(raw)
        if corrupt != "never_gathered":
            all_gather_arena(buf, arena)
        if corrupt == "one_byte" and rank == 1:
            buf[arena.offsets(0)[0] + 5] ^= 1       # one flipped bit in a slice this rank does not own
        if corrupt == "swapped" and rank == 1:
            a, b = arena.offsets(0)[0], arena.offsets(0)[0] + 1
            if buf[a] != buf[b]:
                buf[a], buf[b] = buf[b].clone(), buf[a].clone()   # same byte sum, different positions
            else:
                buf[a] ^= 3
        out[rank] = gathered_arena_consistent(buf, arena)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("corrupt,expected", [("nothing", True), ("one_byte", False), ("swapped", False),
                                              ("never_gathered", False)])
def test_gathered_arena_check_catches_a_rank_that_differs(corrupt, expected):
    # the check bench.py runs after a multi-GPU step, on CPU ranks: identical arenas pass; one flipped bit, two
    # swapped bytes, or slices that never arrived are caught on every rank
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_checksum_worker, args=(world, _free_port(), corrupt, out), nprocs=world, join=True)
        assert dict(out) == {0: expected, 1: expected}


def test_arena_layout_is_disjoint_and_aligned():
    owner, _ = shard_plan(SHAPES, 2)
    arena = Nvfp4Arena(SHAPES, owner, 2, _scales_bytes)
    spans = []
    for slot, (rows, cols) in enumerate(SHAPES):
        co, so, go = arena.offsets(slot)
        e = arena.entries[slot]
        assert co % 16 == 0 and so % 16 == 0 and go % 16 == 0
        assert co // arena.bytes_per_rank == owner[slot] or rows * cols == 0
        spans += [(co, co + e.codes_bytes), (so, so + e.scales_bytes), (go, go + 4)]
    spans = sorted(s for s in spans if s[1] > s[0])
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    assert arena.payload_bytes == sum(r * c // 2 + r * c // 16 + 4 for r, c in SHAPES)


def test_two_rank_all_gather_of_packed_weights():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, -1, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def _raising_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    if rank == 1:
        raise RuntimeError("injected host-side failure before the collective")
    t = torch.zeros(4)
    dist.all_reduce(t)  # the surviving rank's collective must end with an error, not hang


def test_rank_failure_before_the_collective_is_reported():
    # failure detection without a GPU: a rank that raises on the host makes the job fail loudly
    with pytest.raises(Exception):
        mp.spawn(_raising_worker, args=(2, _free_port()), nprocs=2, join=True)
