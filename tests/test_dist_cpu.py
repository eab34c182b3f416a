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

from llmini_b200.dist import Nvfp4Arena, all_gather_arena, all_gather_bucket, bucket_plan, shard_plan

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


def _worker(rank, world, port, buckets, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if buckets > 1:
            bucket, owner = bucket_plan(SHAPES, world, buckets)
        else:
            bucket, (owner, load) = None, shard_plan(SHAPES, world)
        # every rank derives the same plan without communicating
        gathered = [None] * world
        dist.all_gather_object(gathered, (bucket, owner))
        assert all(g == (bucket, owner) for g in gathered)
        arena = Nvfp4Arena(SHAPES, owner, world, _scales_bytes, bucket)
        buf = torch.zeros(arena.total_bytes, dtype=torch.uint8)
        for slot, (rows, cols) in enumerate(SHAPES):
            if owner[slot] != rank or rows * cols == 0:
                continue
            codes, raw, gs = _payload(slot, rows, cols)
            co, so, go = arena.offsets(slot)
            buf[co:co + codes.size] = torch.from_numpy(codes)
            buf[so:so + raw.size] = torch.from_numpy(raw)
            buf[go:go + 4] = torch.from_numpy(np.frombuffer(gs.tobytes(), np.uint8).copy())
        if buckets > 1:
            # bucket by bucket, as a step does it: after bucket b's gather only its region is complete
            for b in range(arena.buckets):
                all_gather_bucket(buf, arena, b)
                later = [e for e in arena.entries if e.bucket > b and e.rank != rank and e.codes_bytes]
                assert all(not buf[arena.offsets(e.slot)[0]:arena.offsets(e.slot)[0] + e.codes_bytes].any() for e in later)
        else:
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
        mp.spawn(_worker, args=(world, port, 1, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_two_rank_all_gather_bucket_by_bucket():
    # the matrices cut into two buckets, each spread over both ranks and gathered by its own all-gather
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, 2, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_bucket_plan_cuts_contiguous_runs_and_balances_each():
    gpt2_layer = [(2304, 768), (768, 768), (3072, 768), (768, 3072)]
    shapes = gpt2_layer * 12
    for world in (2, 4, 8):
        for buckets in (1, 2, 4):
            bucket, owner = bucket_plan(shapes, world, buckets)
            assert bucket == sorted(bucket) and bucket[0] == 0 and bucket[-1] == buckets - 1
            assert all(0 <= r < world for r in owner)
            flops = [4.0 * min(r, c) ** 2 * max(r, c) + 2.0 * min(r, c) ** 3 for r, c in shapes]
            per_bucket = [sum(f for f, b in zip(flops, bucket) if b == k) for k in range(buckets)]
            assert max(per_bucket) <= 1.2 * min(per_bucket)
            # what counts is a rank's total (stages M, N and P run once over all buckets): within 10 % of the mean;
            # a single bucket may be less even, the next one makes up for it
            total = [sum(f for f, r in zip(flops, owner) if r == w) for w in range(world)]
            assert max(total) <= 1.10 * (sum(total) / world)
            for k in range(buckets):
                load = [sum(f for f, b, r in zip(flops, bucket, owner) if b == k and r == w) for w in range(world)]
                assert max(load) <= 1.6 * (sum(load) / world)
            # the layout puts a slot inside its owner's slice of its bucket's region, regions back to back
            arena = Nvfp4Arena(shapes, owner, world, _scales_bytes, bucket)
            end = 0
            for k in range(arena.buckets):
                base, size = arena.region(k)
                assert base == end and size == arena.bucket_bytes_per_rank[k] * world
                end = base + size
            assert end == arena.total_bytes
            for slot in range(len(shapes)):
                e = arena.entries[slot]
                base, _ = arena.region(e.bucket)
                lo = base + e.rank * arena.bucket_bytes_per_rank[e.bucket]
                co, so, go = arena.offsets(slot)
                assert lo <= co and go + 4 <= lo + arena.bucket_bytes_per_rank[e.bucket]
    # more buckets than matrices, and padding slots
    bucket, owner = bucket_plan([(128, 128), (0, 0), (256, 128)], 2, 8)
    assert max(bucket) <= 1 and len(owner) == 3


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
