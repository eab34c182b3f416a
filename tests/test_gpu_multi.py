"""Two-GPU run of the sharded step: every rank updates the matrices it owns, writes packed
NVFP4 weights into its arena slice, and the arenas are all-gathered with the library's own NCCL
communicator (b2_comm_* / b2_allgather_nvfp4) or copied into the other rank's arena through peer memory
(b2_peer_*).  The gathered weights must equal a single-GPU run of all matrices bit for bit.  Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(512, 256), (256, 256), (768, 256), (256, 1024), (384, 128)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_inputs():
    rng = np.random.default_rng(77)
    data = []
    for r, c in SHAPES:
        data.append(((rng.standard_normal(r * c) * 1e-3).astype(np.float32),
                     (rng.standard_normal(r * c) * 0.02).astype(np.float32),
                     (rng.standard_normal(r * c) * 0.02).astype(np.float32)))
    return data


def _run_slots(device, slot_ids, arena, arena_t, data):
    import llmini_b200 as b2

    slots = []
    for i in slot_ids:
        r, c = SHAPES[i]
        g, z, x = data[i]
        co, so, go = arena.offsets(i)
        e = arena.entries[i]
        dev = lambda a: torch.from_numpy(a).to(device).view(r, c)
        slots.append(b2.MuonSlot(grad=dev(g.copy()), momentum=torch.zeros(r, c, dtype=torch.bfloat16, device=device),
                                 z_master=dev(z.copy()), x_master=dev(x.copy()), schedule_amax=torch.zeros(1, device=device),
                                 bytes=arena_t[co:co + e.codes_bytes], scales=arena_t[so:so + e.scales_bytes],
                                 global_scale=arena_t[go:go + 4].view(torch.float32), rows=r, cols=c))
    if not slots:
        return
    plan = b2.MuonPlan([SHAPES[i] for i in slot_ids], scale_layout=b2.SCALES_RAW, device=device)
    b2.OptimizerModule().muon_mega_update(plan, b2.slot_table(slots, device), b2.MuonMegaUpdateArgs(
        learning_rate=0.02, coefficients=np.tile(np.asarray([3.4445, -4.7750, 2.0315], np.float32), (5, 1))))
    torch.cuda.synchronize(device)
    assert plan.status() == 0
    plan.close()


def _layout(world, buckets):
    from llmini_b200.dist import Nvfp4Arena, bucket_plan

    bucket, owner = bucket_plan(SHAPES, world, buckets)
    return bucket, owner, Nvfp4Arena(SHAPES, owner, world, lambda r, c: r * c // 16, bucket)


def _worker(rank, world, port, buckets, gather, out):
    import torch.distributed as dist

    from llmini_b200.dist import Communicator, PeerArena

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # rendezvous only
    try:
        bucket, owner, arena = _layout(world, buckets)
        data = _make_inputs()

        def bcast(b):
            box = [b]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        def exchange(obj):
            got = [None] * world
            dist.all_gather_object(got, obj)
            return got

        side = torch.cuda.Stream(device=device)
        if gather == "p2p":
            # the arena in memory the other rank maps; a bucket is copied into the peer's arena by one small kernel
            peers = PeerArena(arena.total_bytes, rank, world, exchange, device)
            arena_t = peers.tensor
        else:
            comm = Communicator(rank, world, bcast)
            arena_t = torch.zeros(arena.total_bytes, dtype=torch.uint8, device=device)
        # bucket by bucket: this rank's matrices of the bucket, then the bucket's exchange on a second stream
        # while the next bucket is computed
        for b in range(arena.buckets):
            _run_slots(device, [i for i, o_ in enumerate(owner) if o_ == rank and bucket[i] == b], arena, arena_t, data)
            base, _ = arena.region(b)
            n = arena.bucket_bytes_per_rank[b]
            side.wait_stream(torch.cuda.current_stream())
            if gather == "p2p":
                peers.push(base + rank * n, n, side.cuda_stream)
            else:
                comm.all_gather(arena_t.data_ptr() + base, n, side.cuda_stream)
        if gather == "p2p":
            peers.wait(side.cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(device)
        out[rank] = arena_t.cpu().numpy().tobytes()
        if gather == "p2p":
            assert peers.status(torch.cuda.current_stream().cuda_stream) == 0
            dist.barrier()          # nobody unmaps or frees while the other may still be copying
            arena_t = None
            peers.close()
        else:
            comm.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("gather", ["nccl", "p2p"])
@pytest.mark.parametrize("buckets", [1, 2])
def test_sharded_step_and_library_all_gather_match_single_gpu(buckets, gather):
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), buckets, gather, out), nprocs=world, join=True)
        got = {k: np.frombuffer(v, np.uint8) for k, v in out.items()}
    assert np.array_equal(got[0], got[1])
    # single-GPU run of every matrix into the same arena layout
    _, _, arena = _layout(world, buckets)
    device = torch.device("cuda", 0)
    arena_t = torch.zeros(arena.total_bytes, dtype=torch.uint8, device=device)
    _run_slots(device, list(range(len(SHAPES))), arena, arena_t, _make_inputs())
    assert np.array_equal(arena_t.cpu().numpy(), got[0])
