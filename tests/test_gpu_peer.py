"""The peer-memory exchange (b2_peer_*) on one GPU: a second allocation on the same device stands in for the other
rank's buffer, so the copy kernel, its completion counts and the bounded wait are exercised without a second GPU.
(The two-GPU form, through CUDA IPC, is in test_gpu_multi.py.)  No kernel here waits for another that runs at the
same time: the waits are launched after the copies they wait for, or wait for a count that nothing raises and
give up after two milliseconds."""
import ctypes as C

import numpy as np
import pytest
import torch

from llmini_b200 import _ffi
from llmini_b200.dist import _DeviceBytes

pytestmark = pytest.mark.gpu

ARENA = 3 * 1024 * 1024 + 512


class _Pair:
    """Two buffers on one device and the group as each of the two 'ranks' sees it."""

    def __init__(self):
        self.lib = _ffi.lib()
        self.ptr = [C.c_void_p(), C.c_void_p()]
        for p in self.ptr:
            h = (C.c_uint8 * 64)()
            _ffi.check(self.lib.b2_peer_buffer_alloc(ARENA, C.byref(p), h), "peer_buffer_alloc")
        self.group = []
        for rank in range(2):
            g = _ffi.PeerGroup()
            g.world, g.rank, g.arena_bytes = 2, rank, ARENA
            g.base[0], g.base[1] = self.ptr[0].value, self.ptr[1].value
            self.group.append(g)
        total = (ARENA + 255) // 256 * 256 + 256
        self.view = [torch.as_tensor(_DeviceBytes(p.value, total), device="cuda") for p in self.ptr]

    def ctrl(self, rank):
        base = (ARENA + 255) // 256 * 256
        return self.view[rank][base:base + 256].view(torch.int32).cpu().numpy()

    def close(self):
        torch.cuda.synchronize()
        self.view = None
        for p in self.ptr:
            self.lib.b2_peer_buffer_free(p)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_push_copies_the_range_and_counts():
    pair = _Pair()
    try:
        lib = pair.lib
        gen = torch.Generator(device="cuda").manual_seed(3)
        pair.view[0][:ARENA] = torch.randint(0, 256, (ARENA,), dtype=torch.uint8, device="cuda", generator=gen)
        pair.view[1][:ARENA] = 7
        want = pair.view[1][:ARENA].clone()
        pushes = [(0, 1024 * 1024, 0), (1024 * 1024 + 4096, 16, 1), (2 * 1024 * 1024, 1024 * 1024 + 512, 5), (4096, 0, 0)]
        for off, n, ctas in pushes:
            _ffi.check(lib.b2_peer_push(C.byref(pair.group[0]), off, n, ctas, _stream()), "peer_push")
            want[off:off + n] = pair.view[0][off:off + n]
        torch.cuda.synchronize()
        assert torch.equal(pair.view[1][:ARENA], want)                       # the ranges, and nothing else
        assert pair.ctrl(1)[0] == len(pushes)                                # arrived[0] in the peer's control block
        assert pair.ctrl(0)[_ffi.MAX_PEERS] == len(pushes)                   # this rank's own count
        assert pair.ctrl(0)[_ffi.MAX_PEERS + 1] == 0                         # the CTA counter is back at zero
        # offsets and sizes must be multiples of 16 inside the arena
        for off, n in ((8, 16), (0, 24), (ARENA, 16), (16, ARENA)):
            assert lib.b2_peer_push(C.byref(pair.group[0]), off, n, 0, _stream()) == _ffi.ERROR_INVALID_VALUE
    finally:
        pair.close()


def test_wait_passes_once_the_peer_has_caught_up_and_gives_up_otherwise():
    pair = _Pair()
    try:
        lib = pair.lib
        g0, g1 = pair.group
        # rank 0 has pushed twice, its peer once: rank 0's wait cannot pass; it runs out after 2 ms and says so
        _ffi.check(lib.b2_peer_push(C.byref(g0), 0, 4096, 0, _stream()), "peer_push")
        _ffi.check(lib.b2_peer_push(C.byref(g0), 4096, 4096, 0, _stream()), "peer_push")
        _ffi.check(lib.b2_peer_push(C.byref(g1), 8192, 4096, 0, _stream()), "peer_push")
        torch.cuda.synchronize()
        _ffi.check(lib.b2_peer_wait(C.byref(g0), 2_000_000, _stream()), "peer_wait")
        assert lib.b2_peer_status(C.byref(g0), _stream()) == _ffi.ERROR_LAUNCH_TIMEOUT
        assert lib.b2_peer_status(C.byref(g0), _stream()) == 0               # reported once
        # the peer, one copy behind nobody, passes at once
        _ffi.check(lib.b2_peer_wait(C.byref(g1), 2_000_000, _stream()), "peer_wait")
        assert lib.b2_peer_status(C.byref(g1), _stream()) == 0
        # the peer's second copy lands: now rank 0 passes too, and the context is as usable as before
        _ffi.check(lib.b2_peer_push(C.byref(g1), 12288, 4096, 0, _stream()), "peer_push")
        torch.cuda.synchronize()
        _ffi.check(lib.b2_peer_wait(C.byref(g0), 2_000_000, _stream()), "peer_wait")
        assert lib.b2_peer_status(C.byref(g0), _stream()) == 0
        assert pair.ctrl(0)[1] == 2 and pair.ctrl(1)[0] == 2
    finally:
        pair.close()


def test_a_group_of_one_needs_no_peer():
    lib = _ffi.lib()
    p, h = C.c_void_p(), (C.c_uint8 * 64)()
    _ffi.check(lib.b2_peer_buffer_alloc(4096, C.byref(p), h), "peer_buffer_alloc")
    g = _ffi.PeerGroup()
    g.world, g.rank, g.arena_bytes = 1, 0, 4096
    g.base[0] = p.value
    _ffi.check(lib.b2_peer_push(C.byref(g), 0, 4096, 0, _stream()), "peer_push")
    _ffi.check(lib.b2_peer_wait(C.byref(g), 0, _stream()), "peer_wait")
    assert lib.b2_peer_status(C.byref(g), _stream()) == 0
    bad = _ffi.PeerGroup()
    bad.world, bad.rank = 2, 0
    bad.base[0] = p.value                                                    # base[1] missing
    assert lib.b2_peer_push(C.byref(bad), 0, 16, 0, _stream()) == _ffi.ERROR_INVALID_VALUE
    torch.cuda.synchronize()
    lib.b2_peer_buffer_free(p)
