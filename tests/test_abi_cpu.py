"""CPU-side checks of the shipped library: it loads, exports every declared symbol, its
host-only entry points agree with the oracle, and compute entry points fail loudly without a
GPU instead of falling back."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import llmini_b200 as b2
from llmini_b200 import _ffi
from oracle import oracle as o


def test_library_is_in_tree_and_exports_every_declared_symbol():
    assert os.path.exists(_ffi.LIB_PATH)
    L = b2.lib()
    names = _ffi.declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(L, n), n
    assert L.b2_abi_version() == 2
    assert C.sizeof(_ffi.MuonSlotDescriptor) == 104  # args/muon.rs:3-21, padded


def test_csf_host_matches_oracle():
    rng = np.random.default_rng(0)
    for rows, k in [(128, 128), (129, 256), (768, 3072), (1, 128), (1, 4096), (300, 384)]:
        raw = rng.integers(0, 0x79, rows * k // 16).astype(np.uint8)
        enc = b2.csf_encode_host(raw, rows, k)
        assert len(enc) == b2.csf_encoded_len(rows, k) == o.csf_encoded_len(rows, k)
        assert np.array_equal(enc, o.csf_encode(raw, rows, k))
        for g in rng.integers(0, raw.size, 64):
            assert b2.csf_scale_at(enc, int(g)) == raw[g]
    raw = rng.integers(0, 256, 256 * 8).astype(np.uint8)  # high bit set: two mask bytes per row
    assert np.array_equal(b2.csf_encode_host(raw, 256, 128), o.csf_encode(raw, 256, 128))
    with pytest.raises(ValueError):
        b2.csf_encode_host(np.zeros(8, np.uint8), 2, 64)


def test_host_schedules_match_oracle():
    L = o.lib()
    for step in [1, 2, 5, 6, 17, 1000]:
        assert b2.schedule_free_beta(step) == L.orc_schedule_free_beta(step, 5, np.float32(0.2), np.float32(0.5))
        assert b2.warmup_multiplier(step) == L.orc_warmup_only(step, 5, np.float32(0.05))
    avg = b2.AverageCoefficient()
    ws = C.c_float(0.0)
    for step in range(1, 12):
        assert avg.step(step) == L.orc_schedule_free_average_coefficient(step, 5, np.float32(0.05), C.byref(ws))


def test_shard_plan_is_deterministic_and_balanced():
    from llmini_b200.dist import shard_plan
    shapes = []
    for _ in range(48):
        shapes += [(4800, 1600), (1600, 1600), (6400, 1600), (1600, 6400)]
    for world in (1, 2, 4, 8):
        owner, load = shard_plan(shapes, world)
        owner2, _ = shard_plan(shapes, world)
        assert owner == owner2 and set(owner) == set(range(world))
        assert max(load) / (sum(load) / world) < 1.02
    owner, load = shard_plan([(64, 64), (0, 0), (32, 64)], 4)
    assert len(owner) == 3


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_compute_entry_points_fail_loudly_without_a_gpu():
    L = b2.lib()
    rows = (C.c_uint32 * 1)(64)
    cols = (C.c_uint32 * 1)(128)
    n = L.b2_muon_workspace_bytes(rows, cols, 1, None)
    assert n > 0
    h = C.c_void_p()
    rc = L.b2_muon_plan_create(C.byref(h), rows, cols, 1, None, 1024, n, None)
    assert rc != 0 and not h.value
    assert L.b2_verify_storage_layout(None) != 0
    a = _ffi.AdamWUpdateArgs()
    assert L.b2_apply_fp32_adamw_update(C.byref(a), None) == _ffi.ERROR_INVALID_VALUE


def test_argument_validation():
    L = b2.lib()
    rows = (C.c_uint32 * 1)(64)
    cols = (C.c_uint32 * 1)(40)  # not a multiple of 16
    assert L.b2_muon_workspace_bytes(rows, cols, 1, None) == 0
    cols = (C.c_uint32 * 1)(48)  # CSF needs a multiple of 128
    assert L.b2_muon_workspace_bytes(rows, cols, 1, None) == 0
    opt = _ffi.MuonOptions(0, _ffi.SCALES_RAW, 0, 5)
    assert L.b2_muon_workspace_bytes(rows, cols, 1, C.byref(opt)) > 0
    assert L.b2_muon_workspace_bytes(rows, cols, 0, None) == 0


def test_sizes_beyond_the_32_bit_limits_are_refused():
    # elements and 2048-value chunks are indexed in 32 bits and GEMM tile indices in 16: anything larger is
    # refused up front instead of wrapping inside a kernel
    L = b2.lib()
    INVALID = _ffi.ERROR_INVALID_VALUE
    raw = _ffi.MuonOptions(0, _ffi.SCALES_RAW, 0, 5)
    one = lambda r, c: ((C.c_uint32 * 1)(r), (C.c_uint32 * 1)(c))
    rows, cols = one(16 * 1024 * 1024, 16)          # 131072 row tiles of 128: beyond a 16-bit tile index
    assert L.b2_muon_workspace_bytes(rows, cols, 1, C.byref(raw)) == 0
    rows, cols = one(65535 * 128, 16)               # the largest admissible extent
    assert L.b2_muon_workspace_bytes(rows, cols, 1, C.byref(raw)) > 0
    rows, cols = one(65536, 65536)                  # 2^32 elements
    assert L.b2_muon_workspace_bytes(rows, cols, 1, C.byref(raw)) == 0
    big = 0xfffff800                                 # (len + 2047) / 2048 would wrap in 32 bits
    fake = 4096                                      # never dereferenced: the size check comes first
    assert L.b2_tensor_amax_f32(fake, fake, fake, big, None) == INVALID
    assert L.b2_materialize_master(fake, fake, fake, fake, fake, fake, big, _ffi.SCALES_RAW, None) == INVALID
    assert L.b2_fp32_to_nvfp4_four_six(fake, fake, fake, fake, fake, big // 16, _ffi.SCALES_RAW, None) == INVALID
    assert L.b2_materialize_master_static(fake, fake, fake, fake, (1 << 26) + 16, _ffi.SCALES_RAW, None) == INVALID
    sf = _ffi.ScheduleFreeMaterializeArgs(fake, fake, fake, fake, fake, None, fake, big, 1 << 16, 1 << 16, 0.5, 0.0,
                                          _ffi.SCALES_RAW, (C.c_void_p * 6)())
    assert L.b2_materialize_schedule_free(C.byref(sf), None) == INVALID
    ad = _ffi.AdamWUpdateArgs()
    ad.z_master = ad.x_master = ad.grad = ad.first_moment = ad.second_moment = fake
    ad.len = big
    assert L.b2_apply_fp32_adamw_update(C.byref(ad), None) == INVALID
    t = (_ffi.AdamWSlotDescriptor * 1)()
    t[0].z_master = t[0].x_master = t[0].grad = t[0].first_moment = t[0].second_moment = fake
    t[0].len = big
    total = C.c_uint32(0)
    assert L.b2_adamw_table_prepare(t, 1, C.byref(total)) == INVALID


def test_one_pass_prepare_is_refused_for_f16_operands():
    L = b2.lib()
    rows, cols = (C.c_uint32 * 1)(64), (C.c_uint32 * 1)(64)
    opt = _ffi.MuonOptions(_ffi.OPERAND_F16, _ffi.SCALES_RAW, 0, 5, 0, 0, 0, _ffi.NORMALIZE_DEFERRED)
    h = C.c_void_p()
    n = L.b2_muon_workspace_bytes(rows, cols, 1, C.byref(opt))
    assert L.b2_muon_plan_create(C.byref(h), rows, cols, 1, C.byref(opt), 1024, n, None) == _ffi.ERROR_INVALID_VALUE
