"""b2_materialize_master_static: the requantiser for callers that have no scratch buffers to
pass and must not allocate (an export or evaluation hook that only holds the weights).

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test.  The new entry point is called through the C ABI and must reproduce the
regular `materialize_master` bit for bit, on two calls in a row that share the library's
built-in scratch array."""
import numpy as np
import pytest
import torch

import llmini_b200 as b2
from oracle import oracle as o
from tests.gpu_util import host, rcp_table

pytestmark = pytest.mark.gpu


def _reference(opt, x, rows, k, layout):
    n = rows * k
    t = b2.Nvfp4Tensor.empty(rows, k, layout)
    amax = torch.zeros(1, device="cuda")
    chunk = torch.zeros((n + 2047) // 2048, device="cuda")
    opt.materialize_master(t.bytes, t.scales, t.global_scale, x, amax, chunk, n, layout)
    return t


def _static(opt, x, rows, k, layout):
    t = b2.Nvfp4Tensor.empty(rows, k, layout)
    opt.materialize_master_static(t.bytes, t.scales, t.global_scale, x, rows * k, layout)
    return t


def test_static_scratch_matches_materialize_master_on_consecutive_calls():
    opt = b2.OptimizerModule()
    g = torch.Generator(device="cuda").manual_seed(7)
    # the second tensor is shorter and much smaller in magnitude than the first: stale chunk maxima
    # left in the shared array by the first call must not leak into the second
    cases = [(3072, 768, b2.SCALES_CSF, 1.0), (129, 256, b2.SCALES_CSF, 1e-3), (7, 48, b2.SCALES_RAW, 0.02)]
    for rows, k, layout, std in cases:
        x = torch.randn(rows * k, device="cuda", generator=g) * std
        want = _reference(opt, x, rows, k, layout)
        got = _static(opt, x, rows, k, layout)
        torch.cuda.synchronize()
        assert torch.equal(got.bytes, want.bytes)
        assert torch.equal(got.scales, want.scales)
        assert torch.equal(got.global_scale, want.global_scale)
        amax = np.float32(x.abs().max().item())
        assert got.global_scale.item() == np.float32(amax / np.float32(1536.0))
        # and against the CPU oracle, not only against the library's other entry point
        gs = host(got.global_scale)[0]
        codes, raw, ogs, misses = o.nvfp4_quantize(host(x), amax=amax, rcp_table=rcp_table(gs))
        assert misses == 0 and gs == ogs
        assert np.array_equal(host(got.bytes), codes)
        got_raw = host(got.scales) if layout == b2.SCALES_RAW else o.csf_decode_matrix(host(got.scales), rows, k)
        assert np.array_equal(got_raw[: rows * k // 16], raw)


def test_second_call_on_a_device_reserves_nothing():
    # The first call on a device resolves the built-in array's address (and, with lazy module loading, is when
    # the driver sets the array aside); from then on a call must leave the device's free memory untouched.
    opt = b2.OptimizerModule()
    x = torch.randn(4096, device="cuda")
    t = b2.Nvfp4Tensor.empty(1, 4096, b2.SCALES_RAW)
    opt.materialize_master_static(t.bytes, t.scales, t.global_scale, x, 4096, b2.SCALES_RAW)   # warm-up call
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    opt.materialize_master_static(t.bytes, t.scales, t.global_scale, x, 4096, b2.SCALES_RAW)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_static_scratch_at_its_maximum_size():
    # exactly B2_STATIC_MAX_ELEMENTS values (256 MiB of FP32): every entry of the built-in array is in use
    opt = b2.OptimizerModule()
    n = opt.STATIC_MAX_ELEMENTS
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(n, device="cuda", generator=g) * 0.02
    x[n - 1] = 3.0   # the tensor maximum sits in the last chunk
    want = _reference(opt, x, n // 4096, 4096, b2.SCALES_RAW)
    got = _static(opt, x, n // 4096, 4096, b2.SCALES_RAW)
    torch.cuda.synchronize()
    assert got.global_scale.item() == np.float32(np.float32(3.0) / np.float32(1536.0))
    assert torch.equal(got.bytes, want.bytes) and torch.equal(got.scales, want.scales)


def test_static_scratch_limits_are_enforced():
    opt = b2.OptimizerModule()
    x = torch.zeros(32, device="cuda")
    t = b2.Nvfp4Tensor.empty(1, 32, b2.SCALES_RAW)
    with pytest.raises(b2.B2Error) as e:
        opt.materialize_master_static(t.bytes, t.scales, t.global_scale, x, (1 << 26) + 16, b2.SCALES_RAW)
    assert e.value.code == 1
    with pytest.raises(b2.B2Error):
        opt.materialize_master_static(t.bytes, t.scales, t.global_scale, x, 24, b2.SCALES_RAW)  # not a multiple of 16
    # an all-zero tensor still gets the neutral tensor scale
    opt.materialize_master_static(t.bytes, t.scales, t.global_scale, x, 32, b2.SCALES_RAW)
    torch.cuda.synchronize()
    assert float(t.global_scale) == 1.0 and not bool(t.bytes.any())
