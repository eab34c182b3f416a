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
