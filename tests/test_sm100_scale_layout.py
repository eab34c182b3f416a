"""The block-scale operand layout of sm_100 tensor cores (`tcgen05.mma kind::mxf4nvf4.block_scale`):
oracle against the published offset formula (CPU), converter and direct emission against the
oracle (GPU), and a library NVFP4 GEMM consuming codes + scales exactly as this build writes them."""
import numpy as np
import pytest
import torch

import llmini_b200 as b2
from oracle import oracle as o
from tests import _util as U

F = np.float32


@pytest.mark.parametrize("rows,cols", [(128, 64), (1, 16), (200, 1040), (384, 4096), (33, 48)])
def test_oracle_blocked_layout_matches_offset_formula(rows, cols):
    per_row = cols // 16
    raw = np.random.default_rng(rows).integers(0, 256, size=rows * per_row).astype(np.uint8)
    blocked = o.sm100_blocked(raw, rows, cols)
    kb_tiles = -(-per_row // 4)
    assert blocked.size == -(-rows // 128) * kb_tiles * 512 == b2.sm100_scales_bytes(rows, cols)
    r, kb = np.divmod(np.arange(rows * per_row), per_row)
    off = ((r >> 7) * kb_tiles + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)
    assert np.array_equal(blocked[off], raw)
    mask = np.ones(blocked.size, bool)
    mask[off] = False
    assert not blocked[mask].any()          # padding is zero
    assert np.array_equal(o.sm100_unblocked(blocked, rows, cols), raw)


def test_converter_rejects_bad_arguments_without_a_device():
    L = b2.lib()
    assert L.b2_nvfp4_scales_to_sm100(None, 1, 128, 64, None, None) == 1
    # the sm_100 layout needs the row length, which the flat quantiser is not given: it refuses it
    import ctypes as C
    dummy = C.c_void_p(16)
    assert L.b2_fp32_to_nvfp4_four_six(dummy, dummy, dummy, dummy, dummy, 8, b2.SCALES_SM100, None) == 1
    assert b2.sm100_scales_bytes(0, 64) == 0 and b2.sm100_scales_bytes(129, 80) == 2 * 2 * 512


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,src", [(200, 1040, b2.SCALES_RAW), (384, 512, b2.SCALES_CSF),
                                           (128, 128, b2.SCALES_CSF), (7, 16, b2.SCALES_RAW)])
def test_converter_matches_oracle(rows, cols, src):
    from tests.gpu_util import dev, host
    per_row = cols // 16
    raw = np.random.default_rng(7).integers(0, 127, size=rows * per_row).astype(np.uint8)
    stored = raw if src == b2.SCALES_RAW else b2.csf_encode_host(raw, rows, cols)
    got = host(b2.scales_to_sm100(dev(stored), src, rows, cols))
    assert np.array_equal(got, o.sm100_blocked(raw, rows, cols))


@pytest.mark.gpu
def test_muon_step_emits_the_layout_directly():
    # the same update + quantisation with raw and with sm_100 scale storage: same codes, and the
    # sm_100 bytes are the blocked form of the raw plane (padding untouched)
    from tests.gpu_util import dev, host
    shapes = [(384, 256), (100, 48), (0, 0), (128, 1040)]
    outs = {}
    for layout in (b2.SCALES_RAW, b2.SCALES_SM100):
        rng = np.random.default_rng(3)
        slots = [b2.MuonSlot.allocate(r, c, layout) for r, c in shapes]
        plan = b2.MuonPlan(shapes, scale_layout=layout)
        for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
            if r * c:
                s.z_master.copy_(dev(U.weights(rng, r * c)).view(r, c))
                s.x_master.copy_(dev(U.weights(rng, r * c)).view(r, c))
        table = b2.slot_table(slots)
        opt = b2.OptimizerModule()
        opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
        for k, (r, c) in enumerate(shapes):
            if r * c:
                plan.scratch(k, 1).copy_(dev((rng.standard_normal(r * c) * 0.05).astype(F)).view(r, c))
        opt.muon_tma_finish_update(plan, table, b2.MuonMegaUpdateArgs(learning_rate=0.02, average_coefficient=0.3,
                                                                     schedule_beta=0.6))
        torch.cuda.synchronize()
        assert plan.status() == 0
        outs[layout] = [(host(s.bytes).copy(), host(s.scales).copy(), host(s.global_scale).copy()) for s in slots]
        plan.close()
    for (r, c), a, b in zip(shapes, outs[b2.SCALES_RAW], outs[b2.SCALES_SM100]):
        if r * c == 0:
            continue
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[2], b[2])
        assert np.array_equal(b[1], o.sm100_blocked(a[1][: r * c // 16], r, c))


@pytest.mark.gpu
def test_library_nvfp4_gemm_consumes_codes_and_scales_as_written():
    # C = A * W^T on the tensor cores' block-scaled FP4 path (cuBLASLt through torch._scaled_mm),
    # fed with this build's packed codes and its sm_100 scale layout, against the same product of
    # the dequantised operands.  A wrong nibble order or scale placement gives errors of order one.
    from tests.gpu_util import dev, host
    if not hasattr(torch, "float4_e2m1fn_x2"):
        pytest.skip("this torch build has no packed FP4 dtype")
    M, N, K = 256, 384, 512
    rng = np.random.default_rng(11)
    opt = b2.OptimizerModule()

    def quantise(x2d):
        rows, cols = x2d.shape
        n = rows * cols
        t = b2.Nvfp4Tensor.empty(rows, cols, b2.SCALES_RAW)
        opt.materialize_master(t.bytes, t.scales, t.global_scale, dev(x2d.reshape(-1)), torch.zeros(1, device="cuda"),
                               torch.zeros((n + 2047) // 2048, device="cuda"), n, b2.SCALES_RAW)
        torch.cuda.synchronize()
        codes, raw, gs = host(t.bytes), host(t.scales)[: n // 16], float(host(t.global_scale)[0])
        return t, o.nvfp4_dequantize(codes, raw, gs).reshape(rows, cols).astype(np.float64), gs

    # rows of very different magnitude, so that a misplaced scale cannot go unnoticed
    a = (rng.standard_normal((M, K)) * np.exp(rng.uniform(-3, 0, size=(M, 1)))).astype(F)
    w = (rng.standard_normal((N, K)) * 0.02 * np.exp(rng.uniform(-2, 2, size=(N, 1)))).astype(F)
    ta, da, gsa = quantise(a)
    tw, dw, gsw = quantise(w)
    sa = b2.scales_to_sm100(ta.scales, b2.SCALES_RAW, M, K).view(torch.float8_e4m3fn)
    sw = b2.scales_to_sm100(tw.scales, b2.SCALES_RAW, N, K).view(torch.float8_e4m3fn)
    a4 = ta.bytes.view(M, K // 2).view(torch.float4_e2m1fn_x2)
    w4 = tw.bytes.view(N, K // 2).view(torch.float4_e2m1fn_x2)
    try:
        c = torch._scaled_mm(a4, w4.t(), sa, sw, out_dtype=torch.bfloat16)
    except (RuntimeError, NotImplementedError, TypeError) as exc:
        pytest.skip(f"torch._scaled_mm does not take NVFP4 operands here: {str(exc)[:120]}")
    got = host(c.float()).astype(np.float64) * gsa * gsw
    want = da @ dw.T
    err = np.abs(got - want)
    bound = np.abs(da) @ np.abs(dw.T) * 2.0 ** -7 + 1e-12   # bf16 output rounding + fp32 accumulation
    assert np.all(err <= bound), float(np.max(err / bound))
    assert np.linalg.norm(got - want) <= 4e-3 * np.linalg.norm(want)
