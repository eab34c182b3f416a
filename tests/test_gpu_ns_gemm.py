"""Newton-Schulz GEMMs (tcgen05/TMEM/TMA) against the oracle with the same operand rounding.

Tolerances: intermediates after one GEMM differ only by FP32 accumulation order, so 16-bit
results may differ by one unit in the last place on a small fraction of entries; the full
single iteration is held to relative L2 <= 2e-3.  Over five iterations with the fixed
coefficient triple the map amplifies perturbations (|p'(s)| is about 1.6 inside the band the
singular values oscillate in), so two BF16 implementations that round at identical points but
accumulate in a different order already differ by about 1e-2: the five-iteration bound is
relative L2 <= 2e-2 (the stated tolerance of the path), with a loose sanity bound of 1e-1 of the
peak entry on the largest single-entry difference.
"""
import numpy as np
import pytest
import torch

import llmini_b200 as b2
from oracle import oracle as o
from tests import _util as U
from tests.gpu_util import dev, host

pytestmark = pytest.mark.gpu
F = np.float32


def _x0(rng, rows, cols, fmt):
    x = (rng.standard_normal((rows, cols))).astype(F)
    x = x / (np.linalg.norm(x) * 1.01)
    return o.round_bf16(x) if fmt == b2.OPERAND_BF16 else x.astype(np.float16).astype(F)


def _run(shapes, fmt, iterations, coeffs, tile_n, xs, schedule=b2.NS_PER_PHASE):
    opt = b2.OptimizerModule()
    plan = b2.MuonPlan(shapes, operand_format=fmt, scale_layout=b2.SCALES_RAW, tile_n=tile_n, max_iterations=iterations,
                       ns_schedule=schedule)
    for i, x in enumerate(xs):
        t = plan.scratch(i, 0)
        t.copy_(dev(x).to(t.dtype))
    opt.muon_polar(plan, b2.MuonMegaUpdateArgs(iterations=iterations, coefficients=coeffs))
    torch.cuda.synchronize()
    assert plan.status() == 0
    return plan


@pytest.mark.parametrize("schedule", [b2.NS_CHAINED, b2.NS_PER_PHASE, b2.NS_FUSED_GRAM_POLY])
@pytest.mark.parametrize("tile_n", [128, 256, 512])  # 512 = two-CTA 256 x 256 tiles
@pytest.mark.parametrize("fmt", [b2.OPERAND_BF16, b2.OPERAND_F16])
@pytest.mark.parametrize("rows,cols", [(64, 256), (256, 64), (128, 128), (96, 160), (160, 96), (320, 832), (832, 320)])
def test_single_iteration_intermediates(rows, cols, fmt, tile_n, schedule):
    rng = np.random.default_rng(rows * 7 + cols)
    x = _x0(rng, rows, cols, fmt)
    co = o.polar_express_coefficients(1) if fmt == b2.OPERAND_F16 else o.fixed_coefficients(1)
    plan = _run([(rows, cols)], fmt, 1, co, tile_n, [x], schedule)
    mode = o.ROUND_BF16 if fmt == b2.OPERAND_BF16 else o.ROUND_F16
    rnd = (lambda a: o.round_bf16(a)) if fmt == b2.OPERAND_BF16 else (lambda a: np.asarray(a, F).astype(np.float16).astype(F))
    xs = x if rows <= cols else np.ascontiguousarray(x.T)   # polar orientation [n][m]
    n = min(rows, cols)
    G = (xs.astype(np.float64) @ xs.T.astype(np.float64)).astype(F)
    g16 = host(plan.scratch(0, 5).float())
    ulp = 2.0 ** (-7 if fmt == b2.OPERAND_BF16 else -10)  # one unit in the last place of the 16-bit type
    tiny = 0.0 if fmt == b2.OPERAND_BF16 else 2.0 ** -24   # binary16 subnormal spacing
    assert np.all(np.abs(g16 - rnd(G)) <= 1.01 * ulp * np.abs(G) + 1e-6 * np.max(np.abs(G)) + tiny)
    assert np.mean(g16 != rnd(G)) < 0.02
    a, b, c = (F(v) for v in co[0])
    Gr = rnd(G).astype(np.float64)
    Q = (c * (Gr @ Gr) + b * G.astype(np.float64) + a * np.eye(n)).astype(F)
    q16 = host(plan.scratch(0, 6).float())
    assert np.all(np.abs(q16 - rnd(Q)) <= 3 * ulp * np.abs(Q) + 2e-5 * np.max(np.abs(Q)))
    want = o.polar(x, 1, co, round_mode=mode)
    got = host(plan.scratch(0, 1))
    assert U.rel_l2(got, want) <= 2e-3 and U.max_rel_to_peak(got, want) <= 2e-2
    plan.close()


@pytest.mark.parametrize("schedule", [b2.NS_CHAINED, b2.NS_PER_PHASE, b2.NS_FUSED_GRAM_POLY])
@pytest.mark.parametrize("tile_n", [0, 256])
@pytest.mark.parametrize("shapes", [
    [(768, 768), (768, 3072), (3072, 768), (2304, 768)],
    [(1600, 1600), (1600, 320), (48, 1600)],
])
def test_five_iterations_multi_slot(shapes, tile_n, schedule):
    rng = np.random.default_rng(len(shapes) * 97 + shapes[0][0])
    xs = [_x0(rng, r, c, b2.OPERAND_BF16) for r, c in shapes]
    co = o.fixed_coefficients(5)
    plan = _run(shapes, b2.OPERAND_BF16, 5, co, tile_n, xs, schedule)
    for i, x in enumerate(xs):
        want = o.polar(x, 5, co, round_mode=o.ROUND_BF16)
        got = host(plan.scratch(i, 1))
        assert np.isfinite(got).all()
        r2, mx = U.rel_l2(got, want), U.max_rel_to_peak(got, want)
        print(f"slot {shapes[i]}: rel_l2 {r2:.3e} max/peak {mx:.3e}")
        assert r2 <= 2e-2 and mx <= 1e-1
        # orthogonality sanity: the bulk of the singular values sits in the Newton-Schulz band
        sv = np.linalg.svd(got.astype(np.float64), compute_uv=False)
        assert sv.max() < 1.6 and np.median(sv) > 0.5
    plan.close()


@pytest.mark.parametrize("tile_n", [0, 128, 256])
@pytest.mark.parametrize("shapes", [
    [(768, 768), (768, 3072), (3072, 768), (2304, 768), (0, 0), (768, 768)],
    [(1600, 1600), (1600, 320), (48, 1600), (4800, 1600)],
    [(64, 64)],
    # 13 x 13 pair tiles = 91 Gram tiles, more than the device runs CTA pairs at once: the fused form must step
    # aside (a pair waiting for tiles that no resident pair can take would wait for ever)
    [(3328, 3328), (256, 512)],
])
def test_chained_launch_equals_the_per_phase_launches_bit_for_bit(shapes, tile_n):
    # The chained launch runs the same tiles with the same k order as the fifteen per-phase launches; only the
    # ordering between tiles differs (per-matrix progress counts instead of launch boundaries), so every
    # intermediate and the result must be identical, and its progress words must be zero again afterwards.
    rng = np.random.default_rng(31 + len(shapes))
    xs = [_x0(rng, r, c, b2.OPERAND_BF16) if r * c else np.zeros((0, 0), F) for r, c in shapes]
    co = o.fixed_coefficients(5)
    live = [(i, x) for i, x in enumerate(xs) if x.size]

    def run(schedule):
        opt = b2.OptimizerModule()
        plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW, tile_n=tile_n, ns_schedule=schedule)
        for i, x in live:
            t = plan.scratch(i, 0)
            t.copy_(dev(x).to(t.dtype))
        for _ in range(2):   # twice: the second run starts from the words the first one left
            for i, x in live:
                t = plan.scratch(i, 0)
                t.copy_(dev(x).to(t.dtype))
            opt.muon_polar(plan, b2.MuonMegaUpdateArgs(iterations=5, coefficients=co))
        torch.cuda.synchronize()
        assert plan.status() == 0
        assert not host(plan.scratch(0, 11)).any()
        out = [[host(plan.scratch(i, w).float()).copy() for w in (1, 5, 6, 7)] for i, _ in live]
        plan.close()
        return out

    b = run(b2.NS_PER_PHASE)
    # (the fused Gram + polynomial form draws its tiles the same way and keeps the FP32 Gram tile in tensor memory
    # instead of reading it back: the same arithmetic again)
    for schedule in (b2.NS_CHAINED, b2.NS_FUSED_GRAM_POLY):
        a = run(schedule)
        for (i, _), ra, rb in zip(live, a, b):
            for w, ta, tb in zip(("U", "Gram", "Q", "X1"), ra, rb):
                assert np.array_equal(ta, tb), (schedule, shapes[i], w)


def test_steps_with_fewer_iterations_take_the_per_phase_launches():
    # a plan made for five iterations asked for three: the chained list does not apply, the result must not change
    rng = np.random.default_rng(5)
    shapes = [(256, 512), (512, 256)]
    xs = [_x0(rng, r, c, b2.OPERAND_BF16) for r, c in shapes]
    co = o.fixed_coefficients(3)
    plan = _run(shapes, b2.OPERAND_BF16, 3, co, 0, xs, b2.NS_CHAINED)                     # max_iterations = 3: chained
    plan5 = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW, ns_schedule=b2.NS_CHAINED)     # made for 5: per phase for 3
    for i, x in enumerate(xs):
        t = plan5.scratch(i, 0)
        t.copy_(dev(x).to(t.dtype))
    b2.OptimizerModule().muon_polar(plan5, b2.MuonMegaUpdateArgs(iterations=3, coefficients=co))
    torch.cuda.synchronize()
    for i in range(len(shapes)):
        assert torch.equal(plan.scratch(i, 1), plan5.scratch(i, 1))
    plan.close()
    plan5.close()
