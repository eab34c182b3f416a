"""Newton-Schulz GEMMs (tcgen05/TMEM/TMA) against the oracle with the same operand rounding.

Tolerances: intermediates after one GEMM differ only by FP32 accumulation order, so 16-bit
results may differ by one unit in the last place on a small fraction of entries; the full
iteration is held to relative L2 <= 2e-3 and max error <= 2e-2 of the peak entry, an order
tighter than the 2e-2 relative bound the path is specified to.
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
    return o.round_bf16(x) if fmt == b2.OPERAND_BF16 else np.vectorize(o.lib().orc_round_f16, otypes=[F])(x)


def _run(shapes, fmt, iterations, coeffs, tile_n, xs):
    opt = b2.OptimizerModule()
    plan = b2.MuonPlan(shapes, operand_format=fmt, scale_layout=b2.SCALES_RAW, tile_n=tile_n)
    for i, x in enumerate(xs):
        t = plan.scratch(i, 0)
        t.copy_(dev(x).to(t.dtype))
    opt.muon_polar(plan, b2.MuonMegaUpdateArgs(iterations=iterations, coefficients=coeffs))
    torch.cuda.synchronize()
    assert plan.status() == 0
    return plan


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("fmt", [b2.OPERAND_BF16, b2.OPERAND_F16])
@pytest.mark.parametrize("rows,cols", [(64, 256), (256, 64), (128, 128), (96, 160), (160, 96), (320, 832), (832, 320)])
def test_single_iteration_intermediates(rows, cols, fmt, tile_n):
    rng = np.random.default_rng(rows * 7 + cols)
    x = _x0(rng, rows, cols, fmt)
    co = o.polar_express_coefficients(1) if fmt == b2.OPERAND_F16 else o.fixed_coefficients(1)
    plan = _run([(rows, cols)], fmt, 1, co, tile_n, [x])
    mode = o.ROUND_BF16 if fmt == b2.OPERAND_BF16 else o.ROUND_F16
    rnd = np.vectorize(lambda v: o.lib().orc_round_operand(v, mode), otypes=[F])
    xs = x if rows <= cols else np.ascontiguousarray(x.T)   # polar orientation [n][m]
    n = min(rows, cols)
    G = (xs.astype(np.float64) @ xs.T.astype(np.float64)).astype(F)
    g16 = host(plan.scratch(0, 5).float())
    ulp = 2.0 ** (-8 if fmt == b2.OPERAND_BF16 else -11)
    assert np.all(np.abs(g16 - rnd(G)) <= 1.01 * ulp * np.abs(G) + 1e-6 * np.max(np.abs(G)))
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


@pytest.mark.parametrize("shapes", [
    [(768, 768), (768, 3072), (3072, 768), (2304, 768)],
    [(1600, 1600), (1600, 320), (48, 1600)],
])
def test_five_iterations_multi_slot(shapes):
    rng = np.random.default_rng(len(shapes) * 97 + shapes[0][0])
    xs = [_x0(rng, r, c, b2.OPERAND_BF16) for r, c in shapes]
    co = o.fixed_coefficients(5)
    plan = _run(shapes, b2.OPERAND_BF16, 5, co, 0, xs)
    for i, x in enumerate(xs):
        want = o.polar(x, 5, co, round_mode=o.ROUND_BF16)
        got = host(plan.scratch(i, 1))
        assert np.isfinite(got).all()
        r2, mx = U.rel_l2(got, want), U.max_rel_to_peak(got, want)
        print(f"slot {shapes[i]}: rel_l2 {r2:.3e} max/peak {mx:.3e}")
        assert r2 <= 2e-2 and mx <= 2e-2
        # orthogonality sanity: singular values of the result sit in the Newton-Schulz band
        sv = np.linalg.svd(got.astype(np.float64), compute_uv=False)
        assert 0.3 < sv.min() and sv.max() < 1.6
    plan.close()
