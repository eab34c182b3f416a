"""Golden fixtures (tests/golden/, made by make_golden.py from the oracle): the oracle must
keep reproducing them bit for bit on the CPU, and the CUDA library must match them on the GPU."""
import os

import numpy as np
import pytest

from oracle import oracle as o

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "muon_nvfp4_64x128.npz"))
F = np.float32


def test_oracle_reproduces_quantiser_and_csf_golden():
    codes, raw, gs, _ = o.nvfp4_quantize(G["x"])
    assert np.array_equal(codes, G["q_codes"]) and np.array_equal(raw, G["q_raw_scales"]) and gs == G["q_global_scale"]
    assert np.array_equal(o.csf_encode(raw, int(G["rows"]), int(G["cols"])), G["q_csf"])
    assert np.array_equal(o.csf_decode_matrix(G["q_csf"], int(G["rows"]), int(G["cols"])), raw)


def test_oracle_reproduces_elementwise_golden():
    m2, u, ss = o.momentum(G["grad"], G["momentum_bits"], 0.95, 1.0)
    assert np.array_equal(m2, G["mom_bits"]) and np.array_equal(u, G["mom_u"]) and ss == float(G["mom_sumsq"])
    z = G["z"]
    az, ax, ay, a1, a2, am = o.adamw(z, G["x"], G["grad"], np.zeros_like(z), np.zeros_like(z), 1.0, 2e-4, 0.005, 0.9,
                                     0.95, 0.1, 0.05, 1e-10, 0.5, 0.2)
    for got, key in ((az, "adam_z"), (ax, "adam_x"), (ay, "adam_y"), (a1, "adam_m1"), (a2, "adam_m2")):
        assert np.array_equal(got, G[key]), key
    assert am == G["adam_amax"]


def test_oracle_step_golden_within_gemm_reassociation():
    # the oracle's GEMMs are vectorised with reassociation allowed, so the whole step is pinned
    # to a tolerance (and the state that does not depend on the GEMMs bit for bit)
    rows, cols = int(G["rows"]), int(G["cols"])
    r = o.muon_step(G["grad"], G["momentum_bits"], G["z"], G["x"], rows, cols, mu=0.95, grad_scale=1.0, lr=0.02,
                    wd=0.025, c_avg=0.5, sched_beta=0.2, iterations=5, coeffs=o.fixed_coefficients(5),
                    round_mode=o.ROUND_BF16)
    assert np.array_equal(r.momentum_bits, G["step_momentum_bits"])
    assert np.linalg.norm(r.U - G["step_U"]) <= 2e-2 * np.linalg.norm(G["step_U"])
    assert np.max(np.abs(r.z - G["step_z"])) <= 0.02 * 0.2 * np.sqrt(128.0) * 0.1 * np.max(np.abs(G["step_U"]))


@pytest.mark.gpu
def test_gpu_matches_golden():
    import torch

    import llmini_b200 as b2
    from tests.gpu_util import bf16_bits, bf16_from_bits, dev, host, rcp_table

    rows, cols = int(G["rows"]), int(G["cols"])
    n = rows * cols
    # quantiser: bit-exact against the stored codes / CSF storage / tensor scale
    q = b2.Nvfp4QuantModule()
    t = b2.Nvfp4Tensor.empty(rows, cols)
    amax, chunk = torch.zeros(1, device="cuda"), torch.zeros((n + 2047) // 2048, device="cuda")
    b2.OptimizerModule().materialize_master(t.bytes, t.scales, t.global_scale, dev(G["x"]), amax, chunk, n)
    torch.cuda.synchronize()
    gs = host(t.global_scale)[0]
    assert gs == G["q_global_scale"]
    # the fixture was made with the correctly rounded reciprocal; re-derive with the device's
    codes, raw, _, _ = o.nvfp4_quantize(G["x"], rcp_table=rcp_table(gs))
    assert np.array_equal(host(t.bytes), codes)
    assert np.count_nonzero(host(t.bytes) != G["q_codes"]) <= 2
    assert np.array_equal(o.csf_decode_matrix(host(t.scales), rows, cols), G["q_raw_scales"])
    # whole step: BF16 state bit-exact, weights within the Newton-Schulz tolerance
    s = b2.MuonSlot.allocate(rows, cols)
    s.grad.copy_(dev(G["grad"]).view(rows, cols))
    s.momentum.copy_(bf16_from_bits(G["momentum_bits"]).view(rows, cols))
    s.z_master.copy_(dev(G["z"]).view(rows, cols))
    s.x_master.copy_(dev(G["x"]).view(rows, cols))
    plan = b2.MuonPlan([(rows, cols)])
    b2.OptimizerModule().muon_mega_update(plan, b2.slot_table([s]), b2.MuonMegaUpdateArgs(
        learning_rate=0.02, average_coefficient=0.5, schedule_beta=0.2, coefficients=o.fixed_coefficients(5)))
    torch.cuda.synchronize()
    assert plan.status() == 0
    assert np.array_equal(bf16_bits(s.momentum).ravel(), G["step_momentum_bits"])
    U = host(plan.scratch(0, 1))
    assert np.linalg.norm(U - G["step_U"]) <= 2e-2 * np.linalg.norm(G["step_U"])
    assert np.max(np.abs(host(s.z_master).ravel() - G["step_z"])) <= 0.02 * 0.2 * np.sqrt(128.0) * 0.1 * np.max(np.abs(G["step_U"]))
    plan.close()
