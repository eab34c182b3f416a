"""Whole Muon + NVFP4 step through `muon_mega_update` against the oracle and the reference's
own known answers."""
import numpy as np
import pytest
import torch

import llmini_b200 as b2
from oracle import oracle as o
from tests import _util as U
from tests.gpu_util import bf16_bits, bf16_from_bits, decode_scales, dev, host, rcp_table

pytestmark = pytest.mark.gpu
F = np.float32


def _slot(rows, cols, grad, mom_bits, z, x, layout):
    s = b2.MuonSlot.allocate(rows, cols, layout)
    s.grad.copy_(dev(grad).view(rows, cols))
    s.momentum.copy_(bf16_from_bits(mom_bits).view(rows, cols))
    s.z_master.copy_(dev(z).view(rows, cols))
    s.x_master.copy_(dev(x).view(rows, cols))
    return s


@pytest.mark.parametrize("rows,cols", [(64, 64), (64, 32), (32, 64)])
def test_reference_constant_gradient_recurrence(rows, cols):
    # crates/cuda-kernels/tests/optimizer/muon/fixture.rs:12-63 — F16 operands, reference
    # coefficient table, one iteration; every z and x within 1e-7 of the closed form.
    n = rows * cols
    layout = b2.SCALES_RAW if cols % 128 else b2.SCALES_CSF
    s = _slot(rows, cols, np.full(n, 0.5, F), np.zeros(n, np.uint16), np.ones(n, F), np.ones(n, F), layout)
    plan = b2.MuonPlan([(rows, cols)], operand_format=b2.OPERAND_F16, scale_layout=layout)
    b2.OptimizerModule().muon_mega_update(plan, b2.slot_table([s]), b2.MuonMegaUpdateArgs(
        mu=0.95, grad_scale=0.5, learning_rate=0.25, weight_decay=0.1, average_coefficient=1.0, iterations=1))
    torch.cuda.synchronize()
    assert plan.status() == 0
    nest = (F(1.0) - F(0.95)) * (F(1.0) + F(0.95)) * F(0.5) * F(0.5)
    upd = F(o.lib().orc_polar_first_iteration_scalar(F(nest), rows, cols))
    expected = (F(1.0) - F(0.25) * F(0.1)) - F(0.25) * upd * (F(0.2) * np.sqrt(F(max(rows, cols))))
    assert np.max(np.abs(host(s.z_master) - expected)) <= 1e-7
    assert np.max(np.abs(host(s.x_master) - expected)) <= 1e-7
    assert abs(host(s.global_scale)[0] - abs(expected) / F(1536.0)) <= 1e-8
    assert host(s.bytes).any() and host(s.scales).any()
    plan.close()


def test_reference_nonconstant_wide_recurrence():
    # crates/cuda-kernels/tests/optimizer/muon/nonconstant.rs:19-75 — 2e-3 absolute against the
    # host three-product oracle with F16 rounding.
    rows, cols, n = 32, 64, 32 * 64
    i = np.arange(n)
    grad = ((i % 37).astype(F) - F(18.0)) * F(0.0003) + (i // cols).astype(F) * F(0.00001)
    s = _slot(rows, cols, grad, np.zeros(n, np.uint16), np.ones(n, F), np.ones(n, F), b2.SCALES_RAW)
    plan = b2.MuonPlan([(rows, cols)], operand_format=b2.OPERAND_F16, scale_layout=b2.SCALES_RAW)
    b2.OptimizerModule().muon_mega_update(plan, b2.slot_table([s]), b2.MuonMegaUpdateArgs(
        mu=0.95, grad_scale=0.5, learning_rate=0.25, weight_decay=0.1, average_coefficient=1.0, iterations=5))
    torch.cuda.synchronize()
    sg = grad * F(0.5)
    mu = F(0.95)
    nest = np.array([np.float32(np.float64(F(1) - mu) * np.float64(g) + np.float64(mu * (F(1) - mu) * g)) for g in sg], F)
    inv = F(1.0) / (np.sqrt(np.sum(nest * nest, dtype=F)) * F(1.01) + F(1.0e-7))
    polar = o.polar((nest * inv).reshape(rows, cols), 5, o.polar_express_coefficients(5),
                    round_mode=o.ROUND_F16_HOST, form="three_product").reshape(-1)
    expected = (F(1.0) - F(0.25) * F(0.1)) - F(0.25) * (F(0.2) * np.sqrt(F(64.0))) * polar
    assert np.max(np.abs(host(s.x_master).ravel() - expected)) <= 2e-3
    assert np.max(np.abs(host(s.z_master).ravel() - expected)) <= 2e-3
    plan.close()


def _check_step(shapes, layout, fmt, coeffs, target=b2.QUANTIZE_X, seed=0, outliers=True,
                normalize=b2.NORMALIZE_TWO_PASS, update_input=b2.UPDATE_F32, schedule=b2.NS_PER_PHASE):
    rng = np.random.default_rng(seed)
    hp = dict(mu=0.95, grad_scale=1.0, learning_rate=0.02, weight_decay=0.025, average_coefficient=0.5,
              schedule_beta=0.2, iterations=5)
    data, slots = [], []
    for r, c in shapes:
        z = U.weights(rng, r * c)
        x = U.weights(rng, r * c)
        g = U.gradients(rng, r * c, outlier_fraction=0.001 if outliers else 0.0)
        m = o.bf16_bits(U.gradients(rng, r * c, outlier_fraction=0.0))
        data.append((g, m, z, x))
        slots.append(_slot(r, c, g, m, z, x, layout))
    deferred = normalize == b2.NORMALIZE_DEFERRED
    plan = b2.MuonPlan(shapes, operand_format=fmt, scale_layout=layout, quantize_target=target, normalize_mode=normalize,
                       update_input=update_input, ns_schedule=schedule)
    b2.OptimizerModule().muon_mega_update(plan, b2.slot_table(slots), b2.MuonMegaUpdateArgs(coefficients=coeffs, **hp))
    torch.cuda.synchronize()
    assert plan.status() == 0
    mode = o.ROUND_BF16 if fmt == b2.OPERAND_BF16 else o.ROUND_F16
    for i, (s, (r, c)) in enumerate(zip(slots, shapes)):
        if r * c == 0:
            continue
        g, m, z, x = data[i]
        # the oracle rounds the operand where the plan does: after the Frobenius scaling (the reference's
        # order) or before it (one-pass prepare)
        ref = o.muon_step(g, m, z, x, r, c, mu=0.95, grad_scale=1.0, lr=0.02, wd=0.025, c_avg=0.5, sched_beta=0.2,
                          iterations=5, coeffs=coeffs, round_mode=mode, quantize_y=(target == b2.QUANTIZE_Y),
                          deferred_normalize=deferred)
        assert np.array_equal(bf16_bits(s.momentum).ravel(), ref.momentum_bits)   # bit-exact in both orders
        # the Newton-Schulz result as stage U reads it: FP32, or the 16-bit buffer the fifth iteration wrote
        Ug = host(plan.scratch(i, 1)) if update_input == b2.UPDATE_F32 else host(plan.scratch(i, 7).float())
        r2, mx = U.rel_l2(Ug, ref.U), U.max_rel_to_peak(Ug, ref.U)
        print(f"slot {i} {r}x{c}: NS rel_l2 {r2:.3e} max/peak {mx:.3e}")
        assert r2 <= 2e-2 and mx <= 1e-1          # Newton-Schulz in 16-bit operands (see test_gpu_ns_gemm)
        if deferred:
            # Against the reference's rounding order the result differs by one more BF16 rounding of the
            # operand, which five iterations of the fixed triple amplify like any other perturbation: the
            # two oracle orders are 1.5e-2 apart from each other on these shapes.
            ref2 = o.muon_step(g, m, z, x, r, c, mu=0.95, grad_scale=1.0, lr=0.02, wd=0.025, c_avg=0.5,
                               sched_beta=0.2, iterations=5, coeffs=coeffs, round_mode=mode)
            r3 = U.rel_l2(Ug, ref2.U)
            print(f"slot {i}: against the two-pass order {r3:.3e}; oracle orders apart {U.rel_l2(ref.U, ref2.U):.3e}")
            assert r3 <= 3e-2
        # elementwise stages given the device's own U: bit-exact
        z2, x2, y2, ax, ay = o.update(Ug, z, x, r, c, 0.02, 0.025, 0.5, 0.2)
        assert np.array_equal(host(s.z_master).ravel(), z2)
        assert np.array_equal(host(s.x_master).ravel(), x2)
        assert np.array_equal(host(s.grad).ravel(), y2)
        assert host(s.schedule_amax)[0] == ay
        # weights against the all-oracle step: bounded by lr * scale * NS error
        scale = 0.2 * np.sqrt(max(r, c))
        tol = 0.02 * scale * 1e-1 * np.max(np.abs(ref.U)) + 1e-7
        assert np.max(np.abs(host(s.z_master).ravel() - ref.z)) <= tol
        # NVFP4 output: bit-exact given identical FP32 pre-quantisation weights
        src, am = (y2, ay) if target == b2.QUANTIZE_Y else (x2, ax)
        gs = host(s.global_scale)[0]
        codes, raw, ogs, misses = o.nvfp4_quantize(src, amax=am, rcp_table=rcp_table(gs))
        assert misses == 0 and gs == ogs
        assert np.array_equal(host(s.bytes)[: r * c // 2], codes)
        assert np.array_equal(decode_scales(s.scales, r, c, layout), raw)
    plan.close()


def test_config1_single_mlp_matrix_fixed_triple_bf16():
    # one GPT-2 MLP matrix 3072 x 768, fixed coefficient triple, BF16 operands, seed 0
    _check_step([(3072, 768)], b2.SCALES_CSF, b2.OPERAND_BF16, o.fixed_coefficients(5), seed=0)


def test_config1_reference_recipe_f16():
    _check_step([(3072, 768)], b2.SCALES_CSF, b2.OPERAND_F16, o.polar_express_coefficients(5), seed=0)


def test_one_gpt2_layer_mixed_shapes_quantise_y():
    _check_step([(2304, 768), (768, 768), (3072, 768), (768, 3072), (0, 0)], b2.SCALES_CSF, b2.OPERAND_BF16,
                o.fixed_coefficients(5), target=b2.QUANTIZE_Y, seed=1, outliers=False)


def test_ragged_shapes_raw_scales():
    _check_step([(1600, 320), (48, 1600), (200, 208)], b2.SCALES_RAW, b2.OPERAND_BF16, o.fixed_coefficients(5), seed=2)


def test_config1_one_pass_prepare():
    # the same matrix with the Frobenius scale deferred into the first iteration
    _check_step([(3072, 768)], b2.SCALES_CSF, b2.OPERAND_BF16, o.fixed_coefficients(5), seed=0,
                normalize=b2.NORMALIZE_DEFERRED)


def test_one_gpt2_layer_one_pass_prepare():
    _check_step([(2304, 768), (768, 768), (3072, 768), (768, 3072), (0, 0)], b2.SCALES_CSF, b2.OPERAND_BF16,
                o.fixed_coefficients(5), seed=4, normalize=b2.NORMALIZE_DEFERRED)


@pytest.mark.parametrize("fmt,coeffs", [(b2.OPERAND_BF16, "fixed"), (b2.OPERAND_F16, "table")])
def test_update_reads_the_16_bit_result(fmt, coeffs):
    # B2_UPDATE_16BIT: the last Apply stores the operand type and stage U reads it; everything downstream of that
    # buffer is still bit-exact against the oracle
    co = o.fixed_coefficients(5) if coeffs == "fixed" else o.polar_express_coefficients(5)
    _check_step([(2304, 768), (768, 768), (768, 3072), (200, 208)], b2.SCALES_RAW, fmt, co, seed=8,
                update_input=b2.UPDATE_16BIT)


def test_16_bit_result_with_one_pass_prepare_and_y_target():
    _check_step([(3072, 768), (768, 3072)], b2.SCALES_CSF, b2.OPERAND_BF16, o.fixed_coefficients(5),
                target=b2.QUANTIZE_Y, seed=9, normalize=b2.NORMALIZE_DEFERRED, update_input=b2.UPDATE_16BIT)


def test_16_bit_result_is_refused_where_statistics_need_fp32():
    shapes = [(128, 256)]
    s = _slot(128, 256, np.zeros(128 * 256, F), np.zeros(128 * 256, np.uint16), np.zeros(128 * 256, F),
              np.zeros(128 * 256, F), b2.SCALES_CSF)
    s.second_momentum = torch.zeros(256, device="cuda")
    plan = b2.MuonPlan(shapes, update_input=b2.UPDATE_16BIT)
    opt, table = b2.OptimizerModule(), b2.slot_table([s])
    with pytest.raises(b2.B2Error) as e:
        opt.muon_tma_finish_update(plan, table, b2.MuonMegaUpdateArgs(normuon=True))
    assert e.value.code == b2._ffi.ERROR_NOT_SUPPORTED
    with pytest.raises(b2.B2Error) as e:
        opt.muon_tma_finish_hyperball_update_deferred_quantization(plan, table, b2.MuonMegaUpdateArgs())
    assert e.value.code == b2._ffi.ERROR_NOT_SUPPORTED
    plan.close()


def test_one_gpt2_layer_chained_newton_schulz():
    # the whole step with the Newton-Schulz loop as one persistent launch, one-pass prepare feeding its first iteration
    _check_step([(2304, 768), (768, 768), (3072, 768), (768, 3072), (0, 0)], b2.SCALES_CSF, b2.OPERAND_BF16,
                o.fixed_coefficients(5), seed=10, normalize=b2.NORMALIZE_DEFERRED, schedule=b2.NS_CHAINED)
    _check_step([(1600, 320), (48, 1600), (200, 208)], b2.SCALES_RAW, b2.OPERAND_F16, o.polar_express_coefficients(5),
                seed=11, schedule=b2.NS_CHAINED, update_input=b2.UPDATE_16BIT)


def test_one_gpt2_layer_fused_gram_poly_newton_schulz():
    # the whole step with the Gram and polynomial tile of a position fused on one CTA pair, against the oracle: with
    # the one-pass prepare (the held Gram accumulator takes s^2 in the first iteration) and with the reference's
    # F16 recipe on ragged shapes; then a GPT-2 XL layer, whose 1600-wide matrices have 28 tiles each
    _check_step([(2304, 768), (768, 768), (3072, 768), (768, 3072), (0, 0)], b2.SCALES_CSF, b2.OPERAND_BF16,
                o.fixed_coefficients(5), seed=12, normalize=b2.NORMALIZE_DEFERRED, schedule=b2.NS_FUSED_GRAM_POLY)
    _check_step([(1600, 320), (48, 1600), (200, 208)], b2.SCALES_RAW, b2.OPERAND_F16, o.polar_express_coefficients(5),
                seed=13, schedule=b2.NS_FUSED_GRAM_POLY)
    _check_step([(4800, 1600), (1600, 1600), (6400, 1600), (1600, 6400)], b2.SCALES_RAW, b2.OPERAND_BF16,
                o.fixed_coefficients(5), seed=14, normalize=b2.NORMALIZE_DEFERRED, schedule=b2.NS_FUSED_GRAM_POLY)


def test_finish_by_groups_equals_one_finish_launch():
    # stage U + Q launched group by group (what a multi-GPU step does to start a bucket's all-gather early) must
    # leave exactly what the single launch leaves; groups may be empty and a group index must exist
    shapes = [(256, 512), (384, 128), (128, 128), (0, 0), (640, 256), (128, 1024)]
    rng = np.random.default_rng(21)
    data = [((rng.standard_normal(r * c) * 1e-3).astype(F), (rng.standard_normal(r * c) * 0.02).astype(F),
             (rng.standard_normal(r * c) * 0.02).astype(F)) for r, c in shapes]
    args = b2.MuonMegaUpdateArgs(learning_rate=0.02, coefficients=o.fixed_coefficients(5))

    def run(groups):
        slots = [_slot(r, c, g, np.zeros(r * c, np.uint16), z, x, b2.SCALES_RAW) for (r, c), (g, z, x) in zip(shapes, data)]
        plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW, normalize_mode=b2.NORMALIZE_DEFERRED)
        opt, table = b2.OptimizerModule(), b2.slot_table(slots)
        if groups:
            plan.set_finish_groups(groups)
        for _ in range(2):   # twice: the second step starts from the counters the first one left
            opt.muon_tma_prepare_polar(plan, table, args)
            opt.muon_polar(plan, args)
            if groups:
                for g in range(len(groups)):
                    opt.muon_tma_finish_update_group(plan, table, args, g)
            else:
                opt.muon_tma_finish_update(plan, table, args)
        torch.cuda.synchronize()
        assert plan.status() == 0
        if groups:
            with pytest.raises(b2.B2Error):
                opt.muon_tma_finish_update_group(plan, table, args, len(groups))
            with pytest.raises(b2.B2Error):
                plan.set_finish_groups([1, 2])          # must start at slot 0
            with pytest.raises(b2.B2Error):
                plan.set_finish_groups([0, 4, 2])       # must ascend
        out = [[host(t).copy() for t in (s.z_master, s.x_master, s.grad, s.momentum.view(torch.int16), s.bytes, s.scales,
                                         s.global_scale, s.schedule_amax)] for s in slots if s.rows * s.cols]
        plan.close()
        return out

    whole = run(None)
    for groups in ([0, 2, 2, 5], [0, 1, 2, 3, 4, 5], [0]):
        for a, b in zip(run(groups), whole):
            for ta, tb in zip(a, b):
                assert np.array_equal(ta, tb), groups


def test_one_pass_prepare_needs_bf16_operands():
    with pytest.raises(b2.B2Error):
        b2.MuonPlan([(64, 64)], operand_format=b2.OPERAND_F16, scale_layout=b2.SCALES_RAW,
                    normalize_mode=b2.NORMALIZE_DEFERRED)


@pytest.mark.parametrize("normalize", [b2.NORMALIZE_TWO_PASS, b2.NORMALIZE_DEFERRED])
def test_one_gpt2_medium_layer_csf(normalize):
    # the four matrix shapes of a GPT-2-medium layer (d = 1024), CSF scale storage
    _check_step([(3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096)], b2.SCALES_CSF, b2.OPERAND_BF16,
                o.fixed_coefficients(5), seed=5, normalize=normalize)


@pytest.mark.parametrize("normalize", [b2.NORMALIZE_TWO_PASS, b2.NORMALIZE_DEFERRED])
def test_one_gpt2_xl_layer_raw_scales(normalize):
    # the four matrix shapes of a GPT-2-XL layer (d = 1600 = 6.25 tiles of 256: every GEMM clips at the tensor
    # edge); cols % 128 != 0, so the scales are a raw plane
    _check_step([(4800, 1600), (1600, 1600), (6400, 1600), (1600, 6400)], b2.SCALES_RAW, b2.OPERAND_BF16,
                o.fixed_coefficients(5), seed=6, normalize=normalize)


def test_fused_wait_runs_out_and_plan_recovers():
    # The completion-counter wait of the one-launch update + encode, made to run out on purpose: one CTA, one
    # encode span whose matrix has no update chunks in the list, a limit of 3 ms.  The launch must return, report
    # through the status word, leave its ticket / abort / completion words zeroed, and the plan must then work
    # as if nothing had happened.
    rng = np.random.default_rng(9)
    shapes = [(128, 256), (256, 128)]
    hp = dict(mu=0.95, grad_scale=1.0, learning_rate=0.02, weight_decay=0.025, average_coefficient=0.5,
              schedule_beta=0.2, iterations=5, coefficients=o.fixed_coefficients(5))
    data = [(U.gradients(rng, r * c), np.zeros(r * c, np.uint16), U.weights(rng, r * c), U.weights(rng, r * c))
            for r, c in shapes]

    def fresh():
        slots = [_slot(r, c, *d, b2.SCALES_CSF) for (r, c), d in zip(shapes, data)]
        return slots, b2.MuonPlan(shapes), b2.slot_table(slots)

    opt = b2.OptimizerModule()
    slots_a, plan_a, table_a = fresh()
    before = [host(getattr(s, k)).copy() for s in slots_a for k in ("z_master", "x_master", "bytes", "scales")]
    plan_a.debug_fused_wait_expiry(table_a, 1, 3_000_000)
    torch.cuda.synchronize()
    assert plan_a.status() == b2._ffi.ERROR_LAUNCH_TIMEOUT
    assert plan_a.status() == 0                                   # reading the status clears it
    assert not host(plan_a.scratch(0, 10)).any()                  # ticket, abort, exited, completion counts
    after = [host(getattr(s, k)) for s in slots_a for k in ("z_master", "x_master", "bytes", "scales")]
    assert all(np.array_equal(a, b) for a, b in zip(before, after))   # nothing was updated or encoded
    opt.muon_mega_update(plan_a, table_a, b2.MuonMegaUpdateArgs(**hp))
    slots_b, plan_b, table_b = fresh()
    opt.muon_mega_update(plan_b, table_b, b2.MuonMegaUpdateArgs(**hp))
    torch.cuda.synchronize()
    assert plan_a.status() == 0 and plan_b.status() == 0
    for sa, sb in zip(slots_a, slots_b):
        for k in ("grad", "momentum", "z_master", "x_master", "schedule_amax", "bytes", "scales", "global_scale"):
            ta, tb = getattr(sa, k), getattr(sb, k)
            assert torch.equal(ta.view(torch.uint8), tb.view(torch.uint8)), k
    plan_a.close()
    plan_b.close()


def test_second_step_chains_on_state():
    # two consecutive steps: the momentum state and y written by step 1 feed step 2 correctly
    rng = np.random.default_rng(3)
    r, c = 256, 512
    z, x = U.weights(rng, r * c), U.weights(rng, r * c)
    g1, g2 = U.gradients(rng, r * c), U.gradients(rng, r * c)
    s = _slot(r, c, g1, np.zeros(r * c, np.uint16), z, x, b2.SCALES_CSF)
    plan = b2.MuonPlan([(r, c)])
    opt, table = b2.OptimizerModule(), b2.slot_table([s])
    args = b2.MuonMegaUpdateArgs(learning_rate=0.02, coefficients=o.fixed_coefficients(5))
    opt.muon_mega_update(plan, table, args)
    s.grad.copy_(dev(g2).view(r, c))
    opt.muon_mega_update(plan, table, args)
    torch.cuda.synchronize()
    m1, _, _ = o.momentum(g1, np.zeros(r * c, np.uint16), 0.95, 1.0)
    m2, _, _ = o.momentum(g2, m1, 0.95, 1.0)
    assert np.array_equal(bf16_bits(s.momentum).ravel(), m2)
    assert plan.status() == 0
    plan.close()
