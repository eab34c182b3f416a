"""Muon variants on the GPU through the plan entry points: variance-adaptive momentum (Muon-VS),
qk-clip inside the update stage, and sign-Muon; each against the oracle and against the
reference's own test recurrences."""
import numpy as np
import pytest
import torch

import llmini_b200 as b2
from oracle import oracle as o
from tests import _util as U
from tests.gpu_util import bf16_bits, bf16_from_bits, dev, host

pytestmark = pytest.mark.gpu
F = np.float32


def _slot(rows, cols, grad, mom_bits, z, x, var_bits=None):
    s = b2.MuonSlot.allocate(rows, cols, b2.SCALES_RAW)
    s.grad.copy_(dev(grad).view_as(s.grad))
    s.momentum.copy_(bf16_from_bits(mom_bits).view_as(s.momentum))
    s.z_master.copy_(dev(z).view_as(s.z_master))
    s.x_master.copy_(dev(x).view_as(s.x_master))
    if var_bits is not None:
        s.variance = bf16_from_bits(var_bits).view(rows, cols).contiguous()
    return s


def _powi(base, n):
    r = F(1.0)
    for _ in range(n):
        r = F(r * base)
    return r


@pytest.mark.parametrize("rows,cols", [(64, 128), (128, 64)])
@pytest.mark.parametrize("nesterov", [True, False])
def test_muon_vs_prepare_reference_case(rows, cols, nesterov):
    # crates/cuda-kernels/tests/optimizer/muon/tma_prepare.rs:87-208, variance_adaptive = true:
    # six chained steps; BF16 states bit-exact, normalised direction against the oracle
    n = rows * cols
    i = np.arange(n)
    grad = ((i * 73 % 257).astype(F) - F(128.0)) / F(211.0)
    m_bits = o.bf16_bits(((i * 29 % 131).astype(F) - F(65.0)) / F(173.0))
    v_bits = o.bf16_bits(F(0.01) + (i * 17 % 97).astype(F) / F(503.0))
    slot = _slot(rows, cols, grad, m_bits, np.zeros(n, F), np.zeros(n, F), v_bits)
    plan = b2.MuonPlan([(rows, cols)], scale_layout=b2.SCALES_RAW)
    table = b2.slot_table([slot])
    opt = b2.OptimizerModule()
    for step in range(3, 9):
        bci = F(1.0) / (F(1.0) - _powi(F(0.9), step))
        args = b2.MuonMegaUpdateArgs(mu=0.9, grad_scale=0.125, iterations=1, nesterov=nesterov,
                                     variance_adaptive=True, bias_correction_inv=float(bci))
        opt.muon_tma_prepare_polar(plan, table, args)
        torch.cuda.synchronize()
        m_bits, v_bits, u, ss = o.momentum_vs(grad, m_bits, v_bits, 0.9, 0.125, nesterov, bci)
        assert np.array_equal(bf16_bits(slot.momentum).ravel(), m_bits)
        assert np.array_equal(bf16_bits(slot.variance).ravel(), v_bits)
        inv = o.inv_norm(ss)
        got_inv = host(plan.scratch(0, 2))[0]
        assert abs(got_inv - inv) <= 1e-6 * inv
        x0 = host(plan.scratch(0, 0).float()).ravel()
        # sqrt/div are IEEE on both sides; allow one operand ulp for the odd last-bit difference
        want = u * got_inv
        assert np.max(np.abs(x0 - want)) <= np.max(np.abs(want)) * 2.0 ** -7
        assert np.mean(x0 == o.round_bf16(want)) > 0.999
    plan.close()


@pytest.mark.parametrize("variance_adaptive", [False, True])
def test_sign_update_reference_case(variance_adaptive):
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:686-840
    n = 32 * 32
    i = np.arange(n)
    grad = ((i * 41 % 97).astype(F) - F(48.0)) / F(37.0)
    m_bits = o.bf16_bits(((i * 17 % 61).astype(F) - F(30.0)) / F(53.0))
    v_bits = o.bf16_bits(F(0.02) + (i * 19 % 89).astype(F) / F(401.0))
    z = (i.astype(F) - F(511.0)) / F(997.0)
    x = (F(307.0) - i.astype(F)) / F(613.0)
    slot = _slot(32, 32, grad, m_bits, z, x, v_bits)
    slot.learning_rate_multiplier = 0.75
    slot.schedule_amax.fill_(9.0)   # stale value: the call has to reset it
    plan = b2.MuonPlan([(32, 32)], scale_layout=b2.SCALES_RAW)
    table = b2.slot_table([slot])
    args = b2.MuonMegaUpdateArgs(mu=0.9, grad_scale=0.25, learning_rate=0.004, weight_decay=0.1,
                                 average_coefficient=0.3, schedule_beta=0.4, variance_adaptive=variance_adaptive)
    b2.OptimizerModule().muon_tma_sign_update_deferred_quantization(plan, table, args)
    torch.cuda.synchronize()
    y, mb, vb, z2, x2, ax, ay = o.sign_update(grad, m_bits, v_bits, z, x, 32, 32, 0.9, 0.25, variance_adaptive,
                                               F(0.004) * F(0.75), 0.1, 0.3, 0.4)
    assert np.array_equal(bf16_bits(slot.momentum).ravel(), mb)
    assert np.array_equal(bf16_bits(slot.variance).ravel(), vb)
    assert np.array_equal(host(slot.z_master).ravel(), z2) and np.array_equal(host(slot.x_master).ravel(), x2)
    assert np.array_equal(host(slot.grad).ravel(), y)
    assert host(slot.schedule_amax)[0] == ay and host(plan.scratch(0, 3))[0] == ax
    assert not host(slot.bytes).any()   # deferred: nothing quantised
    plan.close()


@pytest.mark.parametrize("input_dim,output_dim", [(2048, 64), (2048, 6272), (64, 256)])
def test_qk_clip_reference_case(input_dim, output_dim):
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:112-262 (exact equality there too)
    rows, cols, head = output_dim, input_dim, 32
    n = rows * cols
    factors = np.where(np.arange(input_dim // head) % 2 == 0, F(0.5), F(0.25)).astype(F)
    m_bits, v_bits = o.bf16_bits(np.full(n, 3.0, F)), o.bf16_bits(np.full(n, 4.0, F))
    slot = _slot(rows, cols, np.zeros(n, F), m_bits, np.full(n, 1.0, F), np.full(n, 2.0, F), v_bits)
    slot.qk_clip_factor_offset, slot.qk_clip_head_dim = 0, head
    plan = b2.MuonPlan([(rows, cols)], scale_layout=b2.SCALES_RAW)
    table = b2.slot_table([slot])
    args = b2.MuonMegaUpdateArgs(learning_rate=0.0, weight_decay=0.0, average_coefficient=0.0, schedule_beta=0.4,
                                 qk_clip_factors=dev(factors))
    opt = b2.OptimizerModule()
    opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
    slot.momentum.copy_(bf16_from_bits(m_bits).view_as(slot.momentum))
    plan.scratch(0, 1).zero_()
    opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
    torch.cuda.synchronize()
    row_factor = np.ones(rows, F)
    for r in range(min(rows, 2 * cols)):
        row_factor[r] = factors[(r % cols) // head]
    f = np.repeat(row_factor, cols)
    ez, ex = np.full(n, 1.0, F) * f, np.full(n, 2.0, F) * f
    assert np.array_equal(host(slot.z_master).ravel(), ez) and np.array_equal(host(slot.x_master).ravel(), ex)
    assert np.array_equal(bf16_bits(slot.momentum).ravel(), o.bf16_bits(np.full(n, 3.0, F) * f))
    assert np.array_equal(bf16_bits(slot.variance).ravel(), o.bf16_bits(np.full(n, 4.0, F) * f * f))
    assert host(slot.schedule_amax)[0] == np.max(np.abs(ez + F(0.4) * (ex - ez)))
    plan.close()


def test_update_with_clip_and_variance_matches_oracle():
    # random data, two slots (one clipped, one not), non-zero learning rate
    rng = np.random.default_rng(5)
    shapes = [(192, 64), (64, 128)]
    factors = (0.25 + 0.75 * rng.random(8)).astype(F)
    factors[5] = 1.0
    slots, data = [], []
    for k, (r, c) in enumerate(shapes):
        z, x = U.weights(rng, r * c), U.weights(rng, r * c)
        mb, vb = o.bf16_bits(U.weights(rng, r * c, 1e-2)), o.bf16_bits(np.abs(U.weights(rng, r * c, 1e-3)))
        s = _slot(r, c, np.zeros(r * c, F), mb, z, x, vb)
        if k == 0:
            s.qk_clip_factor_offset, s.qk_clip_head_dim = 4, 16   # 64 / 16 = 4 heads at offset 4
        slots.append(s)
        data.append((z, x, mb, vb, (rng.standard_normal(r * c) * 0.05).astype(F)))
    plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW)
    table = b2.slot_table(slots)
    opt = b2.OptimizerModule()
    opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
    for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
        s.momentum.copy_(bf16_from_bits(data[k][2]).view_as(s.momentum))
        s.variance.copy_(bf16_from_bits(data[k][3]).view_as(s.variance))
        plan.scratch(k, 1).copy_(dev(data[k][4]).view(r, c))
    args = b2.MuonMegaUpdateArgs(learning_rate=0.02, weight_decay=0.025, average_coefficient=0.3, schedule_beta=0.6,
                                 qk_clip_factors=dev(factors), variance_adaptive=True)
    opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
    torch.cuda.synchronize()
    for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
        z, x, mb, vb, Um = data[k]
        off, hd = (4, 16) if k == 0 else (0xFFFFFFFF, 0)
        z2, x2, y2, m2, v2, ax, ay = o.update_clip(Um, z, x, mb, vb, r, c, 0.02, 0.025, 0.3, 0.6, factors, off, hd)
        assert np.array_equal(host(s.z_master).ravel(), z2) and np.array_equal(host(s.x_master).ravel(), x2)
        assert np.array_equal(host(s.grad).ravel(), y2)
        assert np.array_equal(bf16_bits(s.momentum).ravel(), m2)
        assert np.array_equal(bf16_bits(s.variance).ravel(), v2)
        assert host(s.schedule_amax)[0] == ay and host(plan.scratch(k, 3))[0] == ax
    plan.close()


def _stage_u_inputs(plan, slots, shapes, Us):
    """Resets the amax words through the prepare stage, then places the given updates."""
    opt = b2.OptimizerModule()
    opt.muon_tma_prepare_polar(plan, b2.slot_table(slots), b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
    for k, (r, c) in enumerate(shapes):
        plan.scratch(k, 1).copy_(dev(Us[k]).view(r, c))
    return opt


def test_normuon_reference_case():
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:264-384
    n, lr = 32, F(0.01)
    idx = np.arange(n * n)
    update = ((idx // n + 1).astype(F) * (idx % n % 7 + 1).astype(F) / F(128.0)).astype(F)
    old = (F(0.01) + np.arange(n).astype(F) / F(10000.0)).astype(F)
    slot = _slot(n, n, np.zeros(n * n, F), np.zeros(n * n, np.uint16), np.zeros(n * n, F), np.zeros(n * n, F))
    slot.second_momentum = dev(old)
    plan = b2.MuonPlan([(n, n)], scale_layout=b2.SCALES_RAW)
    opt = _stage_u_inputs(plan, [slot], [(n, n)], [update])
    args = b2.MuonMegaUpdateArgs(learning_rate=float(lr), weight_decay=0.0, average_coefficient=1.0, schedule_beta=0.4,
                                 normuon=True)
    opt.muon_tma_finish_update_deferred_quantization(plan, b2.slot_table([slot]), args)
    torch.cuda.synchronize()
    sm, fa, st = o.normuon_stats(update, n, n, old)
    got_f, got_s = host(plan.scratch(0, 8).view(torch.float32)), host(plan.scratch(0, 9).view(torch.float32))
    assert np.max(np.abs(host(slot.second_momentum) - sm)) <= 2e-6
    assert np.max(np.abs(got_f - fa)) <= 2e-5 and abs(got_s[0] - st[0]) <= 2e-6
    # elementwise stage: bit-exact given the device's own factors and scale
    z2, x2, y2, ax, ay = o.update_normuon(update, np.zeros(n * n, F), np.zeros(n * n, F), n, n, lr, 0.0, 1.0, 0.4,
                                          got_f, got_s[0])
    assert np.array_equal(host(slot.z_master).ravel(), z2) and np.array_equal(host(slot.x_master).ravel(), x2)
    assert np.array_equal(host(slot.grad).ravel(), y2) and host(slot.schedule_amax)[0] == ay
    want = -lr * (F(0.2) * np.sqrt(F(n))) * update * np.repeat(fa, n) * st[0]
    assert np.max(np.abs(host(slot.z_master).ravel() - want)) <= 2e-6
    plan.close()


@pytest.mark.parametrize("hyperball", [False, True])
def test_normuon_and_hyperball_match_oracle_on_mixed_shapes(hyperball):
    # tall, wide (column neurons, ragged 128-column unit), square; random data, second call chains the state
    rng = np.random.default_rng(17)
    shapes = [(384, 128), (96, 400), (128, 128), (0, 0), (40, 48)]
    slots, data = [], []
    for r, c in shapes:
        n = r * c
        z, x = U.weights(rng, n), U.weights(rng, n)
        s = _slot(r, c, np.zeros(n, F), np.zeros(n, np.uint16), z, x) if n else b2.MuonSlot.allocate(0, 0, b2.SCALES_RAW)
        sm = (0.01 + 0.02 * rng.random(max(r, c))).astype(F)
        if n:
            s.second_momentum = dev(sm)
        s.learning_rate_multiplier = 0.75
        slots.append(s)
        data.append([z, x, sm])
    plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW)
    table = b2.slot_table(slots)
    for step in range(2):
        Us = [(rng.standard_normal(r * c) * 0.05).astype(F) for r, c in shapes]
        opt = b2.OptimizerModule()
        opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
        for k, (r, c) in enumerate(shapes):
            if r * c:
                plan.scratch(k, 1).copy_(dev(Us[k]).view(r, c))
        args = b2.MuonMegaUpdateArgs(learning_rate=0.02, weight_decay=0.0 if hyperball else 0.025,
                                     average_coefficient=0.3, schedule_beta=0.6, normuon=True)
        if hyperball:
            opt.muon_tma_finish_hyperball_update_deferred_quantization(plan, table, args, use_schedule_free=step == 0)
        else:
            opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
        torch.cuda.synchronize()
        for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
            if r * c == 0:
                continue
            z, x, sm = data[k]
            sm2, fa, st = o.normuon_stats(Us[k], r, c, sm, z=z if hyperball else None)
            got_f, got_s = host(plan.scratch(k, 8).view(torch.float32)), host(plan.scratch(k, 9).view(torch.float32))
            assert np.allclose(host(s.second_momentum), sm2, rtol=2e-6, atol=0)
            assert np.allclose(got_f, fa, rtol=2e-6, atol=0)
            assert np.allclose(got_s[:2], st[:2], rtol=2e-6, atol=0)
            lr = F(0.02) * F(0.75)
            if hyperball:
                assert np.allclose(got_s[2:], st[2:], rtol=1e-5, atol=1e-6)
                z2, x2, y2, _, _, ax, ay = o.hyperball_update(Us[k], z, x, r, c, lr, 0.3, 0.6, step == 0, got_f, got_s)
                assert abs(np.sqrt(np.sum(z2.astype(np.float64) ** 2)) - got_s[2]) <= 1e-5 * got_s[2]
            else:
                z2, x2, y2, ax, ay = o.update_normuon(Us[k], z, x, r, c, lr, 0.025, 0.3, 0.6, got_f, got_s[0])
            assert np.array_equal(host(s.z_master).ravel(), z2) and np.array_equal(host(s.x_master).ravel(), x2)
            assert np.array_equal(host(s.grad).ravel(), y2)
            assert host(s.schedule_amax)[0] == ay and host(plan.scratch(k, 3))[0] == ax
            data[k] = [z2, x2, host(s.second_momentum).copy()]
    plan.close()


@pytest.mark.parametrize("rows,cols", [(32, 32), (32, 64), (64, 32)])
def test_hyperball_reference_cases(rows, cols):
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:386-676 (square with schedule-free
    # averaging; rectangular without), tolerances as stated there
    n = rows * cols
    idx = np.arange(n)
    pr, pc = min(rows, cols), max(rows, cols)
    if rows == cols:
        storage = (((idx // cols * 13 + idx % cols * 7) % 41).astype(F) / F(37.0) - F(0.5)).astype(F)
        old = (F(0.02) + np.arange(pc).astype(F) / F(20000.0)).astype(F)
        z = (((idx * 29 % 211).astype(F) - F(105.0)) / F(173.0)).astype(F)
        x = (((idx * 17 % 157).astype(F) - F(78.0)) / F(199.0)).astype(F)
        mult, c_avg, use_sf, tol = 0.75, 0.3, True, 3e-5
    else:
        polar = (((idx * 23 % 101).astype(F) - F(50.0)) / F(71.0)).astype(F).reshape(pr, pc)
        storage = (polar.T if rows > cols else polar).reshape(-1).copy()
        old = (F(0.015) + np.arange(pc).astype(F) / F(30000.0)).astype(F)
        z = (((idx * 31 % 193).astype(F) - F(96.0)) / F(151.0)).astype(F)
        x = np.zeros(n, F)
        mult, c_avg, use_sf, tol = 0.625, 1.0, False, 4e-5
    slot = _slot(rows, cols, np.zeros(n, F), np.zeros(n, np.uint16), z, x)
    slot.second_momentum = dev(old)
    slot.learning_rate_multiplier = mult
    plan = b2.MuonPlan([(rows, cols)], scale_layout=b2.SCALES_RAW)
    opt = _stage_u_inputs(plan, [slot], [(rows, cols)], [storage])
    args = b2.MuonMegaUpdateArgs(learning_rate=0.018, average_coefficient=c_avg, schedule_beta=0.4)
    opt.muon_tma_finish_hyperball_update_deferred_quantization(plan, b2.slot_table([slot]), args, use_schedule_free=use_sf)
    torch.cuda.synchronize()
    # host recurrence of the reference test in float64 (its float32 sums agree to the stated tolerance)
    U2 = storage.reshape(rows, cols).astype(np.float64)
    sumsq = (U2 ** 2).sum(axis=1 if rows >= cols else 0)
    fac = 1.0 / np.sqrt(np.maximum(0.95 * old + (1.0 - 0.95) * sumsq / pr, 1e-10))
    direction = (U2 * (fac[:, None] if rows >= cols else fac[None, :])).ravel()
    radius, unorm = np.sqrt(np.sum(z.astype(np.float64) ** 2)), np.sqrt(np.sum(direction ** 2))
    step = float(F(0.018) * F(mult)) * radius / unorm
    cand = z - step * direction
    ez = cand * radius / np.sqrt(np.sum(cand ** 2))
    ex = x + c_avg * (ez - x) if use_sf else ez
    gz, gx = host(slot.z_master).ravel(), host(slot.x_master).ravel()
    assert np.max(np.abs(gz - ez)) <= tol and np.max(np.abs(gx - ex)) <= tol
    assert abs(np.sqrt(np.sum(gz.astype(np.float64) ** 2)) - radius) <= radius * tol
    assert abs(host(plan.scratch(0, 9).view(torch.float32))[1] - unorm) <= unorm * 3e-5
    assert abs(host(slot.schedule_amax)[0] - np.max(np.abs(ez + 0.4 * (ex - ez)))) <= 3e-5
    assert not host(slot.bytes).any()
    plan.close()


@pytest.mark.parametrize("target", [b2.QUANTIZE_X, b2.QUANTIZE_Y])
@pytest.mark.parametrize("ext", [False, True])
def test_fused_update_encode_equals_two_launches(target, ext):
    # the one-launch update + encode (ticketed work list) against the two-kernel form (debug flag 16):
    # masters, y, maxima, tensor scales, codes and block scales bit for bit, on matrices of very
    # different sizes (odd chunk counts, one chunk, an empty slot)
    rng = np.random.default_rng(23)
    shapes = [(768, 768), (40, 48), (0, 0), (2304, 768), (128, 1040), (16, 16), (768, 3072)]
    factors = dev((0.25 + 0.75 * rng.random(64)).astype(F))
    results = []
    for flags in (0, 16):
        rng2 = np.random.default_rng(29)
        slots = []
        for k, (r, c) in enumerate(shapes):
            n = r * c
            s = b2.MuonSlot.allocate(r, c, b2.SCALES_RAW)
            if n:
                s.z_master.copy_(dev(U.weights(rng2, n)).view_as(s.z_master))
                s.x_master.copy_(dev(U.weights(rng2, n)).view_as(s.x_master))
                s.momentum.copy_(bf16_from_bits(o.bf16_bits(U.weights(rng2, n, 1e-2))).view_as(s.momentum))
                s.second_momentum = dev((0.01 + 0.02 * rng2.random(max(r, c))).astype(F))
                if ext and k == 3:
                    s.qk_clip_factor_offset, s.qk_clip_head_dim = 0, 64
            s.learning_rate_multiplier = 1.0 + 0.25 * k
            slots.append(s)
        plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW, quantize_target=target, debug_flags=flags)
        table = b2.slot_table(slots)
        opt = b2.OptimizerModule()
        opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
        for k, (r, c) in enumerate(shapes):
            if r * c:
                plan.scratch(k, 1).copy_(dev((rng2.standard_normal(r * c) * 0.05).astype(F)).view(r, c))
        args = b2.MuonMegaUpdateArgs(learning_rate=0.02, weight_decay=0.025, average_coefficient=0.3, schedule_beta=0.6,
                                     normuon=ext, qk_clip_factors=factors if ext else None)
        opt.muon_tma_finish_update(plan, table, args)
        torch.cuda.synchronize()
        assert plan.status() == 0
        out = []
        for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
            if r * c == 0:
                continue
            out.append([host(t).copy() for t in (s.z_master, s.x_master, s.grad, s.schedule_amax, s.global_scale,
                                                 s.bytes, s.scales, plan.scratch(k, 3))] + [bf16_bits(s.momentum)])
        results.append(out)
        plan.close()
    for a, b in zip(*results):
        for u, v in zip(a, b):
            assert np.array_equal(u, v)
        assert a[5].any() and a[4][0] > 0


def test_deferred_finish_then_master_materialise_equals_finish_update():
    # the deferred finish followed by the stand-alone encode of x' against the one-call finish:
    # masters, y, maxima, tensor scales, codes and block scales bit for bit
    shapes = [(768, 768), (40, 48), (0, 0), (2304, 768), (128, 1040), (16, 16)]
    results = []
    for split in (False, True):
        rng2 = np.random.default_rng(61)
        slots = []
        for k, (r, c) in enumerate(shapes):
            n = r * c
            s = b2.MuonSlot.allocate(r, c, b2.SCALES_RAW)
            if n:
                s.z_master.copy_(dev(U.weights(rng2, n)).view_as(s.z_master))
                s.x_master.copy_(dev(U.weights(rng2, n)).view_as(s.x_master))
            s.learning_rate_multiplier = 1.0 + 0.25 * k
            slots.append(s)
        plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW)
        table = b2.slot_table(slots)
        opt = b2.OptimizerModule()
        opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=1.0, grad_scale=0.0, iterations=1))
        for k, (r, c) in enumerate(shapes):
            if r * c:
                plan.scratch(k, 1).copy_(dev((rng2.standard_normal(r * c) * 0.05).astype(F)).view(r, c))
        args = b2.MuonMegaUpdateArgs(learning_rate=0.02, weight_decay=0.025, average_coefficient=0.3, schedule_beta=0.6)
        if split:
            opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
            opt.muon_materialize_master_weights(plan, table)
        else:
            opt.muon_tma_finish_update(plan, table, args)
        torch.cuda.synchronize()
        assert plan.status() == 0
        out = []
        for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
            if r * c:
                out.append([host(t).copy() for t in (s.z_master, s.x_master, s.grad, s.schedule_amax, s.global_scale,
                                                     s.bytes, s.scales)])
        results.append(out)
        plan.close()
    for a, b in zip(*results):
        for u, v in zip(a, b):
            assert np.array_equal(u, v)
        assert a[5].any() and a[4][0] > 0


def _symexp(raw, beta, e=1.0, l=1.0, c=1.0):
    """SymExpLin forward (crates/cuda-kernels/src/gpt/optimizer/symexp_lin.rs:8-26) in float64."""
    raw = raw.astype(np.float64)
    return np.sign(raw) * (e * (np.exp(beta * c * np.abs(raw)) - 1.0) / beta + l * raw / beta)


@pytest.mark.parametrize("entry", ["finish", "hyperball", "sign"])
def test_symexp_lin_forward_in_the_update_kernels(entry):
    # y = SymExpLin(z' + beta (x' - z')) with per-slot scale scalars (slot 0) and unit scales (slot 1);
    # masters stay bit-exact, y follows the definition to the accuracy of ex2.approx
    import ctypes as C
    from llmini_b200 import _ffi
    rng = np.random.default_rng(41)
    shapes = [(96, 64), (64, 128)]
    sbeta, sym_beta = 0.6, 6.0
    one = lambda v: torch.full((1,), v, device="cuda")
    pairs = [(1.25, 0.75), (0.5, 1.5), (2.0, 1.0)]          # (z, x) of exponential, linear, curvature
    keep = [one(v) for pr in pairs for v in pr]
    descs = (_ffi.SymExpLinSlotDescriptor * 2)()
    for name, t in zip(("exponential_z", "exponential_x", "linear_z", "linear_x", "curvature_z", "curvature_x"), keep):
        setattr(descs[0], name, t.data_ptr())
    table_sx = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
    scal = [tuple(zz + sbeta * (xx - zz) for zz, xx in pairs), (1.0, 1.0, 1.0)]
    slots, data = [], []
    for r, c in shapes:
        n = r * c
        z, x = U.weights(rng, n) * F(20.0), U.weights(rng, n) * F(20.0)   # magnitudes where exp() bends
        g = U.gradients(rng, n)
        mb = o.bf16_bits(U.weights(rng, n, 1e-3))
        s = _slot(r, c, g, mb, z, x)
        s.second_momentum = dev(np.full(max(r, c), 1e-2, F))
        slots.append(s)
        data.append((z, x, g, mb, (rng.standard_normal(n) * 0.05).astype(F)))
    plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW)
    table = b2.slot_table(slots)
    opt = _stage_u_inputs(plan, slots, shapes, [d[4] for d in data])
    for s, d in zip(slots, data):       # the prepare call above moved the momentum: put it back
        s.momentum.copy_(bf16_from_bits(d[3]).view_as(s.momentum))
        s.grad.copy_(dev(d[2]).view_as(s.grad))
    args = b2.MuonMegaUpdateArgs(mu=0.9, grad_scale=0.5, learning_rate=0.02, weight_decay=0.0 if entry == "hyperball" else 0.025,
                                 average_coefficient=0.3, schedule_beta=sbeta, symexp_lin_beta=sym_beta,
                                 symexp_lin_slots=table_sx)
    if entry == "finish":
        opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
    elif entry == "hyperball":
        opt.muon_tma_finish_hyperball_update_deferred_quantization(plan, table, args, use_schedule_free=True)
    else:
        opt.muon_tma_sign_update_deferred_quantization(plan, table, args)
    torch.cuda.synchronize()
    for k, (s, (r, c)) in enumerate(zip(slots, shapes)):
        z, x, g, mb, Um = data[k]
        if entry == "finish":
            z2, x2, y_raw, ax, _ = o.update(Um, z, x, r, c, 0.02, 0.025, 0.3, sbeta)
        elif entry == "hyperball":
            fa, st = host(plan.scratch(k, 8).view(torch.float32)), host(plan.scratch(k, 9).view(torch.float32))
            z2, x2, y_raw, _, _, ax, _ = o.hyperball_update(Um, z, x, r, c, 0.02, 0.3, sbeta, True, fa, st)
        else:
            y_raw, _, _, z2, x2, ax, _ = o.sign_update(g, mb, None, z, x, r, c, 0.9, 0.5, False, 0.02, 0.025, 0.3, sbeta)
        assert np.array_equal(host(s.z_master).ravel(), z2) and np.array_equal(host(s.x_master).ravel(), x2)
        want = _symexp(y_raw, sym_beta, *scal[k])
        got = host(s.grad).ravel().astype(np.float64)
        assert np.max(np.abs(got - want)) <= 4e-6 * np.max(np.abs(want))
        assert np.max(np.abs(want - y_raw)) > 0.05 * np.max(np.abs(y_raw))        # the transform did something
        assert abs(host(s.schedule_amax)[0] - np.max(np.abs(want))) <= 4e-6 * np.max(np.abs(want))
        assert host(plan.scratch(k, 3))[0] == ax
    del keep
    plan.close()


def test_symexp_lin_scalar_adam_reference_case():
    # crates/cuda-kernels/tests/optimizer/adam.rs:165-213 (symexp_lin_batched_scalar_adam_matches_independent_updates)
    from llmini_b200 import _ffi
    one = lambda v: torch.full((1,), float(v), device="cuda")
    fix = {name: dict(z=one(1.0), x=one(1.0), grad=one(g), first=one(0.0), second=one(0.0))
           for name, g in (("exponential", 0.5), ("linear", -0.25), ("curvature", 0.75))}
    descs = (_ffi.SymExpLinSlotDescriptor * 2)()      # entry 1 has no scale scalars and must be skipped
    for name, f in fix.items():
        for field, key in (("z", "z"), ("x", "x"), ("grad", "grad"), ("first", "first"), ("second", "second")):
            setattr(descs[0], f"{name}_{field}", f[key].data_ptr())
    table = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
    opt = b2.OptimizerModule()
    opt.symexp_lin_scale_adamw_update(table, 2, 0.5, 0.25, 0.1, 0.1, 0.9, 0.95, 0.1, 0.05, 1.0e-10, 0.25)
    torch.cuda.synchronize()
    for name, z, x in (("exponential", 0.725, 0.93125), ("linear", 1.225, 1.05625), ("curvature", 0.9, 0.975)):
        assert abs(host(fix[name]["z"])[0] - z) <= 1e-6 and abs(host(fix[name]["x"])[0] - x) <= 1e-6
    opt.symexp_lin_zero_scale_grads(table, 2)
    torch.cuda.synchronize()
    assert all(host(f["grad"])[0] == 0.0 for f in fix.values())


def test_symexp_lin_congruent_inverse_inverts_the_unit_forward():
    # r -> t = sign(r) ((exp(beta |r|) - 1) + |r|) / beta is what the inverse undoes (symexp_lin.rs:60-84)
    beta = 12.5
    r = np.concatenate([np.linspace(-0.4, 0.4, 4001), [0.0, 1e-7, -3e-4]]).astype(F)
    t = (np.sign(r) * ((np.exp(beta * np.abs(r.astype(np.float64))) - 1.0) + np.abs(r)) / beta).astype(F)
    buf = dev(t)
    b2.OptimizerModule().symexp_lin_congruent_inverse_in_place(buf, beta)
    torch.cuda.synchronize()
    got = host(buf)
    assert np.max(np.abs(got - r)) <= 2e-6 + 2e-5 * np.max(np.abs(r))
    assert got[4001] == 0.0
    with pytest.raises(b2.B2Error):
        b2.OptimizerModule().symexp_lin_congruent_inverse_in_place(buf, 0.0)


def test_normuon_without_state_buffer_is_the_plain_update():
    # a slot whose `second_momentum` is NULL keeps factor 1 and scale 1: bit-identical to the plain finish
    rng = np.random.default_rng(53)
    shapes = [(96, 64), (64, 128)]
    outs = []
    for normuon in (False, True):
        rng2 = np.random.default_rng(59)
        slots = []
        for r, c in shapes:
            n = r * c
            slots.append(_slot(r, c, np.zeros(n, F), np.zeros(n, np.uint16), U.weights(rng2, n), U.weights(rng2, n)))
        plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW)
        opt = _stage_u_inputs(plan, slots, shapes, [(rng2.standard_normal(r * c) * 0.05).astype(F) for r, c in shapes])
        opt.muon_tma_finish_update(plan, b2.slot_table(slots),
                                   b2.MuonMegaUpdateArgs(learning_rate=0.02, average_coefficient=0.3, schedule_beta=0.6,
                                                         normuon=normuon))
        torch.cuda.synchronize()
        assert plan.status() == 0
        outs.append([[host(t).copy() for t in (s.z_master, s.x_master, s.grad, s.bytes, s.scales, s.global_scale)]
                     for s in slots])
        plan.close()
    for a, b in zip(*outs):
        for u, v in zip(a, b):
            assert np.array_equal(u, v)
