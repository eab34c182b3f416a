"""Elementwise stages on the GPU against the oracle: momentum / norm (M+N), update (U),
requantisation (Q) through the plan entry points, AdamW, and the reference's known answers."""
import numpy as np
import pytest
import torch

import llmini_b200 as b2
from oracle import oracle as o
from tests import _util as U
from tests.gpu_util import bf16_bits, bf16_from_bits, decode_scales, dev, host, rcp_table

pytestmark = pytest.mark.gpu
F = np.float32


def _fill_slot(slot, grad, mom_bits, z, x):
    slot.grad.copy_(dev(grad).view_as(slot.grad))
    slot.momentum.copy_(bf16_from_bits(mom_bits).view_as(slot.momentum))
    slot.z_master.copy_(dev(z).view_as(slot.z_master))
    slot.x_master.copy_(dev(x).view_as(slot.x_master))


@pytest.mark.parametrize("shapes,layout", [
    ([(64, 128), (128, 256)], b2.SCALES_CSF),
    ([(32, 64), (96, 48), (0, 0), (7, 16), (300, 1040)], b2.SCALES_RAW),
])
def test_prepare_matches_oracle(shapes, layout):
    rng = np.random.default_rng(11)
    opt = b2.OptimizerModule()
    slots = [b2.MuonSlot.allocate(r, c, layout) for r, c in shapes]
    inputs = []
    for s, (r, c) in zip(slots, shapes):
        g = U.gradients(rng, r * c)
        m = o.bf16_bits(U.weights(rng, r * c, 1e-3))
        _fill_slot(s, g, m, np.zeros(r * c, F), np.zeros(r * c, F))
        inputs.append((g, m))
    plan = b2.MuonPlan(shapes, scale_layout=layout)
    table = b2.slot_table(slots)
    for nesterov in (True, False):
        args = b2.MuonMegaUpdateArgs(mu=0.9, grad_scale=0.125, iterations=1, nesterov=nesterov)
        opt.muon_tma_prepare_polar(plan, table, args)
        torch.cuda.synchronize()
        for i, (s, (r, c)) in enumerate(zip(slots, shapes)):
            if r * c == 0:
                continue
            g, m = inputs[i]
            m2, u, ss = o.momentum(g, m, 0.9, 0.125, nesterov=nesterov)
            assert np.array_equal(bf16_bits(s.momentum).ravel(), m2)  # BF16 state: bit-exact
            inv = o.inv_norm(ss)
            got_inv = host(plan.scratch(i, 2))[0]
            assert abs(got_inv - inv) <= 1e-6 * inv
            x0 = host(plan.scratch(i, 0).float()).ravel()
            want = o.round_bf16(u * got_inv)
            assert np.array_equal(x0, want)
            inputs[i] = (g, m2)  # the next call chains on the stored state
    plan.close()


@pytest.mark.parametrize("variance_adaptive", [False, True])
def test_one_pass_prepare_matches_oracle(variance_adaptive):
    # NORMALIZE_DEFERRED: momentum state bit-exact, operand = r16(u) without the Frobenius scale, the scale
    # itself within 1e-6 of the oracle's
    rng = np.random.default_rng(12)
    shapes = [(64, 128), (300, 1040), (0, 0), (7, 16), (256, 64)]
    opt = b2.OptimizerModule()
    slots = [b2.MuonSlot.allocate(r, c, b2.SCALES_RAW) for r, c in shapes]
    inputs = []
    for s, (r, c) in zip(slots, shapes):
        g = U.gradients(rng, r * c)
        m = o.bf16_bits(U.weights(rng, r * c, 1e-3))
        v = o.bf16_bits(np.abs(U.weights(rng, r * c, 1e-6)) + F(1e-8))
        _fill_slot(s, g, m, np.zeros(r * c, F), np.zeros(r * c, F))
        if variance_adaptive:
            s.variance = bf16_from_bits(v).view(r, c) if r * c else None
        inputs.append((g, m, v))
    plan = b2.MuonPlan(shapes, scale_layout=b2.SCALES_RAW, normalize_mode=b2.NORMALIZE_DEFERRED)
    table = b2.slot_table(slots)
    for s in slots:   # the prepare pass clears both maxima of every slot
        s.schedule_amax.fill_(7.0)
    for nesterov in (True, False):
        args = b2.MuonMegaUpdateArgs(mu=0.9, grad_scale=0.125, iterations=1, nesterov=nesterov,
                                     variance_adaptive=variance_adaptive, bias_correction_inv=1.25)
        opt.muon_tma_prepare_polar(plan, table, args)
        torch.cuda.synchronize()
        for i, (s, (r, c)) in enumerate(zip(slots, shapes)):
            if r * c == 0:
                continue
            g, m, v = inputs[i]
            if variance_adaptive:
                m2, v2, u, ss = o.momentum_vs(g, m, v, 0.9, 0.125, nesterov, 1.25)
                assert np.array_equal(bf16_bits(s.variance).ravel(), v2)
            else:
                m2, u, ss = o.momentum(g, m, 0.9, 0.125, nesterov=nesterov)
                v2 = v
            assert np.array_equal(bf16_bits(s.momentum).ravel(), m2)
            inv = o.inv_norm(ss)
            assert abs(host(plan.scratch(i, 2))[0] - inv) <= 1e-6 * inv
            assert np.array_equal(host(plan.scratch(i, 0).float()).ravel(), o.round_bf16(u))
            assert host(s.schedule_amax)[0] == 0.0 and host(plan.scratch(i, 3))[0] == 0.0
            inputs[i] = (g, m2, v2)
    plan.close()


def test_momentum_chain_reference_case():
    # crates/cuda-kernels/tests/optimizer/muon/tma_prepare.rs:87-208 (non-variance branch)
    opt = b2.OptimizerModule()
    for rows, cols in [(64, 128), (128, 64)]:
        n = rows * cols
        i = np.arange(n)
        grad = ((i * 73 % 257).astype(F) - F(128.0)) / F(211.0)
        mom = o.round_bf16(((i * 29 % 131).astype(F) - F(65.0)) / F(173.0))
        slot = b2.MuonSlot.allocate(rows, cols, b2.SCALES_RAW)
        _fill_slot(slot, grad, o.bf16_bits(mom), np.zeros(n, F), np.zeros(n, F))
        plan = b2.MuonPlan([(rows, cols)], scale_layout=b2.SCALES_RAW)
        table = b2.slot_table([slot])
        expected_m = mom.copy()
        for _ in range(6):
            g = grad * F(0.125)
            nxt = F(0.9) * expected_m + (F(1.0) - F(0.9)) * g
            expected_m = o.round_bf16(nxt)
            opt.muon_tma_prepare_polar(plan, table, b2.MuonMegaUpdateArgs(mu=0.9, grad_scale=0.125, iterations=1))
            torch.cuda.synchronize()
            assert np.array_equal(host(slot.momentum.float()).ravel(), expected_m)
        plan.close()


@pytest.mark.parametrize("layout,target", [(b2.SCALES_CSF, b2.QUANTIZE_X), (b2.SCALES_RAW, b2.QUANTIZE_Y)])
def test_finish_update_matches_oracle(layout, target):
    rng = np.random.default_rng(21)
    shapes = [(256, 384), (384, 128), (128, 128)] if layout == b2.SCALES_CSF else [(100, 48), (33, 16), (512, 2064)]
    opt = b2.OptimizerModule()
    slots = [b2.MuonSlot.allocate(r, c, layout) for r, c in shapes]
    plan = b2.MuonPlan(shapes, scale_layout=layout, quantize_target=target)
    data = []
    for i, (s, (r, c)) in enumerate(zip(slots, shapes)):
        z, x = U.weights(rng, r * c), U.weights(rng, r * c)
        Um = (rng.standard_normal(r * c) * 0.05).astype(F)
        _fill_slot(s, np.zeros(r * c, F), np.zeros(r * c, np.uint16), z, x)
        s.learning_rate_multiplier = 1.0 + 0.5 * i
        plan.scratch(i, 1).copy_(dev(Um).view(r, c))
        data.append((z, x, Um))
    table = b2.slot_table(slots)
    args = b2.MuonMegaUpdateArgs(learning_rate=0.02, weight_decay=0.025, average_coefficient=0.3, schedule_beta=0.6)
    # the two amax words are cleared by the prepare stage; do the same here
    opt.muon_tma_prepare_polar(plan, table, args)
    for s, (z, x, _) in zip(slots, data):
        s.grad.zero_()
    for i, (r, c) in enumerate(shapes):
        plan.scratch(i, 1).copy_(dev(data[i][2]).view(r, c))
    opt.muon_tma_finish_update(plan, table, args)
    torch.cuda.synchronize()
    for i, (s, (r, c)) in enumerate(zip(slots, shapes)):
        z, x, Um = data[i]
        lr = F(0.02) * F(s.learning_rate_multiplier)
        z2, x2, y2, ax, ay = o.update(Um, z, x, r, c, lr, 0.025, 0.3, 0.6)
        assert np.array_equal(host(s.z_master).ravel(), z2)   # IEEE elementwise: bit-exact
        assert np.array_equal(host(s.x_master).ravel(), x2)
        assert np.array_equal(host(s.grad).ravel(), y2)
        assert host(s.schedule_amax)[0] == ay and host(plan.scratch(i, 3))[0] == ax
        src, am = (y2, ay) if target == b2.QUANTIZE_Y else (x2, ax)
        gs = host(s.global_scale)[0]
        codes, raw, ogs, misses = o.nvfp4_quantize(src, amax=am, rcp_table=rcp_table(gs))
        assert misses == 0 and gs == ogs
        assert np.array_equal(host(s.bytes)[: r * c // 2], codes)
        assert np.array_equal(decode_scales(s.scales, r, c, layout), raw)
    plan.close()


def test_schedule_amax_reference_case():
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:23-99 (deferred: no quantisation)
    n = 32 * 32
    i = np.arange(n).astype(F)
    z = (i - F(511.0)) / F(997.0)
    x = (F(307.0) - i) / F(613.0)
    expected = np.max(np.abs(z + F(0.4) * (x - z)))
    opt = b2.OptimizerModule()
    slot = b2.MuonSlot.allocate(32, 32, b2.SCALES_RAW)
    _fill_slot(slot, np.zeros(n, F), np.zeros(n, np.uint16), z, x)
    plan = b2.MuonPlan([(32, 32)], scale_layout=b2.SCALES_RAW)
    table = b2.slot_table([slot])
    args = b2.MuonMegaUpdateArgs(learning_rate=0.0, weight_decay=0.0, average_coefficient=0.0, schedule_beta=0.4)
    opt.muon_tma_prepare_polar(plan, table, args)
    plan.scratch(0, 1).zero_()
    opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
    torch.cuda.synchronize()
    assert abs(host(slot.schedule_amax)[0] - expected) <= 1e-7
    assert np.array_equal(host(slot.z_master).ravel(), z) and np.array_equal(host(slot.x_master).ravel(), x)
    assert not host(slot.bytes).any()
    plan.close()


def _adam_buffers(n, layout=b2.SCALES_RAW):
    z = lambda v=0.0: torch.full((n,), v, device="cuda")
    return dict(z_master=z(1.0), x_master=z(1.0), grad=z(0.5), first_moment=z(), second_moment=z(),
                bytes=torch.zeros(n // 2, dtype=torch.uint8, device="cuda"),
                scales=torch.zeros(max(n // 16, 1), dtype=torch.uint8, device="cuda"),
                global_scale=torch.ones(1, device="cuda"), amax=torch.zeros(1, device="cuda"),
                chunk_amax=torch.zeros((n + 2047) // 2048, device="cuda"), scale_layout=layout)


ADAM = dict(grad_scale=0.5, learning_rate=0.25, weight_decay=0.1, beta1=0.9, beta2=0.95, beta1_correction=0.1,
            beta2_correction=0.05, eps=1.0e-10)


def test_adamw_reference_known_answers():
    # crates/cuda-kernels/tests/optimizer/adam.rs:97-162
    opt = b2.OptimizerModule()
    buf = _adam_buffers(32)
    opt.apply_adamw_update(len=32, average_coefficient=1.0, schedule_beta=0.0, **ADAM, **buf)
    torch.cuda.synchronize()
    close = lambda t, v: float((t - v).abs().max()) <= 1e-6
    assert close(buf["z_master"], 0.725) and close(buf["x_master"], 0.725)
    assert close(buf["first_moment"], 0.025) and close(buf["second_moment"], 0.003125)
    assert host(buf["bytes"]).any() and host(buf["scales"]).any()
    assert abs(host(buf["global_scale"])[0] - F(0.725) / F(1536.0)) <= 1e-8
    buf = _adam_buffers(32)
    opt.apply_adamw_update(len=32, average_coefficient=0.25, schedule_beta=0.0, **ADAM, **buf)
    torch.cuda.synchronize()
    assert close(buf["z_master"], 0.725) and close(buf["x_master"], 0.93125)
    buf = _adam_buffers(32)
    opt.apply_adamw_update_deferred_quantization(len=32, average_coefficient=0.25, schedule_beta=0.4, **ADAM, **buf)
    torch.cuda.synchronize()
    zz, xx = host(buf["z_master"])[0], host(buf["x_master"])[0]
    want = abs(zz + F(0.4) * (xx - zz))
    assert close(buf["amax"], want) and close(buf["grad"], want)
    ptrs = torch.tensor([buf["amax"].data_ptr()], dtype=torch.int64, device="cuda")
    opt.zero_f32_pointer_table(ptrs, 1)
    torch.cuda.synchronize()
    assert host(buf["amax"])[0] == 0.0


@pytest.mark.parametrize("n", [16, 2048, 50304 * 16, 4099])
def test_adamw_matches_oracle(n):
    rng = np.random.default_rng(n)
    z, x = U.weights(rng, n), U.weights(rng, n)
    g, m1, m2 = U.gradients(rng, n), U.weights(rng, n, 1e-3), np.abs(U.weights(rng, n, 1e-6))
    hp = dict(grad_scale=0.7, lr=2e-4, wd=0.005, beta1=0.9, beta2=0.95, bc1=0.19, bc2=0.0975, eps=1e-10)
    z2, x2, y2, a2, b2_, am = o.adamw(z, x, g, m1, m2, c_avg=0.5, sched_beta=0.3, **hp)
    opt = b2.OptimizerModule()
    kw = dict(grad_scale=0.7, learning_rate=2e-4, weight_decay=0.005, beta1=0.9, beta2=0.95, beta1_correction=0.19,
              beta2_correction=0.0975, eps=1e-10, average_coefficient=0.5, schedule_beta=0.3, len=n)
    t = dict(z_master=dev(z), x_master=dev(x), grad=dev(g), first_moment=dev(m1), second_moment=dev(m2))
    if n % 16 == 0:
        amax = torch.zeros(1, device="cuda")
        opt.apply_adamw_update_deferred_quantization(amax=amax, **kw, **t)
        torch.cuda.synchronize()
        assert host(amax)[0] == am and np.array_equal(host(t["grad"]), y2)
    else:
        opt.apply_fp32_adamw_update(**kw, **t)
        torch.cuda.synchronize()
        assert np.array_equal(host(t["grad"]), g)  # untouched without the schedule output
    for key, want in (("z_master", z2), ("x_master", x2), ("first_moment", a2), ("second_moment", b2_)):
        assert np.array_equal(host(t[key]), want), key  # IEEE elementwise: bit-exact


@pytest.mark.parametrize("R", [256, 1024])
def test_update_quantise_sweep_shapes_bit_exact(R):
    # bandwidth-sweep shapes [R, 4096]: update input N(0, 0.02) with 0.1 % of entries x 50
    rng = np.random.default_rng(R)
    r, c = R, 4096
    z, x = U.weights(rng, r * c), U.weights(rng, r * c)
    Um = U.with_outliers(rng, U.weights(rng, r * c))
    opt = b2.OptimizerModule()
    s = b2.MuonSlot.allocate(r, c)
    _fill_slot(s, np.zeros(r * c, F), np.zeros(r * c, np.uint16), z, x)
    plan = b2.MuonPlan([(r, c)])
    table = b2.slot_table([s])
    args = b2.MuonMegaUpdateArgs(learning_rate=0.02, average_coefficient=0.5, schedule_beta=0.2)
    opt.muon_tma_prepare_polar(plan, table, args)
    plan.scratch(0, 1).copy_(dev(Um).view(r, c))
    opt.muon_tma_finish_update(plan, table, args)
    torch.cuda.synchronize()
    z2, x2, y2, ax, ay = o.update(Um, z, x, r, c, 0.02, 0.025, 0.5, 0.2)
    assert np.array_equal(host(s.z_master).ravel(), z2) and np.array_equal(host(s.x_master).ravel(), x2)
    assert np.array_equal(host(s.grad).ravel(), y2)
    gs = host(s.global_scale)[0]
    codes, raw, ogs, misses = o.nvfp4_quantize(x2, amax=ax, rcp_table=rcp_table(gs))
    assert misses == 0 and gs == ogs and np.array_equal(host(s.bytes), codes)
    assert np.array_equal(host(s.scales), o.csf_encode(raw, r, c))
    plan.close()


def test_update_quantise_large_shape_properties():
    # 65536 x 4096 (268 M elements): too large for the CPU oracle in a test, so the checks are
    # size-independent: elementwise results against the same IEEE operations done by torch
    # (separate mul / sub kernels, no contraction), tensor maxima, and the packed output against
    # the literal one-thread-per-group device transcription of the reference quantiser.
    r, c = 65536, 4096
    n = r * c
    g = torch.Generator(device="cuda").manual_seed(1)
    z = torch.randn(n, device="cuda", generator=g) * 0.02
    x = torch.randn(n, device="cuda", generator=g) * 0.02
    Um = torch.randn(n, device="cuda", generator=g) * 0.02
    s = b2.MuonSlot.allocate(r, c)
    s.z_master.copy_(z.view(r, c)); s.x_master.copy_(x.view(r, c))
    plan = b2.MuonPlan([(r, c)])
    table = b2.slot_table([s])
    opt = b2.OptimizerModule()
    lr, wd, cavg, beta = 0.02, 0.025, 0.5, 0.2
    args = b2.MuonMegaUpdateArgs(learning_rate=lr, weight_decay=wd, average_coefficient=cavg, schedule_beta=beta)
    opt.muon_tma_prepare_polar(plan, table, args)
    plan.scratch(0, 1).copy_(Um.view(r, c))
    opt.muon_tma_finish_update(plan, table, args)
    torch.cuda.synchronize()
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device="cuda")
    scale = f32(0.2) * torch.sqrt(f32(float(max(r, c))))
    decay = f32(1.0) - f32(lr) * f32(wd)
    nz = z * decay - f32(lr) * (scale * Um)
    nx = x + f32(cavg) * (nz - x)
    ny = nz + f32(beta) * (nx - nz)
    assert torch.equal(s.z_master.view(-1), nz) and torch.equal(s.x_master.view(-1), nx)
    assert torch.equal(s.grad.view(-1), ny)
    assert s.schedule_amax.item() == ny.abs().max().item()
    amax = nx.abs().max().reshape(1)
    assert plan.scratch(0, 3).item() == amax.item()
    del z, x, Um, nz, ny
    lit4, lits, litg = b2.Nvfp4QuantModule().debug_quantize_literal(nx, amax)
    torch.cuda.synchronize()
    assert torch.equal(lit4, s.bytes) and torch.equal(litg, s.global_scale)
    raw = o.csf_decode_matrix(host(s.scales), r, c)
    assert np.array_equal(raw, host(lits))
    plan.close()


def test_grad_clip_reference_case_and_device_scale():
    # crates/cuda-kernels/tests/optimizer/grad_clip.rs:9-44
    opt = b2.OptimizerModule()
    first = dev(np.array([3.0, 4.0, 0.0, 0.0], F))
    second = dev(np.array([12.0, 0.0, 0.0, 0.0], F))
    ptrs = torch.tensor([first.data_ptr(), second.data_ptr()], dtype=torch.int64, device="cuda")
    lens = torch.tensor([4, 4], dtype=torch.int32, device="cuda")
    sums, scale, norm = torch.zeros(2, device="cuda"), torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    opt.clip_gradients(chunk_ptrs=ptrs, chunk_lens=lens, chunk_sums=sums, extra_sums=dev(np.array([27.0], F)),
                       scale=scale, norm=norm, chunk_count=2, extra_sum_count=1, max_norm=7.0, apply=True)
    torch.cuda.synchronize()
    assert np.allclose(host(first), [1.5, 2.0, 0, 0], atol=1e-6) and np.allclose(host(second), [6.0, 0, 0, 0], atol=1e-6)
    assert abs(host(scale)[0] - 0.5) <= 1e-6 and abs(host(norm)[0] - 14.0) <= 1e-6

    # many ragged chunks against the oracle; then the step consumes the scale from device memory
    rng = np.random.default_rng(9)
    r, c = 192, 256
    g = U.gradients(rng, r * c) * F(40.0)
    gd = dev(g)
    cuts = [0, 4096, 8192, 8195, 20000, r * c]
    ptrs = torch.tensor([gd.data_ptr() + 4 * a for a in cuts[:-1]], dtype=torch.int64, device="cuda")
    lens = torch.tensor([b - a for a, b in zip(cuts, cuts[1:])], dtype=torch.int32, device="cuda")
    sums = torch.zeros(5, device="cuda")
    opt.clip_gradients(chunk_ptrs=ptrs, chunk_lens=lens, chunk_sums=sums, extra_sums=None, scale=scale, norm=norm,
                       chunk_count=5, extra_sum_count=0, max_norm=1.0, apply=False)
    torch.cuda.synchronize()
    want_scale, want_norm = o.grad_clip([g[a:b] for a, b in zip(cuts, cuts[1:])], None, 1.0)
    assert want_scale < 1.0
    assert abs(host(norm)[0] - want_norm) <= 1e-6 * want_norm and abs(host(scale)[0] - want_scale) <= 1e-6
    assert np.array_equal(host(gd), g)  # apply = False leaves the gradients alone
    sc = host(scale)[0]
    results = []
    for use_device in (False, True):
        s = b2.MuonSlot.allocate(r, c)
        _fill_slot(s, g, np.zeros(r * c, np.uint16), np.zeros(r * c, F), np.zeros(r * c, F))
        plan = b2.MuonPlan([(r, c)])
        args = b2.MuonMegaUpdateArgs(grad_scale=(123.0 if use_device else float(sc)),
                                     grad_scale_device=(scale if use_device else None), iterations=1)
        opt.muon_tma_prepare_polar(plan, b2.slot_table([s]), args)
        torch.cuda.synchronize()
        results.append((bf16_bits(s.momentum).copy(), host(plan.scratch(0, 0).float()).copy()))
        plan.close()
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1])
    m2, _, _ = o.momentum(g, np.zeros(r * c, np.uint16), 0.95, sc)
    assert np.array_equal(results[1][0].ravel(), m2)


def test_multi_tensor_adamw_equals_per_tensor_calls():
    rng = np.random.default_rng(31)
    opt = b2.OptimizerModule()
    specs = [(768, 0), (4099, 0), (16 * 301, 1), (128 * 40, 2), (2048 * 3, 2), (0, 0), (16, 1)]
    hp = dict(grad_scale=0.7, learning_rate=2e-4, weight_decay=0.005, beta1=0.9, beta2=0.95, beta1_correction=0.19,
              beta2_correction=0.0975, eps=1e-10, average_coefficient=0.5, schedule_beta=0.3)

    def make(stale_amax):
        rng2 = np.random.default_rng(5)
        out = []
        for n, mode in specs:
            t = dict(z_master=dev(U.weights(rng2, n)), x_master=dev(U.weights(rng2, n)), grad=dev(U.gradients(rng2, n)),
                     first_moment=dev(U.weights(rng2, n, 1e-3)), second_moment=dev(np.abs(U.weights(rng2, n, 1e-6))),
                     len=n, mode=mode)
            if mode:
                t["amax"] = torch.full((1,), stale_amax, device="cuda")
            if mode == 2:
                q = b2.Nvfp4Tensor.empty(n // 128, 128)
                t.update(bytes=q.bytes, scales=q.scales, global_scale=q.global_scale,
                         chunk_amax=torch.zeros((n + 2047) // 2048, device="cuda"))
            out.append(t)
        return out

    # the multi-tensor call clears the amax words itself; the per-tensor deferred call raises
    # whatever the caller left there (the reference clears it with zero_f32_pointer_table)
    a, b = make(7.0), make(0.0)
    table, count, chunks = opt.adamw_table(a)
    opt.apply_adamw_update_multi(table, count, chunks, **hp)
    for t in b:
        if t["len"] == 0:
            continue
        kw = {k: v for k, v in t.items() if k != "mode"}
        if t["mode"] == 0:
            opt.apply_fp32_adamw_update(**hp, **kw)
        elif t["mode"] == 1:
            opt.apply_adamw_update_deferred_quantization(**hp, **kw)
        else:
            opt.apply_adamw_update(**hp, **kw)
    torch.cuda.synchronize()
    for ta, tb in zip(a, b):
        for key in ("z_master", "x_master", "grad", "first_moment", "second_moment", "amax", "bytes", "scales", "global_scale"):
            if key in ta:
                assert torch.equal(ta[key], tb[key]), (ta["len"], ta["mode"], key)


def test_multi_tensor_adamw_materialize_equals_per_tensor_precomputed():
    # deferred multi-tensor update, then ONE launch that quantises every deferred tensor's cached
    # y with its cached amax == materialize_schedule_free_precomputed per tensor, with the cached
    # values and with y rebuilt from the masters
    opt = b2.OptimizerModule()
    specs = [(128 * 6, 1), (128 * 40, 1), (4099, 0), (2048 * 3 + 128, 1), (128 * 8, 2)]
    hp = dict(grad_scale=0.7, learning_rate=2e-4, weight_decay=0.005, beta1=0.9, beta2=0.95, beta1_correction=0.19,
              beta2_correction=0.0975, eps=1e-10, average_coefficient=0.5, schedule_beta=0.3)
    rng = np.random.default_rng(77)
    tensors = []
    for n, mode in specs:
        t = dict(z_master=dev(U.weights(rng, n)), x_master=dev(U.weights(rng, n)), grad=dev(U.gradients(rng, n)),
                 first_moment=dev(U.weights(rng, n, 1e-3)), second_moment=dev(np.abs(U.weights(rng, n, 1e-6))),
                 len=n, mode=mode)
        if mode:
            t["amax"] = torch.zeros(1, device="cuda")
            q = b2.Nvfp4Tensor.empty(n // 128, 128)
            t.update(bytes=q.bytes, scales=q.scales, global_scale=q.global_scale, q=q)
        tensors.append(t)
    table, count, chunks = opt.adamw_table(tensors)
    opt.apply_adamw_update_multi(table, count, chunks, **hp)
    torch.cuda.synchronize()
    untouched = {i: (t["bytes"].clone(), t["global_scale"].clone()) for i, t in enumerate(tensors) if t["mode"] == 2}
    for cached in (True, False):
        for t in tensors:
            if t["mode"] == 1:
                t["bytes"].zero_()
                t["global_scale"].zero_()
                t["scales"][128:].zero_()
        opt.adamw_materialize_training_weights(table, count, chunks, hp["schedule_beta"], values_cached=cached)
        torch.cuda.synchronize()
        for i, t in enumerate(tensors):
            if t["mode"] == 2:  # other modes are left alone
                assert torch.equal(t["bytes"], untouched[i][0]) and torch.equal(t["global_scale"], untouched[i][1])
            if t["mode"] != 1:
                continue
            n = t["len"]
            ref = b2.Nvfp4Tensor.empty(n // 128, 128)
            opt.materialize_schedule_free_precomputed(
                bytes=ref.bytes, scales=ref.scales, global_scale=ref.global_scale, z_master=t["z_master"],
                x_master=t["x_master"], precomputed_values=(t["grad"] if cached else None), amax=t["amax"], len=n,
                scale_rows=n // 128, scale_k=128, beta=hp["schedule_beta"])
            torch.cuda.synchronize()
            assert torch.equal(t["bytes"], ref.bytes), (n, cached)
            assert torch.equal(t["scales"], ref.scales), (n, cached)
            assert torch.equal(t["global_scale"], ref.global_scale), (n, cached)
            if cached:  # and against the oracle on the cached values
                y = host(t["grad"]).ravel()
                am = host(t["amax"])[0]
                assert am == np.max(np.abs(y))
                gs = host(t["global_scale"])[0]
                codes, raw, ogs, _ = o.nvfp4_quantize(y, amax=am, rcp_table=rcp_table(gs))
                assert gs == ogs and np.array_equal(host(t["bytes"]), codes)
                assert np.array_equal(host(t["scales"]), o.csf_encode(raw, n // 128, 128))


def test_materialize_training_weights_for_all_slots():
    # deferred finish, then one launch that quantises every slot's cached y with its schedule_amax
    rng = np.random.default_rng(41)
    shapes = [(128, 256), (384, 128)]
    opt = b2.OptimizerModule()
    slots = [b2.MuonSlot.allocate(r, c) for r, c in shapes]
    plan = b2.MuonPlan(shapes)
    for i, (s, (r, c)) in enumerate(zip(slots, shapes)):
        _fill_slot(s, np.zeros(r * c, F), np.zeros(r * c, np.uint16), U.weights(rng, r * c), U.weights(rng, r * c))
    table = b2.slot_table(slots)
    args = b2.MuonMegaUpdateArgs(learning_rate=0.02, average_coefficient=0.5, schedule_beta=0.3)
    opt.muon_tma_prepare_polar(plan, table, args)
    for i, (r, c) in enumerate(shapes):
        plan.scratch(i, 1).copy_(dev((rng.standard_normal(r * c) * 0.05).astype(F)).view(r, c))
    opt.muon_tma_finish_update_deferred_quantization(plan, table, args)
    opt.muon_materialize_training_weights(plan, table)
    torch.cuda.synchronize()
    for s, (r, c) in zip(slots, shapes):
        y = host(s.grad).ravel()
        am = host(s.schedule_amax)[0]
        assert am == np.max(np.abs(y))
        gs = host(s.global_scale)[0]
        codes, raw, ogs, _ = o.nvfp4_quantize(y, amax=am, rcp_table=rcp_table(gs))
        assert gs == ogs and np.array_equal(host(s.bytes), codes)
        assert np.array_equal(host(s.scales), o.csf_encode(raw, r, c))
    plan.close()
