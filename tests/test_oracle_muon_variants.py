"""Oracle pins for the Muon variants: variance-adaptive momentum (Muon-VS), qk-clip in the update
stage and sign-Muon.  Each case restates the host recurrence of the reference's own test in numpy
float32 (one rounding per operation, like the Rust expressions) and holds the oracle to the
tolerance that test states."""
import numpy as np
import pytest

from oracle import oracle as o

F = np.float32


def _bf16(v):
    return o.round_bf16(np.asarray(v, F))


@pytest.mark.parametrize("rows,cols", [(64, 128), (128, 64)])
@pytest.mark.parametrize("nesterov", [True, False])
def test_muon_vs_prepare_recurrence(rows, cols, nesterov):
    # crates/cuda-kernels/tests/optimizer/muon/tma_prepare.rs:87-208, variance_adaptive = true
    n = rows * cols
    i = np.arange(n)
    grad = ((i * 73 % 257).astype(F) - F(128.0)) / F(211.0)
    m = _bf16(((i * 29 % 131).astype(F) - F(65.0)) / F(173.0))
    v = _bf16(F(0.01) + (i * 17 % 97).astype(F) / F(503.0))
    m_bits, v_bits = o.bf16_bits(m), o.bf16_bits(v)
    mu, one = F(0.9), F(1.0)
    for step in range(3, 9):
        bci = F(1.0) / (F(1.0) - _powi(F(0.9), step))
        g = grad * F(0.125)
        nxt = mu * m + (one - mu) * g
        inn = m - g
        nv = mu * v + mu * (one - mu) * inn * inn
        corrected = nxt * bci
        num = g + (mu / (one - mu)) * corrected if nesterov else corrected
        upd = num / (np.sqrt(nv * bci) + F(1.0e-8))
        m, v = _bf16(nxt), _bf16(nv)
        m_bits, v_bits, u, ss = o.momentum_vs(grad, m_bits, v_bits, 0.9, 0.125, nesterov, bci)
        assert np.array_equal(m_bits, o.bf16_bits(m))
        assert np.array_equal(v_bits, o.bf16_bits(v))
        assert np.max(np.abs(u - upd)) <= 5.0e-5
        assert abs(ss - float(np.sum(upd.astype(np.float64) ** 2))) <= 1e-6 * ss


def _powi(base, n):
    """f32 `powi` by repeated multiplication (each product rounded to float32)."""
    r = F(1.0)
    for _ in range(n):
        r = F(r * base)
    return r


@pytest.mark.parametrize("variance_adaptive", [False, True])
def test_sign_update_reference_case(variance_adaptive):
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:686-840
    n = 32 * 32
    i = np.arange(n)
    grad = ((i * 41 % 97).astype(F) - F(48.0)) / F(37.0)
    m = _bf16(((i * 17 % 61).astype(F) - F(30.0)) / F(53.0))
    v = _bf16(F(0.02) + (i * 19 % 89).astype(F) / F(401.0))
    z = (i.astype(F) - F(511.0)) / F(997.0)
    x = (F(307.0) - i.astype(F)) / F(613.0)
    mu, gs, beta, c = F(0.9), F(0.25), F(0.4), F(0.3)
    lr = F(0.004) * F(0.75)
    decay = F(1.0) - lr * F(0.1)
    nm = mu * m + (F(1.0) - mu) * grad * gs
    g = grad * gs
    inn = m - g
    nv = mu * v + mu * (F(1.0) - mu) * inn * inn
    nz = z * decay - lr * np.sign(nm).astype(F)
    nx = x + c * (nz - x)
    amax = np.max(np.abs(nz + beta * (nx - nz)))
    y, mb, vb, z2, x2, ax, ay = o.sign_update(grad, o.bf16_bits(m), o.bf16_bits(v), z, x, 32, 32, mu, gs,
                                               variance_adaptive, lr, 0.1, c, beta)
    assert np.array_equal(mb, o.bf16_bits(_bf16(nm)))
    if variance_adaptive:
        assert np.array_equal(vb, o.bf16_bits(_bf16(nv)))
    else:
        assert np.array_equal(vb, o.bf16_bits(v))
    assert np.max(np.abs(z2 - nz)) <= 1e-6 and np.max(np.abs(x2 - nx)) <= 1e-6
    assert abs(ay - amax) <= 1e-6 and ax == np.max(np.abs(x2))
    assert np.array_equal(y, (z2 + beta * (x2 - z2)).astype(F))


@pytest.mark.parametrize("input_dim,output_dim", [(2048, 64), (2048, 6272), (64, 256)])
def test_qk_clip_reference_case(input_dim, output_dim):
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:112-262: rows = output_dim,
    # cols = input_dim, heads of 32 inputs alternate 0.5 / 0.25, rows >= 2*input_dim are left alone
    n = input_dim * output_dim
    head = 32
    factors = np.where(np.arange(input_dim // head) % 2 == 0, F(0.5), F(0.25)).astype(F)
    z, x = np.full(n, 1.0, F), np.full(n, 2.0, F)
    m, v = np.full(n, 3.0, F), np.full(n, 4.0, F)
    row_factor = np.ones(output_dim, F)
    for r in range(min(output_dim, 2 * input_dim)):
        row_factor[r] = factors[(r % input_dim) // head]
    f = np.repeat(row_factor, input_dim)
    z2, x2, y, mb, vb, ax, ay = o.update_clip(np.zeros(n, F), z, x, o.bf16_bits(m), o.bf16_bits(v), output_dim,
                                              input_dim, 0.0, 0.0, 0.0, 0.4, factors, 0, head)
    assert np.array_equal(z2, z * f) and np.array_equal(x2, x * f)
    assert np.array_equal(mb, o.bf16_bits(_bf16(m * f)))
    assert np.array_equal(vb, o.bf16_bits(_bf16(v * f * f)))
    assert ay == np.max(np.abs(z2 + F(0.4) * (x2 - z2)))


def _seq_sum(v):
    """Left-to-right float32 sum, like `iter().sum::<f32>()`."""
    return np.cumsum(np.asarray(v, F), dtype=F)[-1]


def test_normuon_reference_case():
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:264-384 (32 x 32, beta2 0.95)
    n, lr = 32, F(0.01)
    idx = np.arange(n * n)
    update = ((idx // n + 1).astype(F) * (idx % n % 7 + 1).astype(F) / F(128.0)).astype(F)
    old = (F(0.01) + np.arange(n).astype(F) / F(10000.0)).astype(F)
    U = update.reshape(n, n)
    row_sumsq = np.array([_seq_sum(U[r] ** 2) for r in range(n)], F)
    nxt = F(0.95) * old + (F(1.0) - F(0.95)) * (row_sumsq / F(n))
    fac = F(1.0) / np.sqrt(np.maximum(nxt, F(1e-10)))
    raw, scaled = _seq_sum(row_sumsq), _seq_sum(row_sumsq * fac * fac)
    scale = np.sqrt(raw / max(scaled, F(1e-10)))
    sm, fa, st = o.normuon_stats(update, n, n, old)
    assert np.max(np.abs(sm - nxt)) <= 2e-6 and np.max(np.abs(fa - fac)) <= 2e-5
    assert abs(st[0] - scale) <= 2e-6
    z2, x2, y, ax, ay = o.update_normuon(update, np.zeros(n * n, F), np.zeros(n * n, F), n, n, lr, 0.0, 1.0, 0.4,
                                         fa, st[0])
    want = -lr * (F(0.2) * np.sqrt(F(n))) * update * np.repeat(fac, n) * scale
    assert np.max(np.abs(z2 - want)) <= 2e-6 and np.max(np.abs(x2 - want)) <= 2e-6
    # NorMuon keeps the update's Frobenius norm
    t = update * np.repeat(fa, n) * st[0]
    assert abs(float(np.sum(t.astype(np.float64) ** 2)) - raw) <= raw * 2e-5


def _hyperball_expected(update_storage, factors_neuron, z, x, rows, cols, lr_eff, c_avg, use_sf):
    neuron = (np.arange(rows * cols) // cols) if rows >= cols else (np.arange(rows * cols) % cols)
    direction = update_storage * factors_neuron[neuron]
    radius = np.sqrt(_seq_sum(z * z))
    update_norm = np.sqrt(_seq_sum(direction * direction))
    step = lr_eff * radius / update_norm
    cand = z - step * direction
    proj = radius / np.sqrt(_seq_sum(cand * cand))
    ez = cand * proj
    ex = x + c_avg * (ez - x) if use_sf else ez
    return ez.astype(F), ex.astype(F), radius, update_norm


def test_hyperball_reference_case_square():
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:386-531
    n = 32
    idx = np.arange(n * n)
    update = (((idx // n * 13 + idx % n * 7) % 41).astype(F) / F(37.0) - F(0.5)).astype(F)
    old = (F(0.02) + np.arange(n).astype(F) / F(20000.0)).astype(F)
    z = (((idx * 29 % 211).astype(F) - F(105.0)) / F(173.0)).astype(F)
    x = (((idx * 17 % 157).astype(F) - F(78.0)) / F(199.0)).astype(F)
    sm, fa, st = o.normuon_stats(update, n, n, old, z=z)
    rows_sumsq = np.array([_seq_sum(update.reshape(n, n)[r] ** 2) for r in range(n)], F)
    fac = F(1.0) / np.sqrt(np.maximum(F(0.95) * old + (F(1.0) - F(0.95)) * rows_sumsq / F(n), F(1e-10)))
    ez, ex, radius, unorm = _hyperball_expected(update, fac, z, x, n, n, F(0.018) * F(0.75), F(0.3), True)
    assert abs(st[1] - unorm) <= unorm * 3e-5 and abs(st[2] - radius) <= radius * 3e-5
    z2, x2, y, _, _, ax, ay = o.hyperball_update(update, z, x, n, n, F(0.018) * F(0.75), 0.3, 0.4, True, fa, st)
    assert np.max(np.abs(z2 - ez)) <= 3e-5 and np.max(np.abs(x2 - ex)) <= 3e-5
    r2 = np.sqrt(np.sum(z2.astype(np.float64) ** 2))
    assert abs(r2 - radius) <= radius * 3e-5
    assert abs(ay - np.max(np.abs(ez + F(0.4) * (ex - ez)))) <= 3e-5


@pytest.mark.parametrize("rows,cols", [(32, 64), (64, 32)])
def test_hyperball_reference_case_rectangular(rows, cols):
    # crates/cuda-kernels/tests/optimizer/muon/tma_finish.rs:533-676; the reference hands the update
    # over in polar orientation [min][max], this build keeps it in storage orientation
    n = rows * cols
    pr, pc = min(rows, cols), max(rows, cols)
    idx = np.arange(n)
    polar = (((idx * 23 % 101).astype(F) - F(50.0)) / F(71.0)).astype(F).reshape(pr, pc)
    storage = (polar.T if rows > cols else polar).reshape(-1).copy()
    old = (F(0.015) + np.arange(pc).astype(F) / F(30000.0)).astype(F)
    z = (((idx * 31 % 193).astype(F) - F(96.0)) / F(151.0)).astype(F)
    col_sumsq = np.array([_seq_sum(polar[:, k] ** 2) for k in range(pc)], F)
    fac = F(1.0) / np.sqrt(np.maximum(F(0.95) * old + (F(1.0) - F(0.95)) * col_sumsq / F(pr), F(1e-10)))
    ez, _, radius, _ = _hyperball_expected(storage, fac, z, np.zeros(n, F), rows, cols, F(0.018) * F(0.625), F(1.0),
                                           False)
    sm, fa, st = o.normuon_stats(storage, rows, cols, old, z=z)
    assert np.max(np.abs(fa - fac)) <= 2e-5
    z2, x2, *_ = o.hyperball_update(storage, z, np.zeros(n, F), rows, cols, F(0.018) * F(0.625), 1.0, 0.4, False, fa,
                                    st)
    assert np.max(np.abs(z2 - ez)) <= 4e-5 and np.array_equal(z2, x2)
    assert abs(np.sqrt(np.sum(z2.astype(np.float64) ** 2)) - radius) <= radius * 4e-5
