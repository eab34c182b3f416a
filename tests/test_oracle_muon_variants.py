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
