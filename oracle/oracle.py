"""ctypes/numpy front end of the CPU oracle in ``oracle.c``.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker or the timed CPU
baseline.  The shipped package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

ROUND_NONE, ROUND_F16, ROUND_BF16, ROUND_F16_HOST = 0, 1, 2, 3

# Fixed Newton-Schulz triple named by the benchmark configurations.
FIXED_TRIPLE = (3.4445, -4.7750, 2.0315)


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` with the Makefile beside it (idempotent)."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("oracle.c", "oracle.h", "Makefile"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_m:
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _LIB_PATH


class _RcpTable(C.Structure):
    _fields_ = [("in_bits", C.POINTER(C.c_uint32)), ("out_bits", C.POINTER(C.c_uint32)), ("count", C.c_uint32)]


class _MuonParams(C.Structure):
    _fields_ = [
        ("mu", C.c_float), ("grad_scale", C.c_float), ("learning_rate", C.c_float),
        ("weight_decay", C.c_float), ("average_coefficient", C.c_float), ("schedule_beta", C.c_float),
        ("iterations", C.c_int32), ("nesterov", C.c_int32), ("round_mode", C.c_int32),
        ("contract", C.c_int32), ("quantize_y", C.c_int32), ("deferred_normalize", C.c_int32),
        ("coeffs", C.POINTER(C.c_float)),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        try:
            L = C.CDLL(_LIB_PATH)
        except OSError:
            build(force=True)
            L = C.CDLL(_LIB_PATH)
        f32p, u8p, u16p, u32p = (C.POINTER(t) for t in (C.c_float, C.c_uint8, C.c_uint16, C.c_uint32))
        sig = {
            "orc_f32_to_bf16_bits": (C.c_uint16, [C.c_float]),
            "orc_round_bf16": (C.c_float, [C.c_float]),
            "orc_round_f16": (C.c_float, [C.c_float]),
            "orc_round_f16_host_flush": (C.c_float, [C.c_float]),
            "orc_f32_to_f16_bits": (C.c_uint16, [C.c_float]),
            "orc_f32_to_e4m3": (C.c_uint8, [C.c_float]),
            "orc_f32_to_e2m1": (C.c_uint8, [C.c_float]),
            "orc_e4m3_value": (C.c_float, [C.c_uint8]),
            "orc_e2m1_value": (C.c_float, [C.c_uint8]),
            "orc_rcp_exact_ftz": (C.c_float, [C.c_float]),
            "orc_four_six_global_scale": (C.c_float, [C.c_float]),
            "orc_nvfp4_rcp_inputs": (C.c_uint32, [C.c_float, C.c_int, f32p]),
            "orc_tensor_amax": (C.c_float, [f32p, C.c_uint64]),
            "orc_nvfp4_quantize": (C.c_uint64, [f32p, C.c_uint64, C.c_float, C.c_int, C.POINTER(_RcpTable), u8p, u8p, f32p]),
            "orc_nvfp4_dequantize": (None, [u8p, u8p, C.c_float, C.c_uint64, f32p]),
            "orc_csf_encoded_len": (C.c_uint64, [C.c_uint64, C.c_uint64]),
            "orc_csf_encode": (C.c_uint64, [u8p, C.c_uint64, C.c_uint64, C.c_uint64, u8p, C.c_uint64]),
            "orc_csf_scale_at": (C.c_uint8, [u8p, C.c_uint64]),
            "orc_momentum": (C.c_double, [f32p, u16p, f32p, C.c_uint64, C.c_float, C.c_float, C.c_int, C.c_int]),
            "orc_inv_norm": (C.c_float, [C.c_float, C.c_int]),
            "orc_momentum_vs": (C.c_double, [f32p, u16p, u16p, f32p, C.c_uint64, C.c_float, C.c_float, C.c_int, C.c_float]),
            "orc_update_clip": (None, [f32p, f32p, f32p, f32p, u16p, u16p, C.c_uint64, C.c_uint32, C.c_uint32] + [C.c_float] * 4 + [f32p, C.c_uint32, C.c_uint32, f32p]),
            "orc_normuon_stats": (None, [f32p, f32p, C.c_uint32, C.c_uint32, f32p, f32p, f32p]),
            "orc_update_normuon": (None, [f32p, f32p, f32p, f32p, C.c_uint64, C.c_uint32, C.c_uint32] + [C.c_float] * 4 + [f32p, C.c_float, f32p]),
            "orc_hyperball_update": (None, [f32p, f32p, f32p, f32p, u16p, u16p, C.c_uint32, C.c_uint32] + [C.c_float] * 3 + [C.c_int, f32p, f32p, f32p, C.c_uint32, C.c_uint32, f32p]),
            "orc_sign_update": (None, [f32p, u16p, u16p, f32p, f32p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_int] + [C.c_float] * 4 + [f32p, C.c_uint32, C.c_uint32, f32p]),
            "orc_polar_gram": (None, [f32p, C.c_int, C.c_int, C.c_int, f32p, C.c_int]),
            "orc_polar_gram_tall": (None, [f32p, C.c_int, C.c_int, C.c_int, f32p, C.c_int]),
            "orc_polar_three_product": (None, [f32p, C.c_int, C.c_int, C.c_int, f32p, C.c_int]),
            "orc_polar_gram_scaled": (None, [f32p, C.c_int, C.c_int, C.c_int, f32p, C.c_int, C.c_float]),
            "orc_polar_gram_tall_scaled": (None, [f32p, C.c_int, C.c_int, C.c_int, f32p, C.c_int, C.c_float]),
            "orc_set_threads": (None, [C.c_int]),
            "orc_max_threads": (C.c_int, []),
            "orc_update": (None, [f32p, f32p, f32p, f32p, C.c_uint64, C.c_uint32, C.c_uint32] + [C.c_float] * 4 + [C.c_int, f32p]),
            "orc_schedule_free_values": (C.c_float, [f32p, f32p, f32p, C.c_uint64, C.c_float, C.c_int]),
            "orc_adamw": (C.c_float, [f32p, f32p, f32p, f32p, f32p, f32p, C.c_uint64] + [C.c_float] * 10 + [C.c_int]),
            "orc_polar_first_iteration_scalar": (C.c_float, [C.c_float, C.c_int, C.c_int]),
            "orc_polar_express_coefficients": (None, [C.c_int, f32p]),
            "orc_muon_step": (C.c_uint64, [f32p, u16p, f32p, f32p, C.c_uint32, C.c_uint32, C.POINTER(_MuonParams), C.POINTER(_RcpTable), u8p, u8p, f32p, f32p, f32p]),
            "orc_grad_clip": (C.c_float, [C.POINTER(f32p), u32p, C.c_uint32, f32p, C.c_uint32, C.c_float, f32p]),
            "orc_round_operand": (C.c_float, [C.c_float, C.c_int]),
            "orc_warmup_only": (C.c_float, [C.c_uint32, C.c_uint32, C.c_float]),
            "orc_schedule_free_beta": (C.c_float, [C.c_uint32, C.c_uint32, C.c_float, C.c_float]),
            "orc_schedule_free_average_coefficient": (C.c_float, [C.c_uint32, C.c_uint32, C.c_float, f32p]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(C.POINTER(t))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _rcp(table):
    """table: None or (in_bits uint32[], out_bits uint32[]) -> (struct pointer, keepalive)."""
    if table is None:
        return None, None
    i = np.ascontiguousarray(table[0], dtype=np.uint32)
    o = np.ascontiguousarray(table[1], dtype=np.uint32)
    t = _RcpTable(_p(i, C.c_uint32), _p(o, C.c_uint32), len(i))
    return C.byref(t), (i, o, t)


# ---------------------------------------------------------------- scalar helpers
def round_bf16(a) -> np.ndarray:
    a = _f32(a)
    bits = a.view(np.uint32).astype(np.uint64)
    bias = 0x7FFF + ((bits >> 16) & 1)
    return (((bits + bias) >> 16) << 16).astype(np.uint32).view(np.float32).reshape(a.shape)


def bf16_bits(a) -> np.ndarray:
    a = _f32(a)
    bits = a.view(np.uint32).astype(np.uint64)
    bias = 0x7FFF + ((bits >> 16) & 1)
    return ((bits + bias) >> 16).astype(np.uint16).reshape(a.shape)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def polar_express_coefficients(iterations: int) -> np.ndarray:
    out = np.zeros(3 * iterations, dtype=np.float32)
    lib().orc_polar_express_coefficients(iterations, _p(out, C.c_float))
    return out.reshape(iterations, 3)


def fixed_coefficients(iterations: int) -> np.ndarray:
    return np.tile(np.asarray(FIXED_TRIPLE, dtype=np.float32), (iterations, 1))


def rcp_inputs(global_scale: float, contract: bool = False) -> np.ndarray:
    out = np.zeros(128, dtype=np.float32)
    lib().orc_nvfp4_rcp_inputs(np.float32(global_scale), int(contract), _p(out, C.c_float))
    return out


def four_six_global_scale(amax: float) -> np.float32:
    return np.float32(lib().orc_four_six_global_scale(np.float32(amax)))


# ---------------------------------------------------------------- quantiser
def nvfp4_quantize(x, amax=None, contract=False, rcp_table=None):
    """-> (codes u8[len/2], raw_scales u8[len/16], global_scale f32, table_misses)."""
    x = _f32(x).reshape(-1)
    assert x.size % 16 == 0
    if amax is None:
        amax = lib().orc_tensor_amax(_p(x, C.c_float), x.size)
    codes = np.zeros(x.size // 2, dtype=np.uint8)
    scales = np.zeros(x.size // 16, dtype=np.uint8)
    gs = C.c_float(0)
    tp, keep = _rcp(rcp_table)
    miss = lib().orc_nvfp4_quantize(_p(x, C.c_float), x.size, np.float32(amax), int(contract), tp,
                                    _p(codes, C.c_uint8), _p(scales, C.c_uint8), C.byref(gs))
    del keep
    return codes, scales, np.float32(gs.value), int(miss)


def nvfp4_dequantize(codes, raw_scales, global_scale) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    raw_scales = np.ascontiguousarray(raw_scales, dtype=np.uint8)
    n = codes.size * 2
    out = np.zeros(n, dtype=np.float32)
    lib().orc_nvfp4_dequantize(_p(codes, C.c_uint8), _p(raw_scales, C.c_uint8), np.float32(global_scale), n, _p(out, C.c_float))
    return out


def csf_encoded_len(rows: int, k: int) -> int:
    return int(lib().orc_csf_encoded_len(rows, k))


def csf_encode(raw, rows: int, k: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    cap = 128 + ((rows + 127) // 128) * ((k + 127) // 128) * 1024 + k // 16
    out = np.zeros(cap, dtype=np.uint8)
    n = lib().orc_csf_encode(_p(raw, C.c_uint8), raw.size, rows, k, _p(out, C.c_uint8), cap)
    if n == 0:
        raise ValueError("csf_encode precondition violated")
    return out[:n].copy()


def csf_decode(enc, groups: int) -> np.ndarray:
    enc = np.ascontiguousarray(enc, dtype=np.uint8)
    L = lib()
    p = _p(enc, C.c_uint8)
    return np.fromiter((L.orc_csf_scale_at(p, g) for g in range(groups)), dtype=np.uint8, count=groups)


def csf_decode_matrix(enc, rows: int, k: int) -> np.ndarray:
    """Vectorised decode of a one-mask-byte CSF matrix (numpy; same addressing as csf_decode)."""
    enc = np.ascontiguousarray(enc, dtype=np.uint8)
    if enc[8] == 255:
        return enc[128:128 + k // 16].copy()
    assert enc[9] == 7
    d = enc[128:].astype(np.uint32)
    groups = k // 16
    row = np.repeat(np.arange(rows, dtype=np.uint32), groups)
    kg = np.tile(np.arange(groups, dtype=np.uint32), rows)
    t = row // 128 * (k // 128) + kg // 8
    r = row % 128
    at = t * 896 + (r // 16) * 96 + (r % 8) * 12 + (r % 16 // 8) * 3 + (kg % 8 // 4) * 6
    word = d[at] | (d[at + 1] << 8) | (d[at + 2] << 16)
    q = (word >> ((kg % 4) * 6)) & 63
    mask = d[t * 896 + 768 + r]
    return (q | (((mask >> (kg % 8)) & 1) << 6)).astype(np.uint8)


# ---------------------------------------------------------------- Muon stages
def momentum(grad, momentum_bits, mu, grad_scale, nesterov=True, contract=False):
    """-> (momentum' bf16 bits, u f32, sumsq float64); inputs untouched."""
    g = _f32(grad).reshape(-1)
    m = np.ascontiguousarray(momentum_bits, dtype=np.uint16).reshape(-1).copy()
    u = np.zeros_like(g)
    s = lib().orc_momentum(_p(g, C.c_float), _p(m, C.c_uint16), _p(u, C.c_float), g.size,
                           np.float32(mu), np.float32(grad_scale), int(nesterov), int(contract))
    return m, u, float(s)


def momentum_vs(grad, momentum_bits, variance_bits, mu, grad_scale, nesterov, bias_correction_inv):
    """Muon-VS branch -> (momentum' bits, variance' bits, u, sumsq)."""
    g = _f32(grad).reshape(-1)
    m = np.ascontiguousarray(momentum_bits, dtype=np.uint16).reshape(-1).copy()
    v = np.ascontiguousarray(variance_bits, dtype=np.uint16).reshape(-1).copy()
    u = np.zeros_like(g)
    s = lib().orc_momentum_vs(_p(g, C.c_float), _p(m, C.c_uint16), _p(v, C.c_uint16), _p(u, C.c_float), g.size,
                              np.float32(mu), np.float32(grad_scale), int(nesterov), np.float32(bias_correction_inv))
    return m, v, u, float(s)


def update_clip(U, z, x, momentum_bits, variance_bits, rows, cols, lr, wd, c_avg, beta, factors, offset, head_dim):
    """Stage U with qk-clip -> (z', x', y, momentum bits, variance bits or None, amax_x, amax_y)."""
    U = _f32(U).reshape(-1); z = _f32(z).reshape(-1).copy(); x = _f32(x).reshape(-1).copy()
    y = np.zeros_like(z); am = np.zeros(2, np.float32)
    m = np.ascontiguousarray(momentum_bits, dtype=np.uint16).reshape(-1).copy()
    v = None if variance_bits is None else np.ascontiguousarray(variance_bits, dtype=np.uint16).reshape(-1).copy()
    fa = _f32(factors).reshape(-1)
    f = np.float32
    lib().orc_update_clip(_p(U, C.c_float), _p(z, C.c_float), _p(x, C.c_float), _p(y, C.c_float), _p(m, C.c_uint16),
                          None if v is None else _p(v, C.c_uint16), z.size, rows, cols, f(lr), f(wd), f(c_avg), f(beta),
                          _p(fa, C.c_float), offset, head_dim, _p(am, C.c_float))
    return z, x, y, m, v, am[0], am[1]


def sign_update(grad, momentum_bits, variance_bits, z, x, rows, cols, mu, grad_scale, variance_adaptive, lr, wd, c_avg,
                beta, factors=None, offset=0xFFFFFFFF, head_dim=0):
    """sign-Muon -> (y, momentum bits, variance bits, z', x', amax_x, amax_y)."""
    g = _f32(grad).reshape(-1).copy(); z = _f32(z).reshape(-1).copy(); x = _f32(x).reshape(-1).copy()
    m = np.ascontiguousarray(momentum_bits, dtype=np.uint16).reshape(-1).copy()
    v = np.ascontiguousarray(variance_bits if variance_bits is not None else np.zeros(g.size, np.uint16), dtype=np.uint16).reshape(-1).copy()
    am = np.zeros(2, np.float32)
    fa = None if factors is None else _f32(factors).reshape(-1)
    f = np.float32
    lib().orc_sign_update(_p(g, C.c_float), _p(m, C.c_uint16), _p(v, C.c_uint16), _p(z, C.c_float), _p(x, C.c_float),
                          g.size, rows, cols, f(mu), f(grad_scale), int(variance_adaptive), f(lr), f(wd), f(c_avg),
                          f(beta), None if fa is None else _p(fa, C.c_float), offset, head_dim, _p(am, C.c_float))
    return g, m, v, z, x, am[0], am[1]


def normuon_stats(U, rows, cols, second_momentum, z=None):
    """NorMuon second moment (+ Hyperball statistics when z is given); U in storage orientation.
    -> (second_momentum', factors, stats[normuon_scale, update_norm, radius, dot])."""
    U = _f32(U).reshape(-1)
    sm = _f32(second_momentum).reshape(-1).copy()
    assert sm.size == max(rows, cols) and U.size == rows * cols
    fa = np.zeros_like(sm); st = np.zeros(4, np.float32)
    zz = None if z is None else _f32(z).reshape(-1)
    lib().orc_normuon_stats(_p(U, C.c_float), None if zz is None else _p(zz, C.c_float), rows, cols,
                            _p(sm, C.c_float), _p(fa, C.c_float), _p(st, C.c_float))
    return sm, fa, st


def update_normuon(U, z, x, rows, cols, lr, wd, c_avg, beta, factors, normuon_scale):
    """Stage U with NorMuon factors -> (z', x', y, amax_x, amax_y)."""
    U = _f32(U).reshape(-1); z = _f32(z).reshape(-1).copy(); x = _f32(x).reshape(-1).copy()
    y = np.zeros_like(z); am = np.zeros(2, np.float32); fa = _f32(factors).reshape(-1)
    f = np.float32
    lib().orc_update_normuon(_p(U, C.c_float), _p(z, C.c_float), _p(x, C.c_float), _p(y, C.c_float), z.size, rows, cols,
                             f(lr), f(wd), f(c_avg), f(beta), _p(fa, C.c_float), f(normuon_scale), _p(am, C.c_float))
    return z, x, y, am[0], am[1]


def hyperball_update(U, z, x, rows, cols, lr, c_avg, beta, use_schedule_free, factors, stats, momentum_bits=None,
                     variance_bits=None, clip_factors=None, offset=0xFFFFFFFF, head_dim=0):
    """Hyperball projection -> (z', x', y, momentum bits, variance bits, amax_x, amax_y)."""
    U = _f32(U).reshape(-1); z = _f32(z).reshape(-1).copy(); x = _f32(x).reshape(-1).copy()
    y = np.zeros_like(z); am = np.zeros(2, np.float32)
    fa = _f32(factors).reshape(-1); st = _f32(stats).reshape(-1)
    m = np.zeros(z.size, np.uint16) if momentum_bits is None else np.ascontiguousarray(momentum_bits, dtype=np.uint16).reshape(-1).copy()
    v = None if variance_bits is None else np.ascontiguousarray(variance_bits, dtype=np.uint16).reshape(-1).copy()
    cf = None if clip_factors is None else _f32(clip_factors).reshape(-1)
    f = np.float32
    lib().orc_hyperball_update(_p(U, C.c_float), _p(z, C.c_float), _p(x, C.c_float), _p(y, C.c_float), _p(m, C.c_uint16),
                               None if v is None else _p(v, C.c_uint16), rows, cols, f(lr), f(c_avg), f(beta),
                               int(use_schedule_free), _p(fa, C.c_float), _p(st, C.c_float),
                               None if cf is None else _p(cf, C.c_float), offset, head_dim, _p(am, C.c_float))
    return z, x, y, m, v, am[0], am[1]


def sm100_blocked(raw_scales, rows, cols):
    """Block scales [rows][cols/16] -> the block-scale operand layout of sm_100 tensor cores, as
    published for cuBLASLt's VEC16_UE4M3 scale mode and restated by PyTorch / torchao as
    `to_blocked`: pad to 128 rows x 4 columns, tiles (row/128, col/4) row-major, and inside a
    512-byte tile byte (row % 32) * 16 + (row % 128) // 32 * 4 + col % 4."""
    per_row = cols // 16
    a = np.asarray(raw_scales, np.uint8).reshape(rows, per_row)
    rb, cb = -(-rows // 128), -(-per_row // 4)
    pad = np.zeros((rb * 128, cb * 4), np.uint8)
    pad[:rows, :per_row] = a
    t = pad.reshape(rb, 128, cb, 4).transpose(0, 2, 1, 3)      # [rb][cb][128][4]
    t = t.reshape(rb * cb, 4, 32, 4).transpose(0, 2, 1, 3)       # [tile][32][4][4]
    return np.ascontiguousarray(t).reshape(-1)


def sm100_unblocked(blocked, rows, cols):
    """Inverse of `sm100_blocked` (drops the padding)."""
    per_row = cols // 16
    rb, cb = -(-rows // 128), -(-per_row // 4)
    t = np.asarray(blocked, np.uint8).reshape(rb * cb, 32, 4, 4).transpose(0, 2, 1, 3).reshape(rb, cb, 128, 4)
    return np.ascontiguousarray(t.transpose(0, 2, 1, 3).reshape(rb * 128, cb * 4)[:rows, :per_row]).reshape(-1)


def inv_norm(sumsq, contract=False) -> np.float32:
    return np.float32(lib().orc_inv_norm(np.float32(sumsq), int(contract)))


def set_threads(n: int) -> int:
    """Host threads for the OpenMP loops (the CPU-baseline legs of bench.py); returns the count in effect."""
    lib().orc_set_threads(int(n))
    return int(lib().orc_max_threads())


def polar(X, iterations, coeffs, round_mode=ROUND_BF16, form="gram", first_scale=1.0):
    """Newton-Schulz on a storage-layout matrix [rows][cols]; returns a new array.  `first_scale` != 1:
    X is un-normalised and the Frobenius scale enters through the first iteration (one-pass prepare)."""
    X = _f32(X).copy()
    rows, cols = X.shape
    co = _f32(coeffs).reshape(-1)
    assert co.size >= 3 * iterations
    L = lib()
    if form == "gram":
        fs = np.float32(first_scale)
        if rows > cols:
            L.orc_polar_gram_tall_scaled(_p(X, C.c_float), rows, cols, iterations, _p(co, C.c_float), round_mode, fs)
        else:
            L.orc_polar_gram_scaled(_p(X, C.c_float), rows, cols, iterations, _p(co, C.c_float), round_mode, fs)
        return X
    assert form == "three_product"
    if rows > cols:
        Xt = np.ascontiguousarray(X.T)
        L.orc_polar_three_product(_p(Xt, C.c_float), cols, rows, iterations, _p(co, C.c_float), round_mode)
        return np.ascontiguousarray(Xt.T)
    L.orc_polar_three_product(_p(X, C.c_float), rows, cols, iterations, _p(co, C.c_float), round_mode)
    return X


def update(U, z, x, rows, cols, lr, wd, c_avg, beta, contract=False):
    """-> (z', x', y, amax_x, amax_y)."""
    U = _f32(U).reshape(-1)
    z = _f32(z).reshape(-1).copy()
    x = _f32(x).reshape(-1).copy()
    y = np.zeros_like(z)
    am = np.zeros(2, dtype=np.float32)
    lib().orc_update(_p(U, C.c_float), _p(z, C.c_float), _p(x, C.c_float), _p(y, C.c_float), z.size, rows, cols,
                     np.float32(lr), np.float32(wd), np.float32(c_avg), np.float32(beta), int(contract), _p(am, C.c_float))
    return z, x, y, am[0], am[1]


def schedule_free_values(z, x, beta, contract=False):
    z = _f32(z).reshape(-1)
    x = _f32(x).reshape(-1)
    y = np.zeros_like(z)
    am = lib().orc_schedule_free_values(_p(z, C.c_float), _p(x, C.c_float), _p(y, C.c_float), z.size, np.float32(beta), int(contract))
    return y, np.float32(am)


def adamw(z, x, grad, m1, m2, grad_scale, lr, wd, beta1, beta2, bc1, bc2, eps, c_avg, sched_beta, contract=False):
    """-> (z', x', y, m1', m2', amax_y)."""
    z = _f32(z).reshape(-1).copy(); x = _f32(x).reshape(-1).copy()
    g = _f32(grad).reshape(-1); m1 = _f32(m1).reshape(-1).copy(); m2 = _f32(m2).reshape(-1).copy()
    y = np.zeros_like(z)
    f = np.float32
    am = lib().orc_adamw(_p(z, C.c_float), _p(x, C.c_float), _p(g, C.c_float), _p(y, C.c_float), _p(m1, C.c_float),
                         _p(m2, C.c_float), z.size, f(grad_scale), f(lr), f(wd), f(beta1), f(beta2), f(bc1), f(bc2),
                         f(eps), f(c_avg), f(sched_beta), int(contract))
    return z, x, y, m1, m2, np.float32(am)


def grad_clip(chunks, extra_sums, max_norm):
    """-> (scale, norm) of the global gradient-norm clip over a list of f32 arrays."""
    arrs = [_f32(c).reshape(-1) for c in chunks]
    n = len(arrs)
    ptrs = (C.POINTER(C.c_float) * max(n, 1))(*[_p(a, C.c_float) for a in arrs])
    lens = (C.c_uint32 * max(n, 1))(*[a.size for a in arrs])
    ex = _f32(extra_sums).reshape(-1) if extra_sums is not None and len(extra_sums) else np.zeros(0, np.float32)
    norm = C.c_float(0)
    sc = lib().orc_grad_clip(ptrs, lens, n, _p(ex, C.c_float) if ex.size else None, ex.size, np.float32(max_norm), C.byref(norm))
    return np.float32(sc), np.float32(norm.value)


@dataclass
class MuonResult:
    momentum_bits: np.ndarray
    z: np.ndarray
    x: np.ndarray
    y: np.ndarray
    codes: np.ndarray
    raw_scales: np.ndarray
    global_scale: np.float32
    schedule_amax: np.float32
    U: np.ndarray
    rcp_misses: int


def muon_step(grad, momentum_bits, z, x, rows, cols, *, mu, grad_scale, lr, wd, c_avg, sched_beta,
              iterations, coeffs, nesterov=True, round_mode=ROUND_BF16, contract=False,
              quantize_y=False, rcp_table=None, deferred_normalize=False) -> MuonResult:
    g = _f32(grad).reshape(-1).copy()
    m = np.ascontiguousarray(momentum_bits, dtype=np.uint16).reshape(-1).copy()
    z = _f32(z).reshape(-1).copy(); x = _f32(x).reshape(-1).copy()
    n = rows * cols
    co = _f32(coeffs).reshape(-1)
    prm = _MuonParams(mu, grad_scale, lr, wd, c_avg, sched_beta, iterations, int(nesterov), round_mode,
                      int(contract), int(quantize_y), int(deferred_normalize), _p(co, C.c_float))
    codes = np.zeros(n // 2, dtype=np.uint8); sc = np.zeros(n // 16, dtype=np.uint8)
    gs = C.c_float(0); sa = C.c_float(0)
    U = np.zeros(n, dtype=np.float32)
    tp, keep = _rcp(rcp_table)
    miss = lib().orc_muon_step(_p(g, C.c_float), _p(m, C.c_uint16), _p(z, C.c_float), _p(x, C.c_float), rows, cols,
                               C.byref(prm), tp, _p(codes, C.c_uint8), _p(sc, C.c_uint8), C.byref(gs), C.byref(sa),
                               _p(U, C.c_float))
    del keep
    return MuonResult(m, z, x, g, codes, sc, np.float32(gs.value), np.float32(sa.value), U.reshape(rows, cols), int(miss))
