"""Generates the golden fixtures in this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust + cuda-oxide) cannot be run where this repository is built, so these
vectors are NOT reference outputs: they freeze the oracle's own results on small seeded
inputs, so that a later change to the oracle or to the CUDA kernels that alters any bit of the
quantiser output, the CSF packing, or the elementwise stages is caught.  The oracle itself is
pinned against the reference's known answers in tests/test_oracle_known_answers.py.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as o  # noqa: E402

F = np.float32


def inputs():
    rng = np.random.default_rng(20261125)
    rows, cols = 64, 128
    n = rows * cols
    g = (rng.standard_normal(n) * 1e-3).astype(F)
    g[rng.random(n) < 0.001] *= F(50.0)
    z = (rng.standard_normal(n) * 0.02).astype(F)
    x = (rng.standard_normal(n) * 0.02).astype(F)
    m = o.bf16_bits((rng.standard_normal(n) * 1e-3).astype(F))
    return rows, cols, g, m, z, x


def main():
    rows, cols, g, m, z, x = inputs()
    # quantiser + CSF on the weights themselves
    codes, raw, gs, _ = o.nvfp4_quantize(x)
    csf = o.csf_encode(raw, rows, cols)
    # one whole step, benchmark recipe (BF16 operands, fixed triple)
    r = o.muon_step(g, m, z, x, rows, cols, mu=0.95, grad_scale=1.0, lr=0.02, wd=0.025, c_avg=0.5, sched_beta=0.2,
                    iterations=5, coeffs=o.fixed_coefficients(5), round_mode=o.ROUND_BF16)
    # elementwise stages on their own
    m2, u, ss = o.momentum(g, m, 0.95, 1.0)
    az, ax, ay, a1, a2, aam = o.adamw(z, x, g, np.zeros_like(z), np.zeros_like(z), 1.0, 2e-4, 0.005, 0.9, 0.95, 0.1, 0.05,
                                      1e-10, 0.5, 0.2)
    np.savez_compressed(
        os.path.join(HERE, "muon_nvfp4_64x128.npz"),
        rows=rows, cols=cols, grad=g, momentum_bits=m, z=z, x=x,
        q_codes=codes, q_raw_scales=raw, q_global_scale=gs, q_csf=csf,
        step_momentum_bits=r.momentum_bits, step_z=r.z, step_x=r.x, step_y=r.y, step_codes=r.codes,
        step_raw_scales=r.raw_scales, step_global_scale=r.global_scale, step_schedule_amax=r.schedule_amax, step_U=r.U,
        mom_bits=m2, mom_u=u, mom_sumsq=np.float64(ss),
        adam_z=az, adam_x=ax, adam_y=ay, adam_m1=a1, adam_m2=a2, adam_amax=aam)
    print("wrote", os.path.join(HERE, "muon_nvfp4_64x128.npz"))


if __name__ == "__main__":
    main()
