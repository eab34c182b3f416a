"""Seeded synthetic inputs with the distributions the benchmark configurations name."""
import numpy as np

F = np.float32


def weights(rng, shape, std=0.02):
    return (rng.standard_normal(shape) * std).astype(F)


def gradients(rng, shape, std=1.0e-3, outlier_fraction=0.001, outlier_scale=50.0):
    g = (rng.standard_normal(shape) * std).astype(F)
    if outlier_fraction > 0:
        mask = rng.random(shape) < outlier_fraction
        g = np.where(mask, g * F(outlier_scale), g).astype(F)
    return g


def with_outliers(rng, x, fraction=0.001, scale=50.0):
    mask = rng.random(x.shape) < fraction
    return np.where(mask, x * F(scale), x).astype(F)


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def max_rel_to_peak(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-300))
