"""Shared helpers for the parity tests: seeded inputs and the error measure."""
import numpy as np


def uniform(shape, seed):
    """Uniform[-1, 1) float32 from a seeded generator (the f32 GEMM configurations)."""
    return np.random.default_rng(seed).uniform(-1.0, 1.0, size=shape).astype(np.float32)


def normal(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(size=shape, dtype=np.float32) * np.float32(scale))


def to_bf16_bits(x):
    """float32 -> bf16 (round to nearest even) as torch tensor, plus its float32 upcast."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16)
    return t, t.float().numpy()


def rel_err(got, want, scale=None):
    """max |got - want| relative to the output scale max |want| (the tolerance's measure)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    if scale is None:
        scale = np.abs(want).max()
    return float(np.abs(got - want).max() / max(scale, 1e-30))


def tile_mask(m, n, bm, bn, tile_ids):
    """Boolean [m, n] mask of the elements covered by the listed logical tiles."""
    mask = np.zeros((m, n), bool)
    tiles_n = n // bn
    for t in tile_ids:
        i, j = divmod(int(t), tiles_n)
        mask[i * bm:(i + 1) * bm, j * bn:(j + 1) * bn] = True
    return mask
