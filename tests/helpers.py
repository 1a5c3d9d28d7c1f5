"""Shared builders for the test-suite: seeded voxel clouds and oracle wrappers."""
import numpy as np


def random_cloud(seed, d, n, batch=1, lo=0):
    """`n` distinct voxels per sample in a d^3 cube starting at `lo`; int32 [N,4]."""
    rng = np.random.default_rng(seed)
    out = []
    for b in range(batch):
        lin = rng.choice(d ** 3, n, replace=False)
        xyz = np.stack([lin // (d * d), (lin // d) % d, lin % d], 1) + lo
        out.append(np.concatenate([np.full((n, 1), b), xyz], 1))
    return np.concatenate(out).astype(np.int32)


def surface_cloud(seed, d, batch=1):
    """A wavy 2-D sheet in a d^3 cube: dense in-plane neighbourhoods like a scanned surface."""
    rng = np.random.default_rng(seed)
    out = []
    for b in range(batch):
        x, y = np.meshgrid(np.arange(d), np.arange(d), indexing="ij")
        z = (d / 2 + d / 5 * np.sin(x / 5.0 + b) * np.cos(y / 7.0)).astype(np.int64)
        keep = rng.uniform(size=x.shape) < 0.8
        xyz = np.stack([x[keep], y[keep], z[keep]], 1)
        out.append(np.concatenate([np.full((len(xyz), 1), b), xyz], 1))
    return np.concatenate(out).astype(np.int32)


def cmax_of(coords):
    return coords[:, 1:].max(0).tolist() if len(coords) else [0, 0, 0]
