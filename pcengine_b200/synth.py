"""Seeded synthetic voxel clouds that stand in for the workloads the engine is
measured on (no public dataset is reproduced): a uniform random grid sample, a
spinning-LiDAR-shaped scan, an indoor-room-shaped surface sample and a tiled
multi-room scene.  NumPy only; every generator returns int32 [N,3] voxel
coordinates that are unique and non-negative.
"""
from __future__ import annotations

import numpy as np


def uniform_grid(n: int = 20000, grid: int = 64, seed: int = 1001) -> np.ndarray:
    """``n`` distinct voxels drawn uniformly without replacement from grid^3."""
    rng = np.random.default_rng(seed)
    lin = rng.choice(grid ** 3, size=n, replace=False)
    return np.stack([lin // (grid * grid), (lin // grid) % grid, lin % grid], axis=1).astype(np.int32)


def _voxelise(points: np.ndarray, voxel: float) -> np.ndarray:
    v = np.floor(points / voxel).astype(np.int64)
    v -= v.min(axis=0, keepdims=True)
    v = np.unique(v, axis=0)
    return v.astype(np.int32)


def lidar_scan(seed: int = 2000, beams: int = 64, azimuths: int = 2048, voxel: float = 0.05,
               n_boxes: int = 40, max_range: float = 50.0) -> np.ndarray:
    """64-beam spinning scan: elevations evenly spaced over -25..+3 degrees, each ray
    hits the nearest of a ground plane at z=-1.7 m and ``n_boxes`` axis-aligned boxes
    standing on it (sides 0.5-5 m, centres within 50 m); hits beyond ``max_range``
    are dropped; points are voxelised at ``voxel`` metres."""
    rng = np.random.default_rng(seed)
    el = np.deg2rad(np.linspace(-25.0, 3.0, beams))
    az = np.linspace(0.0, 2.0 * np.pi, azimuths, endpoint=False)
    e, a = np.meshgrid(el, az, indexing="ij")
    d = np.stack([np.cos(e) * np.cos(a), np.cos(e) * np.sin(a), np.sin(e)], axis=-1).reshape(-1, 3)
    t = np.full(len(d), np.inf)
    dz = d[:, 2]
    down = dz < 0
    t[down] = -1.7 / dz[down]
    ang = rng.uniform(0.0, 2.0 * np.pi, n_boxes)
    rad = 50.0 * np.sqrt(rng.uniform(0.0, 1.0, n_boxes))
    side = rng.uniform(0.5, 5.0, (n_boxes, 3))
    ctr = np.stack([rad * np.cos(ang), rad * np.sin(ang), -1.7 + side[:, 2] / 2.0], axis=1)
    for c, s in zip(ctr, side):
        lo, hi = c - s / 2.0, c + s / 2.0
        if np.all(lo < 0) and np.all(hi > 0):
            continue  # a box around the sensor would swallow every ray
        with np.errstate(divide="ignore", invalid="ignore"):
            t1 = lo / d
            t2 = hi / d
        tn = np.nanmax(np.minimum(t1, t2), axis=1)
        tf = np.nanmin(np.maximum(t1, t2), axis=1)
        hit = (tf >= tn) & (tn > 0)
        t = np.where(hit & (tn < t), tn, t)
    keep = t <= max_range
    return _voxelise(d[keep] * t[keep, None], voxel)


def _box_faces(lo, hi):
    lo = np.asarray(lo, float)
    hi = np.asarray(hi, float)
    ext = hi - lo
    faces = []
    for ax in range(3):
        u = np.zeros(3)
        w = np.zeros(3)
        u[(ax + 1) % 3] = ext[(ax + 1) % 3]
        w[(ax + 2) % 3] = ext[(ax + 2) % 3]
        faces.append((lo.copy(), u, w))
        o = lo.copy()
        o[ax] = hi[ax]
        faces.append((o, u, w))
    return faces


def room_points(seed: int, n_points: int, origin=(0.0, 0.0, 0.0)) -> np.ndarray:
    """Area-uniform surface samples of an 8x8x3 m room (6 faces) with 30 boxes
    (sides 0.3-2 m) standing on its floor.  Returns float points [n_points,3]."""
    rng = np.random.default_rng(seed)
    faces = _box_faces((0, 0, 0), (8, 8, 3))
    for _ in range(30):
        s = rng.uniform(0.3, 2.0, 3)
        c = np.array([rng.uniform(s[0] / 2, 8 - s[0] / 2), rng.uniform(s[1] / 2, 8 - s[1] / 2), s[2] / 2])
        faces += _box_faces(c - s / 2, c + s / 2)
    o = np.array([f[0] for f in faces])
    u = np.array([f[1] for f in faces])
    w = np.array([f[2] for f in faces])
    area = np.linalg.norm(np.cross(u, w), axis=1)
    idx = rng.choice(len(faces), n_points, p=area / area.sum())
    ab = rng.uniform(0.0, 1.0, (n_points, 2))
    return o[idx] + ab[:, :1] * u[idx] + ab[:, 1:] * w[idx] + np.asarray(origin, float)


def indoor_room(seed: int = 3001, target_voxels: int = 200000, voxel: float = 0.02):
    """Room surface sample voxelised at ``voxel`` metres; the number of surface
    samples is tuned (deterministically, from the seed) until the voxel count is
    within 3 % of ``target_voxels``.  Returns (coords, samples_used)."""
    m = int(target_voxels * 1.12)
    v = None
    for _ in range(8):
        v = _voxelise(room_points(seed, m) + 1e-9, voxel)
        if abs(len(v) - target_voxels) <= 0.03 * target_voxels:
            break
        m = int(m * target_voxels / len(v) * 1.02)
    return v, m


def tiled_scene(rooms_x: int = 5, rooms_y: int = 4, voxels_per_room: int = 75000, seed0: int = 5000,
                voxel: float = 0.02, pitch: float = 8.0) -> np.ndarray:
    """``rooms_x*rooms_y`` rooms on a grid with ``pitch`` metres spacing, one seed each."""
    per = int(voxels_per_room * 1.06)
    pts = []
    k = 0
    for ix in range(rooms_x):
        for iy in range(rooms_y):
            pts.append(room_points(seed0 + k, per, origin=(ix * pitch, iy * pitch, 0.0)))
            k += 1
    return _voxelise(np.concatenate(pts) + 1e-9, voxel)


def with_batch(xyz: np.ndarray, b: int = 0) -> np.ndarray:
    """Prepend the batch index column: int32 [N,4] = (b,x,y,z)."""
    return np.concatenate([np.full((len(xyz), 1), b, np.int32), xyz.astype(np.int32)], axis=1)
