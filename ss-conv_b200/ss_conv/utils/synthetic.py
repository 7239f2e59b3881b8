"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (object-surface point clouds in the unit cube, as in LineMOD/REAL275-like
data: 1024-16384 points per object on 32^3-64^3 grids).  Per-sample seed = base_seed +
sample id, so a sample is identical no matter which rank generates it."""
import numpy as np


def _rotation(rng):
    q, r = np.linalg.qr(rng.randn(3, 3))
    q = q * np.sign(np.diag(r))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q


def ellipsoid_points(seed, n_pts):
    """n_pts points on a randomly rotated ellipsoid with semi-axes U[0.3,0.5], strictly inside
    the cube [-0.5,0.5]^3 (unit-sphere directions scaled by the axes, then rotated)."""
    rng = np.random.RandomState(seed)
    axes = rng.uniform(0.3, 0.5, 3)
    rot = _rotation(rng)
    d = rng.randn(n_pts, 3)
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    p = (d * axes) @ rot.T
    return np.clip(p, -0.4995, 0.4995).astype(np.float32)


def box_points(seed, n_pts):
    """n_pts points on the faces of a randomly rotated box with half-sizes U[0.15,0.28]."""
    rng = np.random.RandomState(seed)
    half = rng.uniform(0.15, 0.28, 3)
    rot = _rotation(rng)
    p = rng.uniform(-1, 1, (n_pts, 3)) * half
    face = rng.randint(0, 3, n_pts)
    sign = rng.choice([-1.0, 1.0], n_pts)
    p[np.arange(n_pts), face] = sign * half[face]
    p = p @ rot.T
    return np.clip(p, -0.4995, 0.4995).astype(np.float32)


def surface_voxels(sample_ids, V, n_pts, base_seed=0):
    """indices [N,4] int32 (batch position, x, y, z) of voxelised ellipsoid surfaces, sorted
    lexicographically; batch position = index of the sample inside `sample_ids`."""
    rows = []
    for b, sid in enumerate(sample_ids):
        p = ellipsoid_points(base_seed + int(sid), n_pts)
        v = np.floor((p + 0.5) * V).astype(np.int64)
        v = np.unique(v, axis=0)
        rows.append(np.concatenate([np.full((v.shape[0], 1), b, dtype=np.int64), v], axis=1))
    return np.ascontiguousarray(np.concatenate(rows, axis=0), dtype=np.int32)


def bernoulli_voxels(sample_ids, V, occupancy, base_seed=0):
    rows = []
    for b, sid in enumerate(sample_ids):
        rng = np.random.RandomState(base_seed + int(sid))
        occ = np.argwhere(rng.rand(V, V, V) < occupancy)
        rows.append(np.concatenate([np.full((occ.shape[0], 1), b, dtype=np.int64), occ], axis=1))
    return np.ascontiguousarray(np.concatenate(rows, axis=0), dtype=np.int32)


def object_points(sample_ids, n_pts, base_seed=0):
    """(points [B*n,3], feats [B*n,3] U[0,1], batch_ids [B*n]) of ellipsoid / box surfaces
    (alternating by sample id)."""
    pts, fts, ids = [], [], []
    for b, sid in enumerate(sample_ids):
        seed = base_seed + int(sid)
        p = ellipsoid_points(seed, n_pts) if int(sid) % 2 == 0 else box_points(seed, n_pts)
        rng = np.random.RandomState(seed + 7919)
        pts.append(p)
        fts.append(rng.uniform(0, 1, (n_pts, 3)).astype(np.float32))
        ids.append(np.full(n_pts, b, dtype=np.int64))
    return np.concatenate(pts), np.concatenate(fts), np.concatenate(ids)


def features(n, c, seed):
    return np.random.RandomState(seed).randn(n, c).astype(np.float32)
