"""Seeded synthetic scenes: the workloads of the benchmark and of the parity tests.

No public dataset is involved anywhere; these generators define the inputs.  All functions return
numpy arrays; coordinates are int64 [n,3] voxel indices, deduplicated unless stated otherwise.

  boxes_and_spheres   128^3 grid, surfaces of 8 axis-aligned boxes and 4 spheres (~50k voxels)
  next_frame          frame t+1 of the same scene: a 16^3 cube deleted, a sphere inserted, 1% re-drawn
  room                8x8x3 m room at 2 cm (400x400x150 voxels): floor, 4 walls, 20 boxes (~250k voxels)
  sweep_frame         one frame of a camera sweep through the room (new surface voxels in a frustum)
  building            5 rooms x 4 floors (~4M voxels)
"""
import numpy as np


def _unique_rows(c):
    c = np.asarray(c, dtype=np.int64)
    if c.shape[0] == 0:
        return c.reshape(0, 3)
    key = (c[:, 2] << 42) | (c[:, 1] << 21) | c[:, 0]
    _, first = np.unique(key, return_index=True)
    return c[np.sort(first)]


def box_surface(lo, hi):
    """Voxels on the surface of the axis-aligned box [lo, hi] (inclusive corners)."""
    lo = np.asarray(lo, dtype=np.int64)
    hi = np.asarray(hi, dtype=np.int64)
    parts = []
    for d in range(3):
        a, b = [i for i in range(3) if i != d]
        ga, gb = np.meshgrid(np.arange(lo[a], hi[a] + 1), np.arange(lo[b], hi[b] + 1), indexing="ij")
        for v in (lo[d], hi[d]):
            c = np.empty((ga.size, 3), dtype=np.int64)
            c[:, d] = v
            c[:, a] = ga.ravel()
            c[:, b] = gb.ravel()
            parts.append(c)
    return _unique_rows(np.concatenate(parts, 0))


def sphere_surface(center, radius):
    """Voxels whose centre lies within half a voxel of the sphere surface."""
    center = np.asarray(center, dtype=np.int64)
    r = int(radius)
    g = np.arange(-r - 1, r + 2)
    x, y, z = np.meshgrid(g, g, g, indexing="ij")
    d = np.sqrt((x * x + y * y + z * z).astype(np.float64))
    m = np.abs(d - r) <= 0.5
    return np.stack([x[m], y[m], z[m]], 1).astype(np.int64) + center


def boxes_and_spheres(seed=0, grid=128):
    rng = np.random.RandomState(seed)
    parts = []
    for _ in range(8):
        side = rng.randint(8, 49, size=3)
        lo = np.array([rng.randint(1, grid - 1 - s) for s in side])
        parts.append(box_surface(lo, lo + side - 1))
    for _ in range(4):
        r = rng.randint(6, 25)
        c = rng.randint(r + 2, grid - r - 2, size=3)
        parts.append(sphere_surface(c, r))
    c = _unique_rows(np.concatenate(parts, 0))
    keep = ((c >= 1) & (c <= grid - 2)).all(1)
    return c[keep]


def kaiming_uniform(rng, volume, n_in, n_out):
    bound = np.sqrt(6.0 / (volume * n_in))
    return rng.uniform(-bound, bound, size=(volume, n_in, n_out)).astype(np.float32)


def next_frame(coords, feats, seed=0, grid=128):
    """Frame t+1.  Returns a dict with
      coords, feats        the full frame t+1 (for the full recompute)
      new_coords, new_feats the points handed to the incremental path: the inserted sphere voxels and
                           the re-drawn 1% (insert / re-draw only; deletion has no counterpart in the
                           reference's incremental semantics and is checked against the full recompute)
      deleted              boolean mask over the frame-t rows that fell inside the deleted cube
    """
    rng = np.random.RandomState(seed + 1000)
    n = coords.shape[0]
    anchor = coords[rng.randint(n)]
    lo = np.clip(anchor - 8, 1, grid - 18)
    deleted = ((coords >= lo) & (coords < lo + 16)).all(1)
    for _ in range(64):
        c = rng.randint(13, grid - 13, size=3)
        if np.abs(c - (lo + 8)).max() > 30:
            break
    sph = sphere_surface(c, 10)
    have = set(map(tuple, coords.tolist()))
    sph = np.array([p for p in sph.tolist() if tuple(p) not in have], dtype=np.int64).reshape(-1, 3)
    keep = np.nonzero(~deleted)[0]
    redraw = keep[rng.rand(keep.size) < 0.01]
    feats1 = feats.copy()
    feats1[redraw] = rng.randn(redraw.size, feats.shape[1]).astype(np.float32)
    sph_f = rng.randn(sph.shape[0], feats.shape[1]).astype(np.float32)
    return {
        "coords": np.concatenate([coords[keep], sph], 0),
        "feats": np.concatenate([feats1[keep], sph_f], 0),
        "new_coords": np.concatenate([sph, coords[redraw]], 0),
        "new_feats": np.concatenate([sph_f, feats1[redraw]], 0),
        "redraw_old_feats": feats[redraw],
        "deleted": deleted,
    }


def room(seed=0, target=250000, origin=(8, 8, 8), size=(400, 400, 150), n_boxes=20):
    """Floor + 4 walls + n_boxes seeded boxes standing on the floor, thinned to ~target voxels."""
    rng = np.random.RandomState(seed)
    sx, sy, sz = size
    parts = []
    gx, gy = np.meshgrid(np.arange(sx), np.arange(sy), indexing="ij")
    parts.append(np.stack([gx.ravel(), gy.ravel(), np.zeros(gx.size, np.int64)], 1))
    gz = np.arange(sz)
    for x in (0, sx - 1):
        a, b = np.meshgrid(np.arange(sy), gz, indexing="ij")
        parts.append(np.stack([np.full(a.size, x), a.ravel(), b.ravel()], 1))
    for y in (0, sy - 1):
        a, b = np.meshgrid(np.arange(sx), gz, indexing="ij")
        parts.append(np.stack([a.ravel(), np.full(a.size, y), b.ravel()], 1))
    for _ in range(n_boxes):
        side = np.array([rng.randint(20, 81), rng.randint(20, 81), rng.randint(20, 101)])
        lo = np.array([rng.randint(2, sx - side[0] - 2), rng.randint(2, sy - side[1] - 2), 1])
        parts.append(box_surface(lo, lo + side - 1))
    c = _unique_rows(np.concatenate(parts, 0).astype(np.int64))
    if target and c.shape[0] > target:
        # thin the scan the way occlusion does: drop whole 16^3 blocks, keep surfaces dense inside the rest
        blk = c >> 4
        bkey = (blk[:, 2] << 40) | (blk[:, 1] << 20) | blk[:, 0]
        ub, inv = np.unique(bkey, return_inverse=True)
        keep_blk = rng.rand(ub.shape[0]) < float(target) / c.shape[0]
        c = c[keep_blk[inv.reshape(-1)]]
    return c + np.asarray(origin, dtype=np.int64)


def rgb(seed, n):
    return np.random.RandomState(seed + 7).uniform(-1.0, 1.0, size=(n, 3)).astype(np.float32)


def sweep_frame(base_coords, frame, n_frames=100, seed=0, origin=(8, 8, 8), size=(400, 400, 150)):
    """New surface voxels seen by a camera moving along x through the room at `frame`: points of a
    freshly seeded box inside a moving window, 2-8 % of the base scene, plus the indices of 1 % of the
    existing voxels whose colour is perturbed.  Returns (new_coords, perturbed_rows)."""
    rng = np.random.RandomState(seed * 1000 + frame + 1)
    n = base_coords.shape[0]
    frac = rng.uniform(0.02, 0.08)
    cx = int(origin[0] + 40 + (size[0] - 120) * frame / max(n_frames - 1, 1))
    have = None
    parts = []
    total = 0
    want = int(frac * n)
    while total < want:
        side = np.array([rng.randint(10, 41), rng.randint(20, 81), rng.randint(10, 61)])
        lo = np.array([cx + rng.randint(-30, 30), origin[1] + rng.randint(2, size[1] - side[1] - 2),
                       origin[2] + rng.randint(1, size[2] - side[2] - 1)])
        p = box_surface(lo, lo + side - 1)
        parts.append(p)
        total += p.shape[0]
    c = _unique_rows(np.concatenate(parts, 0))[:want]
    pert = np.nonzero(rng.rand(n) < 0.01)[0]
    return c, pert


def building(seed=0, rooms_x=5, floors=4, target=4000000):
    """rooms_x rooms side by side along x, `floors` storeys along z."""
    per = target // (rooms_x * floors) if target else 0
    parts = []
    i = 0
    for f in range(floors):
        for r in range(rooms_x):
            c = room(seed * 100 + i, target=per, origin=(8 + 400 * r, 8, 8 + 150 * f))
            parts.append(c)
            i += 1
    return _unique_rows(np.concatenate(parts, 0))
