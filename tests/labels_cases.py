"""Seeded label-fusion sequences shared by the CPU and GPU tests and by the script that stores what the reference
makes of them (tests/golden/make_golden_ref.py)."""
import numpy as np

CLASSES = 20


def frames(seed=0, n_frames=6, n_scene=4000, per_frame=1500, dup_frac=0.05):
    """A scene of n_scene voxels; every frame scores a random subset of it (so voxels come back with agreeing and
    disagreeing labels) plus a few rows that repeat voxels of the same frame.  Scores are softmax-like rows."""
    rng = np.random.RandomState(seed)
    scene = np.unique(rng.randint(1, 200, size=(n_scene * 2, 3)), axis=0)[:n_scene].astype(np.int64)
    truth = rng.randint(0, CLASSES, scene.shape[0])
    out = []
    for f in range(n_frames):
        idx = rng.choice(scene.shape[0], per_frame, replace=False)
        dups = rng.choice(idx, int(per_frame * dup_frac), replace=True)
        idx = np.concatenate([idx, dups])
        rng.shuffle(idx)
        logits = rng.randn(idx.size, CLASSES).astype(np.float32)
        agree = rng.rand(idx.size) < 0.7
        logits[np.arange(idx.size)[agree], truth[idx][agree]] += 3.0
        e = np.exp(logits - logits.max(1, keepdims=True))
        out.append((scene[idx].copy(), (e / e.sum(1, keepdims=True)).astype(np.float32)))
    return scene, out
