"""One scene split into x-slabs over two gloo ranks on CPU: halo rows exchanged after every submanifold and
strided convolution.  The per-rank compute is the CPU oracle (this is test infrastructure); what is under test
is the slab logic of insconv.slab -- cuts, ghost zone, row lists, exchange -- which is the code the GPU ranks run."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLANES = [8, 16, 24]


def _paths():
    for p in (ROOT, os.path.join(ROOT, "ins-conv_b200"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)


def _model():
    _paths()
    import sparseconvnet as scn
    from test_gpu_unet import small_unet, randomize_bn
    torch.manual_seed(7)
    model = small_unet(scn, PLANES, residual=True, full_scale=128).eval()
    randomize_bn(model, 7)
    return model


def _scene():
    _paths()
    from insconv import synth
    c = synth.boxes_and_spheres(5)
    return c, synth.rgb(5, c.shape[0])


def _worker(rank, world, port, out, sparse_ghost):
    _paths()
    from insconv import slab
    from oracle.scn_graph import GraphRunner
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    model = _model()
    c, f = _scene()
    align = 2 ** (len(PLANES) - 1)
    cuts = slab.cuts_for(c[:, 0].min(), c[:, 0].max(), world, align)
    ext = slab.load_mask(c, cuts, rank, len(PLANES)) if sparse_ghost else slab.extended_mask(c[:, 0], cuts, rank, align)
    own = slab.owned_mask(c[ext][:, 0], cuts, rank)
    ex = slab.SlabExchange(dist, rank, world, cuts, 128)
    runner = GraphRunner(model, post=lambda m, t: ex(t))
    y = runner._run(model.linear, runner._run(model.sparseModel, [torch.from_numpy(c[ext]), torch.from_numpy(f[ext])], False), False)
    out[rank] = (np.nonzero(ext)[0][own], y[torch.from_numpy(own)].numpy(), ex.exchanges, cuts)
    dist.barrier()
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("world,sparse_ghost", [(2, False), (3, True)])
def test_slabs_equal_the_whole_scene(world, sparse_ghost):
    _paths()
    from oracle.scn_graph import GraphRunner
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out, sparse_ghost), nprocs=world, join=True)
    model = _model()
    c, f = _scene()
    runner = GraphRunner(model)
    want = runner._run(model.linear, runner._run(model.sparseModel, [torch.from_numpy(c), torch.from_numpy(f)], False), False).numpy()
    got = np.full_like(want, np.nan)
    for r in range(world):
        idx, y, n_ex, cuts = out[r]
        got[idx] = y
        assert n_ex > 10  # one exchange per submanifold / strided convolution
    assert not np.isnan(got).any()  # every point is owned by exactly one rank
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-5 * scale


def test_cuts_are_aligned_and_cover():
    _paths()
    from insconv import slab
    for world in (1, 2, 3, 8):
        cuts = slab.cuts_for(8, 2007, world, 64)
        assert len(cuts) == world + 1 and cuts[0] <= 8 and cuts[-1] > 2007
        assert all(c % 64 == 0 for c in cuts) and all(b >= a for a, b in zip(cuts, cuts[1:]))
    rng = np.random.RandomState(0)
    pts = np.concatenate([rng.randint(8, 500, 30000), rng.randint(500, 2008, 10000)])  # three quarters in the first quarter
    for world in (1, 2, 4, 8):
        cuts = slab.cuts_balanced(pts, world, 64)
        assert len(cuts) == world + 1 and cuts[0] <= 8 and cuts[-1] > 2007
        assert all(c % 64 == 0 for c in cuts) and all(b > a for a, b in zip(cuts, cuts[1:]))
        own = [int(slab.owned_mask(pts, cuts, r).sum()) for r in range(world)]
        assert sum(own) == pts.size
        even = [int(slab.owned_mask(pts, slab.cuts_for(8, 2007, world, 64), r).sum()) for r in range(world)]
        assert max(own) <= max(even)
    assert slab.cuts_balanced(np.array([5, 70, 130]), 3, 64) == [0, 64, 128, 192]
    x = np.arange(0, 300)
    cuts = slab.cuts_for(0, 299, 2, 64)
    assert (slab.owned_mask(x, cuts, 0) ^ slab.owned_mask(x, cuts, 1)).all()


def test_sparse_ghost_zone_keeps_every_cell_next_to_a_cut():
    """load_mask: at every level the planes next to a rank's cuts hold the same occupied cells as in the whole scene,
    the level-0 planes hold every point, and far fewer points are loaded than with the full ghost zone."""
    _paths()
    from insconv import slab
    c, _ = _scene()
    levels = 5
    align = 2 ** (levels - 1)
    world = 3
    cuts = slab.cuts_for(c[:, 0].min(), c[:, 0].max(), world, align)
    for rank in range(world):
        keep = slab.load_mask(c, cuts, rank, levels)
        full = slab.extended_mask(c[:, 0], cuts, rank, align)
        own = slab.owned_mask(c[:, 0], cuts, rank)
        assert (keep & own).sum() == own.sum() and not (keep & ~full).any()
        assert keep.sum() - own.sum() < 0.35 * (full.sum() - own.sum())
        for lvl in range(levels):
            for plane in ((cuts[rank] >> lvl) - 1, cuts[rank + 1] >> lvl):
                cells = lambda pts: {tuple(v) for v in (pts[(pts[:, 0] >> lvl) == plane] >> lvl)}
                assert cells(c[keep]) == cells(c)
        for plane in (cuts[rank] - 1, cuts[rank + 1]):
            assert (keep[c[:, 0] == plane]).all()
