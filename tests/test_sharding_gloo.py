"""The N > 1 path of the benchmark on CPU: two gloo ranks shard independent scenes, and the only
communication is the reduction of unit counts (sum) and step time (max)."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_scenes, out):
    for p in (ROOT, os.path.join(ROOT, "ins-conv_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from insconv import shard, synth
    from oracle import scn_oracle as O
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    mine = shard.scenes_for_rank(n_scenes, rank, world)
    units = sum(O.Grid(synth.boxes_and_spheres(s, grid=128)).n for s in mine)
    total, tmax = shard.aggregate(dist, torch.device("cpu"), units, 10.0 * (rank + 1))
    out[rank] = (mine, units, total, tmax)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_scenes_without_a_data_collective():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, 5, out), nprocs=2, join=True)
    from insconv import synth
    from oracle import scn_oracle as O
    want = [O.Grid(synth.boxes_and_spheres(s, grid=128)).n for s in range(5)]
    assert out[0][0] == [0, 2, 4] and out[1][0] == [1, 3]
    assert out[0][1] + out[1][1] == sum(want)
    assert out[0][2] == out[1][2] == float(sum(want))
    assert out[0][3] == out[1][3] == 20.0


def test_assignment_covers_every_scene_once():
    from insconv import shard
    for world in (1, 2, 3, 8):
        got = sorted(i for r in range(world) for i in shard.scenes_for_rank(64, r, world))
        assert got == list(range(64))
    assert shard.aggregate(None, None, 7, 3.5) == (7.0, 3.5)
