"""Slab split on real GPUs: two NCCL ranks (one per GPU) run the product's UNet on the two halves of a scene
with halo exchange and must reproduce the single-GPU result.  Needs two GPUs; skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLANES = [32, 64, 96]


def _paths():
    for p in (ROOT, os.path.join(ROOT, "ins-conv_b200"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)


def _worker(rank, world, port, out):
    _paths()
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import sparseconvnet as scn
    from insconv import slab, synth
    from test_gpu_unet import small_unet, randomize_bn
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(11)
    model = small_unet(scn, PLANES, residual=True, full_scale=128).eval()
    randomize_bn(model, 11)
    model = model.to(dev)
    c = synth.boxes_and_spheres(6)
    f = synth.rgb(6, c.shape[0])
    align = 2 ** (len(PLANES) - 1)
    cuts = slab.cuts_for(c[:, 0].min(), c[:, 0].max(), world, align)
    ext = slab.extended_mask(c[:, 0], cuts, rank, align)
    own = slab.owned_mask(c[ext][:, 0], cuts, rank)
    ex = slab.SlabExchange(dist, rank, world, cuts, 128)
    handles = slab.install(model, ex, (scn.SubmanifoldConvolution, scn.Convolution))
    y = model([torch.from_numpy(c[ext]).to(dev), torch.from_numpy(f[ext]).to(dev)])
    res = {"idx": np.nonzero(ext)[0][own], "y": y[torch.from_numpy(own).to(dev)].detach().cpu().numpy(), "n_ex": ex.exchanges}
    if rank == 0:
        for h in handles:
            h.remove()
        res["whole"] = model([torch.from_numpy(c).to(dev), torch.from_numpy(f).to(dev)]).detach().cpu().numpy()
    out[rank] = res
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_slabs_equal_one_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    want = out[0]["whole"]
    got = np.full_like(want, np.nan)
    for r in (0, 1):
        got[out[r]["idx"]] = out[r]["y"]
        assert out[r]["n_ex"] > 10
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
