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


def _worker(rank, world, port, out, precision="fp32", sparse_ghost=False, peer=False):
    _paths()
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import sparseconvnet as scn
    from insconv import slab, synth
    from test_gpu_unet import small_unet, randomize_bn
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world, device_id=dev)
    scn.set_precision(precision)
    torch.manual_seed(11)
    model = small_unet(scn, PLANES, residual=True, full_scale=128).eval()
    randomize_bn(model, 11)
    model = model.to(dev)
    c = synth.boxes_and_spheres(6)
    f = synth.rgb(6, c.shape[0])
    align = 2 ** (len(PLANES) - 1)
    cuts = slab.cuts_for(c[:, 0].min(), c[:, 0].max(), world, align)
    ext = slab.load_mask(c, cuts, rank, len(PLANES)) if sparse_ghost else slab.extended_mask(c[:, 0], cuts, rank, align)
    own = slab.owned_mask(c[ext][:, 0], cuts, rank)
    ex = slab.PeerSlabExchange(dist, rank, world, cuts, 128, dev, slot_bytes=8 << 20) if peer else \
        slab.SlabExchange(dist, rank, world, cuts, 128)
    slab.install(model, ex)
    y = model([torch.from_numpy(c[ext]).to(dev), torch.from_numpy(f[ext]).to(dev)])
    if peer:
        ex.check()
    res = {"loaded": int(ext.sum()), "idx": np.nonzero(ext)[0][own], "y": y[torch.from_numpy(own).to(dev)].detach().cpu().numpy(), "n_ex": ex.exchanges}
    if rank == 0:
        slab.install(model, None)
        res["whole"] = model([torch.from_numpy(c).to(dev), torch.from_numpy(f).to(dev)]).detach().cpu().numpy()
    out[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("precision,sparse_ghost,peer,tol", [("fp32", False, False, 1e-4), ("fp32", True, False, 1e-4),
                                                             ("fp16", True, False, 2e-2), ("fp32", True, True, 1e-4),
                                                             ("fp16", True, True, 2e-2)])
def test_two_gpu_slabs_equal_one_gpu(precision, sparse_ghost, peer, tol):
    """fp32: the split changes nothing but the order of sums.  fp16: the epilogue-fused frame (BatchNorm results
    written as fp16 rows by the convolutions, exchanged as such) against the same fused frame on one GPU.
    peer: rows pushed into the neighbour's memory by the library's own kernels instead of NCCL send/recv."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, out, precision, sparse_ghost, peer), nprocs=2, join=True)
    want = out[0]["whole"]
    got = np.full_like(want, np.nan)
    for r in (0, 1):
        got[out[r]["idx"]] = out[r]["y"]
        assert out[r]["n_ex"] > 10
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
