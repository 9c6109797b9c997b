"""One oversized scene on several GPUs: x-slabs with a halo exchange after every layer that mixes sites.

Rank r owns the sites with x in [cut[r], cut[r+1]); cuts are multiples of `align` = 2^(levels-1) voxels, so a
size-2/stride-2 cell never straddles a cut at any level of the network.  Every rank loads its slab plus a
ghost zone of `align` voxels on each side.  Ghost rows are computed locally like any other row, but only the
first ghost layer next to a cut (one voxel of the level at hand) is guaranteed to be right, and it is the only
ghost layer an owned row ever reads: a submanifold convolution looks one voxel across the cut, a strided
convolution or deconvolution not at all.  The invariant "the first ghost layer holds the owner's values" is
restored after every SubmanifoldConvolution and every Convolution by exchanging those rows with the two
neighbours (grouped send/recv: NCCL on GPUs, gloo in the CPU tests); row-wise layers (BatchNorm, 1x1
convolution, add, concatenate) and the Deconvolution preserve it.  Deeper ghost rows go stale; they only ever
feed other ghost rows.

Both sides of a cut hold the same sites on the planes they exchange and number them in the same (key) order,
so a message is just the feature rows of one plane in row order.  The reference has no multi-GPU path.
"""
import numpy as np
import torch


def cuts_for(x_lo, x_hi, world, align):
    """world+1 cut positions, multiples of `align`, covering [x_lo, x_hi] as evenly as the alignment allows."""
    a_lo = (int(x_lo) // align) * align
    a_hi = ((int(x_hi) + align) // align) * align
    cells = (a_hi - a_lo) // align
    cuts = [a_lo + align * ((cells * r) // world) for r in range(world)] + [a_hi]
    return cuts


def extended_mask(x, cuts, rank, align):
    """Points a rank loads: its slab plus `align` voxels of ghost zone on each side."""
    return (x >= cuts[rank] - align) & (x < cuts[rank + 1] + align)


def owned_mask(x, cuts, rank):
    return (x >= cuts[rank]) & (x < cuts[rank + 1])


class SlabExchange(object):
    """Keeps, per scale, the row lists of the planes next to this rank's two cuts and exchanges them."""

    def __init__(self, dist, rank, world, cuts, full_scale):
        self.dist, self.rank, self.world, self.cuts, self.full_scale = dist, rank, world, cuts, int(full_scale)
        self.cache = {}
        self.exchanges = 0
        self.bytes_sent = 0

    def _rows(self, tensor):
        size = int(tensor.spatial_size[0])
        hit = self.cache.get(size)
        if hit is not None and hit["meta"] is tensor.metadata:  # one entry per scale, replaced when the scene changes
            return hit
        shift = int(round(np.log2(self.full_scale / size)))
        dev = tensor.features.device
        if hasattr(tensor.metadata, "getSpatialLocationsDevice"):  # stays on the GPU
            x = tensor.metadata.getSpatialLocationsDevice(tensor.spatial_size)[0]
        else:
            x = torch.as_tensor(tensor.metadata.getSpatialLocations(tensor.spatial_size))[:, 0]
        lo, hi = self.cuts[self.rank] >> shift, self.cuts[self.rank + 1] >> shift
        rows = {
            "meta": tensor.metadata,
            "send_left": torch.nonzero(x == lo).flatten().to(dev),       # my first owned plane
            "recv_left": torch.nonzero(x == lo - 1).flatten().to(dev),   # left neighbour's last plane
            "send_right": torch.nonzero(x == hi - 1).flatten().to(dev),
            "recv_right": torch.nonzero(x == hi).flatten().to(dev),
        }
        self.cache[size] = rows
        return rows

    def __call__(self, tensor):
        """Overwrites the first ghost layer of `tensor.features` with the neighbours' rows (in place)."""
        if self.world == 1:
            return tensor
        rows = self._rows(tensor)
        f = tensor.features
        ops, landing = [], []
        for side, peer in (("left", self.rank - 1), ("right", self.rank + 1)):
            if peer < 0 or peer >= self.world:
                continue
            send = f.index_select(0, rows["send_" + side]).contiguous()
            recv = f.new_empty((rows["recv_" + side].shape[0], f.shape[1]))
            if send.numel():
                ops.append(self.dist.P2POp(self.dist.isend, send, peer))
                self.bytes_sent += send.numel() * 4
            if recv.numel():
                ops.append(self.dist.P2POp(self.dist.irecv, recv, peer))
                landing.append((rows["recv_" + side], recv))
        if ops:
            for req in self.dist.batch_isend_irecv(ops):
                req.wait()
        for idx, recv in landing:
            f.index_copy_(0, idx, recv)
        self.exchanges += 1
        return tensor


def install(model, exchange, layer_types):
    """Runs `exchange` on the output of every module of the given types (forward hooks); returns the handles."""
    handles = []
    for m in model.modules():
        if isinstance(m, layer_types):
            handles.append(m.register_forward_hook(lambda mod, inp, out: exchange(out)))
    return handles
