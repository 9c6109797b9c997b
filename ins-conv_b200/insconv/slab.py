"""One oversized scene on several GPUs: x-slabs with a halo exchange after every layer that mixes sites.

Rank r owns the sites with x in [cut[r], cut[r+1]); cuts are multiples of `align` = 2^(levels-1) voxels, so a
size-2/stride-2 cell never straddles a cut at any level of the network.  Besides its own points a rank loads a
ghost zone on each side of its slab.  What an owned row ever reads across a cut is the FIRST ghost layer of the
level at hand (a submanifold convolution looks one voxel of its level across the cut, a strided convolution or
deconvolution not at all), so the ghost zone only has to make those layers exist:

  level 0      every point of the plane next to the cut;
  level l > 0  one point (any) for every occupied cell of the level-l plane next to the cut -- a coarse cell exists
               when one point falls into it, and the values of ghost rows are never computed from their children:

the invariant "the first ghost layer holds the owner's values" is restored after every SubmanifoldConvolution
and every Convolution by exchanging those rows with the two neighbours (grouped send/recv: NCCL on GPUs, gloo in
the CPU tests); row-wise layers (BatchNorm, 1x1 convolution, add, concatenate) and the Deconvolution preserve it.
Other ghost rows (the few fine cells the representatives create) hold values that nothing owned reads.
`extended_mask` is the simple variant: the whole ghost zone of `align` voxels, 64 planes of wasted work per side
for a 7-level network.

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


def cuts_balanced(x, world, align):
    """world+1 cut positions, multiples of `align`, that split the points (x: their x coordinates) into slabs whose
    largest point count is as small as the alignment allows (dynamic programme over the aligned cells); every slab
    is at least one cell wide."""
    x = np.asarray(x, dtype=np.int64)
    a_lo = (int(x.min()) // align) * align
    a_hi = ((int(x.max()) + align) // align) * align
    cells = (a_hi - a_lo) // align
    if cells < world:
        raise ValueError("more slabs than aligned cells")
    before = np.concatenate([[0], np.cumsum(np.bincount((x - a_lo) // align, minlength=cells))])  # points left of cell i
    # best[r][i]: smallest possible maximum over r slabs covering cells [0, i)
    inf = float("inf")
    best = [[inf] * (cells + 1) for _ in range(world + 1)]
    arg = [[0] * (cells + 1) for _ in range(world + 1)]
    best[0][0] = 0
    for r in range(1, world + 1):
        for i in range(r, cells - (world - r) + 1):
            for j in range(r - 1, i):
                v = max(best[r - 1][j], before[i] - before[j])
                if v < best[r][i]:
                    best[r][i], arg[r][i] = v, j
    cuts, i = [cells], cells
    for r in range(world, 0, -1):
        i = arg[r][i]
        cuts.append(i)
    return [a_lo + align * i for i in reversed(cuts)]


def extended_mask(x, cuts, rank, align):
    """Points a rank loads, simple variant: its slab plus `align` voxels of ghost zone on each side."""
    return (x >= cuts[rank] - align) & (x < cuts[rank + 1] + align)


def owned_mask(x, cuts, rank):
    return (x >= cuts[rank]) & (x < cuts[rank + 1])


def load_mask(coords, cuts, rank, levels):
    """Points a rank loads: its slab, the two level-0 planes next to its cuts, and for every coarser level one
    point per occupied cell of the two planes of that level next to its cuts.  coords: int array [N, >=3] (x,y,z)."""
    c = np.asarray(coords)
    x = c[:, 0].astype(np.int64)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])
    keep = (x >= lo - 1) & (x <= hi)
    for lvl in range(1, levels):
        for plane in ((lo >> lvl) - 1, hi >> lvl):
            idx = np.nonzero((x >> lvl) == plane)[0]
            if idx.size == 0:
                continue
            cell = ((c[idx, 1].astype(np.int64) >> lvl) << 32) | (c[idx, 2].astype(np.int64) >> lvl)
            if c.shape[1] > 3:
                cell |= c[idx, 3].astype(np.int64) << 48
            _, first = np.unique(cell, return_index=True)
            keep[idx[first]] = True
    return keep


class SlabExchange(object):
    """Keeps, per scale, the row lists of the planes next to this rank's two cuts and exchanges them.

    Called with the SparseConvNetTensor a convolution returned: its fp32 features and, when the convolution also
    formed the next BatchNorm's result as fp16 rows in its epilogue, those rows too are overwritten in place on the
    first ghost layer.  Per tensor: one gather of the rows to send, one grouped send/recv, one scatter."""

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
        if hasattr(tensor.metadata, "getSpatialLocationsDevice"):  # stays on the GPU
            x = tensor.metadata.getSpatialLocationsDevice(tensor.spatial_size)[0]
        else:
            x = torch.as_tensor(tensor.metadata.getSpatialLocations(tensor.spatial_size))[:, 0]
        lo, hi = self.cuts[self.rank] >> shift, self.cuts[self.rank + 1] >> shift
        left, right = self.rank > 0, self.rank + 1 < self.world
        # [send to left, send to right, receive from left, receive from right]; one trip to the host for the four
        # counts, the row lists themselves stay on the device
        planes = torch.stack([(x == lo) if left else torch.zeros_like(x, dtype=torch.bool),
                              (x == hi - 1) if right else torch.zeros_like(x, dtype=torch.bool),
                              (x == lo - 1) if left else torch.zeros_like(x, dtype=torch.bool),
                              (x == hi) if right else torch.zeros_like(x, dtype=torch.bool)])
        counts = [int(v) for v in planes.sum(1).tolist()]
        n = x.shape[0]
        flat = torch.nonzero_static(planes.flatten(), size=sum(counts)).flatten()
        rows = flat - torch.repeat_interleave(torch.arange(4, device=x.device) * n,
                                              torch.tensor(counts, device=x.device), output_size=sum(counts))
        hit = {"meta": tensor.metadata, "counts": counts, "send": rows[:counts[0] + counts[1]],
               "recv": rows[counts[0] + counts[1]:]}
        self.cache[size] = hit
        return hit

    def _swap(self, f, rows):
        n_sl, n_sr, n_rl, n_rr = rows["counts"]
        send = f.index_select(0, rows["send"])
        recv = f.new_empty((n_rl + n_rr, f.shape[1]))
        ops = []
        for peer, s, r in ((self.rank - 1, send[:n_sl], recv[:n_rl]), (self.rank + 1, send[n_sl:], recv[n_rl:])):
            if s.shape[0]:
                ops.append(self.dist.P2POp(self.dist.isend, s, peer))
            if r.shape[0]:
                ops.append(self.dist.P2POp(self.dist.irecv, r, peer))
        if ops:
            for req in self.dist.batch_isend_irecv(ops):
                req.wait()
        if recv.shape[0]:
            f.index_copy_(0, rows["recv"], recv)
        self.bytes_sent += send.numel() * send.element_size()

    def __call__(self, tensor):
        """Overwrites the first ghost layer of the tensor's rows with the neighbours' rows (in place)."""
        if self.world == 1:
            return tensor
        rows = self._rows(tensor)
        if tensor.features is not None and tensor.features.numel():
            self._swap(tensor.features, rows)
        ready = getattr(tensor, "bn_ready", None)
        if ready is not None:
            self._swap(ready[1].features, rows)
        self.exchanges += 1
        return tensor


class PeerSlabExchange(SlabExchange):
    """The same exchange with the library's own kernels: every rank pushes its planes straight into its neighbours'
    memory over NVLink and picks up what they pushed (scn_halo_* of the C ABI: two launches per exchange, none of
    them NCCL's, no host round trip -- row lists and their lengths stay on the device).  The ranks must be processes
    of one box, one GPU each.  check() reads the status word: a neighbour that never answered, or a plane larger than
    a message slot, raises there."""

    def __init__(self, dist, rank, world, cuts, full_scale, device, slot_bytes=128 << 20, max_plane_rows=1 << 20):
        SlabExchange.__init__(self, dist, rank, world, cuts, full_scale)
        import ctypes as C
        from . import cabi
        self.cabi, self.C, self.device, self.max_rows = cabi, C, device, int(max_plane_rows)
        self.track_bytes = False  # True: bytes pushed are summed on the device (two small extra kernels per exchange)
        self.sent_dev = torch.zeros((), dtype=torch.int64, device=device)
        self.h = C.c_void_p()
        cabi.call("scn_halo_create", C.byref(self.h), int(slot_bytes))
        mine = C.create_string_buffer(64)
        cabi.call("scn_halo_ipc_handle", self.h, mine)
        handles = [None] * world
        dist.all_gather_object(handles, bytes(mine.raw))
        for side, peer in ((0, rank - 1), (1, rank + 1)):
            if 0 <= peer < world:
                cabi.call("scn_halo_connect", self.h, side, C.create_string_buffer(handles[peer], 64))
        dist.barrier()

    def _rows(self, tensor):
        size = int(tensor.spatial_size[0])
        hit = self.cache.get(size)
        if hit is not None and hit["meta"] is tensor.metadata:
            return hit
        shift = int(round(np.log2(self.full_scale / size)))
        lo, hi = self.cuts[self.rank] >> shift, self.cuts[self.rank + 1] >> shift
        n = int(tensor.metadata.getNActive(tensor.spatial_size))
        cap = max(min(n, self.max_rows), 1)
        # two launches of the library (no torch ops, no host round trip): ascending rows of the four planes
        lists, counts = tensor.metadata.haloPlaneLists(tensor.spatial_size, lo, hi, self.rank > 0, self.rank + 1 < self.world, cap)
        hit = {"meta": tensor.metadata, "lists": lists, "counts": counts, "cap": cap}
        self.cache[size] = hit
        return hit

    def __call__(self, tensor):
        if self.world == 1:
            return tensor
        rows = self._rows(tensor)
        arrays = []
        if tensor.features is not None and tensor.features.numel():
            arrays.append(tensor.features)
        ready = getattr(tensor, "bn_ready", None)
        if ready is not None:
            arrays.append(ready[1].features)
        assert arrays and all(a.is_contiguous() for a in arrays)
        a = arrays[0]
        b = arrays[1] if len(arrays) > 1 else None
        self.cabi.call("scn_halo_exchange", self.h, rows["lists"].data_ptr(), rows["counts"].data_ptr(), rows["cap"],
                       a.data_ptr(), a.shape[1] * a.element_size(), None if b is None else b.data_ptr(),
                       0 if b is None else b.shape[1] * b.element_size(), torch.cuda.current_stream().cuda_stream)
        if self.track_bytes:
            self.sent_dev += rows["counts"][:2].sum() * sum(t.shape[1] * t.element_size() for t in arrays)
        self.exchanges += 1
        return tensor

    @property
    def bytes_sent(self):
        return int(self.sent_dev.item())

    @bytes_sent.setter
    def bytes_sent(self, v):
        pass

    def check(self):
        """Synchronises the stream and raises when an exchange since the last check gave up or was cut short."""
        t, o = self.C.c_int(0), self.C.c_int(0)
        self.cabi.call("scn_halo_status", self.h, self.C.byref(t), self.C.byref(o), torch.cuda.current_stream().cuda_stream)
        if t.value or o.value:
            raise RuntimeError("halo exchange failed: %s" % ("a neighbour did not answer in time" if t.value else
                                                             "a plane holds more rows than a message slot"))

    def close(self):
        if self.h:
            self.cabi.call("scn_halo_destroy", self.h)
            self.h = None


def install(model, exchange, layer_types=None):
    """Makes every full-frame SubmanifoldConvolution and Convolution of the process run `exchange` on its result
    (sparseconvnet.set_halo_exchange); install(model, None) switches it off."""
    import sparseconvnet
    sparseconvnet.set_halo_exchange(exchange)
