"""The halo-exchange kernels of the C ABI (scn_halo_*) on one GPU: a rank that is its own neighbour on both sides
(periodic boundary) pushes its planes into its own inbox and picks them up, so every part of the two kernels runs --
gather, slot alternation, sequence numbers, scatter, both word widths -- without a second GPU and without any kernel
waiting for another.  The bounded wait is exercised by a side nobody writes to."""
import ctypes as C
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "ins-conv_b200"))


def _lists(n, counts, cap, gen):
    """Four disjoint ascending row lists [4, cap] (unused entries 0) and their counts."""
    perm = torch.randperm(n, generator=gen)
    lists = torch.zeros(4, cap, dtype=torch.int64)
    at = 0
    for i, c in enumerate(counts):
        lists[i, :c] = torch.sort(perm[at:at + c]).values
        at += c
    return lists


def _halo(slot_bytes, sides=(0, 1)):
    from insconv import cabi
    h = C.c_void_p()
    cabi.call("scn_halo_create", C.byref(h), slot_bytes)
    for s in sides:
        cabi.call("scn_halo_connect", h, s, None)
    return cabi, h


def _exchange(cabi, h, lists, counts, a, b=None):
    cabi.call("scn_halo_exchange", h, lists.data_ptr(), counts.data_ptr(), lists.shape[1], a.data_ptr(),
              a.shape[1] * a.element_size(), None if b is None else b.data_ptr(),
              0 if b is None else b.shape[1] * b.element_size(), torch.cuda.current_stream().cuda_stream)


def _status(cabi, h):
    t, o = C.c_int(0), C.c_int(0)
    cabi.call("scn_halo_status", h, C.byref(t), C.byref(o), torch.cuda.current_stream().cuda_stream)
    return t.value, o.value


@pytest.mark.parametrize("planes_a,planes_b", [(32, 32), (64, 0), (3, 0), (6, 10)])
def test_periodic_self_exchange_moves_exactly_the_listed_rows(planes_a, planes_b):
    gen = torch.Generator().manual_seed(planes_a * 100 + planes_b)
    n, cap = 5000, 700
    cabi, h = _halo(1 << 20)
    try:
        for step, counts in enumerate([(300, 200, 200, 300), (1, 700, 700, 1), (0, 5, 5, 0)]):
            lists = _lists(n, counts, cap, gen).cuda()
            cnt = torch.tensor(counts, dtype=torch.int64).cuda()
            a = torch.randn(n, planes_a, generator=gen).cuda()
            b = torch.randn(n, planes_b, generator=gen).half().cuda() if planes_b else None
            a0, b0 = a.clone(), None if b is None else b.clone()
            _exchange(cabi, h, lists, cnt, a, b)
            assert _status(cabi, h) == (0, 0)
            for t, t0 in ((a, a0), (b, b0)):
                if t is None:
                    continue
                want = t0.clone()
                # what goes out to the left comes back in from the right, and the other way round
                want[lists[3, :counts[3]]] = t0[lists[0, :counts[0]]]
                want[lists[2, :counts[2]]] = t0[lists[1, :counts[1]]]
                assert torch.equal(t, want), step
    finally:
        cabi.call("scn_halo_destroy", h)


def test_plane_larger_than_a_slot_is_reported():
    gen = torch.Generator().manual_seed(1)
    n, cap = 4000, 1000
    cabi, h = _halo(64 * 128)  # room for 64 rows of 32 floats
    try:
        counts = (100, 100, 100, 100)
        lists = _lists(n, counts, cap, gen).cuda()
        a = torch.randn(n, 32, generator=gen).cuda()
        a0 = a.clone()
        _exchange(cabi, h, lists, torch.tensor(counts).cuda(), a)
        assert _status(cabi, h) == (0, 1)
        assert _status(cabi, h) == (0, 0)  # reading clears
        assert torch.equal(a[lists[3, :64]], a0[lists[0, :64]]) and torch.equal(a[lists[3, 64:100]], a0[lists[3, 64:100]])
        # a count beyond the list's capacity (the caller's lists were cut short) is reported the same way
        short = lists[:, :40].contiguous()
        _exchange(cabi, h, short, torch.tensor((50, 10, 10, 50)).cuda(), a)
        assert _status(cabi, h) == (0, 1)
    finally:
        cabi.call("scn_halo_destroy", h)


def test_wait_for_a_neighbour_that_never_writes_runs_out_and_reports():
    """Only the left side is connected (to this rank's own inbox): what is pushed left arrives in the right-hand
    inbox, which is not read, and the left-hand inbox is never written.  The wait gives up after its limit, the rows
    stay as they were, the status says so and the context stays usable."""
    gen = torch.Generator().manual_seed(2)
    n, cap = 1000, 100
    cabi, h = _halo(1 << 20, sides=(0,))
    try:
        cabi.call("scn_halo_set_spin_limit", h, 50)
        counts = (10, 10, 10, 10)
        lists = _lists(n, counts, cap, gen).cuda()
        a = torch.randn(n, 32, generator=gen).cuda()
        a0 = a.clone()
        for _ in range(3):  # later exchanges do not wait again
            _exchange(cabi, h, lists, torch.tensor(counts).cuda(), a)
        assert _status(cabi, h) == (1, 0)
        assert torch.equal(a, a0)
        assert torch.equal(a * 2, a0 * 2)  # the device still answers
    finally:
        cabi.call("scn_halo_destroy", h)


def test_bad_arguments_are_refused():
    from insconv import cabi
    h = C.c_void_p()
    with pytest.raises(cabi.ScnError):
        cabi.call("scn_halo_create", C.byref(h), 24)
    cabi2, h = _halo(1 << 16)
    try:
        with pytest.raises(cabi.ScnError):
            cabi.call("scn_halo_connect", h, 0, None)  # connected already
        a = torch.zeros(4, 3, dtype=torch.float16).cuda()  # 6-byte rows
        lists = torch.zeros(4, 4, dtype=torch.int64).cuda()
        with pytest.raises(cabi.ScnError):
            _exchange(cabi, h, lists, torch.zeros(4, dtype=torch.int64).cuda(), a)
    finally:
        cabi.call("scn_halo_destroy", h)


def test_plane_row_lists_match_a_direct_search(cuda):
    """scn_halo_plane_lists (through Metadata.haloPlaneLists): ascending rows of the planes x == lo, hi - 1, lo - 1, hi of a
    scale, with and without neighbours, at the input scale and at a coarse one, and with a capacity that cuts them short."""
    import sparseconvnet as scn
    from insconv import synth
    c = synth.room(3, target=60000)
    il = scn.InputLayer(3, 4096, mode=4)
    t = il([torch.from_numpy(c).to(cuda), torch.ones(c.shape[0], 1, device=cuda)])
    conv = scn.Convolution(3, 1, 1, 2, 2, False).to(cuda)
    coarse = conv(t)
    for tensor, lo, hi in ((t, 100, 228), (t, 8, 9), (coarse, 50, 114)):
        x = tensor.metadata.getSpatialLocationsDevice(tensor.spatial_size)[0]
        n = x.shape[0]
        for left, right in ((True, True), (False, True), (True, False)):
            lists, counts = tensor.metadata.haloPlaneLists(tensor.spatial_size, lo, hi, left, right, n)
            want = [torch.nonzero(x == v).flatten() if on else x.new_empty(0, dtype=torch.long)
                    for v, on in ((lo, left), (hi - 1, right), (lo - 1, left), (hi, right))]
            assert counts.tolist() == [w.numel() for w in want]
            for i, w in enumerate(want):
                assert torch.equal(lists[i, :w.numel()], w)
        lists, counts = tensor.metadata.haloPlaneLists(tensor.spatial_size, lo, hi, True, True, 5)
        full = int((x == lo).sum())
        assert int(counts[0]) == full and torch.equal(lists[0, :min(5, full)], torch.nonzero(x == lo).flatten()[:5])
