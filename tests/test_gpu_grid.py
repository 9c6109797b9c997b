"""Grid (voxel hash), InputLayer rules and rulebooks through the C ABI vs the CPU oracle: bit exact."""
import numpy as np
import pytest
import torch

from insconv import cabi, synth
from oracle import scn_oracle as O

pytestmark = pytest.mark.gpu


def _build(coords, size, cuda, mode=4, on_device=True):
    m = cabi.Metadata()
    t = torch.from_numpy(np.ascontiguousarray(coords, dtype=np.int64))
    n = m.input_layer_build(size, t.to(cuda) if on_device else t, mode=mode)
    return m, n


def _check_grid(m, n, g, size):
    assert n == g.n
    loc = m.spatial_locations(size)
    np.testing.assert_array_equal(loc, g.coords)
    keys, rows = m.hash_dump(size)
    filled = keys != np.uint64(0xFFFFFFFFFFFFFFFF)
    assert int(filled.sum()) == g.n
    assert dict(zip(keys[filled].tolist(), rows[filled].tolist())) == g.hash_contents()
    hdr, rrows = m.input_rules()
    ohdr, orows = O.input_rules(g, int(hdr[0]))
    np.testing.assert_array_equal(hdr, ohdr)
    np.testing.assert_array_equal(rrows, orows)


def _check_rules(got, want):
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        np.testing.assert_array_equal(a, b, err_msg="offset %d" % k)


def test_tiny_hand_checkable(cuda):
    # three voxels in a row along x plus one isolated voxel
    c = np.array([[5, 5, 5], [6, 5, 5], [7, 5, 5], [20, 20, 20]])
    m, n = _build(c, 64, cuda)
    g = O.Grid(c)
    _check_grid(m, n, g, 64)
    rules = m.ssc_rulebook(64)
    _check_rules(rules, O.ssc_rules(g))
    # centre offset holds every site once; +x / -x offsets hold the two chain links
    assert rules[13].tolist() == [[0, 0], [1, 1], [2, 2], [3, 3]]
    assert rules[22].tolist() == [[1, 0], [2, 1]]  # dx=+1: input is the +x neighbour
    assert rules[4].tolist() == [[0, 1], [1, 2]]   # dx=-1


@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("on_device", [True, False])
def test_boxes_and_spheres(cuda, seed, on_device):
    c = synth.boxes_and_spheres(seed)
    rng = np.random.RandomState(seed)
    c = c[rng.permutation(c.shape[0])]
    m, n = _build(c, 128, cuda, on_device=on_device)
    g = O.Grid(c)
    _check_grid(m, n, g, 128)
    _check_rules(m.ssc_rulebook(128), O.ssc_rules(g))
    coarse, crules = O.conv2_rules(g)
    _check_rules(m.conv_rulebook(128, 64), crules)
    assert m.n_active(64) == coarse.n
    np.testing.assert_array_equal(m.spatial_locations(64), coarse.coords)
    _check_rules(m.ssc_rulebook(64), O.ssc_rules(coarse))


def test_duplicates_and_batches(cuda):
    rng = np.random.RandomState(3)
    c = rng.randint(1, 40, size=(20000, 3))
    b = np.sort(rng.randint(0, 3, size=(20000, 1)), 0)
    cb = np.concatenate([c, b], 1)
    for mode in (3, 4):
        m, n = _build(cb, 64, cuda, mode=mode)
        g = O.Grid(cb)
        assert g.n < cb.shape[0]
        _check_grid(m, n, g, 64)
        _check_rules(m.ssc_rulebook(64), O.ssc_rules(g))
        _, crules = O.conv2_rules(g)
        _check_rules(m.conv_rulebook(64, 32), crules)


@pytest.mark.parametrize("extent", [(1, 1, 7), (1, 3, 2), (2, 5, 3), (3, 1, 11), (5, 7, 2), (63, 2, 2), (65, 3, 1)])
def test_narrow_boxes(cuda, extent):
    # bounding boxes whose lines (and planes) are shorter than a 64-cell bitmap word: one word of the ranking
    # structure then covers several lines, planes and batch entries
    rng = np.random.RandomState(sum(extent))
    e = np.array(extent)
    c = rng.randint(0, 1 << 30, size=(400, 3)) % e + np.array([5, 9, 2])
    b = np.sort(rng.randint(0, 4, size=(400, 1)), 0)
    cb = np.concatenate([c, b], 1)
    m, n = _build(cb, 128, cuda)
    g = O.Grid(cb)
    _check_grid(m, n, g, 128)
    _check_rules(m.ssc_rulebook(128), O.ssc_rules(g))
    coarse, crules = O.conv2_rules(g)
    _check_rules(m.conv_rulebook(128, 64), crules)
    np.testing.assert_array_equal(m.spatial_locations(64), coarse.coords)
    _check_rules(m.ssc_rulebook(64), O.ssc_rules(coarse))


def test_permutation_invariance(cuda):
    c = synth.boxes_and_spheres(2)
    m1, _ = _build(c, 128, cuda)
    m2, _ = _build(c[np.random.RandomState(0).permutation(c.shape[0])], 128, cuda)
    np.testing.assert_array_equal(m1.spatial_locations(128), m2.spatial_locations(128))
    _check_rules(m1.ssc_rulebook(128), m2.ssc_rulebook(128))


@pytest.mark.parametrize("pts", [
    [[0, 0, 0], [1, 0, 0], [0, 1, 1]],                                  # low faces of the key range
    [[65534, 65534, 65534], [65533, 65534, 65534], [65534, 65533, 65533]],  # high faces
    [[1023, 2047, 1023], [1024, 2047, 1023], [1024, 2048, 1024]],       # beyond the reference's 10/11/10-bit key
])
def test_border_and_wide_coordinates(cuda, pts):
    # neighbours outside the key range must miss, not alias
    c = np.array(pts)
    m, n = _build(c, 65536, cuda)
    g = O.Grid(c)
    _check_grid(m, n, g, 65536)
    _check_rules(m.ssc_rulebook(65536), O.ssc_rules(g))


def test_empty_and_single(cuda):
    m, n = _build(np.zeros((0, 3), np.int64), 32, cuda)
    assert n == 0 and m.n_active(32) == 0
    assert sum(len(r) for r in m.ssc_rulebook(32)) == 0
    m, n = _build(np.array([[3, 4, 5]]), 32, cuda)
    assert n == 1
    r = m.ssc_rulebook(32)
    assert [len(x) for x in r] == [0] * 13 + [1] + [0] * 13


def test_errors_are_reported_not_fatal(cuda):
    m = cabi.Metadata()
    with pytest.raises(cabi.ScnError) as e:
        m.input_layer_build(64, torch.tensor([[1, 2, 70000]], device=cuda), mode=4)
    assert e.value.code == -3
    with pytest.raises(cabi.ScnError):
        m.input_layer_build(64, torch.tensor([[1, 2, 3]], device=cuda), mode=1)
    with pytest.raises(cabi.ScnError):
        m.ssc_rulebook(64)  # no grid
    # the device is still usable afterwards
    n = m.input_layer_build(64, torch.tensor([[1, 2, 3]], device=cuda), mode=4)
    assert n == 1


def test_query(cuda):
    c = synth.boxes_and_spheres(0)
    m, _ = _build(c, 128, cuda)
    g = O.Grid(c)
    rng = np.random.RandomState(0)
    q = np.concatenate([c[rng.randint(0, c.shape[0], 5000)], rng.randint(0, 128, size=(5000, 3))], 0)
    q4 = np.concatenate([q, np.zeros((q.shape[0], 1), np.int64)], 1)
    soa = torch.from_numpy(np.ascontiguousarray(q4.T.astype(np.int32))).to(cuda)
    rows = m.query(128, soa).cpu().numpy()
    np.testing.assert_array_equal(rows, g.lookup(q4))


def test_build_ahead_changes_when_not_what(cuda):
    # scn_set_build_ahead: coarse scales and neighbour maps built inside the input layer's call, or on first use;
    # grids, hash tables and rulebooks are the same either way
    c = synth.boxes_and_spheres(4)
    d = torch.from_numpy(c).to(cuda)
    results = []
    try:
        for ssc, levels in ((0, 0), (1, 3)):
            cabi.call("scn_set_build_ahead", ssc, levels)
            m = cabi.Metadata()
            n = m.input_layer_build(128, d, mode=4)
            assert (m.n_active(64) >= 0) == (levels >= 1)
            assert (m.n_active(16) >= 0) == (levels >= 3) and m.n_active(8) < 0
            rb = [m.ssc_rulebook(128), m.conv_rulebook(128, 64), m.ssc_rulebook(64), m.conv_rulebook(64, 32),
                  m.conv_rulebook(32, 16)]
            locs = [m.spatial_locations(s) for s in (128, 64, 32, 16)]
            results.append((n, rb, locs))
        with pytest.raises(cabi.ScnError):
            cabi.call("scn_set_build_ahead", 2, 0)
    finally:
        cabi.call("scn_set_build_ahead", -1, -1)
    (n0, rb0, l0), (n1, rb1, l1) = results
    assert n0 == n1
    for a, b in zip(l0, l1):
        assert np.array_equal(a, b)
    for a, b in zip(rb0, rb1):
        assert len(a) == len(b)
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


def _distant_clusters(seed, span):
    """Two clusters of surfaces at opposite corners of a span^3 volume (a bounding box far beyond what a ranking bitmap
    is laid out for), with duplicates, in two batch entries."""
    rng = np.random.RandomState(seed)
    a = synth.boxes_and_spheres(seed, grid=64) + 1
    b = synth.boxes_and_spheres(seed + 1, grid=64) + (span - 70)
    c = np.concatenate([a, b, a[rng.randint(0, a.shape[0], 500)]], 0)
    c = c[rng.permutation(c.shape[0])]
    batch = np.sort(rng.randint(0, 2, size=(c.shape[0], 1)), 0)
    return np.concatenate([c, batch], 1)


@pytest.mark.parametrize("span", [4096, 65534])
def test_scene_spanning_the_whole_volume_builds_and_matches_the_oracle(cuda, span):
    """A scene that spans the 4096^3 volume model.py declares (and one that spans the whole key range): ranked by
    sorting, looked up through the open-addressing table; sites, input rules, hash contents, 3x3x3 and 2x2x2 rulebooks at
    the input scale and down the coarse scales, and coordinate queries, all bit-exact."""
    cb = _distant_clusters(7, span)
    size = 1 << 16
    for mode in (3, 4):
        m, n = _build(cb, size, cuda, mode=mode)
        g = O.Grid(cb)
        assert g.n < cb.shape[0]
        _check_grid(m, n, g, size)
        _check_rules(m.ssc_rulebook(size), O.ssc_rules(g))
        fine = g
        for level in range(1, 5):  # coarse scales: sorted while the box is still too large, bitmaps once it fits
            coarse, crules = O.conv2_rules(fine)
            _check_rules(m.conv_rulebook(size >> (level - 1), size >> level), crules)
            np.testing.assert_array_equal(m.spatial_locations(size >> level), coarse.coords)
            _check_rules(m.ssc_rulebook(size >> level), O.ssc_rules(coarse))
            fine = coarse
    rng = np.random.RandomState(1)
    q = np.concatenate([cb[rng.randint(0, cb.shape[0], 3000)], np.concatenate([rng.randint(0, span, size=(3000, 3)),
                                                                              rng.randint(0, 2, size=(3000, 1))], 1)], 0)
    soa = torch.from_numpy(np.ascontiguousarray(q.T.astype(np.int32))).to(cuda)
    np.testing.assert_array_equal(m.query(size, soa).cpu().numpy(), g.lookup(q))


def test_spread_out_scene_with_build_ahead_and_incremental_maps(cuda):
    """The same kind of scene through the build-ahead chain (coarse scales built by the input layer) and as the saved
    frame of an incremental update: pre-exist map and incremental rulebook bit-exact."""
    cb = _distant_clusters(9, 4096)[:, :3]
    rng = np.random.RandomState(2)
    new = np.concatenate([cb[rng.randint(0, cb.shape[0], 400)], cb[rng.randint(0, cb.shape[0], 400)] + rng.randint(-1, 2, size=(400, 3)),
                          synth.sphere_surface([2000, 2000, 2000], 6)], 0)
    new = np.clip(new, 0, 65534)
    try:
        cabi.call("scn_set_build_ahead", 1, 4)
        pre, _ = _build(cb, 4096, cuda)
        m, _ = _build(new, 4096, cuda)
    finally:
        cabi.call("scn_set_build_ahead", -1, -1)
    pg, g = O.Grid(cb), O.Grid(new)
    np.testing.assert_array_equal(m.spatial_locations(4096), g.coords)
    np.testing.assert_array_equal(m.pre_exist(pre, 4096), O.pre_exist(g, pg))
    _check_rules(m.incre_ssc_rulebook(pre, 4096), O.incre_ssc_rules(g, pg))
    fine, pfine = g, pg
    for level in range(1, 5):
        coarse, crules = O.conv2_rules(fine)
        pcoarse, _ = O.conv2_rules(pfine)
        _check_rules(m.conv_rulebook(4096 >> (level - 1), 4096 >> level), crules)
        np.testing.assert_array_equal(m.pre_exist(pre, 4096 >> level), O.pre_exist(coarse, pcoarse))
        _check_rules(m.incre_ssc_rulebook(pre, 4096 >> level), O.incre_ssc_rules(coarse, pcoarse))
        fine, pfine = coarse, pcoarse


def test_rebuilding_on_one_metadata_with_a_scene_that_leaves_the_previous_box(cuda):
    """A metadata object that is built on again lays its bitmap out for the previous scene's box (no round trip to
    measure); a scene that does not fit is built again with its own box.  Same results either way."""
    a = synth.boxes_and_spheres(1, grid=96) + 20
    m = cabi.Metadata()
    for shift in ((0, 0, 0), (3, -2, 5), (60, 0, 0), (-19, -19, -19), (300, 500, 10), (0, 0, 0)):
        c = a + np.array(shift)
        rng = np.random.RandomState(abs(shift[0]) + 1)
        c = np.concatenate([c, c[rng.randint(0, c.shape[0], 300)]], 0)[rng.permutation(c.shape[0] + 300)]
        n = m.input_layer_build(1024, torch.from_numpy(c).to(cuda), mode=4)
        g = O.Grid(c)
        _check_grid(m, n, g, 1024)
        _check_rules(m.ssc_rulebook(1024), O.ssc_rules(g))
        coarse, crules = O.conv2_rules(g)
        _check_rules(m.conv_rulebook(1024, 512), crules)
        np.testing.assert_array_equal(m.spatial_locations(512), coarse.coords)
    # an out-of-range coordinate on a hinted build is still an error, and the next build works
    bad = a.copy()
    bad[5] = [70000, 1, 1]
    with pytest.raises(cabi.ScnError) as e:
        m.input_layer_build(1024, torch.from_numpy(bad).to(cuda), mode=4)
    assert e.value.code == -3
    n = m.input_layer_build(1024, torch.from_numpy(a).to(cuda), mode=4)
    _check_grid(m, n, O.Grid(a), 1024)
