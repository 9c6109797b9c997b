"""Label fusion on the GPU (sparseconvnet.SCN.Result_3 / ResultOfWeight over the C ABI's scn_labels_*) against the
CPU restatement of the reference's classes and against what the reference itself produced (tests/golden/ref_labels.npz).
Integer results: bit-exact."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from labels_cases import CLASSES, frames  # noqa: E402
from oracle import scn_labels as L  # noqa: E402

pytestmark = pytest.mark.gpu


def _scn():
    import sparseconvnet as scn
    return scn.SCN


def _rows(t):
    return {tuple(v) for v in np.asarray(t).tolist()}


@pytest.mark.parametrize("name,maximum", [("default", 0.7), ("cap3", 3.0)])
def test_vote_table_equals_the_reference_vectors_and_the_oracle(cuda, name, maximum):
    fx = np.load(os.path.join(HERE, "golden", "ref_labels.npz"))
    scene, fr = frames(0)
    d_scene = torch.from_numpy(scene).to(cuda)
    r, o = _scn().Result_3(maximum), L.Result(maximum)
    serial = 0
    for f, (ps, sc) in enumerate(fr):
        # points and scores already on the GPU, as a network's output is; every other frame from the host
        if f % 2 == 0:
            r.update(torch.from_numpy(ps).to(cuda), torch.from_numpy(sc).to(cuda))
        else:
            r.update(torch.from_numpy(ps), torch.from_numpy(sc))
        o.update(ps, sc)
        serial += r.rowsAppliedSerially()
        got = r.multiQuery(d_scene).numpy()
        assert np.array_equal(got, fx[name + "_labels_after_each_frame"][f]) and np.array_equal(got, o.multiQuery(scene))
    assert serial > 0  # the cases name some voxels twice in one call
    assert r.size() == int(fx[name + "_size"])
    assert _rows(r.get_all_points_labels()) == _rows(o.get_all_points_labels())
    assert r.query(torch.from_numpy(scene[7])) == int(o.query(scene[7])) and r.query(torch.tensor([1, 2, 60000])) == -1
    r.finalize(torch.from_numpy(scene[::3]))
    o.finalize(scene[::3])
    assert np.array_equal(r.multiQuery(d_scene).numpy(), fx[name + "_labels_after_finalize"]) and r.size() == len(o.result)
    r.set(torch.from_numpy(scene[:50]), torch.from_numpy(fr[0][1][:50]))
    assert np.array_equal(r.multiQuery(d_scene).numpy(), fx[name + "_labels_after_set"])
    # confidences are not readable through the reference's interface; they show in what later votes do: the same
    # frames once more, against the oracle that went through the same finalize and set
    o.set(scene[:50], fr[0][1][:50])
    for ps, sc in fr:
        r.update(torch.from_numpy(ps).to(cuda), torch.from_numpy(sc).to(cuda))
        o.update(ps, sc)
        assert np.array_equal(r.multiQuery(d_scene).numpy(), o.multiQuery(scene))
    r.clear()
    assert r.size() == 0 and int(r.multiQuery(d_scene).max()) == -1


def test_weight_table_equals_the_reference_vectors_and_the_oracle(cuda):
    fx = np.load(os.path.join(HERE, "golden", "ref_labels.npz"))
    scene, fr = frames(0)
    d_scene = torch.from_numpy(scene).to(cuda)
    r, o = _scn().ResultOfWeight(), L.ResultOfWeight()
    assert int(r.multiQuery(d_scene).max()) == -1 and r.size() == 0
    for ps, sc in fr:
        r.update(torch.from_numpy(ps).to(cuda), torch.from_numpy(sc).to(cuda))
        o.update(ps, sc)
        assert np.array_equal(r.multiQuery(d_scene).numpy(), o.multiQuery(scene))
    assert np.array_equal(r.multiQuery(d_scene).numpy(), fx["weight_labels"])
    assert _rows(r.get_all_points_labels()) == _rows(o.get_all_points_labels())
    r.finalize(d_scene[:500])
    o.finalize(scene[:500])
    assert r.size() == len(o.result) and np.array_equal(r.multiQuery(d_scene).numpy(), o.multiQuery(scene))


def test_table_grows_and_keeps_its_entries(cuda):
    """300k voxels in three calls: the table is rebuilt with more slots twice on the way; every entry survives, batch
    indices are part of the key, coordinates outside the key range are refused."""
    rng = np.random.RandomState(3)
    pts = np.unique(rng.randint(0, 600, size=(400000, 3)), axis=0)[:300000].astype(np.int64)
    pts = np.concatenate([pts, rng.randint(0, 3, size=(pts.shape[0], 1))], 1)
    lab = rng.randint(0, CLASSES, pts.shape[0])
    sc = np.full((pts.shape[0], CLASSES), 0.01, np.float32)
    sc[np.arange(pts.shape[0]), lab] = 0.8
    r = _scn().Result_3(5.0)
    for part in np.array_split(np.arange(pts.shape[0]), 3):
        r.update(torch.from_numpy(pts[part]).to(cuda), torch.from_numpy(sc[part]).to(cuda))
    assert r.size() == pts.shape[0]
    assert np.array_equal(r.multiQuery(torch.from_numpy(pts).to(cuda)).numpy(), lab)
    other_batch = pts.copy()
    other_batch[:, 3] += 5
    assert int(r.multiQuery(torch.from_numpy(other_batch[:1000]).to(cuda)).max()) == -1
    bad = torch.tensor([[1, 2, 70000]])
    r.update(bad.to(cuda), torch.ones(1, CLASSES, device=cuda))
    with pytest.raises(RuntimeError):
        r.size()
    assert r.size() == pts.shape[0]  # reported once, the table is as it was
