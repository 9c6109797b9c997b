"""The CPU oracle against vectors produced by the reference itself (tests/golden/ref_*.npz, written by
tests/golden/make_golden_ref.py and make_golden_model.py from the reference compiled for the host), and the
product's module tree against the reference's (ref_model.json).  Integer results bit for bit; fp32 within 1e-5
relative of the reference's outputs (its kernels sum in another order)."""
import json
import os
import sys

import numpy as np
import pytest
import torch

from oracle import scn_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden_model as GM  # noqa: E402
import make_golden_ref as G  # noqa: E402
from insconv import synth  # noqa: E402


def load(name):
    return np.load(os.path.join(HERE, "golden", name))


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max()) / max(float(np.abs(b).max()), 1e-12)


def check_sampled(x, fx, name, tol=1e-5):
    x = np.asarray(x, np.float32)
    assert list(x.shape) == fx[name + "_shape"].tolist()
    assert rel(x[::G.STEP], fx[name + "_rows"]) <= tol
    assert rel(x.astype(np.float64).sum(0), fx[name + "_colsum"]) <= 10 * tol


def test_config0_scene_rulebooks_and_ssc_output_equal_the_reference():
    fx = load("ref_c1.npz")
    coords, feats, weight = G.c1_inputs()
    assert np.array_equal(G.digest(coords), fx["coords_digest"]), "the scene generator changed: regenerate the fixtures"
    g = O.Grid(coords)
    assert g.n == int(fx["n_active"]) == 50208
    assert np.array_equal(G.digest(g.coords), fx["site_coords_digest"])
    rules = O.ssc_rules(g)
    assert [len(r) for r in rules] == fx["ssc_counts"].tolist()
    assert np.array_equal(G.rules_digest(rules), fx["ssc_pairs_digest"])
    vox = O.input_forward(feats, g, 4)
    check_sampled(O.conv_forward(vox, weight, rules, g.n).numpy(), fx, "out")
    coarse, crules = O.conv2_rules(g)
    assert [len(r) for r in crules] == fx["conv_counts"].tolist()
    assert np.array_equal(G.rules_digest(crules), fx["conv_pairs_digest"])
    assert np.array_equal(G.digest(coarse.coords), fx["coarse_coords_digest"])


def test_config1_incremental_maps_and_residuals_equal_the_reference():
    fx = load("ref_c2.npz")
    coords, feats, weight = G.c1_inputs()
    nf = synth.next_frame(coords, feats, G.C1_SEED)
    assert np.array_equal(G.digest(nf["new_coords"]), fx["new_coords_digest"])
    pg, g = O.Grid(coords), O.Grid(nf["new_coords"])
    assert g.n == int(fx["n_active"])
    assert np.array_equal(G.digest(g.coords), fx["site_coords_digest"])
    assert np.array_equal(G.digest(O.pre_exist(g, pg)), fx["pre_exist_digest"])
    assert np.array_equal(G.rules_digest(O.ssc_rules(g)), fx["ssc_pairs_digest"])
    irules = O.incre_ssc_rules(g, pg)
    assert [len(r) for r in irules] == fx["incre_counts"].tolist()
    assert np.array_equal(G.rules_digest(irules), fx["incre_pairs_digest"])
    vox = O.input_forward(feats, pg, 4)
    res = O.incre_input_forward(nf["new_feats"], g, 4, pg, vox)
    assert rel(res.numpy(), fx["input_residual"]) <= 1e-5
    assert rel(O.incre_ssc_forward(res, weight, g, pg, vox).numpy(), fx["ssc_residual"]) <= 1e-5


def oracle_chain():
    """The network of make_golden_ref.py's chain on the oracle: (full-frame output, incremental output)."""
    coords0 = synth.boxes_and_spheres(0)
    rng = np.random.RandomState(0)
    feats0 = rng.randn(coords0.shape[0], 16).astype(np.float32)
    nf = synth.next_frame(coords0, feats0, 0)
    p = G.chain_params()
    bn = (p["mean"], p["var"], p["gamma"], p["beta"], 1e-4, 0.0)
    g0 = O.Grid(coords0)
    c0, r0 = O.conv2_rules(g0)
    v0 = O.input_forward(feats0, g0, 4)
    a = O.conv_forward(v0, p["w1"], O.ssc_rules(g0), g0.n)
    b = O.bn_forward(a, *bn)
    c = O.conv_forward(b, p["w2"], r0, c0.n)
    d = O.conv_forward(c, p["w3"], O.ssc_rules(c0), c0.n)
    e = O.conv_forward(d, p["w4"], r0, g0.n, reverse=True)
    full = O.output_forward(e, g0)
    g1 = O.Grid(nf["new_coords"])
    c1, r1 = O.conv2_rules(g1)
    x = O.incre_input_forward(nf["new_feats"], g1, 4, g0, v0)
    x = O.incre_ssc_forward(x, p["w1"], g1, g0, v0)
    x = O.incre_bn_forward(x, *bn, g1, g0, b, a)
    x = O.conv_forward(x, p["w2"], r1, c1.n)
    x = O.incre_ssc_forward(x, p["w3"], c1, c0, c)
    x = O.incre_deconv_forward(x, p["w4"], g1, c1, r1, g0, c0, d)
    inc = O.incre_output_forward(x, g1, g0, e)
    return coords0, nf, full.numpy(), inc.numpy(), {"after_ssc1": a, "after_bn": b, "after_conv": c, "after_ssc2": d,
                                                    "after_deconv": e}


def test_operator_chain_full_and_incremental_equals_the_reference():
    fx = load("ref_chain.npz")
    coords0, nf, full, inc, mid = oracle_chain()
    assert np.array_equal(G.digest(coords0), fx["coords_digest"])
    assert np.array_equal(G.digest(nf["new_coords"]), fx["new_coords_digest"])
    for name, x in mid.items():
        assert rel(x.double().sum(0).numpy(), fx[name + "_colsum"]) <= 1e-4, name
    check_sampled(full, fx, "full")
    assert rel(inc, fx["incremental"]) <= 1e-5


def model_py_network():
    """The network of the reference's model.py:9-26, built from this repository's sparseconvnet package."""
    import sparseconvnet as scn

    class Naive_UNet(torch.nn.Module):
        def __init__(self):
            torch.nn.Module.__init__(self)
            m = 32
            self.sparseModel = scn.Sequential().add(scn.InputLayer(3, 4096, mode=4)).add(
                scn.SubmanifoldConvolution(3, 3, m, 3, False)).add(
                scn.UNet(3, 2, [m, 2 * m, 3 * m, 4 * m, 5 * m, 6 * m, 7 * m], True)).add(scn.BatchNormReLU(m)).add(
                scn.OutputLayer(3))
            self.linear = torch.nn.Linear(m, 20)

        def forward(self, x, increment=False):
            return self.linear(self.sparseModel(x, increment))

    return Naive_UNet().eval()


def test_product_module_tree_equals_the_reference_model_py():
    """state_dict keys and shapes, and the module tree with every layer's constructor-derived attributes, against
    what the reference's own model.py + sparseconvnet package build (ref_model.json)."""
    with open(os.path.join(HERE, "golden", "ref_model.json")) as f:
        fx = json.load(f)
    net = model_py_network()
    assert {k: list(v.shape) for k, v in net.state_dict().items()} == fx["state_dict"]
    assert GM.tree(net) == fx["tree"]


def test_oracle_topology_builder_equals_the_reference_model_py():
    """oracle/scn_topology.py (the module tree the timed CPU baseline walks, built without the product package)."""
    from oracle import scn_topology as T
    with open(os.path.join(HERE, "golden", "ref_model.json")) as f:
        fx = json.load(f)
    net = T.Naive_UNet().eval()
    assert {k: list(v.shape) for k, v in net.state_dict().items()} == fx["state_dict"]
    assert GM.tree(net) == fx["tree"]


def test_oracle_walks_the_product_tree_as_it_walks_the_reference_tree():
    """ref_model_run.npz holds what the oracle computed walking the REFERENCE's module tree; walking the product's
    tree with the same seeded weights must give the same numbers (same torch-CPU arithmetic: exact)."""
    from oracle.scn_graph import GraphRunner
    fx = load("ref_model_run.npz")
    net = model_py_network()
    shapes = {k: list(v.shape) for k, v in net.state_dict().items()}
    net.load_state_dict({k: torch.from_numpy(v) for k, v in GM.seeded_state(shapes).items()}, strict=False)
    coords, feats, new, new_feats = GM.small_scene()
    run = GraphRunner(net)
    full = run([torch.from_numpy(coords), torch.from_numpy(feats)])
    inc = run([torch.from_numpy(new), torch.from_numpy(new_feats)], True)
    assert np.array_equal(full.numpy(), fx["full"]) and np.array_equal(inc.numpy(), fx["incremental"])


@pytest.mark.skipif(not os.path.isdir("/root/reference"), reason="needs the reference tree")
def test_committed_model_fixture_is_what_the_reference_builds_today():
    import subprocess
    r = subprocess.run([sys.executable, "-c", (
        "import sys, json; sys.path.insert(0, %r); import make_golden_model as GM\n"
        "from unittest import mock; sys.path.insert(0, GM.REFERENCE); sys.modules['sparseconvnet.SCN'] = mock.MagicMock()\n"
        "import model; net = model.Naive_UNet({'dimension': 3, 'full_scale': 4096})\n"
        "print(json.dumps({'state_dict': {k: list(v.shape) for k, v in net.state_dict().items()}, 'tree': GM.tree(net)}, sort_keys=True))"
    ) % os.path.join(HERE, "golden")], capture_output=True, text=True, check=True)
    with open(os.path.join(HERE, "golden", "ref_model.json")) as f:
        assert json.loads(r.stdout.strip().splitlines()[-1]) == json.load(f)


def test_label_fusion_oracle_equals_the_reference_vectors():
    """oracle/scn_labels.py against what the reference's Result<3> / ResultOfWeight<3> produced (ref_labels.npz)."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from labels_cases import frames
    from oracle import scn_labels as L
    fx = load("ref_labels.npz")
    for name, maximum in (("default", 0.7), ("cap3", 3.0)):
        scene, fr = frames(0)
        assert np.array_equal(G.digest(scene), fx["scene_digest"]), "the case generator changed: regenerate the fixtures"
        o = L.Result(maximum)
        for f, (ps, sc) in enumerate(fr):
            o.update(ps, sc)
            assert np.array_equal(o.multiQuery(scene), fx[name + "_labels_after_each_frame"][f])
        conf = np.array([o.result.get(tuple(int(v) for v in p), (0, -1.0))[1] for p in scene], np.float32)
        assert np.array_equal(conf, fx[name + "_confidence"]) and len(o.result) == int(fx[name + "_size"])
        o.finalize(scene[::3])
        assert np.array_equal(o.multiQuery(scene), fx[name + "_labels_after_finalize"])
        o.set(scene[:50], fr[0][1][:50])
        assert np.array_equal(o.multiQuery(scene), fx[name + "_labels_after_set"])
    w = L.ResultOfWeight()
    for ps, sc in fr:
        w.update(ps, sc)
    assert np.array_equal(w.multiQuery(scene), fx["weight_labels"])
