"""The CPU oracle against hand-derived cases (worked out from the reference's rule definitions) and
against the committed fixtures in tests/golden/."""
import os

import numpy as np
import torch

from oracle import scn_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_key_order_matches_the_reference_key_inside_its_range():
    rng = np.random.RandomState(0)
    c = np.stack([rng.randint(0, 1024, 5000), rng.randint(0, 2048, 5000), rng.randint(0, 1024, 5000)], 1)
    k31 = O.ref_key31(c[:, 0], c[:, 1], c[:, 2])
    k64 = O.key64(c[:, 0], c[:, 1], c[:, 2], np.zeros(5000, np.int64))
    # same ordering (ties included): ranks agree
    assert np.array_equal(np.argsort(k31, kind="stable"), np.argsort(k64, kind="stable"))
    assert np.array_equal(np.unique(k31, return_inverse=True)[1], np.unique(k64, return_inverse=True)[1])


def test_site_numbering_is_rank_of_key_z_major():
    # keys order by z, then y, then x (CUDPPWrapper.cu:110-119: z<<21 | y<<10 | x)
    c = np.array([[5, 1, 1], [1, 5, 1], [1, 1, 5], [2, 1, 1], [1, 1, 1]])
    g = O.Grid(c)
    assert g.coords[:, :3].tolist() == [[1, 1, 1], [2, 1, 1], [5, 1, 1], [1, 5, 1], [1, 1, 5]]
    assert g.src_row.tolist() == [2, 3, 4, 1, 0]
    assert g.lookup(np.array([[1, 5, 1, 0], [9, 9, 9, 0], [-1, 0, 0, 0]])).tolist() == [3, -1, -1]


def test_input_rules_layout_and_mean():
    # three points share voxel (1,1,1); rule rows hold ascending point indices (IOLayers.cu:7-12)
    c = np.array([[1, 1, 1], [2, 1, 1], [1, 1, 1], [1, 1, 1]])
    g = O.Grid(c)
    hdr, rows = O.input_rules(g, 4)
    assert hdr.tolist() == [4, 3, 4, 2]
    assert rows.tolist() == [[3, 0, 2, 3], [1, 1, 0, 0]]
    f = torch.tensor([[1.0], [10.0], [2.0], [6.0]])
    assert O.input_forward(f, g, 4).flatten().tolist() == [3.0, 10.0]
    assert O.input_forward(f, g, 3).flatten().tolist() == [9.0, 10.0]
    assert O.output_forward(torch.tensor([[7.0], [8.0]]), g).flatten().tolist() == [7.0, 8.0, 7.0, 7.0]


def test_ssc_offsets_and_pairs():
    # offset index (dx+1)*9 + (dy+1)*3 + (dz+1); input site = output + offset (SubmanifoldRules_cuda.cu:61-74,104-109)
    offs = O.ssc_offsets()
    assert offs[0] == (-1, -1, -1) and offs[13] == (0, 0, 0) and offs[26] == (1, 1, 1) and offs[22] == (1, 0, 0)
    c = np.array([[5, 5, 5], [6, 5, 5], [5, 5, 6]])
    g = O.Grid(c)  # rows: (5,5,5)=0, (6,5,5)=1, (5,5,6)=2
    r = O.ssc_rules(g)
    assert r[13].tolist() == [[0, 0], [1, 1], [2, 2]]
    assert r[22].tolist() == [[1, 0]]      # +x neighbour of row 0 is row 1
    assert r[4].tolist() == [[0, 1]]       # -x neighbour of row 1 is row 0
    assert r[14].tolist() == [[2, 0]]      # +z neighbour of row 0 is row 2
    assert r[12].tolist() == [[0, 2]]
    assert r[5].tolist() == [[2, 1]]       # (-1,0,+1): rows 1 and 2 are diagonal neighbours
    assert r[21].tolist() == [[1, 2]]      # (+1,0,-1)
    assert sum(len(x) for x in r) == 9


def test_stride2_rules():
    # k = (x&1)*4 + (y&1)*2 + (z&1), pair (fine, coarse) (SubmanifoldRules_cuda.cu:760-766)
    c = np.array([[2, 2, 2], [3, 2, 2], [2, 3, 3], [4, 2, 2]])
    g = O.Grid(c)
    coarse, rules = O.conv2_rules(g)
    assert coarse.coords[:, :3].tolist() == [[1, 1, 1], [2, 1, 1]]
    fine_rows = {tuple(v): i for i, v in enumerate(g.coords[:, :3].tolist())}
    assert rules[0].tolist() == [[fine_rows[(2, 2, 2)], 0], [fine_rows[(4, 2, 2)], 1]]
    assert rules[4].tolist() == [[fine_rows[(3, 2, 2)], 0]]
    assert rules[3].tolist() == [[fine_rows[(2, 3, 3)], 0]]


def test_conv_and_deconv_arithmetic():
    c = np.array([[5, 5, 5], [6, 5, 5]])
    g = O.Grid(c)
    w = torch.zeros(27, 1, 1)
    w[13] = 2.0
    w[22] = 10.0  # weight of the +x neighbour
    x = torch.tensor([[1.0], [3.0]])
    out = O.conv_forward(x, w, O.ssc_rules(g), g.n, bias=torch.tensor([0.5]))
    assert out.flatten().tolist() == [2 * 1 + 10 * 3 + 0.5, 2 * 3 + 0.5]
    coarse, rules = O.conv2_rules(O.Grid(np.array([[2, 2, 2], [3, 2, 2]])))
    w8 = torch.arange(8, dtype=torch.float32).reshape(8, 1, 1) + 1
    down = O.conv_forward(x, w8, rules, coarse.n)
    assert down.flatten().tolist() == [1 * 1 + 5 * 3]
    up = O.conv_forward(torch.tensor([[2.0]]), w8, rules, 2, reverse=True)
    assert up.flatten().tolist() == [2.0, 10.0]


def test_bn_formula():
    x = torch.tensor([[1.0, -2.0]])
    y = O.bn_forward(x, torch.tensor([0.5, 0.0]), torch.tensor([4.0 - 1e-4, 1.0 - 1e-4]), torch.tensor([2.0, 1.0]),
                     torch.tensor([0.0, 1.0]), 1e-4, 0.0)
    assert torch.allclose(y, torch.tensor([[0.5, 0.0]]), atol=1e-6)
    y = O.bn_forward(x, torch.zeros(2), torch.ones(2) - 1e-4, None, None, 1e-4, 0.5)
    assert torch.allclose(y, torch.tensor([[1.0, -1.0]]), atol=1e-6)


def test_incremental_input_residual_formula():
    # saved voxel holds 2 points with mean 4; one new point of value 10 -> new mean 6, residual 2 (IOLayers.cu:82-106)
    pre = O.Grid(np.array([[1, 1, 1], [1, 1, 1], [3, 3, 3]]))
    pre_out = O.input_forward(torch.tensor([[3.0], [5.0], [7.0]]), pre, 4)
    g = O.Grid(np.array([[1, 1, 1], [9, 9, 9]]))
    res = O.incre_input_forward(torch.tensor([[10.0], [1.5]]), g, 4, pre, pre_out)
    assert torch.allclose(res.flatten(), torch.tensor([2.0, 1.5]))
    full = O.incre_output_forward(res, g, pre, pre_out)
    assert torch.allclose(full.flatten(), torch.tensor([6.0, 1.5]))


def test_incremental_ssc_rules_only_feed_new_sites():
    pre = O.Grid(np.array([[5, 5, 5], [6, 5, 5]]))
    g = O.Grid(np.array([[6, 5, 5], [7, 5, 5]]))  # row 0 existed, row 1 is new
    assert O.pre_exist(g, pre).tolist() == [1, -1]
    r = O.incre_ssc_rules(g, pre)
    assert r[4].tolist() == [[1, 1]]  # -x neighbour of the new site is saved row 1
    assert sum(len(x) for x in r) == 1


def test_golden_fixtures():
    z = np.load(os.path.join(GOLDEN, "c1_small.npz"))
    g = O.Grid(z["coords"])
    assert np.array_equal(g.coords, z["site_coords"])
    assert np.array_equal(g.src_row, z["src_row"])
    rules = O.ssc_rules(g)
    assert np.array_equal(np.array([len(r) for r in rules]), z["ssc_counts"])
    assert np.array_equal(np.concatenate(rules, 0), z["ssc_pairs"])
    coarse, crules = O.conv2_rules(g)
    assert np.array_equal(np.concatenate(crules, 0), z["conv_pairs"])
    out = O.conv_forward(z["feats"], z["weight"], rules, g.n)
    assert np.allclose(out.numpy(), z["ssc_out"], rtol=1e-5, atol=1e-6)
