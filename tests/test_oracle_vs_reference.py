"""Pins the Python oracle (oracle/scn_oracle.py) to the reference implementation itself.

oracle/_ref/libscn_ref.so is the reference's own Metadata, rulebook builders, cuda_* operators (kernels run
by a CUDA-on-host emulation) and cpu_* operators, compiled from the reference tree by oracle/build_ref.py.
Every function of the oracle that the GPU parity tests rely on is compared here with what the reference
computes on the same seeded inputs: integer results bit for bit, fp32 results to 1e-5 relative (the
reference's kernels accumulate in another order, partly in fp64; the parity bar itself is 1e-4).

The tests skip when neither the reference tree nor a prebuilt library is present.
"""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import scn_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "ins-conv_b200"))
from insconv import synth  # noqa: E402

SPATIAL = 64


@pytest.fixture(scope="module")
def R():
    from oracle import build_ref
    try:
        path = build_ref.build()
    except Exception as e:  # noqa: BLE001
        pytest.fail("the reference could not be compiled for the host: %s" % (e,))
    if path is None:
        pytest.skip("no reference tree and no prebuilt oracle/_ref/libscn_ref.so")
    from oracle import scn_ref
    return scn_ref


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max()) / max(float(np.abs(b).max()), 1e-12)


def scene(seed, n_points=2600, lo=3, hi=40, batch=1):
    """Points on a few box and sphere surfaces inside [lo, hi)^3, with duplicates, sorted by batch index."""
    rng = np.random.RandomState(seed)
    parts = []
    for b in range(batch):
        pts = [synth.box_surface([lo + 2, lo + 3, lo + 1], [lo + 14 + b, lo + 12, lo + 9]),
               synth.sphere_surface([lo + 22, lo + 20, lo + 18], 7 + b),
               synth.box_surface([lo + 18, lo + 2, lo + 20], [lo + 30, lo + 9, lo + 33])]
        c = np.concatenate(pts, 0)
        c = c[rng.permutation(c.shape[0])[:n_points // batch]]
        dup = c[rng.randint(0, c.shape[0], c.shape[0] // 6)]  # some voxels get several points
        c = np.concatenate([c, dup], 0)
        c = c[rng.permutation(c.shape[0])]
        parts.append(np.concatenate([c, np.full((c.shape[0], 1), b, np.int64)], 1))
    coords = np.concatenate(parts, 0)
    assert coords[:, :3].min() >= 1 and coords[:, :3].max() <= 1022
    return coords


def same_rulebook(got, want):
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        assert np.array_equal(np.asarray(a).reshape(-1, 2), np.asarray(b).reshape(-1, 2)), "offset %d" % k


@pytest.mark.parametrize("batch,mode", [(1, 4), (2, 3)])
def test_site_numbering_input_rules_and_io_layers(R, batch, mode):
    """Multival_Point_Hashtable + inputLayerRulesSimple + InputLayer_fp_/InputLayer_bp_ (CUDA/CUDPPWrapper.hpp:736-1010,
    Metadata/IOLayersRules.h:135-203, CUDA/IOLayers.cu:18-76) and CPU/IOLayers.cpp:12-29."""
    coords = scene(1, batch=batch)
    rng = np.random.RandomState(2)
    feats = rng.randn(coords.shape[0], 5).astype(np.float32)
    m = R.Metadata()
    out = R.input_layer(m, SPATIAL, coords, feats, batch, mode)
    g = O.Grid(coords)
    assert m.n_active(SPATIAL) == g.n
    assert np.array_equal(m.spatial_locations(SPATIAL), g.coords)  # row i = i-th smallest key, batch-major
    header, rows = m.input_rules()
    o_header, o_rows = O.input_rules(g, mode)
    assert header.tolist() == o_header.tolist()
    for i in range(g.n):  # the reference leaves the padding of a row uninitialised
        assert np.array_equal(rows[i, :1 + rows[i, 0]], o_rows[i, :1 + o_rows[i, 0]])
    want = O.input_forward(feats, g, mode).numpy()
    assert rel(out, want) <= 1e-6
    assert rel(R.cpu_input_forward(m, feats), want) <= 1e-6
    vox = rng.randn(g.n, 7).astype(np.float32)
    assert np.array_equal(R.output_layer(m, vox), O.output_forward(vox, g).numpy())
    assert np.array_equal(R.cpu_output_forward(m, vox), O.output_forward(vox, g).numpy())


def test_ssc_rulebook_and_forward(R):
    """SubmanifoldBuildObject + _dGenerateRulebook (CUDA/SubmanifoldRules_cuda.cpp:38-228, .cu:45-114); feature
    kernels: the chunk kernel for planes % 8 == 0, dConvolution_forward2 otherwise (CUDA/Convolution.cu:1001-1028,
    1068-1158, 1296-1395), and the CPU operator (CPU/Convolution.cpp:115-149)."""
    coords = scene(3, batch=2)
    rng = np.random.RandomState(4)
    m = R.Metadata()
    R.input_layer(m, SPATIAL, coords, np.zeros((coords.shape[0], 1), np.float32), 2, 4)
    g = O.Grid(coords)
    rules = O.ssc_rules(g)
    same_rulebook(m.ssc_rulebook(SPATIAL), rules)
    # (planes that are multiples of 8 but not of 16 are left out: the reference sends them to its chunk kernel, which
    # works in tiles of 16 planes -- input_nPlanes / 16 passes, output_nPlanes / 16 blocks -- and drops the rest)
    for n_in, n_out, bias in ((16, 16, False), (3, 32, True), (32, 48, True)):
        x = rng.randn(g.n, n_in).astype(np.float32)
        w = (rng.randn(27, n_in, n_out) * 0.2).astype(np.float32)
        b = rng.randn(n_out).astype(np.float32) if bias else None
        want = O.conv_forward(x, w, rules, g.n, b).numpy()
        got, flops = R.ssc(m, SPATIAL, x, w, b)
        assert rel(got, want) <= 1e-5, (n_in, n_out)
        got_cpu, flops_cpu = R.ssc(m, SPATIAL, x, w, b, cpu=True)
        assert rel(got_cpu, want) <= 1e-5
        assert flops_cpu == O.rule_flops(rules, n_in, n_out)


def test_stride2_rulebook_conv_and_deconv(R):
    """Convolution_InputSgToRulesAndOutputSg_FastDownSampleMode + _d_Convolution_GenerateOutputRules
    (Metadata/ConvolutionRules.h:344-380, CUDA/SubmanifoldRules_cuda.cu:744-840); dConvolution_KMxKN_forwardA/B and
    the deconvolution kernels (CUDA/Convolution.cu:81-253, CUDA/Deconvolution.cu:10-333); CPU operators."""
    coords = scene(5, batch=2)
    rng = np.random.RandomState(6)
    m = R.Metadata()
    R.input_layer(m, SPATIAL, coords, np.zeros((coords.shape[0], 1), np.float32), 2, 4)
    g = O.Grid(coords)
    coarse, rules = O.conv2_rules(g)
    same_rulebook(m.conv_rulebook(SPATIAL), rules)
    assert m.n_active(SPATIAL // 2) == coarse.n
    assert np.array_equal(m.spatial_locations(SPATIAL // 2), coarse.coords)
    same_rulebook(m.ssc_rulebook(SPATIAL // 2), O.ssc_rules(coarse))  # the coarse grid serves lookups too
    for n_in, n_out, bias in ((16, 32, False), (5, 7, True)):
        x = rng.randn(g.n, n_in).astype(np.float32)
        w = (rng.randn(8, n_in, n_out) * 0.3).astype(np.float32)
        b = rng.randn(n_out).astype(np.float32) if bias else None
        want = O.conv_forward(x, w, rules, coarse.n, b).numpy()
        assert rel(R.conv(m, SPATIAL, x, w, b)[0], want) <= 1e-5
        assert rel(R.conv(m, SPATIAL, x, w, b, cpu=True)[0], want) <= 1e-5
        xc = rng.randn(coarse.n, n_out).astype(np.float32)
        wd = (rng.randn(8, n_out, n_in) * 0.3).astype(np.float32)
        bd = rng.randn(n_in).astype(np.float32) if bias else None
        want = O.conv_forward(xc, wd, rules, g.n, bd, reverse=True).numpy()
        assert rel(R.deconv(m, SPATIAL // 2, xc, wd, bd)[0], want) <= 1e-5
        assert rel(R.deconv(m, SPATIAL // 2, xc, wd, bd, cpu=True)[0], want) <= 1e-5


def test_batchnorm_and_nin(R):
    """BatchNormalization_f_test / _f_train (CUDA/BatchNormalization.cu:14-107), CPU/BatchNormalization.cpp:13-62,
    NetworkInNetwork (CUDA/NetworkInNetwork.cpp:9-25, CPU/NetworkInNetwork.cpp:8-23)."""
    rng = np.random.RandomState(7)
    for planes in (32, 24):
        x = (rng.randn(300, planes) * 2 + 0.5).astype(np.float32)
        mean, var = rng.randn(planes).astype(np.float32), (rng.rand(planes) + 0.5).astype(np.float32)
        gamma, beta = rng.randn(planes).astype(np.float32), rng.randn(planes).astype(np.float32)
        for leak in (0.0, 0.333, 1.0):
            want = O.bn_forward(x, mean, var, gamma, beta, 1e-4, leak).numpy()
            assert rel(R.bn(x, mean, var, gamma, beta, 1e-4, leak), want) <= 1e-5
            assert rel(R.bn(x, mean, var, gamma, beta, 1e-4, leak, cpu=True), want) <= 1e-5
            assert rel(R.bn(x, mean, var, None, None, 1e-4, leak), O.bn_forward(x, mean, var, None, None, 1e-4, leak).numpy()) <= 1e-5
        want, rm, rv = O.bn_forward_train(x, mean, var, gamma, beta, 1e-4, 0.9, 0.0)
        for cpu in (False, True):
            got, grm, grv = R.bn(x, mean, var, gamma, beta, 1e-4, 0.0, train=True, momentum=0.9, cpu=cpu)
            assert rel(got, want.numpy()) <= 1e-4 and rel(grm, rm.numpy()) <= 1e-5 and rel(grv, rv.numpy()) <= 1e-4
    x = rng.randn(200, 64).astype(np.float32)
    w = (rng.randn(64, 32) * 0.2).astype(np.float32)
    b = rng.randn(32).astype(np.float32)
    for bias in (None, b):
        want = O.nin_forward(x, w, bias).numpy()
        assert rel(R.nin(x, w, bias)[0], want) <= 1e-5
        assert rel(R.nin(x, w, bias, cpu=True)[0], want) <= 1e-5


def incremental_frames(seed):
    """Frame t and the points of frame t+1: some fall into voxels of frame t, some open new voxels (next to old
    ones and far from them)."""
    coords = scene(seed)
    rng = np.random.RandomState(seed + 100)
    old = coords[rng.randint(0, coords.shape[0], 150)]
    near = coords[rng.randint(0, coords.shape[0], 200)].copy()
    near[:, :3] += rng.randint(-1, 2, size=(200, 3))
    far = np.concatenate([synth.sphere_surface([50, 50, 50], 5), np.zeros((0, 3), np.int64)], 0)
    far = np.concatenate([far, np.zeros((far.shape[0], 1), np.int64)], 1)
    new = np.concatenate([old, near, far], 0)
    new = new[rng.permutation(new.shape[0])]
    return coords, new


def test_incremental_maps_and_operators(R):
    """getPreExistMaps (Metadata/Metadata.cpp:609-626), IncreSubmanifoldBuildObject + _dGenerateIncreRulebook
    (CUDA/SubmanifoldRules_cuda.cpp:233-472, .cu:131-156), InputLayer_inc_fp_/_inc_bp_ (CUDA/IOLayers.cu:82-155),
    cuda_Incre_SubmanifoldConvolution_updateOutput (CUDA/Convolution.cpp:221-303), Incre_BatchNormalization_f_test
    (CUDA/BatchNormalization.cu:112-150), cuda_Incre_Convolution_updateOutput (CUDA/Convolution.cpp:83-113),
    cuda_Incre_Deconvolution_updateOutput (CUDA/Deconvolution.cpp:61-96, CUDA/Deconvolution.cu:82-155)."""
    coords, new = incremental_frames(11)
    rng = np.random.RandomState(12)
    feats = rng.randn(coords.shape[0], 16).astype(np.float32)
    new_feats = rng.randn(new.shape[0], 16).astype(np.float32)
    pre = R.Metadata()
    pre_vox = R.input_layer(pre, SPATIAL, coords, feats, 1, 4)
    pg = O.Grid(coords)
    m = R.Metadata()
    res = R.incre_input_layer(m, SPATIAL, new, new_feats, 1, 4, pre, pre_vox)
    g = O.Grid(new)
    assert np.array_equal(m.spatial_locations(SPATIAL), g.coords)
    pe = O.pre_exist(g, pg)
    assert (pe >= 0).any() and (pe < 0).any()
    assert np.array_equal(m.pre_exist(pre, SPATIAL), pe)
    want = O.incre_input_forward(new_feats, g, 4, pg, pre_vox).numpy()
    assert rel(res, want) <= 1e-5
    # rulebook of the saved neighbours of new sites
    same_rulebook(m.incre_ssc_rulebook(pre, SPATIAL), O.incre_ssc_rules(g, pg))
    # SSC: planes % 8 == 0 takes the chunk path, 3 -> 32 the flat rulebook path
    for n_in, n_out in ((16, 16), (3, 32)):
        x = rng.randn(g.n, n_in).astype(np.float32)
        px = rng.randn(pg.n, n_in).astype(np.float32)
        w = (rng.randn(27, n_in, n_out) * 0.2).astype(np.float32)
        want = O.incre_ssc_forward(x, w, g, pg, px).numpy()
        assert rel(R.incre_ssc(m, SPATIAL, x, w, None, pre, px)[0], want) <= 1e-5, (n_in, n_out)
    # BatchNorm + ReLU residual
    planes = 32
    x, px = rng.randn(g.n, planes).astype(np.float32), rng.randn(pg.n, planes).astype(np.float32)
    mean, var = rng.randn(planes).astype(np.float32), (rng.rand(planes) + 0.5).astype(np.float32)
    gamma, beta = rng.randn(planes).astype(np.float32), rng.randn(planes).astype(np.float32)
    py = O.bn_forward(px, mean, var, gamma, beta, 1e-4, 0.0).numpy()
    want = O.incre_bn_forward(x, mean, var, gamma, beta, 1e-4, 0.0, g, pg, py, px).numpy()
    assert rel(R.incre_bn(x, mean, var, gamma, beta, 1e-4, 0.0, m, pre, py, px, SPATIAL), want) <= 1e-5
    # stride-2 convolution of the residual = the plain operator on the incremental grid
    coarse, rules = O.conv2_rules(g)
    pcoarse, prules = O.conv2_rules(pg)
    R.conv(pre, SPATIAL, np.zeros((pg.n, 1), np.float32), np.zeros((8, 1, 1), np.float32))  # builds pre's coarse grid
    x = rng.randn(g.n, 16).astype(np.float32)
    w = (rng.randn(8, 16, 24) * 0.3).astype(np.float32)
    want = O.conv_forward(x, w, rules, coarse.n).numpy()
    assert rel(R.conv(m, SPATIAL, x, w, None, incremental=True)[0], want) <= 1e-5
    assert np.array_equal(m.pre_exist(pre, SPATIAL // 2), O.pre_exist(coarse, pcoarse))
    # deconvolution: residual rows, plus the saved coarse row where the coarse site existed and the fine site is new
    xc, pxc = rng.randn(coarse.n, 24).astype(np.float32), rng.randn(pcoarse.n, 24).astype(np.float32)
    wd = (rng.randn(8, 24, 16) * 0.3).astype(np.float32)
    want = O.incre_deconv_forward(xc, wd, g, coarse, rules, pg, pcoarse, pxc).numpy()
    assert rel(R.incre_deconv(m, SPATIAL // 2, xc, wd, None, pre, pxc)[0], want) <= 1e-5
    # OutputLayer: residual + saved full row
    vox, pvox = rng.randn(g.n, 8).astype(np.float32), rng.randn(pg.n, 8).astype(np.float32)
    want = O.incre_output_forward(vox, g, pg, pvox).numpy()
    assert rel(R.incre_output_layer(m, vox, pre, pvox), want) <= 1e-6


def test_label_fusion_equals_the_reference_classes(R):
    """Result<3> (votes with a confidence, with the default cap -- held as 0 by the reference's int member -- and with
    a cap of 3) and ResultOfWeight<3> over six frames of scores that revisit voxels with agreeing and disagreeing
    labels and name some voxels twice in one call: labels after every frame, every confidence, finalize, set."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from labels_cases import frames
    from oracle import scn_labels as L
    for maximum in (0.7, 3.0):
        scene, fr = frames(1)
        r, o = R.Result(maximum), L.Result(maximum)
        for ps, sc in fr:
            r.update(ps, sc)
            o.update(ps, sc)
            assert np.array_equal(r.multiQuery(scene), o.multiQuery(scene))
        assert r.size() == len(o.result)
        for k, (lab, conf) in o.result.items():
            assert r.confidence(*k) == float(conf), k
        got = r.get_all_points_labels()
        assert {tuple(v) for v in got.tolist()} == {tuple(v) for v in o.get_all_points_labels().tolist()}
        r.finalize(scene[::3])
        o.finalize(scene[::3])
        assert r.size() == len(o.result) and np.array_equal(r.multiQuery(scene), o.multiQuery(scene))
        r.set(scene[:40], fr[0][1][:40])
        o.set(scene[:40], fr[0][1][:40])
        assert np.array_equal(r.multiQuery(scene), o.multiQuery(scene))
        assert all(r.confidence(*[int(v) for v in p]) == 0.0 for p in scene[:40])
    rw, ow = R.ResultOfWeight(), L.ResultOfWeight()
    for ps, sc in fr:
        rw.update(ps, sc)
        ow.update(ps, sc)
        assert np.array_equal(rw.multiQuery(scene), ow.multiQuery(scene))
    rw.finalize(scene[:500])
    ow.finalize(scene[:500])
    assert rw.size() == len(ow.result) == 500 - int((ow.multiQuery(scene[:500]) < 0).sum())
