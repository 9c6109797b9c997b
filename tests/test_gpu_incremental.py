"""The incremental ("Incre_*") entry points of the C ABI, one operator at a time, against the CPU oracle (itself
pinned to the reference's Incre_* code by tests/test_oracle_vs_reference.py).

Integer results -- pre-exist maps and the incremental rulebooks -- must be bit-exact; fp32 outputs within 1e-4
relative; tf32 outputs within 2e-2 relative per operator."""
import numpy as np
import pytest
import torch

from insconv import cabi, synth
from oracle import scn_oracle as O

pytestmark = pytest.mark.gpu
TOL = {cabi.PREC_FP32: 1e-4, cabi.PREC_TF32: 2e-2}


def rel(got, want):
    want = torch.as_tensor(want)
    got = got.detach().cpu()
    assert got.shape == want.shape
    return float((got - want).abs().max()) / max(float(want.abs().max()), 1e-6)


def frames(seed, batches=1, duplicates=True):
    """Frame t and the points of frame t+1 (some in old voxels, some in new voxels beside old ones, some far away)."""
    rng = np.random.RandomState(seed)
    parts, new_parts = [], []
    for b in range(batches):
        c = synth.boxes_and_spheres(seed + b, grid=96)
        if duplicates:
            c = np.concatenate([c, c[rng.randint(0, c.shape[0], c.shape[0] // 5)]], 0)
        c = c[rng.permutation(c.shape[0])]
        near = c[rng.randint(0, c.shape[0], 3000)] + rng.randint(-1, 2, size=(3000, 3))
        near = np.clip(near, 1, 94)
        far = synth.sphere_surface([70 - 20 * b, 20, 75], 9)
        new = np.concatenate([c[rng.randint(0, c.shape[0], 2000)], near, far, far[:50]], 0)
        new = new[rng.permutation(new.shape[0])]
        if batches > 1:
            c = np.concatenate([c, np.full((c.shape[0], 1), b)], 1)
            new = np.concatenate([new, np.full((new.shape[0], 1), b)], 1)
        parts.append(c)
        new_parts.append(new)
    return np.concatenate(parts, 0).astype(np.int64), np.concatenate(new_parts, 0).astype(np.int64)


def build(cuda, coords, size=96):
    m = cabi.Metadata()
    m.input_layer_build(size, torch.from_numpy(coords).to(cuda), mode=4)
    return m


def same_rules(got, want):
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        np.testing.assert_array_equal(a, np.asarray(b).reshape(-1, 2), err_msg="offset %d" % k)


@pytest.mark.parametrize("batches", [1, 3])
def test_pre_exist_maps_and_incremental_rulebooks_bit_exact(cuda, batches):
    """Metadata::getPreExistMaps (Metadata/Metadata.cpp:609-626) and getIncreSubmanifoldRuleBook
    (Metadata.cpp:543-565; CUDA/SubmanifoldRules_cuda.cpp:233-472) at the input scale and one coarse scale."""
    coords, new = frames(4, batches)
    pre, m = build(cuda, coords), build(cuda, new)
    pg, g = O.Grid(coords), O.Grid(new)
    assert m.n_active(96) == g.n and g.n < new.shape[0]
    pe = O.pre_exist(g, pg)
    assert (pe >= 0).sum() > 100 and (pe < 0).sum() > 100
    np.testing.assert_array_equal(m.pre_exist(pre, 96), pe)
    want = O.incre_ssc_rules(g, pg)
    assert sum(len(r) for r in want) > 1000
    same_rules(m.incre_ssc_rulebook(pre, 96), want)
    # the next coarser scale: both metadata objects go down one stride-2 level
    pc, _ = O.conv2_rules(pg)
    c, _ = O.conv2_rules(g)
    pre.conv_rulebook(96, 48)
    m.conv_rulebook(96, 48)
    np.testing.assert_array_equal(m.pre_exist(pre, 48), O.pre_exist(c, pc))
    same_rules(m.incre_ssc_rulebook(pre, 48), O.incre_ssc_rules(c, pc))


def test_incremental_rulebook_of_a_frame_with_nothing_new_is_empty(cuda):
    coords, _ = frames(5)
    pre, m = build(cuda, coords), build(cuda, coords[:4000])
    assert (m.pre_exist(pre, 96) >= 0).all()
    assert sum(len(r) for r in m.incre_ssc_rulebook(pre, 96)) == 0


@pytest.mark.parametrize("precision", [cabi.PREC_FP32, cabi.PREC_TF32])
def test_incremental_operators_one_by_one(cuda, precision):
    """InputLayer_inc_fp_ / _inc_bp_ (CUDA/IOLayers.cu:82-155), cuda_Incre_SubmanifoldConvolution_updateOutput
    (CUDA/Convolution.cpp:221-303), Incre_BatchNormalization_f_test (CUDA/BatchNormalization.cu:112-150),
    cuda_Incre_Convolution_updateOutput (CUDA/Convolution.cpp:83-113), cuda_Incre_Deconvolution_updateOutput
    (CUDA/Deconvolution.cpp:61-96)."""
    tol = TOL[precision]
    coords, new = frames(6)
    rng = np.random.RandomState(9)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(cuda)
    pre, m = build(cuda, coords), build(cuda, new)
    pg, g = O.Grid(coords), O.Grid(new)
    # input layer residual (fp32 arithmetic in both precisions: no tensor cores involved)
    feats, new_feats = rng.randn(coords.shape[0], 16).astype(np.float32), rng.randn(new.shape[0], 16).astype(np.float32)
    pre_vox = pre.input_forward(t(feats))
    assert rel(pre_vox, O.input_forward(feats, pg, 4)) <= 1e-5
    pre_vox_o = O.input_forward(feats, pg, 4)
    res = m.incre_input_forward(pre, t(new_feats), pre_vox)
    assert rel(res, O.incre_input_forward(new_feats, g, 4, pg, pre_vox_o)) <= 1e-4
    # submanifold convolution: narrow (warp-level kernel in tf32), wide (tcgen05), ragged planes, with bias
    for n_in, n_out, bias in ((16, 16, False), (32, 64, True), (96, 96, False), (3, 32, False)):
        x, px = rng.randn(g.n, n_in).astype(np.float32), rng.randn(pg.n, n_in).astype(np.float32)
        w = synth.kaiming_uniform(rng, 27, n_in, n_out)
        b = rng.randn(n_out).astype(np.float32) if bias else None
        want = O.incre_ssc_forward(x, w, g, pg, px, b)
        got, flops = m.incre_ssc_forward(pre, 96, t(x), t(w), t(px), t(b) if bias else None, precision)
        assert rel(got, want) <= tol, (n_in, n_out)
        assert flops == O.rule_flops(O.ssc_rules(g), n_in, n_out) + O.rule_flops(O.incre_ssc_rules(g, pg), n_in, n_out)
    # BatchNorm + ReLU / leaky / none
    for planes, leak in ((32, 0.0), (96, 0.333), (5, 1.0)):
        x, px = rng.randn(g.n, planes).astype(np.float32), rng.randn(pg.n, planes).astype(np.float32)
        mean, var = rng.randn(planes).astype(np.float32), rng.uniform(0.5, 2, planes).astype(np.float32)
        gamma, beta = rng.randn(planes).astype(np.float32), rng.randn(planes).astype(np.float32)
        py = O.bn_forward(px, mean, var, gamma, beta, 1e-4, leak)
        want = O.incre_bn_forward(x, mean, var, gamma, beta, 1e-4, leak, g, pg, py, px)
        got = m.incre_bn_forward(pre, 96, t(x), t(mean), t(var), t(gamma), t(beta), 1e-4, leak, t(py.numpy()), t(px))
        assert rel(got, want) <= 1e-4
    # stride-2 convolution of the residual, then the incremental deconvolution back
    coarse, rules = O.conv2_rules(g)
    pcoarse, _ = O.conv2_rules(pg)
    pre.conv_rulebook(96, 48)
    for n_in, n_out in ((32, 64), (96, 128), (3, 5)):
        x = rng.randn(g.n, n_in).astype(np.float32)
        w = synth.kaiming_uniform(rng, 8, n_in, n_out)
        got, _ = m.conv_forward(96, 48, t(x), t(w), None, precision)
        assert rel(got, O.conv_forward(x, w, rules, coarse.n)) <= tol
        xc, pxc = rng.randn(coarse.n, n_out).astype(np.float32), rng.randn(pcoarse.n, n_out).astype(np.float32)
        wd = synth.kaiming_uniform(rng, 8, n_out, n_in)
        want = O.incre_deconv_forward(xc, wd, g, coarse, rules, pg, pcoarse, pxc)
        got, _ = m.incre_deconv_forward(pre, 48, 96, t(xc), t(wd), t(pxc), None, precision)
        assert rel(got, want) <= tol, (n_in, n_out)
    # output layer: residual + saved full row
    vox, pvox = rng.randn(g.n, 20).astype(np.float32), rng.randn(pg.n, 20).astype(np.float32)
    got = m.incre_output_forward(pre, t(vox), t(pvox))
    assert rel(got, O.incre_output_forward(vox, g, pg, pvox)) <= 1e-6
    cabi.check_errors()


def test_incremental_operators_on_fp16_rows(cuda):
    """SCN_PREC_F16 in the incremental operators: residual rows and saved rows are fp16 (as a BatchNorm in front of the
    layer writes them), weights are the fp16 pack; the incremental BatchNorm writes its residual as fp16 rows and reads
    the saved frame's output as fp16 rows.  Against the oracle's formulas on the same fp16-rounded inputs."""
    import ctypes as C
    stream = torch.cuda.current_stream().cuda_stream
    coords, new = frames(7)
    rng = np.random.RandomState(11)
    pre, m = build(cuda, coords), build(cuda, new)
    pg, g = O.Grid(coords), O.Grid(new)
    h = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(cuda).half()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(cuda)

    def packed(w):
        p = torch.empty(cabi.lib().scn_packed_size_f16(w.shape[0], w.shape[1], w.shape[2]), dtype=torch.float16, device=cuda)
        dw = t(w)
        cabi.call("scn_pack_weights_f16", cabi.ptr(dw), w.shape[0], w.shape[1], w.shape[2], cabi.ptr(p), stream)
        torch.cuda.synchronize()
        return p

    fl = C.c_double(0)
    for n_in, n_out in ((32, 32), (64, 32), (96, 96), (128, 160)):  # warp-level kernels, slab kernel
        x, px = h(rng.randn(g.n, n_in)), h(rng.randn(pg.n, n_in))
        w = synth.kaiming_uniform(rng, 27, n_in, n_out)
        want = O.incre_ssc_forward(x.float().cpu().numpy(), w, g, pg, px.float().cpu().numpy(), None)
        out = torch.empty(g.n, n_out, dtype=torch.float32, device=cuda)
        pw = packed(w)
        cabi.call("scn_incre_ssc_forward", m.h, pre.h, cabi.size3(96), cabi.ptr(x), n_in, cabi.ptr(out), n_out, cabi.ptr(pw), None,
                  cabi.ptr(px), n_in, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
        assert rel(out, want) <= 2e-2, (n_in, n_out)
        assert fl.value == O.rule_flops(O.ssc_rules(g), n_in, n_out) + O.rule_flops(O.incre_ssc_rules(g, pg), n_in, n_out)
        # with the maps cached, both gathers (changed neighbours, saved neighbours of new sites) are ONE launch
        assert sum(len(r) for r in O.incre_ssc_rules(g, pg)) > 0
        l0 = cabi.lib().scn_launch_count()
        cabi.call("scn_incre_ssc_forward", m.h, pre.h, cabi.size3(96), cabi.ptr(x), n_in, cabi.ptr(out), n_out, cabi.ptr(pw), None,
                  cabi.ptr(px), n_in, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
        assert cabi.lib().scn_launch_count() - l0 == 1, (n_in, n_out)
        assert rel(out, want) <= 2e-2, (n_in, n_out)
    # BatchNorm residual as fp16 rows
    for planes, leak in ((32, 0.0), (96, 0.333)):
        x, px = rng.randn(g.n, planes).astype(np.float32), rng.randn(pg.n, planes).astype(np.float32)
        mean, var = rng.randn(planes).astype(np.float32), rng.uniform(0.5, 2, planes).astype(np.float32)
        gamma, beta = rng.randn(planes).astype(np.float32), rng.randn(planes).astype(np.float32)
        py = h(O.bn_forward(px, mean, var, gamma, beta, 1e-4, leak).numpy())  # what the saved frame wrote
        want = O.incre_bn_forward(x, mean, var, gamma, beta, 1e-4, leak, g, pg, py.float().cpu(), px)
        out = torch.empty(g.n, planes, dtype=torch.float16, device=cuda)
        dx, dpx, dm, dv, dg, db = t(x), t(px), t(mean), t(var), t(gamma), t(beta)
        cabi.call("scn_incre_bn_forward_f16", m.h, pre.h, cabi.size3(96), cabi.ptr(dx), planes, cabi.ptr(out), planes, planes,
                  cabi.ptr(dm), cabi.ptr(dv), cabi.ptr(dg), cabi.ptr(db), 1e-4, leak, cabi.ptr(py), planes, cabi.ptr(dpx), planes,
                  stream)
        torch.cuda.synchronize()
        assert rel(out.float(), want) <= 2e-3
    # incremental deconvolution on fp16 rows
    coarse, rules = O.conv2_rules(g)
    pcoarse, _ = O.conv2_rules(pg)
    pre.conv_rulebook(96, 48)
    m.conv_rulebook(96, 48)
    for n_in, n_out in ((64, 32), (128, 96)):
        xc, pxc = h(rng.randn(coarse.n, n_in)), h(rng.randn(pcoarse.n, n_in))
        wd = synth.kaiming_uniform(rng, 8, n_in, n_out)
        want = O.incre_deconv_forward(xc.float().cpu().numpy(), wd, g, coarse, rules, pg, pcoarse, pxc.float().cpu().numpy())
        out = torch.empty(g.n, n_out, dtype=torch.float32, device=cuda)
        pw = packed(wd)
        cabi.call("scn_incre_deconv_forward", m.h, pre.h, cabi.size3(48), cabi.size3(96), cabi.ptr(xc), n_in, cabi.ptr(out), n_out,
                  cabi.ptr(pw), None, cabi.ptr(pxc), n_in, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
        assert rel(out, want) <= 2e-2, (n_in, n_out)
    cabi.check_errors()


def test_incremental_batchnorm_in_the_convolution_epilogue(cuda):
    """scn_incre_ssc_forward_ex / scn_incre_conv_forward_ex with the incremental BatchNorm (and a residual addend) in the
    epilogue against the same operators followed by scn_incre_bn_forward_f16: equal fp32 results, fp16 rows equal to
    rounding (the warp-level kernel at 32 planes, the slab kernel at 96, the tcgen05 kernel -- which runs the BatchNorm as
    a launch of its own inside the library -- for the stride-2 convolution 64 -> 96)."""
    import ctypes as C
    stream = torch.cuda.current_stream().cuda_stream
    coords, new = frames(8)
    rng = np.random.RandomState(12)
    pre, m = build(cuda, coords), build(cuda, new)
    pg, g = O.Grid(coords), O.Grid(new)
    h = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(cuda).half()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(cuda)

    def packed(w):
        p = torch.empty(cabi.lib().scn_packed_size_f16(w.shape[0], w.shape[1], w.shape[2]), dtype=torch.float16, device=cuda)
        dw = t(w)
        cabi.call("scn_pack_weights_f16", cabi.ptr(dw), w.shape[0], w.shape[1], w.shape[2], cabi.ptr(p), stream)
        torch.cuda.synchronize()
        return p

    fl = C.c_double(0)
    for n_in, n_out in ((32, 32), (96, 96)):
        x, px = h(rng.randn(g.n, n_in)), h(rng.randn(pg.n, n_in))
        pw = packed(synth.kaiming_uniform(rng, 27, n_in, n_out))
        addend = t(rng.randn(g.n, n_out))
        scale, shift = t(rng.uniform(0.5, 1.5, n_out)), t(rng.randn(n_out))
        saved_in, saved_out = t(rng.randn(pg.n, n_out)), h(rng.randn(pg.n, n_out))
        raw = torch.empty(g.n, n_out, dtype=torch.float32, device=cuda)
        rows = torch.empty(g.n, n_out, dtype=torch.float16, device=cuda)
        epi = cabi.Epilogue(cabi.ptr(addend), n_out, cabi.ptr(scale), cabi.ptr(shift), 0.0, cabi.ptr(rows), n_out, 0,
                            cabi.ptr(saved_in), n_out, cabi.ptr(saved_out), n_out)
        cabi.call("scn_incre_ssc_forward_ex", m.h, pre.h, cabi.size3(96), cabi.ptr(x), n_in, cabi.ptr(raw), n_out, cabi.ptr(pw), None,
                  cabi.ptr(px), n_in, n_in, n_out, cabi.PREC_F16, C.byref(epi), stream, C.byref(fl))
        plain = torch.empty_like(raw)
        cabi.call("scn_incre_ssc_forward", m.h, pre.h, cabi.size3(96), cabi.ptr(x), n_in, cabi.ptr(plain), n_out, cabi.ptr(pw), None,
                  cabi.ptr(px), n_in, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
        want_raw = plain + addend
        assert float((raw - want_raw).abs().max()) <= 1e-5 * float(want_raw.abs().max())
        # the BatchNorm kernel with scale/shift as gamma/beta on zero mean, unit variance, eps 0
        want_rows = torch.empty_like(rows)
        zero, one = torch.zeros(n_out, device=cuda), torch.ones(n_out, device=cuda)
        cabi.call("scn_incre_bn_forward_f16", m.h, pre.h, cabi.size3(96), cabi.ptr(want_raw), n_out, cabi.ptr(want_rows), n_out, n_out,
                  cabi.ptr(zero), cabi.ptr(one), cabi.ptr(scale), cabi.ptr(shift), 0.0, 0.0, cabi.ptr(saved_out), n_out,
                  cabi.ptr(saved_in), n_out, stream)
        torch.cuda.synchronize()
        assert float((rows.float() - want_rows.float()).abs().max()) <= 2e-3 * float(want_rows.float().abs().max())
    # stride-2 convolution of the residual with the incremental BatchNorm of the coarse scale
    pre.conv_rulebook(96, 48)
    n_c = C.c_int64(0)
    cabi.call("scn_conv_prepare", m.h, cabi.size3(96), cabi.size3(48), stream, C.byref(n_c))
    n_c, n_pc = int(n_c.value), pre.n_active(48)
    for n_in, n_out in ((32, 64), (64, 96)):
        x = h(rng.randn(g.n, n_in))
        pw = packed(synth.kaiming_uniform(rng, 8, n_in, n_out))
        scale, shift = t(rng.uniform(0.5, 1.5, n_out)), t(rng.randn(n_out))
        saved_in, saved_out = t(rng.randn(n_pc, n_out)), h(rng.randn(n_pc, n_out))
        raw = torch.empty(n_c, n_out, dtype=torch.float32, device=cuda)
        rows = torch.empty(n_c, n_out, dtype=torch.float16, device=cuda)
        epi = cabi.Epilogue(None, 0, cabi.ptr(scale), cabi.ptr(shift), 0.0, cabi.ptr(rows), n_out, 0, cabi.ptr(saved_in), n_out,
                            cabi.ptr(saved_out), n_out)
        cabi.call("scn_incre_conv_forward_ex", m.h, pre.h, cabi.size3(96), cabi.size3(48), cabi.ptr(x), n_in, cabi.ptr(raw), n_out,
                  cabi.ptr(pw), None, n_in, n_out, cabi.PREC_F16, C.byref(epi), stream, C.byref(fl))
        plain = torch.empty_like(raw)
        cabi.call("scn_conv_forward", m.h, cabi.size3(96), cabi.size3(48), cabi.ptr(x), n_in, cabi.ptr(plain), n_out, cabi.ptr(pw),
                  None, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
        assert float((raw - plain).abs().max()) <= 1e-5 * float(plain.abs().max())
        want_rows = torch.empty_like(rows)
        zero, one = torch.zeros(n_out, device=cuda), torch.ones(n_out, device=cuda)
        cabi.call("scn_incre_bn_forward_f16", m.h, pre.h, cabi.size3(48), cabi.ptr(plain), n_out, cabi.ptr(want_rows), n_out, n_out,
                  cabi.ptr(zero), cabi.ptr(one), cabi.ptr(scale), cabi.ptr(shift), 0.0, 0.0, cabi.ptr(saved_out), n_out,
                  cabi.ptr(saved_in), n_out, stream)
        torch.cuda.synchronize()
        assert float((rows.float() - want_rows.float()).abs().max()) <= 2e-3 * float(want_rows.float().abs().max())
    # the saved-row fields belong to the incremental operators
    with pytest.raises(cabi.ScnError):
        cabi.call("scn_ssc_forward_ex", m.h, cabi.size3(96), cabi.ptr(x), n_in, cabi.ptr(raw), n_out, cabi.ptr(pw), None, n_in, n_out,
                  cabi.PREC_F16, C.byref(epi), stream, C.byref(fl))
    cabi.check_errors()
