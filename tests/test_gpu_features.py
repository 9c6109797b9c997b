"""Feature kernels through the C ABI vs the CPU oracle.

Tolerances: fp32 outputs within 1e-4 relative, the parity bar for fp32; the metric used
is max|a-b| / max(|b|_max, 1e-6) per tensor plus an element-wise allclose with rtol = atol = 1e-4.
"""
import numpy as np
import pytest
import torch

from insconv import cabi, synth
from oracle import scn_oracle as O

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-4


def close(got, want, tol=FP32_TOL):
    got = got.detach().cpu()
    want = torch.as_tensor(want)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.numel() == 0:
        return
    scale = max(float(want.abs().max()), 1e-6)
    err = float((got - want).abs().max()) / scale
    assert err <= tol, "relative error %.3g > %.1g" % (err, tol)
    assert torch.allclose(got, want, rtol=tol, atol=tol * scale)


def _scene(cuda, seed=0, size=128):
    c = synth.boxes_and_spheres(seed, grid=size)
    m = cabi.Metadata()
    n = m.input_layer_build(size, torch.from_numpy(c).to(cuda), mode=4)
    g = O.Grid(c)
    assert n == g.n
    return m, g


@pytest.mark.parametrize("n_in,n_out,bias", [(16, 16, False), (3, 32, False), (32, 32, True), (64, 32, False),
                                             (32, 64, True), (96, 96, False), (5, 7, True), (224, 224, False)])
def test_ssc_forward(cuda, n_in, n_out, bias):
    m, g = _scene(cuda, 0)
    rng = np.random.RandomState(n_in * 1000 + n_out)
    x = rng.randn(g.n, n_in).astype(np.float32)
    w = synth.kaiming_uniform(rng, 27, n_in, n_out)
    b = rng.randn(n_out).astype(np.float32) if bias else None
    rules = O.ssc_rules(g)
    want = O.conv_forward(x, w, rules, g.n, b)
    got, flops = m.ssc_forward(128, torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda),
                               torch.from_numpy(b).to(cuda) if bias else None)
    close(got, want)
    assert flops == O.rule_flops(rules, n_in, n_out)


@pytest.mark.parametrize("n_in,n_out", [(32, 64), (16, 16), (3, 5), (96, 128)])
def test_conv_deconv_forward(cuda, n_in, n_out):
    m, g = _scene(cuda, 1)
    rng = np.random.RandomState(7)
    coarse, rules = O.conv2_rules(g)
    x = rng.randn(g.n, n_in).astype(np.float32)
    w = synth.kaiming_uniform(rng, 8, n_in, n_out)
    b = rng.randn(n_out).astype(np.float32)
    want = O.conv_forward(x, w, rules, coarse.n, b)
    got, flops = m.conv_forward(128, 64, torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda),
                                torch.from_numpy(b).to(cuda))
    close(got, want)
    assert flops == O.rule_flops(rules, n_in, n_out)
    # deconvolution back to the fine scale with the same rulebook, pair reversed
    wd = synth.kaiming_uniform(rng, 8, n_out, n_in)
    y = rng.randn(coarse.n, n_out).astype(np.float32)
    want = O.conv_forward(y, wd, rules, g.n, None, reverse=True)
    got, _ = m.deconv_forward(64, 128, torch.from_numpy(y).to(cuda), torch.from_numpy(wd).to(cuda))
    close(got, want)


@pytest.mark.parametrize("planes,leak", [(32, 0.0), (3, 0.333), (224, 0.0), (17, 1.0)])
def test_bn_forward(cuda, planes, leak):
    rng = np.random.RandomState(planes)
    x = rng.randn(5003, planes).astype(np.float32)
    mean = rng.randn(planes).astype(np.float32)
    var = rng.uniform(0.5, 2.0, planes).astype(np.float32)
    gamma = rng.randn(planes).astype(np.float32)
    beta = rng.randn(planes).astype(np.float32)
    want = O.bn_forward(x, mean, var, gamma, beta, 1e-4, leak)
    t = lambda a: torch.from_numpy(a).to(cuda)
    got = cabi.bn_forward(t(x), t(mean), t(var), t(gamma), t(beta), 1e-4, leak)
    close(got, want, 1e-5)
    got = cabi.bn_forward(t(x), t(mean), t(var), None, None, 1e-4, leak)
    close(got, O.bn_forward(x, mean, var, None, None, 1e-4, leak), 1e-5)


@pytest.mark.parametrize("pa,pb,leak", [(32, 32, 0.0), (224, 224, 0.0), (64, 96, 0.333), (4, 8, 1.0)])
def test_join_then_batchnorm_in_one_pass(cuda, pa, pb, leak):
    """scn_join_bn_forward_f16: the joined fp32 rows bit for bit, the BatchNorm of the joined rows (the oracle's formula
    on the concatenation, scale / shift as the modules derive them) as fp16 rows to fp16 rounding."""
    rng = np.random.RandomState(pa + pb)
    rows = 5003
    a, b = rng.randn(rows, pa).astype(np.float32), rng.randn(rows, pb).astype(np.float32)
    planes = pa + pb
    mean, var = rng.randn(planes).astype(np.float32), rng.uniform(0.5, 2.0, planes).astype(np.float32)
    gamma, beta = rng.randn(planes).astype(np.float32), rng.randn(planes).astype(np.float32)
    scale = (gamma / np.sqrt(var + 1e-4)).astype(np.float32)
    shift = (beta - mean * scale).astype(np.float32)
    t = lambda x: torch.from_numpy(x).to(cuda)
    da, db, dsc, dsh = t(a), t(b), t(scale), t(shift)
    joined = torch.empty(rows, planes, dtype=torch.float32, device=cuda)
    half = torch.empty(rows, planes, dtype=torch.float16, device=cuda)
    cabi.call("scn_join_bn_forward_f16", cabi.ptr(da), pa, pa, cabi.ptr(db), pb, pb, rows, cabi.ptr(joined), planes, cabi.ptr(dsc),
              cabi.ptr(dsh), leak, cabi.ptr(half), planes, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    cat = np.concatenate([a, b], 1)
    assert np.array_equal(joined.cpu().numpy(), cat)
    want = O.bn_forward(cat, mean, var, gamma, beta, 1e-4, leak).numpy()
    got = half.float().cpu().numpy()
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max() + 1e-6


@pytest.mark.parametrize("n_in,n_out,bias", [(64, 32, False), (6, 3, True), (448, 224, False)])
def test_nin_forward(cuda, n_in, n_out, bias):
    rng = np.random.RandomState(n_in)
    x = rng.randn(4099, n_in).astype(np.float32)
    w = (rng.randn(n_in, n_out) * np.sqrt(2.0 / n_in)).astype(np.float32)
    b = rng.randn(n_out).astype(np.float32) if bias else None
    t = lambda a: torch.from_numpy(a).to(cuda)
    got, flops = cabi.nin_forward(t(x), t(w), t(b) if bias else None)
    close(got, O.nin_forward(x, w, b))
    assert flops == 4099.0 * n_in * n_out


@pytest.mark.parametrize("mode", [3, 4])
def test_input_output_layers(cuda, mode):
    rng = np.random.RandomState(11)
    c = rng.randint(1, 30, size=(30000, 3))
    f = rng.randn(30000, 3).astype(np.float32)
    m = cabi.Metadata()
    m.input_layer_build(32, torch.from_numpy(c).to(cuda), mode=mode)
    g = O.Grid(c)
    vox = m.input_forward(torch.from_numpy(f).to(cuda))
    close(vox, O.input_forward(f, g, mode), 1e-5)
    h = rng.randn(g.n, 32).astype(np.float32)
    pts = m.output_forward(torch.from_numpy(h).to(cuda))
    assert torch.equal(pts.cpu(), O.output_forward(h, g))
    h3 = rng.randn(g.n, 3).astype(np.float32)  # a plane count that is not a multiple of 4: the scalar kernel
    assert torch.equal(m.output_forward(torch.from_numpy(h3).to(cuda)).cpu(), O.output_forward(h3, g))


def test_linearity_at_full_size(cuda):
    # size-independent property on the 250k-voxel room: SSC(a*x + y) == a*SSC(x) + SSC(y)
    c = synth.room(0)
    m = cabi.Metadata()
    n = m.input_layer_build(4096, torch.from_numpy(c).to(cuda), mode=4)
    assert n == c.shape[0]
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(n, 32, generator=g).to(cuda)
    y = torch.randn(n, 32, generator=g).to(cuda)
    w = (torch.randn(27, 32, 32, generator=g) * 0.05).to(cuda)
    a, _ = m.ssc_forward(4096, 2.5 * x + y, w)
    b1, _ = m.ssc_forward(4096, x, w)
    b2, _ = m.ssc_forward(4096, y, w)
    close(a, (2.5 * b1 + b2).cpu(), 1e-4)
    # and the centre-only filter is a plain matmul
    w0 = torch.zeros_like(w)
    w0[13] = w[13]
    c0, _ = m.ssc_forward(4096, x, w0)
    close(c0, (x @ w[13]).cpu(), 1e-4)


# ---- tensor-core (tf32) paths, tcgen05 and warp-level: 2e-2 relative per layer -------------------------------------
TF32_TOL = 2e-2


@pytest.mark.parametrize("n_in,n_out,bias", [(3, 32, True), (1, 16, False), (4, 64, False), (16, 16, False), (32, 32, False), (64, 32, True), (32, 64, False),
                                             (64, 64, True), (16, 64, False), (64, 16, True), (96, 96, True),
                                             (224, 224, False), (448, 224, False)])
def test_ssc_forward_tf32(cuda, n_in, n_out, bias):
    m, g = _scene(cuda, 0)
    rng = np.random.RandomState(n_in * 1000 + n_out + 1)
    x = rng.randn(g.n, n_in).astype(np.float32)
    w = synth.kaiming_uniform(rng, 27, n_in, n_out)
    b = rng.randn(n_out).astype(np.float32) if bias else None
    want = O.conv_forward(x, w, O.ssc_rules(g), g.n, b)
    got, _ = m.ssc_forward(128, torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda),
                           torch.from_numpy(b).to(cuda) if bias else None, precision=cabi.PREC_TF32)
    cabi.check_errors()
    close(got, want, TF32_TOL)
    # tf32 keeps 10 mantissa bits: the error should in fact be far below the stated bar
    err = float((got.cpu() - want).abs().max()) / float(want.abs().max())
    assert err < 5e-3, err


@pytest.mark.parametrize("n_in,n_out,prec", [(32, 32, "fp32"), (32, 32, "tf32"), (64, 32, "tf32"), (96, 96, "tf32"),
                                             (224, 224, "tf32"), (3, 32, "tf32")])
def test_ssc_forward_add(cuda, n_in, n_out, prec):
    # out = addend + convolution, formed in the epilogue (direct, split-K reduction and warp-level kernels)
    m, g = _scene(cuda, 3)
    rng = np.random.RandomState(n_in + n_out)
    x = torch.from_numpy(rng.randn(g.n, n_in).astype(np.float32)).to(cuda)
    w = torch.from_numpy(synth.kaiming_uniform(rng, 27, n_in, n_out)).to(cuda)
    base = torch.from_numpy(rng.randn(g.n, n_out + 4).astype(np.float32)).to(cuda)[:, :n_out]  # strided rows
    p = cabi.PREC_TF32 if prec == "tf32" else cabi.PREC_FP32
    plain, fl0 = m.ssc_forward(128, x, w, None, p)
    got, fl1 = m.ssc_forward_add(128, x, w, base, p)
    cabi.check_errors()
    assert fl0 == fl1
    want = plain + base
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())


@pytest.mark.parametrize("n_in,n_out", [(32, 32), (32, 64), (64, 32), (64, 64), (96, 96), (64, 96), (160, 128), (96, 32),
                                        (224, 224)])
def test_f16_activations_bn_then_convolutions(cuda, n_in, n_out):
    # BatchNorm+ReLU writing fp16 rows, then SSC / stride-2 convolution / deconvolution reading them (warp-level fp16
    # kernel for 32/64 planes, tcgen05 kind::f16 kernel above, with n_in padded to a multiple of 64), against the
    # oracle's fp32 result of the same two layers
    import ctypes as C
    m, g = _scene(cuda, 1)
    rng = np.random.RandomState(n_in * 7 + n_out)
    stream = torch.cuda.current_stream().cuda_stream
    t = lambda a: torch.from_numpy(a).to(cuda)

    def bn_f16(x, planes):
        mean, var = rng.randn(planes).astype(np.float32), rng.uniform(0.5, 2, planes).astype(np.float32)
        gamma, beta = rng.randn(planes).astype(np.float32), rng.randn(planes).astype(np.float32)
        want = torch.as_tensor(O.bn_forward(x, mean, var, gamma, beta, 1e-4, 0.0)).numpy()
        xd, dm, dv, dg, db = t(x), t(mean), t(var), t(gamma), t(beta)  # kept alive until the kernel has run
        out = torch.empty(x.shape[0], planes, dtype=torch.float16, device=cuda)
        cabi.call("scn_bn_forward_f16", cabi.ptr(xd), planes, cabi.ptr(out), planes, x.shape[0], planes, cabi.ptr(dm),
                  cabi.ptr(dv), cabi.ptr(dg), cabi.ptr(db), 1e-4, 0.0, stream)
        torch.cuda.synchronize()
        assert float(np.abs(out.float().cpu().numpy() - want).max()) <= 1e-3 * float(np.abs(want).max())
        return out, want

    def packed(w):
        size = cabi.lib().scn_packed_size_f16(w.shape[0], w.shape[1], w.shape[2])
        assert size >= w.size
        p = torch.empty(size, dtype=torch.float16, device=cuda)
        dw = t(w)
        cabi.call("scn_pack_weights_f16", cabi.ptr(dw), w.shape[0], w.shape[1], w.shape[2], cabi.ptr(p), stream)
        torch.cuda.synchronize()
        return p

    assert cabi.lib().scn_weights_packable_f16(27, n_in, n_out) == 1 and cabi.lib().scn_weights_packable_f16(27, 48, 96) == 0
    assert cabi.lib().scn_weights_packable_f16(27, 256, 256) == 0
    fl = C.c_double(0)
    # submanifold convolution
    h, ref = bn_f16(rng.randn(g.n, n_in).astype(np.float32), n_in)
    w = synth.kaiming_uniform(rng, 27, n_in, n_out)
    out = torch.empty(g.n, n_out, dtype=torch.float32, device=cuda)
    pw = packed(w)
    cabi.call("scn_ssc_forward", m.h, cabi.size3(128), cabi.ptr(h), n_in, cabi.ptr(out), n_out, cabi.ptr(pw), None, n_in,
              n_out, cabi.PREC_F16, stream, C.byref(fl))
    torch.cuda.synchronize()
    want = torch.as_tensor(O.conv_forward(ref, w, O.ssc_rules(g), g.n, None))
    close(out, want, TF32_TOL)
    assert float((out.cpu() - want).abs().max()) / float(want.abs().max()) < 3e-3
    # stride-2 convolution and deconvolution
    coarse, rules = O.conv2_rules(g)
    w8 = synth.kaiming_uniform(rng, 8, n_in, n_out)
    pw8 = packed(w8)
    n_cc = C.c_int64(0)
    cabi.call("scn_conv_prepare", m.h, cabi.size3(128), cabi.size3(64), stream, C.byref(n_cc))
    n_c = int(n_cc.value)
    assert n_c == coarse.n
    out = torch.empty(n_c, n_out, dtype=torch.float32, device=cuda)
    cabi.call("scn_conv_forward", m.h, cabi.size3(128), cabi.size3(64), cabi.ptr(h), n_in, cabi.ptr(out), n_out,
              cabi.ptr(pw8), None, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
    close(out, O.conv_forward(ref, w8, rules, coarse.n, None), TF32_TOL)
    hc, refc = bn_f16(rng.randn(coarse.n, n_in).astype(np.float32), n_in)
    out = torch.empty(g.n, n_out, dtype=torch.float32, device=cuda)
    cabi.call("scn_deconv_forward", m.h, cabi.size3(64), cabi.size3(128), cabi.ptr(hc), n_in, cabi.ptr(out), n_out,
              cabi.ptr(pw8), None, n_in, n_out, cabi.PREC_F16, stream, C.byref(fl))
    close(out, O.conv_forward(refc, w8, rules, g.n, None, reverse=True), TF32_TOL)
    cabi.check_errors()


def test_f16_rows_saturate_instead_of_overflowing(cuda):
    """Activations beyond the fp16 range (|y| > 65504) are written as +-65504, never as infinity, both by the
    BatchNorm kernel that writes fp16 rows and by the convolution epilogue that applies a BatchNorm; NaN-free
    downstream.  Leakiness 1 (no activation) keeps the negative side large too."""
    import ctypes as C
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.RandomState(4)
    n, planes = 4096, 32
    x = (rng.randn(n, planes) * 1e5).astype(np.float32)  # a third of the entries beyond +-65504
    one, zero = torch.ones(planes, device=cuda), torch.zeros(planes, device=cuda)
    xd = torch.from_numpy(x).to(cuda)
    out = torch.empty(n, planes, dtype=torch.float16, device=cuda)
    cabi.call("scn_bn_forward_f16", cabi.ptr(xd), planes, cabi.ptr(out), planes, n, planes, cabi.ptr(zero), cabi.ptr(one),
              cabi.ptr(one), cabi.ptr(zero), 0.0, 1.0, stream)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all() and got.max() == 65504.0 and got.min() == -65504.0
    inside = np.abs(x) < 6e4
    assert np.abs(got[inside] - x[inside]).max() <= 1e-3 * 6e4
    assert (np.abs(got[np.abs(x) > 65504]) == 65504.0).all()
    # the same through a convolution epilogue: an SSC that only has its centre offset, rows of size ~100 times 1000
    m, g = _scene(cuda, 1)
    h = torch.from_numpy((rng.randn(g.n, planes) * 100).astype(np.float32)).to(cuda).half()
    w = np.zeros((27, planes, planes), np.float32)
    w[13] = np.eye(planes) * 1000
    dw = torch.from_numpy(w).to(cuda)
    pw = torch.empty(cabi.lib().scn_packed_size_f16(27, planes, planes), dtype=torch.float16, device=cuda)
    cabi.call("scn_pack_weights_f16", cabi.ptr(dw), 27, planes, planes, cabi.ptr(pw), stream)
    raw = torch.empty(g.n, planes, dtype=torch.float32, device=cuda)
    rows = torch.empty(g.n, planes, dtype=torch.float16, device=cuda)
    epi = cabi.Epilogue(None, 0, cabi.ptr(one), cabi.ptr(zero), 1.0, cabi.ptr(rows), planes, 0)
    fl = C.c_double(0)
    cabi.call("scn_ssc_forward_ex", m.h, cabi.size3(128), cabi.ptr(h), planes, cabi.ptr(raw), planes, cabi.ptr(pw), None,
              planes, planes, cabi.PREC_F16, C.byref(epi), stream, C.byref(fl))
    torch.cuda.synchronize()
    cabi.check_errors()
    want = h.float() * 1000
    assert float((raw - want).abs().max()) <= 1e-3 * float(want.abs().max())  # the fp32 result is not clipped
    r = rows.float()
    assert bool(torch.isfinite(r).all()) and float(r.max()) == 65504.0 and float(r.min()) == -65504.0
    assert bool((r[want.abs() > 65504].abs() == 65504.0).all())


@pytest.mark.parametrize("n_in,n_out", [(96, 96), (128, 160), (160, 128), (224, 224), (192, 32)])
def test_f16_wide_layers_on_small_grids(cuda, n_in, n_out):
    # a few thousand rows and many planes (the deep levels of a UNet): the slab kernel, 16 rows x 32 output planes per
    # warp, instead of the tcgen05 kernel with split reductions
    import ctypes as C
    c = np.concatenate([synth.sphere_surface((30, 30, 30), 11), synth.sphere_surface((60, 50, 40), 8)], 0)
    m = cabi.Metadata()
    n = m.input_layer_build(128, torch.from_numpy(c).to(cuda), mode=4)
    g = O.Grid(c)
    assert n == g.n and n < 4096
    rng = np.random.RandomState(n_in + 3 * n_out)
    stream = torch.cuda.current_stream().cuda_stream
    x = np.maximum(rng.randn(g.n, n_in), 0).astype(np.float32)  # like a BatchNorm+ReLU output
    h = torch.from_numpy(x).to(cuda).half()
    ref = h.float().cpu().numpy()
    w = synth.kaiming_uniform(rng, 27, n_in, n_out)
    dw = torch.from_numpy(w).to(cuda)
    pw = torch.empty(cabi.lib().scn_packed_size_f16(27, n_in, n_out), dtype=torch.float16, device=cuda)
    cabi.call("scn_pack_weights_f16", cabi.ptr(dw), 27, n_in, n_out, cabi.ptr(pw), stream)
    out = torch.empty(g.n, n_out, dtype=torch.float32, device=cuda)
    fl = C.c_double(0)
    cabi.call("scn_ssc_forward", m.h, cabi.size3(128), cabi.ptr(h), n_in, cabi.ptr(out), n_out, cabi.ptr(pw), None, n_in, n_out,
              cabi.PREC_F16, stream, C.byref(fl))
    torch.cuda.synchronize()
    cabi.check_errors()
    want = torch.as_tensor(O.conv_forward(ref, w, O.ssc_rules(g), g.n, None))
    close(out, want, TF32_TOL)
    assert float((out.cpu() - want).abs().max()) / float(want.abs().max()) < 3e-3


@pytest.mark.parametrize("n_in,n_out,scene", [(32, 32, "c1"), (64, 64, "c1"), (32, 64, "c1"), (96, 96, "spheres"), (160, 128, "spheres"),
                                              (128, 128, "c1"), (96, 160, "tiny"), (224, 224, "tiny")])
def test_f16_fused_epilogue_residual_sum_and_batchnorm(cuda, n_in, n_out, scene):
    """scn_ssc/conv_forward_ex: the residual sum and the BatchNorm + ReLU behind a convolution formed in its epilogue, in
    every fp16 kernel (warp-level 32/64 planes, slab kernel on a few thousand rows, tcgen05 kernel on many rows and --
    with split reductions -- on a few hundred).  The fp32 result must equal the plain call's plus the addend, the fp16
    rows must be the BatchNorm of exactly that result, and skip_raw must leave the fp16 rows unchanged."""
    import ctypes as C
    if scene == "c1":
        c = synth.boxes_and_spheres(0)
    elif scene == "spheres":
        c = np.concatenate([synth.sphere_surface((30, 30, 30), 11), synth.sphere_surface((60, 50, 40), 8)], 0)
    else:
        c = synth.sphere_surface((20, 20, 20), 4)
    m = cabi.Metadata()
    n = m.input_layer_build(128, torch.from_numpy(c).to(cuda), mode=4)
    rng = np.random.RandomState(n_in + 7 * n_out)
    stream = torch.cuda.current_stream().cuda_stream
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(cuda)
    h = t(np.maximum(rng.randn(n, n_in), 0)).half()
    addend = t(rng.randn(n, n_out))
    scale, shift = t(rng.uniform(0.5, 1.5, n_out)), t(rng.randn(n_out))
    fl = C.c_double(0)

    def packed(w):
        dw = t(w)
        p = torch.empty(cabi.lib().scn_packed_size_f16(w.shape[0], n_in, n_out), dtype=torch.float16, device=cuda)
        cabi.call("scn_pack_weights_f16", cabi.ptr(dw), w.shape[0], n_in, n_out, cabi.ptr(p), stream)
        return p

    def run(fn, sizes, rows_in, rows_out, pw, with_addend, leak):
        plain = torch.empty(rows_out, n_out, dtype=torch.float32, device=cuda)
        cabi.call(fn, m.h, *sizes, cabi.ptr(rows_in), n_in, cabi.ptr(plain), n_out, cabi.ptr(pw), None, n_in, n_out, cabi.PREC_F16,
                  stream, C.byref(fl))
        add = addend[:rows_out].contiguous() if with_addend else None
        raw = torch.full((rows_out, n_out), float("nan"), dtype=torch.float32, device=cuda)
        rows = torch.zeros(rows_out, n_out, dtype=torch.float16, device=cuda)
        e = cabi.Epilogue(cabi.ptr(add), n_out, cabi.ptr(scale), cabi.ptr(shift), leak, cabi.ptr(rows), n_out, 0)
        cabi.call(fn + "_ex", m.h, *sizes, cabi.ptr(rows_in), n_in, cabi.ptr(raw), n_out, cabi.ptr(pw), None, n_in, n_out,
                  cabi.PREC_F16, C.byref(e), stream, C.byref(fl))
        want_raw = plain + add if with_addend else plain
        assert torch.equal(raw, want_raw) or float((raw - want_raw).abs().max()) <= 1e-6 * float(want_raw.abs().max())
        y = raw * scale + shift
        y = torch.where(y > 0, y, y * leak).clamp(-65504, 65504)
        assert float((rows.float() - y).abs().max()) <= 2e-3 * max(float(y.abs().max()), 1.0)  # half a unit in the last fp16 place
        rows2 = torch.zeros_like(rows)
        e2 = cabi.Epilogue(cabi.ptr(add), n_out, cabi.ptr(scale), cabi.ptr(shift), leak, cabi.ptr(rows2), n_out, 1)
        cabi.call(fn + "_ex", m.h, *sizes, cabi.ptr(rows_in), n_in, None, n_out, cabi.ptr(pw), None, n_in, n_out, cabi.PREC_F16,
                  C.byref(e2), stream, C.byref(fl))
        assert torch.equal(rows, rows2)

    run("scn_ssc_forward", (cabi.size3(128),), h, n, packed(synth.kaiming_uniform(rng, 27, n_in, n_out)), True, 0.0)
    run("scn_ssc_forward", (cabi.size3(128),), h, n, packed(synth.kaiming_uniform(rng, 27, n_in, n_out)), False, 0.333)
    n_cc = C.c_int64(0)
    cabi.call("scn_conv_prepare", m.h, cabi.size3(128), cabi.size3(64), stream, C.byref(n_cc))
    run("scn_conv_forward", (cabi.size3(128), cabi.size3(64)), h, int(n_cc.value), packed(synth.kaiming_uniform(rng, 8, n_in, n_out)),
        False, 0.0)
    # refused where no kernel carries the epilogue: fp32 rows
    e = cabi.Epilogue(None, 0, cabi.ptr(scale), cabi.ptr(shift), 0.0, cabi.ptr(torch.zeros(n, n_out, dtype=torch.float16, device=cuda)),
                      n_out, 0)
    with pytest.raises(cabi.ScnError):
        cabi.call("scn_ssc_forward_ex", m.h, cabi.size3(128), cabi.ptr(h.float()), n_in, cabi.ptr(torch.empty(n, n_out, device=cuda)),
                  n_out, cabi.ptr(t(synth.kaiming_uniform(rng, 27, n_in, n_out))), None, n_in, n_out, cabi.PREC_TF32, C.byref(e), stream,
                  C.byref(fl))
    cabi.check_errors()


def test_conv_deconv_nin_tf32(cuda):
    m, g = _scene(cuda, 1)
    rng = np.random.RandomState(17)
    coarse, rules = O.conv2_rules(g)
    x = rng.randn(g.n, 32).astype(np.float32)
    w = synth.kaiming_uniform(rng, 8, 32, 64)
    got, _ = m.conv_forward(128, 64, torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda), None, cabi.PREC_TF32)
    close(got, O.conv_forward(x, w, rules, coarse.n, None), TF32_TOL)
    wd = synth.kaiming_uniform(rng, 8, 64, 32)
    y = rng.randn(coarse.n, 64).astype(np.float32)
    got, _ = m.deconv_forward(64, 128, torch.from_numpy(y).to(cuda), torch.from_numpy(wd).to(cuda), None, cabi.PREC_TF32)
    close(got, O.conv_forward(y, wd, rules, g.n, None, reverse=True), TF32_TOL)
    wn = (rng.randn(64, 32) * np.sqrt(2.0 / 64)).astype(np.float32)
    z = rng.randn(5000, 64).astype(np.float32)
    got, _ = cabi.nin_forward(torch.from_numpy(z).to(cuda), torch.from_numpy(wn).to(cuda), None, cabi.PREC_TF32)
    close(got, O.nin_forward(z, wn), TF32_TOL)
    cabi.check_errors()


def test_bn_train_mode(cuda):
    rng = np.random.RandomState(21)
    x = (rng.randn(30011, 32) * 2 + 0.7).astype(np.float32)
    rm = rng.randn(32).astype(np.float32)
    rv = rng.uniform(0.5, 2, 32).astype(np.float32)
    gamma = rng.randn(32).astype(np.float32)
    beta = rng.randn(32).astype(np.float32)
    want, want_rm, want_rv = O.bn_forward_train(x, rm, rv, gamma, beta, 1e-4, 0.9, 0.0)
    t = lambda a: torch.from_numpy(a.copy()).to(cuda)
    d_rm, d_rv = t(rm), t(rv)
    got, sm, si = cabi.bn_forward_train(t(x), d_rm, d_rv, t(gamma), t(beta), 1e-4, 0.9, 0.0)
    close(got, want, 1e-4)
    close(d_rm, want_rm, 1e-5)
    close(d_rv, want_rv, 1e-5)
    close(sm, torch.from_numpy(x).double().mean(0).float(), 1e-5)


@pytest.mark.parametrize("rows", [1, 7, 128, 129, 300])
def test_tf32_tiny_row_counts(cuda, rows):
    # one-row and ragged tiles through the persistent tensor-core kernel (1x1 convolution and a tiny grid)
    rng = np.random.RandomState(rows)
    x = rng.randn(rows, 64).astype(np.float32)
    w = (rng.randn(64, 96) * 0.2).astype(np.float32)
    b = rng.randn(96).astype(np.float32)
    got, _ = cabi.nin_forward(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda), torch.from_numpy(b).to(cuda),
                              cabi.PREC_TF32)
    cabi.check_errors()
    close(got, O.nin_forward(x, w, b), TF32_TOL)
    # the same through the warp-level kernel (narrow layer)
    got, _ = cabi.nin_forward(torch.from_numpy(x).to(cuda), torch.from_numpy(w[:, :32].copy()).to(cuda),
                              torch.from_numpy(b[:32].copy()).to(cuda), cabi.PREC_TF32)
    close(got, O.nin_forward(x, w[:, :32], b[:32]), TF32_TOL)
    # a chain of `rows` voxels along x: every site has at most two neighbours
    c = np.stack([np.arange(rows) + 3, np.full(rows, 5), np.full(rows, 7)], 1)
    m = cabi.Metadata()
    m.input_layer_build(4096, torch.from_numpy(c).to(cuda), mode=4)
    g = O.Grid(c)
    xs = rng.randn(rows, 32).astype(np.float32)
    ws = synth.kaiming_uniform(rng, 27, 32, 32)
    got, _ = m.ssc_forward(4096, torch.from_numpy(xs).to(cuda), torch.from_numpy(ws).to(cuda), None, cabi.PREC_TF32)
    cabi.check_errors()
    close(got, O.conv_forward(xs, ws, O.ssc_rules(g), g.n), TF32_TOL)


@pytest.mark.parametrize("n_in,n_out,seed,size", [(64, 256, 0, 128), (256, 256, 0, 128), (256, 256, 1, 64), (32, 256, 3, 128)])
def test_tf32_256_output_planes_per_tile_kernel(cuda, n_in, n_out, seed, size):
    """256 output planes with 27 offsets leave too little shared memory for the persistent tcgen05 kernel's
    stages: these shapes run the one-tile-per-CTA tcgen05 kernel -- through the neighbour map, with the
    reduction of a tile split over several CTAs on the small scenes (partial sums + reduction kernel) and not
    split on the large one, with a bias, and with the addend read from the output array itself."""
    import ctypes as C
    m, g = _scene(cuda, seed, size)
    rng = np.random.RandomState(n_in + n_out + seed)
    x = rng.randn(g.n, n_in).astype(np.float32)
    w = synth.kaiming_uniform(rng, 27, n_in, n_out)
    b = rng.randn(n_out).astype(np.float32)
    want = O.conv_forward(x, w, O.ssc_rules(g), g.n, b)
    dx, dw, db = torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda), torch.from_numpy(b).to(cuda)
    got, _ = m.ssc_forward(size, dx, dw, db, precision=cabi.PREC_TF32)
    cabi.check_errors()
    close(got, want, TF32_TOL)
    assert float((got.cpu() - want).abs().max()) / float(want.abs().max()) < 5e-3
    # out = out + convolution: the addend is the output array (read and written by the same thread of the epilogue)
    plain, _ = m.ssc_forward(size, dx, dw, None, cabi.PREC_TF32)
    base = torch.from_numpy(rng.randn(g.n, n_out).astype(np.float32)).to(cuda)
    out = base.clone()
    fl = C.c_double(0)
    cabi.call("scn_ssc_forward_add", m.h, cabi.size3(size), cabi.ptr(dx), n_in, cabi.ptr(out), n_out, cabi.ptr(dw),
              cabi.ptr(out), n_out, n_in, n_out, cabi.PREC_TF32, torch.cuda.current_stream().cuda_stream, C.byref(fl))
    cabi.check_errors()
    assert float((out - (plain + base)).abs().max()) <= 1e-5 * float((plain + base).abs().max())


@pytest.mark.parametrize("n_in,n_out", [(64, 32), (96, 128)])
def test_packed_weights_match_unpacked(cuda, n_in, n_out):
    # (64, 32) runs the warp-level kernel, (96, 128) the tcgen05 kernel; each has its own packed layout
    import ctypes as C
    m, g = _scene(cuda, 2)
    rng = np.random.RandomState(5)
    x = torch.from_numpy(rng.randn(g.n, n_in).astype(np.float32)).to(cuda)
    w = torch.from_numpy(synth.kaiming_uniform(rng, 27, n_in, n_out)).to(cuda)
    assert cabi.lib().scn_weights_packable(27, n_in, n_out) == 1 and cabi.lib().scn_weights_packable(27, 3, 32) == 0
    packed = torch.empty_like(w)
    cabi.call("scn_pack_weights", cabi.ptr(w), 27, n_in, n_out, cabi.ptr(packed), torch.cuda.current_stream().cuda_stream)
    if n_in > 64:
        assert torch.equal(packed.view(27, n_out, n_in), w.transpose(1, 2).contiguous())
    else:  # a permutation of the weights rounded to tf32 (13 low mantissa bits cleared)
        bits = packed.view(torch.int32)
        assert int((bits & 0x1FFF).abs().max()) == 0
        assert torch.allclose(packed.flatten().sort().values, w.flatten().sort().values, rtol=1e-3, atol=0)
    a, _ = m.ssc_forward(128, x, w, None, cabi.PREC_TF32)
    out = torch.empty_like(a)
    fl = C.c_double(0)
    cabi.call("scn_ssc_forward", m.h, cabi.size3(128), cabi.ptr(x), n_in, cabi.ptr(out), n_out, cabi.ptr(packed), None, n_in,
              n_out, cabi.PREC_TF32_PACKED, torch.cuda.current_stream().cuda_stream, C.byref(fl))
    cabi.check_errors()
    assert torch.equal(a, out)
