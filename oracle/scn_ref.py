"""ctypes binding of oracle/_ref/libscn_ref.so: the reference implementation itself, compiled for the
host by oracle/build_ref.py (its kernels run on a CUDA-on-host emulation).  TEST INFRASTRUCTURE ONLY: it
pins the Python oracle (oracle/scn_oracle.py) to the reference's own code; nothing the library ships
imports it.

The reference packs a voxel into a 31-bit key (x 10 bits, y 11 bits, z 10 bits) and aliases outside that
range, so scenes fed through this binding keep coordinates in [1,1022] x [1,2046] x [1,1022]; its
InputLayer reads 4-column coordinates (x, y, z, batch) and wants them sorted by batch index.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libscn_ref.so")
_lib = None

_F = ctypes.POINTER(ctypes.c_float)
_L = ctypes.POINTER(ctypes.c_long)
_I = ctypes.POINTER(ctypes.c_int32)


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        import torch  # noqa: F401  (loads libtorch_cpu / libc10, which the library links against)
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.ref_last_error.restype = ctypes.c_char_p
        _lib.ref_metadata_new.restype = ctypes.c_void_p
        for name in ("ref_result_rows", "ref_result_cols", "ref_rules_size", "ref_n_active"):
            getattr(_lib, name).restype = ctypes.c_long
    return _lib


def _check(rc):
    if rc != 0:
        raise RuntimeError("reference: " + lib().ref_last_error().decode(errors="replace"))


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F)


def _fopt(a):
    if a is None:
        return None, None
    return _f(a)


def _result_f32():
    L = lib()
    out = np.empty((L.ref_result_rows(), L.ref_result_cols()), np.float32)
    if out.size:
        _check(L.ref_result_copy_f32(out.ctypes.data_as(_F)))
    return out


def _rules(counts):
    L = lib()
    flat = np.empty(L.ref_rules_size(), np.int32)
    if flat.size:
        L.ref_rules_copy(flat.ctypes.data_as(_I))
    pairs = flat.reshape(-1, 2)
    out, at = [], 0
    for c in counts:
        out.append(pairs[at:at + int(c)].copy())
        at += int(c)
    return out


_c = ctypes.c_long
_cf = ctypes.c_float
_vp = ctypes.c_void_p


class Metadata(object):
    """The reference's Metadata<3> (Metadata/Metadata.h:218-386)."""

    def __init__(self):
        self.h = _vp(lib().ref_metadata_new())

    def __del__(self):
        if getattr(self, "h", None) is not None and _lib is not None:
            _lib.ref_metadata_free(self.h)
            self.h = None

    def n_active(self, spatial):
        return int(lib().ref_n_active(self.h, _c(spatial)))

    def spatial_locations(self, spatial):
        """[n,4] int64 (x,y,z,batch) in row order (Metadata::getSpatialLocations, Metadata.cpp:793-821)."""
        L = lib()
        _check(L.ref_spatial_locations(self.h, _c(spatial)))
        out = np.empty((L.ref_result_rows(), L.ref_result_cols()), np.int64)
        if out.size:
            _check(L.ref_result_copy_i64(out.ctypes.data_as(_L)))
        return out

    def input_rules(self):
        """(header [mode, maxActive, nIn, nOut], rows [nOut, 1+maxActive])."""
        L = lib()
        header = np.zeros(4, np.int32)
        _check(L.ref_input_rules(self.h, header.ctypes.data_as(_I)))
        flat = np.empty(L.ref_rules_size(), np.int32)
        if flat.size:
            L.ref_rules_copy(flat.ctypes.data_as(_I))
        return header, flat.reshape(int(header[3]), 1 + int(header[1]))

    def ssc_rulebook(self, spatial):
        counts = np.zeros(27, np.int32)
        _check(lib().ref_ssc_rulebook(self.h, _c(spatial), counts.ctypes.data_as(_I)))
        return _rules(counts)

    def conv_rulebook(self, in_spatial):
        counts = np.zeros(8, np.int32)
        _check(lib().ref_conv_rulebook(self.h, _c(in_spatial), counts.ctypes.data_as(_I)))
        return _rules(counts)

    def incre_ssc_rulebook(self, pre, spatial):
        counts = np.zeros(27, np.int32)
        _check(lib().ref_incre_ssc_rulebook(self.h, pre.h, _c(spatial), counts.ctypes.data_as(_I)))
        return _rules(counts)

    def pre_exist(self, pre, spatial):
        n = self.n_active(spatial)
        out = np.empty(n, np.int32)
        _check(lib().ref_pre_exist(self.h, pre.h, _c(spatial), out.ctypes.data_as(_I), _c(n)))
        return out


def _coords4(coords):
    c = np.ascontiguousarray(coords, dtype=np.int64)
    if c.shape[1] == 3:
        c = np.concatenate([c, np.zeros((c.shape[0], 1), np.int64)], 1)
    return np.ascontiguousarray(c)


def input_layer(m, spatial, coords, feats, batch_size, mode):
    c = _coords4(coords)
    x, xp = _f(feats)
    _check(lib().ref_input_layer(m.h, _c(spatial), c.ctypes.data_as(_L), _c(c.shape[0]), _c(4), xp, _c(x.shape[1]),
                                 _c(batch_size), _c(mode)))
    return _result_f32()


def incre_input_layer(m, spatial, coords, feats, batch_size, mode, pre, pre_out):
    c = _coords4(coords)
    x, xp = _f(feats)
    po, pop = _f(pre_out)
    _check(lib().ref_incre_input_layer(m.h, _c(spatial), c.ctypes.data_as(_L), _c(c.shape[0]), _c(4), xp, _c(x.shape[1]),
                                       _c(batch_size), _c(mode), pre.h, pop, _c(po.shape[0])))
    return _result_f32()


def output_layer(m, x):
    x, xp = _f(x)
    _check(lib().ref_output_layer(m.h, xp, _c(x.shape[0]), _c(x.shape[1])))
    return _result_f32()


def incre_output_layer(m, x, pre, pre_in):
    x, xp = _f(x)
    p, pp = _f(pre_in)
    _check(lib().ref_incre_output_layer(m.h, xp, _c(x.shape[0]), _c(x.shape[1]), pre.h, pp, _c(p.shape[0])))
    return _result_f32()


def _conv_like(fn, m, spatial, x, w, bias, extra=()):
    x, xp = _f(x)
    w, wp = _f(w)
    b, bp = _fopt(bias)
    flops = ctypes.c_double(0)
    _check(fn(m.h, _c(spatial), xp, _c(x.shape[0]), _c(w.shape[1]), wp, bp, _c(w.shape[2]), *extra, ctypes.byref(flops)))
    return _result_f32(), flops.value


def ssc(m, spatial, x, w, bias=None, cpu=False):
    """cuda_SubmanifoldConvolution_updateOutput (CUDA/Convolution.cpp:152-218), or with cpu=True
    cpu_SubmanifoldConvolution_updateOutput (CPU/Convolution.cpp:115-149) on the same rulebook."""
    return _conv_like(lib().ref_cpu_ssc if cpu else lib().ref_ssc, m, spatial, x, w, bias)


def incre_ssc(m, spatial, x, w, bias, pre, pre_in):
    p, pp = _f(pre_in)
    return _conv_like(lib().ref_incre_ssc, m, spatial, x, w, bias, (pre.h, pp, _c(p.shape[0])))


def conv(m, in_spatial, x, w, bias=None, incremental=False, cpu=False):
    if cpu:
        return _conv_like(lib().ref_cpu_conv, m, in_spatial, x, w, bias)
    return _conv_like(lib().ref_conv, m, in_spatial, x, w, bias, (ctypes.c_int(1 if incremental else 0),))


def deconv(m, in_spatial, x, w, bias=None, cpu=False):
    return _conv_like(lib().ref_cpu_deconv if cpu else lib().ref_deconv, m, in_spatial, x, w, bias)


def incre_deconv(m, in_spatial, x, w, bias, pre, pre_in):
    p, pp = _f(pre_in)
    return _conv_like(lib().ref_incre_deconv, m, in_spatial, x, w, bias, (pre.h, pp, _c(p.shape[0])))


def bn(x, mean, var, gamma, beta, eps, leakiness, train=False, momentum=0.9, cpu=False):
    """Returns out (test mode) or (out, new_running_mean, new_running_var) (train mode)."""
    x, xp = _f(x)
    mean, mp = _f(mean)
    var, vp = _f(var)
    g, gp = _fopt(gamma)
    b, bp = _fopt(beta)
    mo, vo = np.empty_like(mean), np.empty_like(var)
    fn = lib().ref_cpu_bn if cpu else lib().ref_bn
    _check(fn(xp, _c(x.shape[0]), _c(x.shape[1]), mp, vp, gp, bp, _cf(eps), _cf(momentum), ctypes.c_int(1 if train else 0),
              _cf(leakiness), mo.ctypes.data_as(_F), vo.ctypes.data_as(_F)))
    out = _result_f32()
    return (out, mo, vo) if train else out


def incre_bn(x, mean, var, gamma, beta, eps, leakiness, m, pre, pre_out, pre_in, spatial):
    x, xp = _f(x)
    mean, mp = _f(mean)
    var, vp = _f(var)
    g, gp = _fopt(gamma)
    b, bp = _fopt(beta)
    po, pop = _f(pre_out)
    pi, pip = _f(pre_in)
    _check(lib().ref_incre_bn(xp, _c(x.shape[0]), _c(x.shape[1]), mp, vp, gp, bp, _cf(eps), _cf(leakiness), m.h, pre.h, pop, pip,
                              _c(po.shape[0]), _c(spatial)))
    return _result_f32()


def nin(x, w, bias=None, cpu=False):
    x, xp = _f(x)
    w, wp = _f(w)
    b, bp = _fopt(bias)
    flops = ctypes.c_double(0)
    fn = lib().ref_cpu_nin if cpu else lib().ref_nin
    _check(fn(xp, _c(x.shape[0]), _c(w.shape[0]), wp, bp, _c(w.shape[1]), ctypes.byref(flops)))
    return _result_f32(), flops.value


def cpu_input_forward(m, x):
    x, xp = _f(x)
    _check(lib().ref_cpu_input_forward(m.h, xp, _c(x.shape[0]), _c(x.shape[1])))
    return _result_f32()


def cpu_output_forward(m, x):
    x, xp = _f(x)
    _check(lib().ref_cpu_output_forward(m.h, xp, _c(x.shape[0]), _c(x.shape[1])))
    return _result_f32()


# ---- label fusion: the reference's Result<3> / ResultOfWeight<3> (Metadata/resultHash.h) ---------------------------
def _pts(ps):
    p = np.ascontiguousarray(np.asarray(ps, np.int64)[:, :3])
    return p, p.ctypes.data_as(_L)


class Result(object):
    def __init__(self, maximum=0.7):
        L = lib()
        L.ref_result_new.restype = ctypes.c_void_p
        L.ref_result_new.argtypes = [ctypes.c_float]
        L.ref_result_size.restype = ctypes.c_long
        L.ref_result_confidence.restype = ctypes.c_float
        self.h = ctypes.c_void_p(L.ref_result_new(ctypes.c_float(maximum)))

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_result_free(self.h)
            self.h = None

    def _apply(self, fn, ps, label):
        p, pp = _pts(ps)
        s = np.ascontiguousarray(label, np.float32)
        _check(fn(self.h, pp, ctypes.c_long(p.shape[0]), s.ctypes.data_as(_F), ctypes.c_long(s.shape[1])))

    def update(self, ps, label):
        self._apply(lib().ref_result_update, ps, label)

    def set(self, ps, label):
        self._apply(lib().ref_result_set, ps, label)

    def multiQuery(self, ps):
        p, pp = _pts(ps)
        out = np.empty(p.shape[0], np.int64)
        _check(lib().ref_result_multiquery(self.h, pp, ctypes.c_long(p.shape[0]), out.ctypes.data_as(_L)))
        return out

    def size(self):
        return int(lib().ref_result_size(self.h))

    def get_all_points_labels(self):
        out = np.empty((self.size(), 4), np.int64)
        _check(lib().ref_result_all(self.h, out.ctypes.data_as(_L)))
        return out

    def finalize(self, ps):
        p, pp = _pts(ps)
        _check(lib().ref_result_finalize(self.h, pp, ctypes.c_long(p.shape[0])))

    def confidence(self, x, y, z):
        return float(lib().ref_result_confidence(self.h, ctypes.c_long(x), ctypes.c_long(y), ctypes.c_long(z)))


class ResultOfWeight(object):
    def __init__(self):
        L = lib()
        L.ref_weight_new.restype = ctypes.c_void_p
        L.ref_weight_size.restype = ctypes.c_long
        self.h = ctypes.c_void_p(L.ref_weight_new())

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_weight_free(self.h)
            self.h = None

    def update(self, ps, label):
        p, pp = _pts(ps)
        s = np.ascontiguousarray(label, np.float32)
        _check(lib().ref_weight_update(self.h, pp, ctypes.c_long(p.shape[0]), s.ctypes.data_as(_F), ctypes.c_long(s.shape[1])))

    def multiQuery(self, ps):
        p, pp = _pts(ps)
        out = np.empty(p.shape[0], np.int64)
        _check(lib().ref_weight_multiquery(self.h, pp, ctypes.c_long(p.shape[0]), out.ctypes.data_as(_L)))
        return out

    def size(self):
        return int(lib().ref_weight_size(self.h))

    def finalize(self, ps):
        p, pp = _pts(ps)
        _check(lib().ref_weight_finalize(self.h, pp, ctypes.c_long(p.shape[0])))
