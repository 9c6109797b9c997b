"""ctypes binding of libinsconv_b200.so (C ABI: include/insconv_b200.h).

The binding is deliberately thin: it loads the library, declares every prototype, turns negative
status codes into ScnError, and offers a small Metadata wrapper that passes torch CUDA tensors by
data pointer.  There is no fallback: if the shared library is missing or a CUDA call fails, the
call raises.
"""
import ctypes as C
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libinsconv_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "include", "insconv_b200.h")

PREC_FP32 = 0
PREC_TF32 = 1
PREC_TF32_PACKED = 2
PREC_F16 = 3


class ScnError(RuntimeError):
    def __init__(self, code, msg):
        RuntimeError.__init__(self, "insconv_b200 error %d: %s" % (code, msg))
        self.code = code


_p = C.c_void_p
_i64 = C.c_int64
_i64p = C.POINTER(C.c_int64)
_int = C.c_int
_dbl = C.c_double

# name -> (restype, argtypes); status-returning functions have restype int
PROTOTYPES = {
    "scn_last_error": (C.c_char_p, []),
    "scn_version": (C.c_char_p, []),
    "scn_launch_count": (C.c_uint64, []),
    "scn_set_slab_share": (_int, [_int]),
    "scn_set_slab_max_rows": (_int, [_i64]),
    "scn_n_rulebook_bits": (_int, []),
    "scn_check_errors": (_int, [_p]),
    "scn_metadata_create": (_int, [C.POINTER(_p)]),
    "scn_metadata_destroy": (None, [_p]),
    "scn_metadata_clear": (_int, [_p, _p]),
    "scn_metadata_n_active": (_i64, [_p, _i64p]),
    "scn_metadata_spatial_locations": (_int, [_p, _i64p, _p, _p]),
    "scn_metadata_site_coords": (_int, [_p, _i64p, C.POINTER(_p), _i64p]),
    "scn_metadata_hash_dump": (_int, [_p, _i64p, _p, _p, _i64p, _p]),
    "scn_metadata_query": (_int, [_p, _i64p, _p, _i64, _p, _p]),
    "scn_input_layer_build": (_int, [_p, _i64p, _p, _int, _i64, _int, _i64, _int, _p, _i64p]),
    "scn_input_layer_forward": (_int, [_p, _p, _p, _i64, _p]),
    "scn_output_layer_forward": (_int, [_p, _p, _p, _i64, _p]),
    "scn_input_layer_n_points": (_i64, [_p]),
    "scn_metadata_input_n_active": (_i64, [_p]),
    "scn_input_layer_set_site_counts": (_int, [_p, _p, _i64, _p]),
    "scn_input_layer_rules": (_int, [_p, _p, _p, _p]),
    "scn_ssc_rulebook": (_int, [_p, _i64p, _p, _p, _p]),
    "scn_conv_rulebook": (_int, [_p, _i64p, _i64p, _p, _p, _p]),
    "scn_weights_packable": (_int, [_i64, _i64, _i64]),
    "scn_pack_weights": (_int, [_p, _i64, _i64, _i64, _p, _p]),
    "scn_ssc_forward": (_int, [_p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_set_build_ahead": (_int, [_int, _int]),
    "scn_metadata_set_build_ahead": (_int, [_p, _int, _int]),
    "scn_metadata_build_used": (_int, [_p, C.POINTER(_int), C.POINTER(_int)]),
    "scn_metadata_inherit": (_int, [_p, _p]),
    "scn_packed_size_f16": (_i64, [_i64, _i64, _i64]),
    "scn_weights_packable_f16": (_int, [_i64, _i64, _i64]),
    "scn_pack_weights_f16": (_int, [_p, _i64, _i64, _i64, _p, _p]),
    "scn_join_bn_forward_f16": (_int, [_p, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _p, _p, _dbl, _p, _i64, _p]),
    "scn_bn_forward_f16": (_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _p, _p, _p, _dbl, _dbl, _p]),
    "scn_ssc_forward_add": (_int, [_p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_conv_prepare": (_int, [_p, _i64p, _i64p, _p, _i64p]),
    "scn_conv_forward": (_int, [_p, _i64p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_deconv_forward": (_int, [_p, _i64p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_bn_forward": (_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _p, _p, _p, _dbl, _dbl, _p]),
    "scn_bn_forward_train": (_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _dbl, _dbl, _dbl, _p]),
    "scn_nin_forward": (_int, [_p, _i64, _p, _i64, _i64, _p, _p, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_nin_forward_noalloc": (_int, [_p, _i64, _p, _i64, _i64, _p, _p, _i64, _i64, _p]),
    "scn_incre_pre_exist": (_int, [_p, _p, _i64p, C.POINTER(_p), _i64p, _p]),
    "scn_incre_input_layer_forward": (_int, [_p, _p, _p, _p, _p, _i64, _p]),
    "scn_incre_output_layer_forward": (_int, [_p, _p, _p, _p, _p, _i64, _p]),
    "scn_incre_ssc_forward": (_int, [_p, _p, _i64p, _p, _i64, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_incre_ssc_rulebook": (_int, [_p, _p, _i64p, _p, _p, _p]),
    "scn_incre_deconv_forward": (_int, [_p, _p, _i64p, _i64p, _p, _i64, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _int, _p, C.POINTER(_dbl)]),
    "scn_incre_bn_forward": (_int, [_p, _p, _i64p, _p, _i64, _p, _i64, _i64, _p, _p, _p, _p, _dbl, _dbl, _p, _p, _p]),
    "scn_incre_bn_forward_f16": (_int, [_p, _p, _i64p, _p, _i64, _p, _i64, _i64, _p, _p, _p, _p, _dbl, _dbl, _p, _i64, _p, _i64, _p]),
}



class Epilogue(C.Structure):
    """scn_epilogue of include/insconv_b200.h."""
    _fields_ = [("addend", _p), ("addend_stride", _i64), ("bn_scale", _p), ("bn_shift", _p), ("bn_leakiness", _dbl),
                ("bn_out", _p), ("bn_out_stride", _i64), ("skip_raw", _int), ("bn_pre_in", _p), ("bn_pre_in_stride", _i64),
                ("bn_pre_out", _p), ("bn_pre_out_stride", _i64)]


PROTOTYPES.update({
    "scn_ssc_forward_ex": (_int, [_p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, C.POINTER(Epilogue), _p, C.POINTER(_dbl)]),
    "scn_conv_forward_ex": (_int, [_p, _i64p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, C.POINTER(Epilogue), _p,
                                   C.POINTER(_dbl)]),
    "scn_incre_ssc_forward_ex": (_int, [_p, _p, _i64p, _p, _i64, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _int, C.POINTER(Epilogue), _p,
                                        C.POINTER(_dbl)]),
    "scn_incre_conv_forward_ex": (_int, [_p, _p, _i64p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, C.POINTER(Epilogue), _p,
                                         C.POINTER(_dbl)]),
    "scn_deconv_forward_ex": (_int, [_p, _i64p, _i64p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _int, C.POINTER(Epilogue), _p,
                                     C.POINTER(_dbl)]),
})

PROTOTYPES.update({
    "scn_halo_create": (_int, [C.POINTER(_p), _i64]),
    "scn_halo_destroy": (None, [_p]),
    "scn_halo_ipc_handle": (_int, [_p, _p]),
    "scn_halo_connect": (_int, [_p, _int, _p]),
    "scn_halo_set_spin_limit": (_int, [_p, _i64]),
    "scn_halo_exchange": (_int, [_p, _p, _p, _i64, _p, _i64, _p, _i64, _p]),
    "scn_halo_status": (_int, [_p, C.POINTER(_int), C.POINTER(_int), _p]),
    "scn_halo_plane_lists": (_int, [_p, _i64p, _int, _int, _int, _int, _i64, _p, _p, _p]),
})

PROTOTYPES.update({
    "scn_labels_create": (_int, [C.POINTER(_p), _int, _dbl]),
    "scn_labels_destroy": (None, [_p]),
    "scn_labels_clear": (_int, [_p, _p]),
    "scn_labels_update": (_int, [_p, _p, _int, _i64, _p, _i64, _i64, _p]),
    "scn_labels_set": (_int, [_p, _p, _int, _i64, _p, _i64, _i64, _p]),
    "scn_labels_query": (_int, [_p, _p, _int, _i64, _p, _p]),
    "scn_labels_size": (_int, [_p, _i64p, _i64p, _p]),
    "scn_labels_dump": (_int, [_p, _p, _i64, _i64p, _p]),
    "scn_labels_finalize": (_int, [_p, _p, _int, _i64, _p]),
})

_STATUS = {n for n, (r, _) in PROTOTYPES.items() if r is _int and n not in ("scn_n_rulebook_bits", "scn_weights_packable")}


def declared_symbols():
    """Names of the functions include/insconv_b200.h declares."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"SCN_API\s+[\w\s\*]+?\b(scn_\w+)\s*\(", text)))


_lib = None


def lib():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ScnError(-2, "libinsconv_b200.so is not built (run python ins-conv_b200/build.py)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def call(name, *args):
    """Calls a status-returning entry point and raises ScnError on failure."""
    L = lib()
    r = getattr(L, name)(*args)
    if name in _STATUS and r != 0:
        raise ScnError(r, L.scn_last_error().decode())
    return r


def size3(v):
    """int or 3-sequence -> ctypes int64[3]."""
    if isinstance(v, int):
        v = (v, v, v)
    v = [int(x) for x in v]
    assert len(v) == 3
    return (C.c_int64 * 3)(*v)


def ptr(t):
    """Data pointer of a torch tensor / numpy array (None -> NULL)."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    if t.numel() == 0:
        return None
    return t.data_ptr()


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


class Metadata(object):
    """Owns one scn_metadata.  Tensor arguments are torch CUDA fp32 tensors."""

    def __init__(self):
        h = _p()
        call("scn_metadata_create", C.byref(h))
        self.h = h

    def __del__(self):
        try:
            if self.h:
                lib().scn_metadata_destroy(self.h)
                self.h = None
        except Exception:
            pass

    # -- grids ---------------------------------------------------------------------------------
    def input_layer_build(self, size, coords, mode=4, batch_size=0):
        """coords: int64 [n, 3|4] torch tensor (CPU or CUDA) or numpy array (host)."""
        import torch
        if isinstance(coords, np.ndarray):
            coords = torch.from_numpy(np.ascontiguousarray(coords, dtype=np.int64))
        coords = coords.contiguous()
        assert coords.dtype == torch.int64 and coords.dim() == 2
        n = _i64(0)
        call("scn_input_layer_build", self.h, size3(size), ptr(coords), 0 if coords.is_cuda else 1,
             coords.shape[0], coords.shape[1], batch_size, mode, _stream(), C.byref(n))
        self._n_input = n.value
        return n.value

    def n_active(self, size):
        return lib().scn_metadata_n_active(self.h, size3(size))

    def n_points(self):
        return lib().scn_input_layer_n_points(self.h)

    def spatial_locations(self, size):
        n = self.n_active(size)
        out = np.zeros((max(n, 0), 4), dtype=np.int64)
        call("scn_metadata_spatial_locations", self.h, size3(size), out.ctypes.data, _stream())
        return out

    def hash_dump(self, size):
        cap = _i64(0)
        call("scn_metadata_hash_dump", self.h, size3(size), None, None, C.byref(cap), _stream())
        keys = np.zeros(cap.value, dtype=np.uint64)
        rows = np.zeros(cap.value, dtype=np.int32)
        call("scn_metadata_hash_dump", self.h, size3(size), keys.ctypes.data, rows.ctypes.data, C.byref(cap), _stream())
        return keys, rows

    def query(self, size, coords_soa):
        """coords_soa: int32 CUDA tensor [4, n]; returns int32 CUDA tensor [n]."""
        import torch
        coords_soa = coords_soa.contiguous()
        n = coords_soa.shape[1]
        rows = torch.empty(n, dtype=torch.int32, device=coords_soa.device)
        call("scn_metadata_query", self.h, size3(size), ptr(coords_soa), n, ptr(rows), _stream())
        return rows

    def input_rules(self):
        hdr = np.zeros(4, dtype=np.int32)
        call("scn_input_layer_rules", self.h, hdr.ctypes.data, None, _stream())
        rows = np.zeros((int(hdr[3]), 1 + int(hdr[1])), dtype=np.int32)
        if rows.size:
            call("scn_input_layer_rules", self.h, hdr.ctypes.data, rows.ctypes.data, _stream())
        return hdr, rows

    def ssc_rulebook(self, size):
        counts = np.zeros(27, dtype=np.int64)
        call("scn_ssc_rulebook", self.h, size3(size), counts.ctypes.data, None, _stream())
        pairs = np.zeros((int(counts.sum()), 2), dtype=np.int32)
        if pairs.size:
            call("scn_ssc_rulebook", self.h, size3(size), counts.ctypes.data, pairs.ctypes.data, _stream())
        return _split(pairs, counts)

    def conv_rulebook(self, in_size, out_size):
        counts = np.zeros(8, dtype=np.int64)
        call("scn_conv_rulebook", self.h, size3(in_size), size3(out_size), counts.ctypes.data, None, _stream())
        pairs = np.zeros((int(counts.sum()), 2), dtype=np.int32)
        if pairs.size:
            call("scn_conv_rulebook", self.h, size3(in_size), size3(out_size), counts.ctypes.data, pairs.ctypes.data,
                 _stream())
        return _split(pairs, counts)

    def incre_ssc_rulebook(self, pre, size):
        counts = np.zeros(27, dtype=np.int64)
        call("scn_incre_ssc_rulebook", self.h, pre.h, size3(size), counts.ctypes.data, None, _stream())
        pairs = np.zeros((int(counts.sum()), 2), dtype=np.int32)
        if pairs.size:
            call("scn_incre_ssc_rulebook", self.h, pre.h, size3(size), counts.ctypes.data, pairs.ctypes.data, _stream())
        return _split(pairs, counts)

    def pre_exist(self, pre, size):
        """int32 numpy array [n_active(size)]: row in `pre` or -1."""
        import torch
        mp = _p()
        n = _i64(0)
        call("scn_incre_pre_exist", self.h, pre.h, size3(size), C.byref(mp), C.byref(n), _stream())
        out = torch.empty(n.value, dtype=torch.int32, device="cuda")
        if n.value:
            torch.cuda.current_stream().synchronize()
            _memcpy_d2d(out.data_ptr(), mp.value, n.value * 4)
        return out.cpu().numpy()

    # -- feature ops ---------------------------------------------------------------------------
    def input_forward(self, feats):
        import torch
        feats = feats.contiguous()
        n = self.n_active_input()
        out = torch.empty(n, feats.shape[1], dtype=torch.float32, device=feats.device)
        call("scn_input_layer_forward", self.h, ptr(feats), ptr(out), feats.shape[1], _stream())
        return out

    def n_active_input(self):
        return self._n_input

    def output_forward(self, feats):
        import torch
        feats = feats.contiguous()
        out = torch.empty(self.n_points(), feats.shape[1], dtype=torch.float32, device=feats.device)
        call("scn_output_layer_forward", self.h, ptr(feats), ptr(out), feats.shape[1], _stream())
        return out

    def ssc_forward(self, size, x, weight, bias=None, precision=PREC_FP32):
        import torch
        x = x.contiguous()
        weight = weight.contiguous()
        n_out = weight.shape[2]
        out = torch.empty(x.shape[0], n_out, dtype=torch.float32, device=x.device)
        fl = _dbl(0)
        call("scn_ssc_forward", self.h, size3(size), ptr(x), x.stride(0), ptr(out), n_out, ptr(weight), ptr(bias),
             weight.shape[1], n_out, precision, _stream(), C.byref(fl))
        return out, fl.value

    def ssc_forward_add(self, size, x, weight, addend, precision=PREC_FP32):
        import torch
        x = x.contiguous()
        n_out = weight.shape[2]
        out = torch.empty(x.shape[0], n_out, dtype=torch.float32, device=x.device)
        fl = _dbl(0)
        call("scn_ssc_forward_add", self.h, size3(size), ptr(x), x.stride(0), ptr(out), n_out, ptr(weight), ptr(addend),
             addend.stride(0), weight.shape[1], n_out, precision, _stream(), C.byref(fl))
        return out, fl.value

    def conv_forward(self, in_size, out_size, x, weight, bias=None, precision=PREC_FP32):
        import torch
        x = x.contiguous()
        weight = weight.contiguous()
        n = _i64(0)
        call("scn_conv_prepare", self.h, size3(in_size), size3(out_size), _stream(), C.byref(n))
        n_out = weight.shape[2]
        out = torch.empty(n.value, n_out, dtype=torch.float32, device=x.device)
        fl = _dbl(0)
        call("scn_conv_forward", self.h, size3(in_size), size3(out_size), ptr(x), x.stride(0), ptr(out), n_out,
             ptr(weight), ptr(bias), weight.shape[1], n_out, precision, _stream(), C.byref(fl))
        return out, fl.value

    def deconv_forward(self, in_size, out_size, x, weight, bias=None, precision=PREC_FP32):
        import torch
        x = x.contiguous()
        weight = weight.contiguous()
        n_out = weight.shape[2]
        out = torch.empty(self.n_active(out_size), n_out, dtype=torch.float32, device=x.device)
        fl = _dbl(0)
        call("scn_deconv_forward", self.h, size3(in_size), size3(out_size), ptr(x), x.stride(0), ptr(out), n_out,
             ptr(weight), ptr(bias), weight.shape[1], n_out, precision, _stream(), C.byref(fl))
        return out, fl.value

    # -- incremental ("Incre_*") ops: self holds the frame's changed sites, `pre` the last full frame -------------
    def incre_input_forward(self, pre, feats, pre_out):
        import torch
        feats = feats.contiguous()
        out = torch.empty(self.n_active_input(), feats.shape[1], dtype=torch.float32, device=feats.device)
        call("scn_incre_input_layer_forward", self.h, pre.h, ptr(feats), ptr(out), ptr(pre_out.contiguous()), feats.shape[1],
             _stream())
        return out

    def incre_output_forward(self, pre, feats, pre_in):
        import torch
        feats = feats.contiguous()
        out = torch.empty(self.n_points(), feats.shape[1], dtype=torch.float32, device=feats.device)
        call("scn_incre_output_layer_forward", self.h, pre.h, ptr(feats), ptr(out), ptr(pre_in.contiguous()), feats.shape[1],
             _stream())
        return out

    def incre_ssc_forward(self, pre, size, x, weight, pre_in, bias=None, precision=PREC_FP32):
        import torch
        x, weight, pre_in = x.contiguous(), weight.contiguous(), pre_in.contiguous()
        n_out = weight.shape[2]
        out = torch.empty(x.shape[0], n_out, dtype=torch.float32, device=x.device)
        fl = _dbl(0)
        call("scn_incre_ssc_forward", self.h, pre.h, size3(size), ptr(x), x.shape[1], ptr(out), n_out, ptr(weight), ptr(bias),
             ptr(pre_in), pre_in.shape[1], weight.shape[1], n_out, precision, _stream(), C.byref(fl))
        return out, fl.value

    def incre_deconv_forward(self, pre, in_size, out_size, x, weight, pre_in, bias=None, precision=PREC_FP32):
        import torch
        x, weight, pre_in = x.contiguous(), weight.contiguous(), pre_in.contiguous()
        n_out = weight.shape[2]
        out = torch.empty(self.n_active(out_size), n_out, dtype=torch.float32, device=x.device)
        fl = _dbl(0)
        call("scn_incre_deconv_forward", self.h, pre.h, size3(in_size), size3(out_size), ptr(x), x.shape[1], ptr(out), n_out,
             ptr(weight), ptr(bias), ptr(pre_in), pre_in.shape[1], weight.shape[1], n_out, precision, _stream(), C.byref(fl))
        return out, fl.value

    def incre_bn_forward(self, pre, size, x, mean, var, gamma, beta, eps, leak, pre_out, pre_in):
        import torch
        x = x.contiguous()
        out = torch.empty_like(x)
        call("scn_incre_bn_forward", self.h, pre.h, size3(size), ptr(x), x.shape[1], ptr(out), x.shape[1], x.shape[1], ptr(mean),
             ptr(var), ptr(gamma), ptr(beta), float(eps), float(leak), ptr(pre_out.contiguous()), ptr(pre_in.contiguous()),
             _stream())
        return out


_cudart = None


def _memcpy_d2d(dst, src, nbytes):
    """cudaMemcpy(device -> device) through the CUDA runtime torch has already loaded."""
    global _cudart
    import torch  # noqa: F401
    if _cudart is None:
        _cudart = C.CDLL("libcudart.so.12")
        _cudart.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        _cudart.cudaMemcpy.restype = C.c_int
    r = _cudart.cudaMemcpy(dst, src, nbytes, 3)  # cudaMemcpyDeviceToDevice
    if int(r) != 0:
        raise ScnError(-2, "cudaMemcpy failed: %s" % r)


def _split(pairs, counts):
    out, o = [], 0
    for c in counts:
        out.append(pairs[o:o + int(c)])
        o += int(c)
    return out


def check_errors():
    """Synchronises the current stream and raises if a kernel flagged an asynchronous error."""
    call("scn_check_errors", _stream())


def bn_forward(x, mean, var, gamma, beta, eps, leak):
    import torch
    x = x.contiguous()
    out = torch.empty_like(x)
    call("scn_bn_forward", ptr(x), x.stride(0) if x.dim() == 2 and x.shape[0] else x.shape[1], ptr(out), x.shape[1],
         x.shape[0], x.shape[1], ptr(mean), ptr(var), ptr(gamma), ptr(beta), float(eps), float(leak), _stream())
    return out


def bn_forward_train(x, running_mean, running_var, gamma, beta, eps, momentum, leak):
    """Returns (out, save_mean, save_invstd); running_mean / running_var are updated in place."""
    import torch
    x = x.contiguous()
    out = torch.empty_like(x)
    sm = torch.empty(x.shape[1], dtype=torch.float32, device=x.device)
    si = torch.empty(x.shape[1], dtype=torch.float32, device=x.device)
    call("scn_bn_forward_train", ptr(x), x.shape[1], ptr(out), x.shape[1], x.shape[0], x.shape[1], ptr(running_mean),
         ptr(running_var), ptr(sm), ptr(si), ptr(gamma), ptr(beta), float(eps), float(momentum), float(leak), _stream())
    return out, sm, si


def nin_forward(x, weight, bias=None, precision=PREC_FP32):
    import torch
    x = x.contiguous()
    weight = weight.contiguous()
    out = torch.empty(x.shape[0], weight.shape[1], dtype=torch.float32, device=x.device)
    fl = _dbl(0)
    call("scn_nin_forward", ptr(x), x.shape[1], ptr(out), weight.shape[1], x.shape[0], ptr(weight), ptr(bias),
         weight.shape[0], weight.shape[1], precision, _stream(), C.byref(fl))
    return out, fl.value
