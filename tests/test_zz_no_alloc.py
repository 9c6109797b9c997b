"""The 1x1 convolution entry point that never allocates (scn_nin_forward_noalloc).

Some hosts hand out all device memory at start-up and must not see a library touch an allocator
afterwards; for them the library keeps the one piece of scratch this op needs (the transposed weights)
in a fixed buffer of its own.  The test drives the entry point through the C ABI and checks it against the
ordinary scn_nin_forward on the tensor-core path, with plane counts that entry point also gives to a tcgen05
kernel (it hands narrower layers to a warp-level kernel).  The two entry points run different tcgen05 kernels (one
tile per CTA here, the persistent kernel there) that add the same tf32 products in the same order of 32-plane steps,
so the results must agree to fp32 rounding.
Two calls in a row with different shapes and weights make sure nothing stale in the shared buffer leaks
from one call into the next.  This file is collected last so that a failure here cannot hide others.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from insconv import cabi

pytestmark = pytest.mark.gpu


def _noalloc(x, w, b):
    out = torch.empty(x.shape[0], w.shape[1], dtype=torch.float32, device=x.device)
    cabi.call("scn_nin_forward_noalloc", cabi.ptr(x), x.shape[1], cabi.ptr(out), w.shape[1], x.shape[0], cabi.ptr(w),
              cabi.ptr(b), w.shape[0], w.shape[1], torch.cuda.current_stream().cuda_stream)
    return out


def test_two_calls_match_the_allocating_entry_point(cuda):
    g = torch.Generator().manual_seed(5)
    for rows, n_in, n_out, with_bias in ((20000, 96, 64, False), (20011, 128, 96, True)):
        x = torch.randn(rows, n_in, generator=g).to(cuda)
        w = (torch.randn(n_in, n_out, generator=g) * (2.0 / n_in) ** 0.5).to(cuda)
        b = torch.randn(n_out, generator=g).to(cuda) if with_bias else None
        want, _ = cabi.nin_forward(x, w, b, cabi.PREC_TF32)
        got = _noalloc(x, w, b)
        cabi.check_errors()
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 1e-5 * scale
        # and both sit within the tensor-core tolerance of an fp32 product
        ref = x @ w + (b if with_bias else 0)
        assert float((got - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


def _pool_counters():
    """(reserved now, reserved high-water mark, used now, used high-water mark) of the device's stream-ordered pool,
    the one the library's temporaries come from."""
    rt = C.CDLL("libcudart.so.12")
    pool = C.c_void_p()
    assert rt.cudaDeviceGetDefaultMemPool(C.byref(pool), C.c_int(torch.cuda.current_device())) == 0
    vals = []
    for attr in (5, 6, 7, 8):  # cudaMemPoolAttrReservedMemCurrent, ReservedMemHigh, UsedMemCurrent, UsedMemHigh
        v = C.c_uint64(0)
        assert rt.cudaMemPoolGetAttribute(pool, C.c_int(attr), C.byref(v)) == 0
        vals.append(v.value)
    return tuple(vals), rt, pool


def test_no_allocator_is_touched(cuda):
    """Neither the stream-ordered pool of the device (high-water marks reset just before, unchanged after) nor
    torch's allocator sees the call; the ordinary entry point, run the same way, does move the pool's mark."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(30000, 128, generator=g).to(cuda)
    w = (torch.randn(128, 96, generator=g) * 0.1).to(cuda)
    out = torch.empty(30000, 96, device=cuda)
    args = (cabi.ptr(x), 128, cabi.ptr(out), 96, 30000, cabi.ptr(w), None, 128, 96, torch.cuda.current_stream().cuda_stream)
    cabi.call("scn_nin_forward_noalloc", *args)  # first call: module load, function attributes
    torch.cuda.synchronize()
    _, rt, pool = _pool_counters()
    zero = C.c_uint64(0)
    for attr in (6, 8):  # high-water marks can be reset to zero = to the current value
        assert rt.cudaMemPoolSetAttribute(pool, C.c_int(attr), C.byref(zero)) == 0
    before, _, _ = _pool_counters()
    torch_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    for _ in range(3):
        cabi.call("scn_nin_forward_noalloc", *args)
    torch.cuda.synchronize()
    after, _, _ = _pool_counters()
    assert after == before, (before, after)
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before
    cabi.check_errors()
    # the same probe does see the allocating entry point (it takes its transposed weights from the pool)
    fl = C.c_double(0)
    cabi.call("scn_nin_forward", cabi.ptr(x), 128, cabi.ptr(out), 96, 30000, cabi.ptr(w), None, 128, 96, cabi.PREC_TF32,
              torch.cuda.current_stream().cuda_stream, C.byref(fl))
    torch.cuda.synchronize()
    moved, _, _ = _pool_counters()
    assert moved[3] > before[3], (before, moved)


def test_sizes_beyond_the_fixed_buffer_are_refused(cuda):
    x = torch.zeros(256, 1024, device=cuda)
    w = torch.zeros(1024, 256, device=cuda)  # 262144 weights > 131072
    with pytest.raises(cabi.ScnError) as e:
        _noalloc(x, w, None)
    assert e.value.code == -4 and "scratch" in str(e.value)
    with pytest.raises(cabi.ScnError):
        _noalloc(torch.zeros(8, 48, device=cuda), torch.zeros(48, 32, device=cuda), None)  # 48 is not a multiple of 32
    # the device is still fine and the next valid call works
    xs = torch.ones(130, 32, device=cuda)
    ws = torch.eye(32, device=cuda)
    assert torch.allclose(_noalloc(xs, ws, None), xs)
