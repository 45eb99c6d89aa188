"""The allocation-free LayerNorm backward entry point, checked against the regular one and against the CPU oracle.

Some users of this library run where device allocation is not allowed at call time (inside a
framework's capture/replay region, under a fixed memory budget, or as a plugin that only owns the
buffers it is given).  `vb_layernorm_backward_noalloc` serves them: raw pointers in and out, partial
sums in a fixed array inside the library.  This test drives it through the C ABI twice in a row (the
array keeps the previous call's contents, so the second call must not depend on a clean array) and
compares with `vb_layernorm_backward` and with the CPU oracle's `layernorm_backward` at the tolerance the
other GPU tests use.

Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-5, 1e-4


def _close(got, want, name):
    err = np.abs(got - want) - (ATOL + RTOL * np.abs(want))
    assert err.max() <= 0, "%s: worst excess %.3e" % (name, err.max())


def _buffer(vb, arr=None, n=None):
    """A device slot (the test may allocate; the entry point under test does not) and its raw pointer."""
    L = vb.lib()
    slot = C.c_uint32(0)
    n = arr.size if arr is not None else n
    vb.vb_check(L.vb_alloc(n, 1, C.byref(slot)))
    if arr is not None:
        a = np.ascontiguousarray(arr, np.float32)
        vb.vb_check(L.vb_write(slot.value, 0, a.ctypes.data_as(vb.c_f32p), a.size))
    p = C.c_void_p()
    vb.vb_check(L.vb_ptr(slot.value, C.byref(p)))
    return slot.value, p


def _read(vb, slot, shape):
    out = np.empty(shape, np.float32)
    vb.vb_check(vb.lib().vb_read(slot, 0, out.ctypes.data_as(vb.c_f32p), out.size))
    return out


@pytest.mark.parametrize("rows,c", [(4096, 768), (37, 1024), (5, 12)])
def test_noalloc_layernorm_backward_matches_regular_entry_point(rows, c):
    import vearo_b200 as vb
    vb.init()
    L = vb.lib()
    L.vb_layernorm_backward_noalloc.argtypes = [C.c_void_p] * 6 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]
    stream = C.c_void_p()
    vb.vb_check(L.vb_stream(C.byref(stream)))
    rng = np.random.default_rng(7)
    for call in range(2):                      # two calls in a row share the library's scratch array
        x0 = (rng.standard_normal((rows, c)) * 2 + 0.3).astype(np.float32)
        w0 = rng.standard_normal(c).astype(np.float32)
        g0 = (rng.standard_normal((rows, c)) * 0.02).astype(np.float32)      # gradient-sized values: column sums over
        # thousands of rows then stay far above the absolute part of the tolerance
        # regular entry point
        x, w, b, g = (vb.Tensor.from_numpy(a) for a in (x0, w0, np.zeros(c, np.float32), g0))
        gx, gw, gb = vb.VbTensor(), vb.VbTensor(), vb.VbTensor()
        vb.vb_check(L.vb_layernorm_backward(C.byref(x.desc()), C.byref(w.desc()), C.byref(b.desc()), C.byref(g.desc()), 1e-5,
                                            C.byref(gx), C.byref(gw), C.byref(gb)))
        want = [_read(vb, gx.slot, (rows, c)), _read(vb, gw.slot, (c,)), _read(vb, gb.slot, (c,))]
        for t in (gx, gw, gb):
            vb.vb_check(L.vb_release(t.slot, None))
        # allocation-free entry point on caller-owned buffers
        sx, px = _buffer(vb, x0); sw, pw = _buffer(vb, w0); sg, pg = _buffer(vb, g0)
        sgx, pgx = _buffer(vb, n=rows * c); sgw, pgw = _buffer(vb, n=c); sgb, pgb = _buffer(vb, n=c)
        before = vb.memory_stats()
        vb.vb_check(L.vb_layernorm_backward_noalloc(px, pw, pg, pgx, pgw, pgb, rows, c, 1e-5, stream), "noalloc")
        after = vb.memory_stats()
        assert (after["live_bytes"], after["cached_bytes"]) == (before["live_bytes"], before["cached_bytes"])
        got = [_read(vb, sgx, (rows, c)), _read(vb, sgw, (c,)), _read(vb, sgb, (c,))]
        for s in (sx, sw, sg, sgx, sgw, sgb):
            vb.vb_check(L.vb_release(s, None))
        for a, b_, name in zip(got, want, ("gx", "gw", "gb")):
            _close(a, b_, "call %d %s" % (call, name))
        # ... and against the CPU oracle directly (crates/vearo-backend-cpu/src/lib.rs:745-858 through the LayerNorm arm)
        from oracle import oracle as orc
        orc.reset_all()
        ox, ow, ob = orc.Tensor.from_numpy(x0, True), orc.Tensor.from_numpy(w0, True), orc.Tensor.from_numpy(np.zeros(c, np.float32), True)
        n = rows * c
        ox.layernorm(ow, ob, 1e-5).mul(orc.Tensor.from_numpy(g0)).reshape([1, n]).matmul(
            orc.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        for a, t, name in zip(got, (ox, ow, ob), ("gx", "gw", "gb")):
            _close(a, t.grad().numpy(), "call %d %s vs oracle" % (call, name))


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    import vearo_b200 as vb
    vb.init()
    L = vb.lib()
    L.vb_layernorm_backward_noalloc.argtypes = [C.c_void_p] * 6 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]
    s, p = _buffer(vb, n=4096)
    for c in (2048, 1028, 6):
        assert L.vb_layernorm_backward_noalloc(p, p, p, p, p, p, 1, c, 1e-5, None) != 0
        assert b"at most 1024" in L.vb_last_error()
    vb.vb_check(L.vb_release(s, None))
