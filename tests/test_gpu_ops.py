"""Per-op parity: the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Bar (north star): |gpu - cpu| <= 1e-5 + 1e-4 * |cpu| per element, f32, with a guard against
degenerate all-zero outputs in the style of crates/vearo/tests/fused_attention_parity.rs:114-116.
Every case is written once, as a function of the tensor class, and run on both sides.
"""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-5, 1e-4


@pytest.fixture(scope="module")
def vb():
    import vearo_b200 as v
    v.init()
    return v


def assert_close(gpu, cpu, name="", atol=ATOL, rtol=RTOL, guard=True):
    gpu = np.asarray(gpu); cpu = np.asarray(cpu)
    assert gpu.shape == cpu.shape, (name, gpu.shape, cpu.shape)
    if cpu.size == 0:
        return
    assert np.isfinite(gpu).all(), name
    if guard and cpu.size > 4:
        assert np.abs(cpu).max() > 1e-6, "degenerate oracle output in " + name
    err = np.abs(gpu - cpu) - (atol + rtol * np.abs(cpu))
    assert err.max() <= 0, "%s: worst excess %.3e at %s (gpu %r cpu %r)" % (
        name, err.max(), np.unravel_index(err.argmax(), err.shape), gpu.flat[err.argmax()], cpu.flat[err.argmax()])


def both(vb, fn, **kw):
    """Run `fn(T, mod)` on the oracle and on the GPU; compare every returned array."""
    orc.reset_all()
    cpu = fn(orc.Tensor, orc)
    cpu = [c.numpy() for c in cpu]
    vb.zero_gradients(); vb.reset_active_tape()
    gpu = fn(vb.Tensor, vb)
    gpu = [g.numpy() for g in gpu]
    vb.check_errors()
    assert len(cpu) == len(gpu)
    for i, (g, c) in enumerate(zip(gpu, cpu)):
        assert_close(g, c, "%s[%d]" % (fn.__name__, i), **kw)


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


# ---- elementwise + broadcasting (crates/vearo-backend-cuda/src/lib.rs:1643-1699, 1713-1826) ----------
@pytest.mark.parametrize("sa,sb", [((2, 3), (2, 3)), ((1, 3), (2, 1)), ((4, 5, 6), (6,)), ((4, 5, 6), (1,)), ((1,), (7, 3)),
                                   ((3, 1, 5), (4, 1)), ((1037,), (1037,)), ((2, 0, 3), (3,)), ((8, 16, 64), (8, 1, 64))])
def test_binary_broadcast(vb, sa, sb):
    a, b = rnd(1, *sa), rnd(2, *sb) + 3.0

    def case(T, m):
        x, y = T.from_numpy(a), T.from_numpy(b)
        return [x.add(y), x.sub(y), x.mul(y), x.div(y)]
    both(vb, case, guard=False)


def test_binary_on_views(vb):
    a, b = rnd(3, 6, 4), rnd(4, 4, 6)

    def case(T, m):
        x, y = T.from_numpy(a), T.from_numpy(b)
        return [x.transpose(0, 1).add(y), x.mul(y.transpose(0, 1)), x.reshape([2, 3, 4]).permute([2, 0, 1]).contiguous()]
    both(vb, case)


@pytest.mark.parametrize("sa,sb,ta,tb", [((5, 7), (7, 3), False, False), ((130, 70), (70, 129), False, False), ((64, 32), (48, 32), False, True),
                                         ((32, 64), (32, 48), True, False), ((2, 3, 9, 5), (2, 3, 5, 4), False, False),
                                         ((4, 16, 8), (8, 12), False, False), ((1, 6, 8), (5, 8, 7), False, False), ((3, 0, 4), (4, 5), False, False)])
def test_matmul(vb, sa, sb, ta, tb):
    a, b = rnd(5, *sa), rnd(6, *sb)

    def case(T, m):
        x, y = T.from_numpy(a), T.from_numpy(b)
        if ta: x = x.transpose(len(sa) - 2, len(sa) - 1)
        if tb: y = y.transpose(len(sb) - 2, len(sb) - 1)
        return [x.matmul(y)]
    both(vb, case, guard=False)


def test_matmul_backward_with_broadcast_batch(vb):
    a, b = rnd(7, 3, 10, 6), rnd(8, 6, 5)

    def case(T, m):
        x, y = T.from_numpy(a, True), T.from_numpy(b, True)
        out = x.matmul(y)
        out.mul(out).reshape([1, 150]).matmul(T.from_numpy(np.ones((150, 1), np.float32))).reshape([1]).backward()
        return [out, x.grad(), y.grad()]
    both(vb, case)


def test_linear_fused_matches_reference_op_sequence(vb):
    """Linear::forward = transpose, matmul, add (crates/vearo-nn/src/lib.rs:120-128); the fused
    `linear` op must give the same values and gradients as that sequence on the oracle."""
    x0, w0, b0 = rnd(9, 4, 9, 24), rnd(10, 17, 24), rnd(11, 17)
    tgt = rnd(12, 4, 9, 17)

    def run(T, fused):
        x, w, b = T.from_numpy(x0, True), T.from_numpy(w0, True), T.from_numpy(b0, True)
        y = x.linear(w, b) if fused else x.matmul(w.transpose(0, 1)).add(b)
        loss = y.mul(T.from_numpy(tgt)).reshape([1, tgt.size]).matmul(T.from_numpy(np.ones((tgt.size, 1), np.float32))).reshape([1])
        loss.backward()
        return [t.numpy() for t in (y, x.grad(), w.grad().contiguous(), b.grad())]
    orc.reset_all()
    cpu = run(orc.Tensor, False)
    for fused in (True, False):
        vb.zero_gradients(); vb.reset_active_tape()
        for g, c, n in zip(run(vb.Tensor, fused), cpu, "y gx gw gb".split()):
            assert_close(g, c, "linear fused=%s %s" % (fused, n))


# ---- activations, reductions, softmax --------------------------------------------------------------
def test_relu_gelu_forward_backward(vb):
    a = rnd(13, 33, 129, scale=2.0)
    a.flat[:4] = [0.0, -0.0, 1e-30, -1e-30]
    go = rnd(14, 33, 129)

    def case(T, m):
        outs = []
        for name in ("relu", "gelu"):
            x = T.from_numpy(a, True)
            y = getattr(x, name)()
            y.mul(T.from_numpy(go)).reshape([1, a.size]).matmul(T.from_numpy(np.ones((a.size, 1), np.float32))).reshape([1]).backward()
            outs += [y, x.grad()]
        return outs
    both(vb, case)


@pytest.mark.parametrize("shape,dim", [((6, 11), 1), ((6, 11), 0), ((3, 4, 7), 1), ((5, 1024), 1), ((2, 3, 5000), 2)])
def test_sum_mean_softmax(vb, shape, dim):
    a, go = rnd(15, *shape), rnd(16, *shape)

    def case(T, m):
        x = T.from_numpy(a, True)
        y = x.softmax(dim)
        n = a.size
        y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        x2 = T.from_numpy(a)
        return [y, x.grad(), x2.sum(dim, False), x2.sum(dim, True), x2.mean(dim, False), x2.transpose(0, 1).sum(0, False)]
    both(vb, case)


def test_sum_mean_backward(vb):
    a = rnd(17, 5, 6)

    def case(T, m):
        x = T.from_numpy(a, True)
        x.mul(x).mean(1, False).sum(0, False).backward()
        return [x.grad()]
    both(vb, case)


@pytest.mark.parametrize("target", [(7,), (1, 7), (5, 1), (3, 1, 1), (1,), (3, 5, 7), (5, 7)])
def test_reduce_to(vb, target):
    g = rnd(18, 3, 5, 7)
    orc.reset_all()
    cpu = orc.Tensor.from_numpy(g).reduce_to(target).numpy()
    import ctypes as C
    t = vb.Tensor.from_numpy(g)
    out = vb.VbTensor()
    dims = (C.c_int64 * len(target))(*target)
    vb.vb_check(vb.lib().vb_reduce_to(C.byref(t.desc()), dims, len(target), C.byref(out)), "vb_reduce_to")
    got = np.empty(target, np.float32)
    vb.vb_check(vb.lib().vb_read(out.slot, 0, got.ctypes.data_as(vb.c_f32p), got.size))
    vb.vb_check(vb.lib().vb_release(out.slot, None))
    assert_close(got, cpu, "reduce_to %r" % (target,))


# ---- layernorm -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,c", [(5, 12), (64, 768), (33, 100), (7, 1024), (3, 13), (4, 2048), (257, 256)])
def test_layernorm_forward_backward(vb, rows, c):
    x0, w0, b0, go = rnd(19, rows, c) * 2 + 0.5, rnd(20, c), rnd(21, c), rnd(22, rows, c)

    def case(T, m):
        x, w, b = T.from_numpy(x0), T.from_numpy(w0), T.from_numpy(b0)
        y = x.layernorm(w, b, 1e-5)
        xr = T.from_numpy(x0, True); wr = T.from_numpy(w0, True); br = T.from_numpy(b0, True)
        n = x0.size
        xr.layernorm(wr, br, 1e-5).mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [y, xr.grad(), wr.grad(), br.grad()]
    both(vb, case)


def test_layernorm_3d_and_noncontiguous(vb):
    x0, w0, b0 = rnd(23, 6, 8, 16), rnd(24, 16), rnd(25, 16)

    def case(T, m):
        x = T.from_numpy(x0)
        return [x.layernorm(T.from_numpy(w0), T.from_numpy(b0), 1e-5),
                x.transpose(0, 1).layernorm(T.from_numpy(w0), T.from_numpy(b0), 1e-5),
                T.from_numpy(np.zeros((2, 0, 16), np.float32)).layernorm(T.from_numpy(w0), T.from_numpy(b0), 1e-5)]
    both(vb, case)


def test_layernorm_backward_is_bit_reproducible(vb):
    x0, w0, go = rnd(26, 4096, 768), rnd(27, 768), rnd(28, 4096, 768)
    outs = []
    for _ in range(2):
        x, w, b, g = (vb.Tensor.from_numpy(a) for a in (x0, w0, np.zeros(768, np.float32), go))
        import ctypes as C
        gx, gw, gb = vb.VbTensor(), vb.VbTensor(), vb.VbTensor()
        vb.vb_check(vb.lib().vb_layernorm_backward(C.byref(x.desc()), C.byref(w.desc()), C.byref(b.desc()), C.byref(g.desc()), 1e-5,
                                                   C.byref(gx), C.byref(gw), C.byref(gb)))
        res = []
        for t in (gx, gw, gb):
            a = np.empty(t.shape, np.float32)
            vb.vb_check(vb.lib().vb_read(t.slot, 0, a.ctypes.data_as(vb.c_f32p), a.size))
            vb.vb_check(vb.lib().vb_release(t.slot, None))
            res.append(a)
        outs.append(res)
    for a, b in zip(*outs):
        assert (a.view(np.uint32) == b.view(np.uint32)).all()
    # size-independent property: with gamma fixed, each dx row sums to ~0
    assert np.abs(outs[0][0].sum(1)).max() < 1e-3


# ---- embedding / cross-entropy --------------------------------------------------------------------------
def test_embedding_forward_backward(vb):
    w0 = rnd(29, 50, 24); ids = np.random.default_rng(30).integers(0, 50, (3, 17)).astype(np.float32); go = rnd(31, 3, 17, 24)
    ids[0, :5] = 7   # repeated ids accumulate

    def case(T, m):
        w = T.from_numpy(w0, True)
        y = T.from_numpy(ids).embedding(w)
        n = go.size
        y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [y, w.grad()]
    both(vb, case)


@pytest.mark.parametrize("vocab,d,shape", [(300, 128, (2, 100)), (4000, 768, (3, 700)), (64, 8, (2, 40))])
def test_embedding_backward_owner_scan(vb, vocab, d, shape):
    """Fewer positions than table rows: the warp of the first position naming a row sums all its duplicates in order
    (bit-identical to the sequential sum of the CPU backend), untouched rows are exact zeros."""
    w0 = rnd(34, vocab, d); go = rnd(36, *shape, d)
    ids = np.random.default_rng(35).integers(0, vocab, shape).astype(np.float32)
    ids[0, :9] = 5; ids[-1, -3:] = 5; ids[0, 20:24] = vocab - 1

    def run(T):
        w = T.from_numpy(w0, True)
        y = T.from_numpy(ids).embedding(w)
        n = go.size
        y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return w.grad().numpy()
    orc.reset_all()
    ref = run(orc.Tensor)
    vb.zero_gradients(); vb.reset_active_tape()
    got = run(vb.Tensor)
    want = np.zeros((vocab, d), np.float32)
    for pos, i in enumerate(ids.reshape(-1).astype(np.int64)):      # sequential f32 sum in position order
        want[i] += go.reshape(-1, d)[pos]
    assert np.array_equal(got, want)
    assert_close(got, ref, "embedding backward")
    vb.check_errors()


@pytest.mark.parametrize("ids,msg", [([-1.0, 0.0], "negative"), ([2.0, 0.0], "out of")])
def test_invalid_ids_are_reported_not_skipped(vb, ids, msg):
    """CPU contract (crates/vearo-backend-cpu/src/lib.rs:2865-2899): invalid ids are an error."""
    w = vb.Tensor.from_numpy(np.zeros((2, 3), np.float32))
    vb.Tensor.from_numpy(np.array(ids, np.float32)).embedding(w)
    with pytest.raises(vb.VearoError, match=msg):
        vb.check_errors()
    vb.check_errors()   # flag is cleared by the read
    vb.Tensor.from_numpy(np.zeros((2, 2), np.float32)).cross_entropy(vb.Tensor.from_numpy(np.array(ids, np.float32)))
    with pytest.raises(vb.VearoError, match=msg):
        vb.check_errors()


@pytest.mark.parametrize("rows,v", [(6, 11), (4, 1000), (3, 50304), (9, 4097)])
def test_cross_entropy(vb, rows, v):
    l0 = rnd(32, rows, v, scale=3.0); t0 = np.random.default_rng(33).integers(0, v, rows).astype(np.float32)

    def case(T, m):
        l = T.from_numpy(l0, True)
        loss = l.cross_entropy(T.from_numpy(t0))
        loss.backward()
        return [loss, l.grad()]
    both(vb, case, guard=False)


@pytest.mark.parametrize("rows,v,scale", [(7, 1001, None), (64, 4096, None), (5, 50304, 0.5)])
def test_cross_entropy_fused_forward_backward(vb, rows, v, scale):
    """The one-pass form (loss out, logits overwritten with their gradient) against the oracle's two calls; with a loss that
    is scaled afterwards the upstream gradient is not 1 and the stored gradient is multiplied by it."""
    x0, w0 = rnd(232, rows, 24, scale=1.0), rnd(233, 24, v, scale=0.8)
    t0 = np.random.default_rng(234).integers(0, v, rows).astype(np.float32)

    def case(T, m):
        x, w = T.from_numpy(x0, True), T.from_numpy(w0, True)
        logits = x.matmul(w)
        loss = logits.cross_entropy_consuming(T.from_numpy(t0)) if m is not orc else logits.cross_entropy(T.from_numpy(t0))
        del logits
        out = loss if scale is None else loss.mul(T.from_numpy(np.array([scale], np.float32)))
        out.backward()
        return [loss, x.grad(), w.grad().contiguous()]
    both(vb, case, guard=False)


def test_cross_entropy_stability_and_backward_without_stats(vb):
    import ctypes as C
    loss = vb.Tensor.from_numpy(np.array([[1000.0, -1000.0]], np.float32)).cross_entropy(vb.Tensor.from_numpy(np.array([0.0], np.float32)))
    assert abs(loss.numpy()[0]) < 1e-4 and loss.shape == (1,)
    l0 = rnd(34, 5, 777, scale=2.0); t0 = np.random.default_rng(35).integers(0, 777, 5).astype(np.float32)
    orc.reset_all()
    cpu = orc.Tensor.from_numpy(l0).cross_entropy_backward(orc.Tensor.from_numpy(t0), orc.Tensor.from_numpy(np.array([0.5], np.float32))).numpy()
    l, t, g = vb.Tensor.from_numpy(l0), vb.Tensor.from_numpy(t0), vb.Tensor.from_numpy(np.array([0.5], np.float32))
    out = vb.VbTensor()
    vb.vb_check(vb.lib().vb_cross_entropy_backward(C.byref(l.desc()), C.byref(t.desc()), C.byref(g.desc()), None, C.byref(out)))
    got = np.empty((5, 777), np.float32)
    vb.vb_check(vb.lib().vb_read(out.slot, 0, got.ctypes.data_as(vb.c_f32p), got.size))
    vb.vb_check(vb.lib().vb_release(out.slot, None))
    assert_close(got, cpu, "ce backward (no stats)")


# ---- conv / pool / batchnorm (crates/vearo-backend-cuda/src/lib.rs:1829-1979, crates/vearo/tests/batchnorm.rs) ----
@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 0, 3), (1, 0, 2), (2, 1, 3)])
def test_conv2d_forward_backward(vb, stride, pad, k):
    x0, w0, b0 = rnd(36, 3, 4, 9, 8), rnd(37, 5, 4, k, k), rnd(38, 5)

    def case(T, m):
        x, w, b = T.from_numpy(x0, True), T.from_numpy(w0, True), T.from_numpy(b0, True)
        y = x.conv2d(w, b, stride, pad)
        go = np.sin(np.arange(int(np.prod(y.shape)), dtype=np.float32) * 0.37 + 1).reshape(y.shape)
        n = go.size
        y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [y, x.grad(), w.grad(), b.grad()]
    both(vb, case)


@pytest.mark.parametrize("n,cin,cout,hw,stride,pad,k", [
    (6, 16, 32, (14, 12), 1, 1, 3),     # the ConvNet layer shape in small: unfolded rows, MN-major operands
    (4, 3, 64, (32, 32), 1, 1, 3),      # first layer: 27 taps (row length padded to 28), input gradient still asked for
    (5, 24, 40, (13, 11), 2, 0, 3),     # stride 2, no padding, ragged tiles everywhere
    (3, 8, 48, (10, 10), 1, 0, 2),      # even kernel
])
def test_conv2d_tensor_core_path(vb, n, cin, cout, hw, stride, pad, k):
    """Convolutions with enough work are unfolded and run as tensor-core GEMMs; same results as the direct sum."""
    x0, w0, b0 = rnd(80, n, cin, *hw, scale=0.5), rnd(81, cout, cin, k, k, scale=0.2), rnd(82, cout)

    def case(T, m):
        x, w, b = T.from_numpy(x0, True), T.from_numpy(w0, True), T.from_numpy(b0, True)
        y = x.conv2d(w, b, stride, pad)
        go = (np.sin(np.arange(int(np.prod(y.shape)), dtype=np.float32) * 0.37 + 1) * 0.05).reshape(y.shape)
        cnt = go.size
        y.mul(T.from_numpy(go)).reshape([1, cnt]).matmul(T.from_numpy(np.ones((cnt, 1), np.float32))).reshape([1]).backward()
        return [y, x.grad(), w.grad(), b.grad()]
    both(vb, case)


@pytest.mark.parametrize("k,s,p", [(2, 2, 0), (3, 2, 1), (3, 1, 1), (2, 1, 0)])
def test_pools_forward_backward(vb, k, s, p):
    x0 = rnd(39, 2, 3, 9, 7)
    x0[0, 0, :2, :2] = 5.0   # ties: the first maximum in scan order wins

    def case(T, m):
        outs = []
        for name in ("maxpool2d", "avgpool2d"):
            x = T.from_numpy(x0, True)
            y = getattr(x, name)(k, s, p)
            go = np.cos(np.arange(int(np.prod(y.shape)), dtype=np.float32) * 0.11 + 2).reshape(y.shape)
            n = go.size
            y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
            outs += [y, x.grad()]
        return outs
    both(vb, case)


@pytest.mark.parametrize("training", [True, False])
def test_batchnorm(vb, training):
    x0 = rnd(40, 6, 5, 7, 4) * 2 + 1; g0, b0, go = rnd(41, 5), rnd(42, 5), rnd(43, 6, 5, 7, 4)
    rm0 = np.linspace(-0.5, 0.5, 5).astype(np.float32); rv0 = np.linspace(0.5, 1.5, 5).astype(np.float32)

    def case(T, m):
        x, g, b = T.from_numpy(x0, True), T.from_numpy(g0, True), T.from_numpy(b0, True)
        rm, rv = T.from_numpy(rm0), T.from_numpy(rv0)
        y = x.batchnorm(g, b, rm, rv, training, 0.1, 1e-5)
        n = go.size
        y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [y, rm, rv, x.grad(), g.grad(), b.grad()]
    both(vb, case)


@pytest.mark.parametrize("B,S,H,dk,masked", [(2, 40, 3, 8, True), (1, 256, 2, 64, True), (2, 64, 4, 16, False)])
def test_fused_attention_packed(vb, B, S, H, dk, masked):
    """Attention over the packed [B, S, 3*D] projection (q | k | v column blocks) against the oracle fed with the three
    head-split tensors; the single packed gradient must be the three gradients side by side."""
    D = H * dk
    qkv0 = (rnd(90, B, S, 3 * D) * 0.5).astype(np.float32); go = rnd(91, B, S, D)
    mask0 = np.triu(np.full((S, S), -1e9, np.float32), 1)

    orc.reset_all()
    parts = [orc.Tensor.from_numpy(np.ascontiguousarray(qkv0[:, :, i * D:(i + 1) * D].reshape(B, S, H, dk).transpose(0, 2, 1, 3)), True) for i in range(3)]
    o = parts[0].fused_attention(parts[1], parts[2], orc.Tensor.from_numpy(mask0) if masked else None)
    o = o.transpose(1, 2).reshape([B, S, D])
    n = go.size
    o.mul(orc.Tensor.from_numpy(go)).reshape([1, n]).matmul(orc.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
    want_o = o.numpy()
    want_g = np.concatenate([p.grad().numpy().transpose(0, 2, 1, 3).reshape(B, S, D) for p in parts], axis=2)

    vb.zero_gradients(); vb.reset_active_tape()
    x = vb.Tensor.from_numpy(qkv0, True)
    y = x.fused_attention_packed(H, vb.Tensor.from_numpy(mask0) if masked else None)
    y.mul(vb.Tensor.from_numpy(go)).reshape([1, n]).matmul(vb.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
    assert_close(y.numpy(), want_o, "packed attention out")
    assert_close(x.grad().numpy(), want_g, "packed attention dqkv")
    vb.check_errors()


@pytest.mark.parametrize("shape,training", [((6, 5, 8, 12), True), ((3, 7, 9, 7), True), ((4, 3, 6, 6), False), ((40, 16, 16, 16), True)])
def test_bn_relu_maxpool_fused(vb, shape, training):
    """The fused op against the reference's three separate ops (and their three backward arms) on the CPU oracle;
    odd heights / widths leave elements outside every pooling window, exact ties and all-negative windows included."""
    n, c, h, w = shape
    x0 = rnd(44, *shape) * 1.5 + 0.2
    x0[0, 0, :2, :2] = 0.7            # a window of four equal values: the first tap takes the gradient
    x0[0, 1, :2, :2] = -5.0           # a window the rectifier zeroes entirely
    g0, b0 = (rnd(45, c) * 0.3 + 1).astype(np.float32), rnd(46, c) * 0.2
    go = rnd(47, n, c, h // 2, w // 2)
    rm0 = np.linspace(-0.5, 0.5, c).astype(np.float32); rv0 = np.linspace(0.5, 1.5, c).astype(np.float32)

    def run(T, fused):
        x, g, b = T.from_numpy(x0, True), T.from_numpy(g0, True), T.from_numpy(b0, True)
        rm, rv = T.from_numpy(rm0), T.from_numpy(rv0)
        y = x.bn_relu_maxpool(g, b, rm, rv, training, 0.1, 1e-5) if fused else x.batchnorm(g, b, rm, rv, training, 0.1, 1e-5).relu().maxpool2d(2, 2, 0)
        cnt = go.size
        y.mul(T.from_numpy(go)).reshape([1, cnt]).matmul(T.from_numpy(np.ones((cnt, 1), np.float32))).reshape([1]).backward()
        return [t.numpy() for t in (y, rm, rv, x.grad(), g.grad(), b.grad())]
    orc.reset_all()
    cpu = run(orc.Tensor, False)
    vb.zero_gradients(); vb.reset_active_tape()
    got = run(vb.Tensor, True)
    for a, b_, name in zip(got, cpu, "y running_mean running_var dx dgamma dbeta".split()):
        assert_close(a, b_, "bn_relu_maxpool " + name)
    vb.check_errors()


# ---- attention (crates/vearo/tests/fused_attention_parity.rs) ------------------------------------------------
@pytest.mark.parametrize("B,H,S,dk,masked", [(2, 3, 6, 4, True), (1, 2, 33, 16, True), (2, 2, 130, 64, True), (1, 1, 7, 8, False),
                                                (1, 2, 256, 64, True), (2, 1, 128, 32, True), (1, 2, 384, 64, True), (1, 2, 256, 64, "random")])
def test_fused_attention(vb, B, H, S, dk, masked):
    idx = np.arange(B * H * S * dk, dtype=np.float32)
    fill = lambda ph: (np.sin(0.37 * idx + ph) / 2 + np.cos(0.11 * idx + ph) / 4).reshape(B, H, S, dk).astype(np.float32)
    q0, k0, v0, go = fill(0.0), fill(1.0), fill(2.0), fill(3.0)
    mask0 = np.triu(np.full((S, S), -1e9, np.float32), 1)      # S a multiple of 128 takes the triangular (causal) fast path
    if masked == "random":
        mask0 = (np.random.default_rng(5).standard_normal((S, S)) * 2).astype(np.float32)

    def case(T, m):
        q, k, v = T.from_numpy(q0, True), T.from_numpy(k0, True), T.from_numpy(v0, True)
        mask = T.from_numpy(mask0) if masked else None
        o = q.fused_attention(k, v, mask)
        n = go.size
        o.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [o, q.grad(), k.grad(), v.grad()]
    both(vb, case)


def test_fused_attention_on_head_split_views(vb):
    """q, k, v as the [B,S,H,dk] -> transpose(1,2) views MultiHeadAttention feeds (crates/vearo-nn/src/lib.rs:598-600)."""
    B, S, H, dk = 2, 9, 3, 8
    q0, k0, v0 = rnd(44, B, S, H * dk), rnd(45, B, S, H * dk), rnd(46, B, S, H * dk)
    m4 = rnd(47, B, 1, S, S)

    def case(T, m):
        q, k, v = (T.from_numpy(a).reshape([B, S, H, dk]).transpose(1, 2) for a in (q0, k0, v0))
        return [q.fused_attention(k, v, T.from_numpy(m4)), q.fused_attention(k, v, None)]
    both(vb, case)


# ---- optimizers ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["adamw", "sgd"])
def test_optimizer_steps_match_oracle(vb, kind):
    w0 = [rnd(48, 37), rnd(49, 5, 1031), rnd(50, 16384 * 2 + 3)]
    gs = [[rnd(100 + 10 * s + i, *w.shape) for i, w in enumerate(w0)] for s in range(3)]

    def case(T, m):
        ws = [T.from_numpy(w, True) for w in w0]
        opt = m.AdamW(ws, 1e-2, 0.9, 0.999, 1e-8, 0.1) if kind == "adamw" else m.SGD(ws, 0.1, 0.9, 0.01)
        for s in range(3):
            m.zero_gradients(); m.reset_active_tape()
            loss = None
            for w, g in zip(ws[:2] if s == 1 else ws, gs[s]):   # step 1: the last parameter gets no gradient
                n = g.size
                term = w.mul(T.from_numpy(g)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1])
                loss = term if loss is None else loss.add(term)
            loss.backward()
            opt.step()
        return ws
    both(vb, case)


def test_adamw_8bit_matches_oracle_bit_for_bit(vb):
    """AdamW8bit (crates/vearo-optim/src/lib.rs:211-303): after every step the int8 moments, their block scales and the
    weights equal the CPU restatement's exactly -- the kernel uses single-rounding arithmetic in the reference's order,
    so no update can fall on the other side of a quantizer boundary.  Sizes cover a partial last block, a tensor of
    several chunks with an unaligned tail, a parameter skipped for one step, and a block of zero gradients."""
    w0 = [rnd(148, 37), rnd(149, 5, 1031), rnd(150, 16384 * 2 + 259), rnd(151, 512)]
    gs = [[rnd(200 + 10 * s + i, *w.shape) for i, w in enumerate(w0)] for s in range(4)]
    for s in range(4):
        gs[s][3][:256] = 0.0                     # m and v of that block stay zero: scale 0, zeros stored

    def run(T, m):
        ws = [T.from_numpy(w, True) for w in w0]
        opt = m.AdamW8bit(ws, 1e-2, 0.9, 0.999, 1e-8, 0.1)
        out = []
        for s in range(4):
            m.zero_gradients(); m.reset_active_tape()
            loss = None
            for w, g in zip(ws[:2] + ws[3:] if s == 1 else ws, gs[s][:2] + gs[s][3:] if s == 1 else gs[s]):
                term = w.mul(T.from_numpy(g)).reshape([1, g.size]).sum(1, False).reshape([1])
                loss = term if loss is None else loss.add(term)
            loss.backward()
            opt.step()
            out.append([w.numpy().copy() for w in ws] + [a.copy() for i in range(len(ws)) for a in opt.state(i)])
        return out
    orc.reset_all()
    want = run(orc.Tensor, orc)
    vb.zero_gradients(); vb.reset_active_tape()
    got = run(vb.Tensor, vb)
    for s, (a, b) in enumerate(zip(got, want)):
        for k, (x, y) in enumerate(zip(a, b)):
            assert x.dtype == y.dtype and np.array_equal(x, y), "step %d item %d differs (max %g)" % (
                s, k, np.abs(x.astype(np.float64) - y.astype(np.float64)).max())
    # the reference's own test (lib.rs:461-505): 8-bit stays within 1e-2 of plain AdamW after five steps
    wa, wb = vb.Tensor.from_numpy(np.array([1, 2, 3, 4], np.float32), True), vb.Tensor.from_numpy(np.array([1, 2, 3, 4], np.float32), True)
    oa, ob = vb.AdamW([wa], 0.1, 0.9, 0.999, 1e-8, 0.01), vb.AdamW8bit([wb], 0.1, 0.9, 0.999, 1e-8, 0.01)
    for _ in range(5):
        vb.zero_gradients(); vb.reset_active_tape()
        wa.mul(wa).sum(0, False).backward(); oa.step()
        vb.zero_gradients(); vb.reset_active_tape()
        wb.mul(wb).sum(0, False).backward(); ob.step()
    assert np.abs(wa.numpy() - wb.numpy()).max() < 1e-2
    vb.check_errors()


def test_clip_grad_norm_known_answer_and_fused_clip(vb):
    """crates/vearo-optim/src/lib.rs:438-459: grads [6, 8] -> norm 10, clipped to [3, 4]."""
    x = vb.Tensor.from_numpy(np.array([3.0, 4.0], np.float32), True)
    x.mul(x).sum(0, False).backward()
    norm = vb.clip_grad_norm([x], 5.0)
    assert abs(norm - 10.0) < 1e-4
    np.testing.assert_allclose(x.grad().numpy(), [3.0, 4.0], atol=1e-3)
    # fused clip + SGD step equals clip, then step, on the oracle
    w0, g0 = rnd(51, 1000), rnd(52, 1000)

    def case(T, m):
        w = T.from_numpy(w0, True)
        opt = m.SGD([w], 0.1, 0.0, 0.0)
        w.mul(T.from_numpy(g0)).sum(0, False).backward()
        if m is orc:
            n = m.clip_grad_norm([w], 1.0); opt.step()
        else:
            n = opt.clip_and_step(1.0)
        return [w, T.from_numpy(np.array([n], np.float32))]
    both(vb, case)


def test_single_tensor_adamw_through_raw_abi(vb):
    """vb_adamw_step is the drop-in for Tensor::adamw_step (crates/vearo-core/src/tensor.rs:931-1023)."""
    import ctypes as C
    w0, gsteps = rnd(53, 4099), [rnd(54 + i, 4099) for i in range(3)]
    orc.reset_all()
    w = orc.Tensor.from_numpy(w0, True); opt = orc.AdamW([w], 3e-3, 0.9, 0.999, 1e-8, 0.05)
    for g in gsteps:
        orc.zero_gradients(); orc.reset_active_tape()
        w.mul(orc.Tensor.from_numpy(g)).sum(0).backward(); opt.step()
    L = vb.lib()
    slots = [C.c_uint32(0) for _ in range(4)]
    for s in slots:
        vb.vb_check(L.vb_alloc(4099, 1, C.byref(s)))
    vb.vb_check(L.vb_write(slots[0].value, 0, w0.ctypes.data_as(vb.c_f32p), 4099))
    wt = vb.VbTensor.contiguous(slots[0].value, (4099,)); gt = vb.VbTensor.contiguous(slots[1].value, (4099,))
    for t, g in enumerate(gsteps, 1):
        vb.vb_check(L.vb_write(slots[1].value, 0, g.ctypes.data_as(vb.c_f32p), 4099))
        vb.vb_check(L.vb_adamw_step(C.byref(wt), C.byref(gt), slots[2].value, slots[3].value, t, 3e-3, 0.9, 0.999, 1e-8, 0.05))
    got = np.empty(4099, np.float32)
    vb.vb_check(L.vb_read(slots[0].value, 0, got.ctypes.data_as(vb.c_f32p), 4099))
    for s in slots:
        vb.vb_check(L.vb_release(s.value, None))
    assert_close(got, w.numpy(), "vb_adamw_step")


def test_slot_lifecycle(vb):
    """Refcount protocol of the slot table (mirrors crates/vearo-core/src/lib.rs:194-226)."""
    import ctypes as C
    L = vb.lib()
    before = vb.memory_stats()["live_slots"]
    s = C.c_uint32(0)
    vb.vb_check(L.vb_alloc(100, 1, C.byref(s)))
    vb.vb_check(L.vb_retain(s.value))
    freed = C.c_int(-1)
    vb.vb_check(L.vb_release(s.value, C.byref(freed))); assert freed.value == 0
    vb.vb_check(L.vb_release(s.value, C.byref(freed))); assert freed.value == 1
    assert L.vb_release(s.value, C.byref(freed)) != 0          # already gone: an error, not a crash
    assert vb.memory_stats()["live_slots"] == before


# ---- tensor-core GEMM (3xTF32 on tcgen05): sizes large enough to leave the CUDA-core kernel -----------------
@pytest.mark.parametrize("M,N,K,ta,tb", [
    (300, 260, 200, False, False),    # partial tiles in M, N and K; B needs the K-contiguous repack
    (256, 512, 768, False, True),     # both operands K-contiguous as stored: x . W^T
    (512, 192, 136, True, False),     # A transposed view (weight-gradient shape), narrow N
    (128, 64, 2048, True, True),      # BN = 64 tile
    (256, 256, 8192, False, True),    # few tiles, long K: split-K
    (1000, 1000, 72, False, True),    # short K (attention-score shape)
    (1100, 700, 1000, False, True),   # stream-K: ragged tiles in M and N, k ranges straddling tiles
    (4096, 768, 768, False, True),    # stream-K: one CTA per slot, 3-4 parts per tile
    (768, 1536, 4096, True, False),   # stream-K on a weight-gradient shape (A transposed view, long K)
    (2048, 300, 520, False, False),   # stream-K with 128-wide tiles (a 256-wide last tile would be mostly padding)
    (2048, 384, 300, False, True),    # 192-wide tiles (a single wave either way, less padding work than 256)
    (1024, 500, 264, True, False),    # 192-wide tiles with a ragged last tile, A as a transposed view
    (4096, 3072, 512, False, True),   # stream-K because whole tiles would fill one wave and a fraction of a second (384 tiles, 296 slots)
    (384, 64, 1000, False, False),    # 64-wide tiles take 32-wide k-blocks: K ragged against 32, B row-major (MN-major)
    (384, 48, 328, False, True),      # ... both operands K-contiguous (128-byte swizzled rows), ragged N and K
    (640, 64, 1064, True, False),     # ... both operands MN-major (attention dV = P^T . dO shape)
    (200, 40, 96, True, True),        # ... A MN-major with rows not a multiple of 32, three k-blocks
])
def test_matmul_tensor_core(vb, M, N, K, ta, tb):
    a = rnd(60, *((K, M) if ta else (M, K)), scale=0.05)
    b = rnd(61, *((N, K) if tb else (K, N)), scale=0.05)

    def case(T, m):
        x, y = T.from_numpy(a), T.from_numpy(b)
        if ta: x = x.transpose(0, 1)
        if tb: y = y.transpose(0, 1)
        return [x.matmul(y)]
    both(vb, case)
    # the split-precision product must sit at FP32 accuracy (a sequential f32 dot product of this length is no better), far from plain TF32's 1e-3
    x = vb.Tensor.from_numpy(a); y = vb.Tensor.from_numpy(b)
    if ta: x = x.transpose(0, 1)
    if tb: y = y.transpose(0, 1)
    got = x.matmul(y).numpy().astype(np.float64)
    ref = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    scale = np.abs(a.T if ta else a).astype(np.float64) @ np.abs(b.T if tb else b).astype(np.float64)
    assert (np.abs(got - ref) / scale).max() < 4e-6


def test_matmul_stream_k_repeatable_and_counters_reset(vb):
    """Tiles shared by several CTAs are summed in k order by whichever CTA arrives last: the result may not
    depend on that, and the arrival counters must be back at zero for the next product of another shape."""
    a, b = rnd(70, 2304, 640, scale=0.05), rnd(71, 896, 640, scale=0.05)
    c, d = rnd(72, 1280, 1200, scale=0.05), rnd(73, 1200, 384, scale=0.05)
    x, y = vb.Tensor.from_numpy(a), vb.Tensor.from_numpy(b).transpose(0, 1)
    u, v = vb.Tensor.from_numpy(c), vb.Tensor.from_numpy(d)
    first, first2 = x.matmul(y).numpy(), u.matmul(v).numpy()
    for _ in range(5):
        assert np.array_equal(x.matmul(y).numpy(), first)
        assert np.array_equal(u.matmul(v).numpy(), first2)
    ref = a.astype(np.float64) @ b.T.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b.T).astype(np.float64)
    assert (np.abs(first - ref) / scale).max() < 2e-6
    vb.check_errors()


def test_matmul_tensor_core_batched_views(vb):
    """Head-split views [B,S,H,dk] -> [B,H,S,dk] consumed in place, both batch levels strided."""
    B, S, H, dk = 2, 256, 4, 64
    q0, k0, v0 = rnd(62, B, S, H * dk, scale=0.1), rnd(63, B, S, H * dk, scale=0.1), rnd(64, B, S, H * dk, scale=0.3)

    def case(T, m):
        q, k, v = (T.from_numpy(a).reshape([B, S, H, dk]).transpose(1, 2) for a in (q0, k0, v0))
        s = q.matmul(k.transpose(2, 3))
        return [s, s.matmul(v), s.transpose(2, 3).matmul(v)]
    both(vb, case)


def test_linear_weight_lo_plane_exact_and_never_stale(vb):
    """A Linear weight of 2^18 elements or more keeps its TF32 remainders beside it and the GEMM loads them instead of
    recomputing them.  The product must be bit-identical to the same product without the plane (a plain matmul with the
    transposed view), and the plane must follow every change of the weight: a write through the ABI, an in-place
    accumulate, an optimizer step."""
    x0, w0, w1 = rnd(401, 1024, 512, scale=0.5), rnd(402, 512, 512, scale=0.05), rnd(403, 512, 512, scale=0.05)
    T = vb.Tensor
    x, w = T.from_numpy(x0), T.from_numpy(w0, True)

    def check(tag):
        a = x.linear(w, None).numpy()
        b = x.matmul(w.transpose(0, 1)).numpy()
        assert np.array_equal(a, b), tag
        return a
    y0 = check("fresh plane")
    assert np.array_equal(check("plane reused"), y0)
    w.write(w1)                                            # vb_write advances the slot's serial
    y1 = check("after write")
    assert not np.array_equal(y0, y1)
    ref = x0.astype(np.float64) @ w1.T.astype(np.float64)
    assert np.abs(y1 - ref).max() < 1e-4
    opt = vb.AdamW([w], 1e-2, 0.9, 0.999, 1e-8, 0.0)      # the update rewrites the plane itself
    for _ in range(2):
        vb.zero_gradients(); vb.reset_active_tape()
        x.linear(w, None).mul(T.from_numpy(rnd(404, 1024, 512))).sum(1, False).sum(0, False).backward()
        opt.step()
        y2 = check("after optimizer step")
    assert not np.array_equal(y1, y2)
    gx = T.from_numpy(x0, True)                            # the input-gradient product uses the plane too
    vb.zero_gradients(); vb.reset_active_tape()
    go = rnd(405, 1024, 512)
    gx.linear(w, None).mul(T.from_numpy(go)).sum(1, False).sum(0, False).backward()
    want = T.from_numpy(go).matmul(w).numpy()
    assert np.array_equal(gx.grad().numpy(), want)
    vb.check_errors()


def test_activation_lo_plane_follows_in_place_writers(vb):
    """A LayerNorm output of 2^18 elements or more carries a lo plane.  Entry points that overwrite such a slot in place
    (the fused cross-entropy leaves the gradient where the logits were; vb_linear_backward_into writes into a given
    destination) must void the plane: the next product over the slot has to equal the plane-free product bit for bit."""
    import ctypes as C
    T = vb.Tensor
    x0, w0 = rnd(411, 1024, 512), rnd(412, 512, 512, scale=0.05)
    g1, b1 = T.from_numpy(np.ones(512, np.float32)), T.from_numpy(np.zeros(512, np.float32))
    w = T.from_numpy(w0)
    y = T.from_numpy(x0).layernorm(g1, b1, 1e-5)           # [1024, 512]: gets a plane from the kernel that writes it
    before = y.linear(w, None).numpy()
    assert np.array_equal(before, y.matmul(w.transpose(0, 1)).numpy())
    tg = T.from_numpy(np.random.default_rng(3).integers(0, 512, 1024).astype(np.float32))
    loss = vb.VbTensor()
    yd, td = y.desc(), tg.desc()
    vb.vb_check(vb.lib().vb_cross_entropy_fused(C.byref(yd), C.byref(td), C.byref(loss)), "vb_cross_entropy_fused")
    vb.vb_check(vb.lib().vb_release(loss.slot, None))
    after = y.linear(w, None).numpy()
    assert not np.array_equal(before, after)
    assert np.array_equal(after, y.matmul(w.transpose(0, 1)).numpy()), "stale lo plane after the fused cross-entropy"
    # a destination written by vb_linear_backward_into: a second LayerNorm output, of the shape of a [1024, 512] weight gradient
    z = T.from_numpy(rnd(413, 1024, 512)).layernorm(g1, b1, 1e-5)       # 2^19 elements -> plane
    assert np.array_equal(z.linear(w, None).numpy(), z.matmul(w.transpose(0, 1)).numpy())       # (plane in use: 1024 rows)
    x1, w2, go = T.from_numpy(rnd(414, 256, 512)), T.from_numpy(rnd(416, 1024, 512, scale=0.05)), T.from_numpy(rnd(415, 256, 1024))
    zd, xd, wd, gd = z.desc(), x1.desc(), w2.desc(), go.desc()
    gx = vb.VbTensor()
    L = vb.lib()
    vb.vb_check(L.vb_linear_backward_into(C.byref(xd), C.byref(wd), C.byref(gd), C.byref(gx), C.byref(zd), None), "vb_linear_backward_into")
    vb.vb_check(L.vb_release(gx.slot, None))
    assert np.array_equal(z.linear(w, None).numpy(), z.matmul(w.transpose(0, 1)).numpy()), "stale lo plane after linear_backward_into"
    vb.check_errors()


@pytest.mark.parametrize("rows,inf,outf", [(1024, 768, 3072), (512, 384, 640), (260, 96, 200), (6, 5, 7)])
def test_linear_gelu_epilogue_equals_the_two_ops(vb, rows, inf, outf):
    """fc1 -> gelu with the activation formed in the GEMM's epilogue: same values as linear followed by gelu, bit for bit, and the
    same gradients (the tape holds the same two nodes); against the oracle at the usual bar."""
    x0, w0, b0, go = rnd(71, rows, inf, scale=0.3), rnd(72, outf, inf, scale=0.08), rnd(73, outf, scale=0.3), rnd(74, rows, outf, scale=0.01)

    def run(T, fused):
        x, w, b = T.from_numpy(x0, True), T.from_numpy(w0, True), T.from_numpy(b0, True)
        a = x.linear_gelu(w, b) if fused else x.matmul(w.transpose(0, 1)).add(b).gelu()
        n = go.size
        a.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [t.numpy() for t in (a, x.grad(), w.grad().contiguous(), b.grad())]
    orc.reset_all()
    cpu = run(orc.Tensor, False)
    vb.zero_gradients(); vb.reset_active_tape()
    got = run(vb.Tensor, True)
    vb.check_errors()
    for g, c, n in zip(got, cpu, "act gx gw gb".split()):
        assert_close(g, c, "linear_gelu %s" % n)
    # the two-op form on the device (vb_linear, then vb_gelu): identical bits
    vb.zero_gradients(); vb.reset_active_tape()
    x, w, b = vb.Tensor.from_numpy(x0), vb.Tensor.from_numpy(w0), vb.Tensor.from_numpy(b0)
    assert np.array_equal(x.linear(w, b).gelu().numpy(), x.linear_gelu(w, b).numpy())


def test_linear_tensor_core_with_bias_and_backward(vb):
    x0, w0, b0, go = rnd(65, 512, 384, scale=0.5), rnd(66, 640, 384, scale=0.05), rnd(67, 640), rnd(68, 512, 640, scale=0.1)

    def run(T, fused):
        x, w, b = T.from_numpy(x0, True), T.from_numpy(w0, True), T.from_numpy(b0, True)
        y = x.linear(w, b) if fused else x.matmul(w.transpose(0, 1)).add(b)
        n = go.size
        y.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [t.numpy() for t in (y, x.grad(), w.grad().contiguous(), b.grad())]
    orc.reset_all()
    cpu = run(orc.Tensor, False)
    vb.zero_gradients(); vb.reset_active_tape()
    for g, c, n in zip(run(vb.Tensor, True), cpu, "y gx gw gb".split()):
        assert_close(g, c, "linear(tc) " + n)
    vb.check_errors()


# ---- bias gradients from the producer's column sums; LayerNorm backward that adds into an existing gradient --------------------
def _raw_out(vb, t):
    a = np.empty(t.shape, np.float32)
    vb.vb_check(vb.lib().vb_read(t.slot, 0, a.ctypes.data_as(vb.c_f32p), a.size))
    return a


@pytest.mark.parametrize("rows,c", [(2048, 768), (1536, 1024), (1100, 200), (64, 96), (33, 50)])
def test_layernorm_backward_accum_matches_oracle(vb, rows, c):
    """grad_in += dx in the kernel that forms dx (vearo-autograd/src/lib.rs:733-741 does the addition on the gradient map):
    against the oracle's LayerNorm backward plus the existing gradient, for the register kernel (with and without masked
    columns), for short inputs and for a row length the generic route takes."""
    import ctypes as C
    x0, w0, b0, go, acc0 = rnd(501, rows, c) * 1.5 + 0.3, rnd(502, c), rnd(503, c), rnd(504, rows, c, scale=0.05), rnd(505, rows, c, scale=0.05)
    # (gradients of size 0.05: dgamma / dbeta are sums over up to 2048 rows, and the absolute part of the bar is 1e-5)
    orc.reset_all()
    xr, wr, br = orc.Tensor.from_numpy(x0, True), orc.Tensor.from_numpy(w0, True), orc.Tensor.from_numpy(b0, True)
    n = x0.size
    xr.layernorm(wr, br, 1e-5).mul(orc.Tensor.from_numpy(go)).reshape([1, n]).matmul(orc.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
    want_x, want_w, want_b = xr.grad().numpy() + acc0, wr.grad().numpy(), br.grad().numpy()
    T = vb.Tensor
    x, w, b, g, acc = (T.from_numpy(a) for a in (x0, w0, b0, go, acc0))
    gw, gb = vb.VbTensor(), vb.VbTensor()
    L = vb.lib()
    xd, wd, bd, gd, ad = x.desc(), w.desc(), b.desc(), g.desc(), acc.desc()
    vb.vb_check(L.vb_layernorm_backward_accum(C.byref(xd), C.byref(wd), C.byref(bd), C.byref(gd), 1e-5, C.byref(ad), C.byref(gw), C.byref(gb)),
                "vb_layernorm_backward_accum")
    assert_close(acc.numpy(), want_x, "grad_in + dx")
    assert_close(_raw_out(vb, gw), want_w, "dgamma"); assert_close(_raw_out(vb, gb), want_b, "dbeta")
    # the accumulated gradient as the output gradient of a Linear layer: its bias gradient is the column sum of what is there NOW
    xin, wl = T.from_numpy(rnd(506, rows, 32)), T.from_numpy(rnd(507, c, 32, scale=0.1))
    for step in range(2):
        gbias = vb.VbTensor()
        xi, wi = xin.desc(), wl.desc()
        vb.vb_check(L.vb_linear_backward(C.byref(xi), C.byref(wi), C.byref(ad), None, None, C.byref(gbias)), "vb_linear_backward")
        now = acc.numpy()
        assert_close(_raw_out(vb, gbias), now.astype(np.float64).sum(0).astype(np.float32), "bias gradient, pass %d" % step, atol=1e-4 * np.sqrt(rows))
        vb.vb_check(L.vb_release(gbias.slot, None))
        if step == 0:       # an in-place writer voids the kept sums
            extra = T.from_numpy(rnd(508, rows, c)); ed = extra.desc()
            vb.vb_check(L.vb_accumulate(C.byref(ad), C.byref(ed)), "vb_accumulate")
    for t in (gw, gb):
        vb.vb_check(L.vb_release(t.slot, None))
    vb.check_errors()


@pytest.mark.parametrize("rows,c", [(2048, 3072), (1024, 1028), (1024, 132), (300, 256)])
def test_activation_backward_leaves_the_bias_gradient(vb, rows, c):
    """GELU / ReLU backward over a large [rows, c] gradient also sums its columns; Linear backward given that tensor as grad_out
    takes the sums as its bias gradient.  Values against the oracle (dx) and against an f64 column sum of the dx actually
    produced; VB200_COLSUM_REUSE=0 is the same computation through the separate column-sum kernel (small case: never summed)."""
    import ctypes as C
    x0, go = rnd(511, rows, c), rnd(512, rows, c, scale=0.1)
    T = vb.Tensor
    L = vb.lib()
    for op, fwd in (("gelu", "gelu"), ("relu", "relu")):
        orc.reset_all()
        xr = orc.Tensor.from_numpy(x0, True)
        n = x0.size
        getattr(xr, fwd)().mul(orc.Tensor.from_numpy(go)).reshape([1, n]).matmul(orc.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        want = xr.grad().numpy()
        x, g = T.from_numpy(x0), T.from_numpy(go)
        gx, gbias = vb.VbTensor(), vb.VbTensor()
        xd, gd = x.desc(), g.desc()
        vb.vb_check(getattr(L, "vb_%s_backward" % op)(C.byref(xd), C.byref(gd), C.byref(gx)), op)
        got = _raw_out(vb, gx)
        assert_close(got, want, op + " backward")
        xin, wl = T.from_numpy(rnd(513, rows, 16)), T.from_numpy(rnd(514, c, 16, scale=0.1))
        xi, wi = xin.desc(), wl.desc()
        vb.vb_check(L.vb_linear_backward(C.byref(xi), C.byref(wi), C.byref(gx), None, None, C.byref(gbias)), "vb_linear_backward")
        assert_close(_raw_out(vb, gbias), got.astype(np.float64).sum(0).astype(np.float32), op + " bias gradient", atol=1e-4 * np.sqrt(rows))
        for t in (gx, gbias):
            vb.vb_check(L.vb_release(t.slot, None))
    vb.check_errors()


def test_a_device_side_wait_that_runs_out_is_reported_and_survived(vb):
    """Failure detection on the device, without a fault: a kernel waits (bounded, 4096 polls) on a barrier nothing arrives on,
    gives up and raises the wait-timeout bit -- the path every tensor-core kernel of the library takes if a copy or a partner
    never shows up.  The host must see the error at the next check, the error must be cleared by reporting it, and the next
    tensor-core product must be right."""
    import ctypes as C
    L = vb.lib()
    L.vb_selftest_wait_timeout.argtypes = [C.c_uint32, C.POINTER(C.c_double)]
    vb.check_errors()
    ms = C.c_double(0.0)
    vb.vb_check(L.vb_selftest_wait_timeout(4096, C.byref(ms)), "vb_selftest_wait_timeout")
    assert 0.0 < ms.value < 2000.0, ms.value            # bounded: the kernel came back by itself
    with pytest.raises(vb.VearoError, match="a device-side wait ran out"):
        vb.check_errors()
    vb.check_errors()                                    # reported once, then clear
    x0, w0 = rnd(601, 512, 256, scale=0.3), rnd(602, 384, 256, scale=0.1)
    before = C.c_int64(0); after = C.c_int64(0)
    L.vb_tc_launch_count(C.byref(before))
    y = vb.Tensor.from_numpy(x0).linear(vb.Tensor.from_numpy(w0), None).numpy()
    L.vb_tc_launch_count(C.byref(after))
    assert after.value > before.value, "the product after the timeout did not run on the tensor-core kernel"
    assert_close(y, (x0.astype(np.float64) @ w0.astype(np.float64).T).astype(np.float32), "product after a timeout")
    vb.check_errors()
    print("give-up time: %.3f ms for 4096 polls -> about %.1f s for the production limit of 2^20" % (ms.value, ms.value * 256 / 1000.0))
