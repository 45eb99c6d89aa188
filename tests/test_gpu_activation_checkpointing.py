"""Activation checkpointing (crates/vearo-autograd/src/lib.rs:649-730, 897-959): a block run under `checkpoint` keeps
only its input and is run again during backward.  The gradients must be those of the plain graph -- here they are compared
for equality, since the recomputation launches the same kernels on the same values -- stateful layers must not advance
twice, and the peak memory of a GPT step must drop."""
import numpy as np
import pytest

from oracle import oracle as orc
from vearo_b200 import modelspec as ms
from tests.test_gpu_ops import assert_close, rnd

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vb():
    import vearo_b200 as v
    v.init()
    return v


def test_reference_known_answer(vb):
    """vearo-autograd/src/lib.rs:1584-1618: x [1,2] . w [[2,-1],[3,0.5]] -> relu -> sum; with and without checkpoint."""
    T = vb.Tensor
    w = T.from_numpy(np.array([[2.0, -1.0], [3.0, 0.5]], np.float32), True)
    x = T.from_numpy(np.array([[1.0, 2.0]], np.float32), True)
    vb.zero_gradients(); vb.reset_active_tape()
    x.matmul(w).relu().sum(0, False).sum(0, False).backward()
    gx_std, gw_std = x.grad().numpy().copy(), w.grad().contiguous().numpy().copy()
    vb.zero_gradients(); vb.reset_active_tape()
    calls = []

    def block(inp):
        calls.append(vb.is_recomputing())
        return inp.matmul(w).relu()
    vb.checkpoint(x, block).sum(0, False).sum(0, False).backward()
    assert calls == [False, True]                      # once in forward, once more inside backward
    assert np.array_equal(x.grad().numpy(), gx_std) and np.array_equal(w.grad().contiguous().numpy(), gw_std)
    # x.w = [8, 0]; relu passes only the first column (0 is not > 0): dx = [2, 3], dw = [[1, 0], [2, 0]]
    assert np.array_equal(gx_std, [[2.0, 3.0]]) and np.array_equal(gw_std, [[1.0, 0.0], [2.0, 0.0]])
    vb.check_errors()


def test_shared_parameter_and_nested_blocks(vb):
    """A weight used by two checkpointed blocks (one nested in another) and once outside: the contributions add up."""
    w0, x0 = rnd(301, 24, 24, scale=0.3), rnd(302, 5, 24)

    def run(T, m, ckpt):
        w, x = T.from_numpy(w0, True), T.from_numpy(x0, True)
        inner = lambda t: t.matmul(w).gelu()
        outer = lambda t: (m.checkpoint(t, inner) if ckpt else inner(t)).matmul(w).relu()
        h = m.checkpoint(x, outer) if ckpt else outer(x)
        h = (m.checkpoint(h, inner) if ckpt else inner(h)).matmul(w)
        h.mul(h).sum(1, False).sum(0, False).backward()
        return [x.grad().numpy().copy(), w.grad().contiguous().numpy().copy()]
    vb.zero_gradients(); vb.reset_active_tape()
    plain = run(vb.Tensor, vb, False)
    vb.zero_gradients(); vb.reset_active_tape()
    ck = run(vb.Tensor, vb, True)
    orc.reset_all()
    ref = run(orc.Tensor, None, False)
    for a, b, c, n in zip(plain, ck, ref, ("dx", "dw")):
        assert_close(a, c, "plain " + n)
        assert_close(b, c, "checkpointed " + n)
        np.testing.assert_allclose(b, a, rtol=2e-6, atol=1e-7)       # same terms, summed in another order
    vb.check_errors()


def test_dropout_matches_oracle_and_is_reproducible_under_checkpoint(vb):
    """crates/vearo/tests/checkpoint_hazards.rs:30-82: a block containing dropout gives the same gradient with and without
    checkpointing, because the recomputation rewinds the call counter and draws the same mask.  The mask itself is the
    reference's (xorshift64 seeded with seed ^ call * 0x9E3779B97F4A7C15, keep where u >= p, scale 1 / (1 - p))."""
    x0 = np.array([0.5, -1.5, 2.0, 0.25, 1.0, -0.75], np.float32).reshape(2, 3)
    big = rnd(310, 37, 29)

    def run(T, m, ckpt):
        m.set_training(True); m.set_rng_counter(0)
        x, y = T.from_numpy(x0, True), T.from_numpy(big, True)
        m.zero_gradients(); m.reset_active_tape()
        f = lambda t: t.dropout(0.25, 7)
        out = (m.checkpoint(x, f) if ckpt else f(x))
        z = y.dropout(0.5, 11).mul(y)                       # a second draw after the block: counter 1 in both variants
        out.sum(0, False).sum(0, False).add(z.sum(0, False).sum(0, False)).backward()
        return [out.numpy().copy(), x.grad().numpy().copy(), y.grad().numpy().copy()], m.rng_counter()
    orc.reset_all()
    ref, ref_ctr = run(orc.Tensor, orc, False)
    plain, c1 = run(vb.Tensor, vb, False)
    ck, c2 = run(vb.Tensor, vb, True)
    assert ref_ctr == c1 == c2 == 2
    for a, b, c in zip(ref, plain, ck):
        assert np.array_equal(a, b) and np.array_equal(b, c)
    assert (plain[0] == 0).sum() + (big.size - np.count_nonzero(plain[2])) > 0      # something was dropped
    vb.set_training(False)
    t = vb.Tensor.from_numpy(x0)
    assert np.array_equal(t.dropout(0.25, 7).numpy(), x0)                              # identity outside training
    vb.set_training(True)
    vb.check_errors()


def test_batchnorm_running_stats_advance_once(vb):
    """crates/vearo/tests/checkpoint_hazards.rs:84-140: the block runs twice, the running statistics move once."""
    T = vb.Tensor
    x0 = np.array([1, 2, 3, 4, 5, 6, 7, 8], np.float32).reshape(2, 2, 1, 2)
    stats = []
    for ckpt in (False, True):
        x = T.from_numpy(x0, True)
        g, b = T.from_numpy(np.ones(2, np.float32), True), T.from_numpy(np.zeros(2, np.float32), True)
        rm, rv = T.from_numpy(np.zeros(2, np.float32)), T.from_numpy(np.ones(2, np.float32))
        vb.set_training(True); vb.zero_gradients(); vb.reset_active_tape()
        f = lambda t: t.batchnorm(g, b, rm, rv, True, 0.1, 1e-5)
        y = vb.checkpoint(x, f) if ckpt else f(x)
        y.mul(y).sum(0, False).sum(0, False).sum(0, False).sum(0, False).backward()
        stats.append((rm.numpy().copy(), rv.numpy().copy(), x.grad().numpy().copy(), g.grad().numpy().copy()))
    for a, b in zip(stats[0], stats[1]):
        assert np.array_equal(a, b)
    # one update with momentum 0.1 from (0, 1): mean of channel 0 is (1+2+5+6)/4 = 3.5 -> 0.35
    assert abs(stats[0][0][0] - 0.35) < 1e-6
    vb.check_errors()


def test_gpt_blocks_checkpointed(vb):
    """SimpleGPT with every block under checkpoint: same loss and gradients as the plain graph (and as the oracle's),
    the same weights after optimizer steps, and a lower peak of live device memory."""
    vocab, T_, d, heads, layers, ff, B = 128, 64, 64, 4, 4, 256, 4
    params = ms.gpt_params(vocab, T_, d, layers, ff, std=0.1)
    ids, tg = ms.gpt_batch(vocab, B, T_)
    out = {}
    for ckpt in (False, True):
        gm = vb.SimpleGPT(vocab, T_, d, heads, layers, ff); gm.load(params)
        gm.set_checkpointing(ckpt)
        opt = vb.AdamW(gm.parameters(), 1e-3, 0.9, 0.999, 1e-8, 0.1)
        vb.zero_gradients(); vb.reset_active_tape()
        loss = gm.loss(vb.Tensor.from_numpy(ids), vb.Tensor.from_numpy(tg)); loss.backward()
        grads = [p.grad().contiguous().numpy().copy() for p in gm.parameters()]
        losses = [float(loss.numpy().reshape(-1)[0])]
        for _ in range(3):
            l, _n = gm.train_step(opt, ids, tg, 1.0)
            losses.append(l)
        out[ckpt] = (grads, losses, [p.numpy().copy() for p in gm.parameters()])
    for a, b in zip(out[False][0], out[True][0]):
        assert np.array_equal(a, b)
    assert out[False][1] == out[True][1]
    for a, b in zip(out[False][2], out[True][2]):
        assert np.array_equal(a, b)
    vb.check_errors()


def test_gpt_peak_memory_drops(vb):
    vocab, T_, d, heads, layers, ff, B = 512, 256, 256, 4, 6, 1024, 8
    params = ms.gpt_params(vocab, T_, d, layers, ff)
    ids, tg = ms.gpt_batch(vocab, B, T_)
    L = vb.lib()
    peaks = {}
    for ckpt in (False, True):
        gm = vb.SimpleGPT(vocab, T_, d, heads, layers, ff); gm.load(params)
        gm.set_checkpointing(ckpt)
        vb.zero_gradients(); vb.reset_active_tape()
        vb.vb_check(L.vb_memory_reset_peak())
        base = vb.memory_stats()["live_bytes"]
        gm.loss(vb.Tensor.from_numpy(ids), vb.Tensor.from_numpy(tg)).backward()
        vb.sync()
        peaks[ckpt] = vb.memory_stats()["peak_bytes"] - base
        vb.zero_gradients(); vb.reset_active_tape()
        del gm
    # per block the plain graph keeps ~12 activations of [B,T,d] and two of [B,H,T,T]; with checkpointing only its input
    assert peaks[True] < 0.5 * peaks[False], peaks
    vb.check_errors()
