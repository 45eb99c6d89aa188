"""Pins the CPU oracle against the reference's own known-answer tests and NumPy fixtures.

Each test names the reference test it restates (paths relative to the reference root).
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import Tensor as T

HERE = os.path.dirname(os.path.abspath(__file__))
REF_JSON = os.path.join(os.environ.get("VEARO_REFERENCE_DIR", "/root/reference"), "test_data/oracles.json")


def f32(*v, shape=None):
    a = np.array(v, dtype=np.float32)
    return a if shape is None else a.reshape(shape)


def _run_forward_case(c):
    ins = [np.array(i["data"], dtype=np.float32).reshape(i["shape"]) for i in c["inputs"]]
    op = c["op"]
    if op == "add_transposed":
        # the reference builds the first operand as a transposed view of a [2,3] tensor
        # (crates/vearo/tests/verification_harness.rs:45-103)
        base = T.from_numpy(ins[0].T.copy())
        return base.transpose(0, 1).add(T.from_numpy(ins[1]))
    t = [T.from_numpy(a) for a in ins]
    if op in ("add", "add_broadcasted"): return t[0].add(t[1])
    if op == "sub": return t[0].sub(t[1])
    if op == "mul": return t[0].mul(t[1])
    if op == "div": return t[0].div(t[1])
    if op in ("matmul_2d", "matmul_batched"): return t[0].matmul(t[1])
    if op == "reshape": return t[0].reshape([6])
    if op == "transpose": return t[0].transpose(0, 1)
    if op == "permute": return t[0].permute([2, 0, 1])
    raise AssertionError(op)


def test_numpy_forward_fixture():
    """crates/vearo/tests/verification_harness.rs:45-103, tolerance 1e-5."""
    cases = json.load(open(os.path.join(HERE, "golden", "forward_cases.json")))
    assert len(cases) == 11
    for c in cases:
        out = _run_forward_case(c)
        want = np.array(c["output"]["data"], dtype=np.float32).reshape(c["output"]["shape"])
        assert out.shape == tuple(c["output"]["shape"]), c["op"]
        np.testing.assert_allclose(out.numpy(), want, atol=1e-5, rtol=0, err_msg=c["op"])


@pytest.mark.skipif(not os.path.exists(REF_JSON), reason="reference tree not present")
def test_fixture_equals_reference_fixture():
    mine = json.load(open(os.path.join(HERE, "golden", "forward_cases.json")))
    ref = json.load(open(REF_JSON))
    assert [c["op"] for c in mine] == [c["op"] for c in ref]
    for a, b in zip(mine, ref):
        assert a["output"] == b["output"] and a["inputs"] == b["inputs"], a["op"]


def test_cpu_backend_known_answers():
    """crates/vearo-backend-cpu/src/lib.rs:2636-2830 and 2915-2927."""
    assert T.from_numpy(f32(1, 2, 3)).add(T.from_numpy(f32(4, 5, 6))).numpy().tolist() == [5, 7, 9]
    z = T.from_numpy(f32(1, 2, 3, 4, shape=(2, 2))).matmul(T.from_numpy(f32(5, 6, 7, 8, shape=(2, 2))))
    assert z.numpy().flatten().tolist() == [19, 22, 43, 50]
    z = T.from_numpy(f32(1, 2, 3, shape=(1, 3))).add(T.from_numpy(f32(10, 20, shape=(2, 1))))
    assert z.shape == (2, 3) and z.numpy().flatten().tolist() == [11, 12, 13, 21, 22, 23]
    xt = T.from_numpy(f32(1, 2, 3, 4, 5, 6, shape=(2, 3))).transpose(0, 1)
    z = xt.add(T.from_numpy(f32(10, 20, 30, 40, 50, 60, shape=(3, 2))))
    assert z.numpy().flatten().tolist() == [11, 24, 32, 45, 53, 66]
    a = np.arange(1, 13, dtype=np.float32)
    z = T.from_numpy(a.reshape(2, 2, 3)).matmul(T.from_numpy(a.reshape(2, 3, 2)))
    assert z.numpy().flatten().tolist() == [22, 28, 49, 64, 220, 244, 301, 334]
    assert T.from_numpy(f32(1, -2, 3, -0.5)).relu().numpy().tolist() == [1, 0, 3, 0]
    x = T.from_numpy(f32(1, 2, 3, 4, 5, 6, shape=(2, 3)))
    assert x.sum(1).numpy().tolist() == [6, 15] and x.sum(0).numpy().tolist() == [5, 7, 9]
    assert x.sum(1, True).shape == (2, 1)
    assert x.mean(1).numpy().tolist() == [2, 5] and x.mean(0).numpy().tolist() == [2.5, 3.5, 4.5]
    assert x.transpose(0, 1).sum(1).numpy().tolist() == [5, 7, 9]
    # conv corner picker
    x = T.from_numpy(np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3))
    out = x.conv2d(T.from_numpy(f32(1, 0, 0, 1, shape=(1, 1, 2, 2))), T.from_numpy(f32(0)), 1, 0)
    assert out.shape == (1, 1, 2, 2) and out.numpy().flatten().tolist() == [6, 8, 12, 14]
    # cross-entropy stability with +-1000 logits
    loss = T.from_numpy(f32(1000, -1000, shape=(1, 2))).cross_entropy(T.from_numpy(f32(0)))
    assert abs(loss.numpy()[0]) < 1e-4 and loss.shape == (1,)


def test_empty_and_noncontiguous_inputs():
    """crates/vearo-backend-cpu/src/lib.rs:2832-2863."""
    x = T.from_numpy(np.zeros((2, 0, 3), np.float32))
    r = x.transpose(0, 1).reshape([0, 6])
    assert r.shape == (0, 6)
    assert r.add(T.from_numpy(np.zeros((0, 6), np.float32))).shape == (0, 6)
    w, b = T.from_numpy(np.ones(4, np.float32)), T.from_numpy(np.zeros(4, np.float32))
    assert T.from_numpy(np.zeros((2, 0, 4), np.float32)).layernorm(w, b, 1e-5).shape == (2, 0, 4)
    xt = T.from_numpy(np.arange(1, 9, dtype=np.float32).reshape(2, 4)).transpose(0, 1)
    out = xt.layernorm(T.from_numpy(np.ones(2, np.float32)), T.from_numpy(np.zeros(2, np.float32)), 1e-5)
    assert out.shape == (4, 2)
    np.testing.assert_allclose(out.numpy()[:, 0], -out.numpy()[:, 1], atol=1e-6)


@pytest.mark.parametrize("build,msg", [
    (lambda: T.from_numpy(f32(-1, 0)).embedding(T.from_numpy(np.zeros((2, 3), np.float32))), "Token ID cannot be negative"),
    (lambda: T.from_numpy(f32(2, 0)).embedding(T.from_numpy(np.zeros((2, 3), np.float32))), "out of vocabulary bound"),
    (lambda: T.from_numpy(np.zeros((2, 3), np.float32)).cross_entropy(T.from_numpy(f32(-1, 0))), "Target class cannot be negative"),
    (lambda: T.from_numpy(np.zeros((2, 3), np.float32)).cross_entropy(T.from_numpy(f32(3, 0))), "out of vocab bounds"),
])
def test_invalid_ids_are_errors(build, msg):
    """The four should_panic tests, crates/vearo-backend-cpu/src/lib.rs:2865-2899."""
    with pytest.raises(orc.OracleError, match=msg):
        build()


def test_backward_known_answers():
    """crates/vearo-autograd/src/lib.rs:996-1024 and 1100-1121."""
    x, y, w = (T.from_numpy(f32(v), True) for v in (2, 3, 4))
    x.add(y).mul(w).backward()
    assert (x.grad().numpy()[0], y.grad().numpy()[0], w.grad().numpy()[0]) == (4, 4, 5)
    x, y = T.from_numpy(f32(2), True), T.from_numpy(f32(3), True)
    for _ in range(2):   # two passes reuse the same leaves
        x.mul(y).backward()
        assert x.grad().numpy()[0] == 3 and y.grad().numpy()[0] == 2


def test_broadcast_add_mul_gradients():
    """f = sum((x + y) * x), y broadcast over rows (crates/vearo-autograd/src/lib.rs:1026-1098)."""
    xd = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    yd = f32(10, 20, 30, shape=(1, 3))
    x, y = T.from_numpy(xd, True), T.from_numpy(yd, True)
    ones = T.from_numpy(np.ones((6, 1), np.float32))
    x.add(y).mul(x).reshape([1, 6]).matmul(ones).reshape([1]).backward()
    np.testing.assert_allclose(x.grad().numpy(), 2 * xd + yd, atol=1e-5)
    np.testing.assert_allclose(y.grad().numpy(), xd.sum(0, keepdims=True), atol=1e-5)


def test_optimizer_known_answers():
    """crates/vearo-optim/src/lib.rs:389-403 (SGD 0.989), 415-436 (cosine), 438-459 (clip 10 -> [3,4])."""
    x = T.from_numpy(f32(1, 2), True)
    # grad [0.1, 0.2] through loss = sum(x * c)
    c = T.from_numpy(f32(0.1, 0.2))
    x.mul(c).sum(0).backward()
    opt = orc.SGD([x], 0.1, 0.9, 0.01)
    opt.step()
    assert abs(x.numpy()[0] - 0.989) < 1e-5
    assert abs(orc.cosine_lr(0.1, 0.01, 10, 100, 0) - 0.1 / 11) < 1e-6
    assert abs(orc.cosine_lr(0.1, 0.01, 10, 100, 9) - 0.1 * 10 / 11) < 1e-6
    assert abs(orc.cosine_lr(0.1, 0.01, 10, 100, 10) - 0.1) < 1e-6
    assert abs(orc.cosine_lr(0.1, 0.01, 10, 100, 55) - 0.055) < 1e-6
    assert abs(orc.cosine_lr(0.1, 0.01, 10, 100, 100) - 0.01) < 1e-6
    assert abs(orc.cosine_lr(0.1, 0.01, 10, 100, 200) - 0.01) < 1e-6
    orc.reset_all()
    x = T.from_numpy(f32(3, 4), True)
    x.mul(x).sum(0).backward()
    norm = orc.clip_grad_norm([x], 5.0)
    assert abs(norm - 10.0) < 1e-4
    np.testing.assert_allclose(x.grad().numpy(), [3, 4], atol=1e-3)


def test_adamw_8bit_known_answers():
    """crates/vearo-optim/src/lib.rs:461-505: five steps of loss = sum(w * w) from w = [1,2,3,4] with lr 0.1,
    betas (0.9, 0.999), eps 1e-8, weight decay 0.01 -- the 8-bit optimizer must stay within 1e-2 of plain AdamW.
    Plus the quantizer's definition (lib.rs:157-208) on a hand-checkable block: scale = max|x| / 127,
    q = round-half-away(x * 127 / max|x|) clamped to [-127, 127], x' = q * scale."""
    orc.reset_all()
    w_std, w_8 = T.from_numpy(f32(1, 2, 3, 4), True), T.from_numpy(f32(1, 2, 3, 4), True)
    o_std, o_8 = orc.AdamW([w_std], 0.1, 0.9, 0.999, 1e-8, 0.01), orc.AdamW8bit([w_8], 0.1, 0.9, 0.999, 1e-8, 0.01)
    for _ in range(5):
        orc.zero_gradients(); orc.reset_active_tape()
        w_std.mul(w_std).sum(0).backward(); o_std.step()
        orc.zero_gradients(); orc.reset_active_tape()
        w_8.mul(w_8).sum(0).backward(); o_8.step()
    assert np.abs(w_std.numpy() - w_8.numpy()).max() < 1e-2
    # after the first step of a fresh optimizer m = 0.1 g and v = 0.001 g^2; with g = [2, -1, 0.5, 0.0078125]:
    orc.reset_all()
    w = T.from_numpy(f32(1, 1, 1, 1), True)
    g = f32(2, -1, 0.5, 0.0078125)
    w.mul(T.from_numpy(g)).sum(0).backward()
    o = orc.AdamW8bit([w], 0.1, 0.9, 0.999, 1e-8, 0.0)
    o.step()
    m8, ms, v8, vs = o.state(0)
    m = np.float32(0.1) * g                      # (1 - 0.9) * g in f32, as the reference forms it
    m = (np.float32(1.0) - np.float32(0.9)) * g
    assert ms[0] == np.float32(np.abs(m).max() / np.float32(127.0))
    # 127 * [1, -0.5, 0.25, 0.00390625] -> 127, -63.5 -> -64 (half away from zero), 31.75 -> 32, 0.496 -> 0
    assert m8.tolist() == [127, -64, 32, 0]
    v = (np.float32(1.0) - np.float32(0.999)) * g * g
    assert vs[0] == np.float32(v.max() / np.float32(127.0))
    assert v8.tolist() == [127, 32, 8, 0]        # 127 * [1, 0.25, 0.0625, 1.5e-5] -> 127, 31.75 -> 32, 7.94 -> 8, 0


def test_dropout_definition():
    """crates/vearo-nn/src/lib.rs:308-357 with SimpleRng (lib.rs:14-50): mask element i keeps (value 1 / (1 - p)) where the
    i-th xorshift64 draw, as f32 / 2^64, is >= p; the generator is seeded with seed ^ call * 0x9E3779B97F4A7C15 and the call
    counter advances once per forward; identity when p <= 0 or outside training.  Checked against a Python restatement."""
    def mask(seed, call, p, n):
        st = (seed ^ (call * 0x9E3779B97F4A7C15)) & 0xFFFFFFFFFFFFFFFF
        if st == 0: st = 0x123456789ABCDEF0
        out = []
        for _ in range(n):
            st ^= (st << 13) & 0xFFFFFFFFFFFFFFFF; st ^= st >> 7; st ^= (st << 17) & 0xFFFFFFFFFFFFFFFF
            u = np.float32(st) / np.float32(2.0 ** 64)
            out.append(np.float32(1.0) / (np.float32(1.0) - np.float32(p)) if u >= np.float32(p) else np.float32(0.0))
        return np.array(out, np.float32)
    orc.reset_all()
    x = T.from_numpy(np.ones(64, np.float32))
    a, b = x.dropout(0.25, 7).numpy(), x.dropout(0.25, 7).numpy()
    assert np.array_equal(a, mask(7, 0, 0.25, 64)) and np.array_equal(b, mask(7, 1, 0.25, 64)) and orc.rng_counter() == 2
    assert 0 < (a == 0).sum() < 64 and not np.array_equal(a, b)
    orc.set_rng_counter(0)
    assert np.array_equal(x.dropout(0.25, 7).numpy(), a)               # rewinding the counter reproduces the draw
    assert np.array_equal(x.dropout(0.0, 7).numpy(), np.ones(64, np.float32)) and orc.rng_counter() == 1
    orc.set_training(False)
    assert np.array_equal(x.dropout(0.9, 7).numpy(), np.ones(64, np.float32))
    orc.set_training(True)


def test_batchnorm_running_stats():
    """crates/vearo/tests/batchnorm_review.rs:119-174."""
    n, c, h, w = 2, 2, 2, 2
    xd = np.zeros((n, c, h, w), np.float32); xd[:, 0] = 2.0; xd[:, 1] = 6.0
    x = T.from_numpy(xd)
    g, b = T.from_numpy(np.ones(c, np.float32)), T.from_numpy(np.zeros(c, np.float32))
    rm, rv = T.from_numpy(np.zeros(c, np.float32)), T.from_numpy(np.ones(c, np.float32))
    x.batchnorm(g, b, rm, rv, True, 0.1, 1e-5)
    np.testing.assert_allclose(rm.numpy(), [0.2, 0.6], atol=1e-5)
    np.testing.assert_allclose(rv.numpy(), [0.9, 0.9], atol=1e-5)
    before = (rm.numpy().copy(), rv.numpy().copy())
    x.batchnorm(g, b, rm, rv, False, 0.1, 1e-5)
    assert (rm.numpy() == before[0]).all() and (rv.numpy() == before[1]).all()


def test_matmul_block_matches_reference_assembly_bit_for_bit():
    """The oracle's 4x8 block against the reference's own kernel assembled from
    crates/vearo-backend-cpu/src/asm/x86_64/matmul.s (built into oracle/_ref)."""
    path = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libvearo_ref_matmul.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (reference tree absent)")
    ref = C.CDLL(path)
    fp = C.POINTER(C.c_float)
    ref.matmul_block_4x8_avx2_asm.argtypes = [fp, fp, fp, C.c_size_t, C.c_size_t]
    rng = np.random.default_rng(3)
    for k, n in ((1, 8), (7, 16), (768, 24), (3072, 8)):
        a = rng.standard_normal((4, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        o1 = np.zeros((4, n), np.float32); o2 = np.zeros((4, n), np.float32)
        for c0 in range(0, n, 8):
            ref.matmul_block_4x8_avx2_asm(o1[:, c0:].ctypes.data_as(fp), a.ctypes.data_as(fp), b[:, c0:].ctypes.data_as(fp), k, n)
            orc.lib().orc_block_4x8(o2[:, c0:].ctypes.data_as(fp), a.ctypes.data_as(fp), b[:, c0:].ctypes.data_as(fp), k, n)
        assert (o1.view(np.uint32) == o2.view(np.uint32)).all()
        # and the full matmul (threads, 4-row groups, column tails, single rows) is the same fma chain
        for m in (4, 6, 9):
            am = rng.standard_normal((m, k)).astype(np.float32)
            bn = rng.standard_normal((k, n + 3)).astype(np.float32)
            got = T.from_numpy(am).matmul(T.from_numpy(bn)).numpy()
            want = np.zeros((m, n + 3), np.float32)
            for kk in range(k):   # sequential-k fused chain in float64-exact emulation of fmaf
                want = (am[:, kk:kk + 1].astype(np.float64) * bn[kk:kk + 1, :].astype(np.float64) + want.astype(np.float64)).astype(np.float32)
            assert (got.view(np.uint32) == want.view(np.uint32)).all()
