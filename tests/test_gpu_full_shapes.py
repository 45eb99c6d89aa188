"""Parity at the shapes the benchmark workloads really run: the CUDA path against the CPU oracle, value for value.

The per-op tests use small shapes; the kernels pick other instances, tile walks and split factors at the
workloads' widths (sequence 1024 under a causal mask, d_model 768 / 1024, the 50304-wide vocabulary, the
conv net's 64 / 128 / 256 channels).  These cases run those code paths on inputs the oracle still finishes
in seconds: one sequence through a one-block model of full width, four heads of full-length attention, the
fused-op chain on 1024 rows, the conv net on eight full-size images.

Bar: |gpu - cpu| <= 1e-5 + 1e-4 |cpu| per element, and (because most gradients of these models are far
below 1e-5 in magnitude, where the absolute term alone would pass anything) a relative L2 error of the
whole tensor of at most 2e-4.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle import models as om
from vearo_b200 import modelspec as ms
from tests.test_gpu_ops import assert_close, rnd

pytestmark = pytest.mark.gpu

REL_L2 = 2e-4


@pytest.fixture(scope="module")
def vb():
    import vearo_b200 as v
    v.init()
    return v


def close_and_l2(gpu, cpu, name):
    assert_close(gpu, cpu, name, guard=False)
    c = np.asarray(cpu, np.float64); g = np.asarray(gpu, np.float64)
    den = np.sqrt((c * c).sum())
    # (a gradient that is zero in exact arithmetic -- the key bias under softmax's shift invariance, a conv bias ahead of a
    # BatchNorm -- is rounding noise on both sides: only the element-wise bar applies)
    if den > 0 and np.abs(c).max() >= 1e-7:
        rel = np.sqrt(((g - c) ** 2).sum()) / den
        assert rel <= REL_L2, "%s: relative L2 error %.3e" % (name, rel)


# ---- attention at full sequence length (crates/vearo/tests/fused_attention_parity.rs; cpu lib.rs:2368-2630) ----------
@pytest.mark.parametrize("B,H,S,dk,masked", [(1, 4, 1024, 64, True), (2, 2, 768, 64, True), (1, 2, 1024, 64, False), (1, 3, 512, 64, True),
                                                (1, 2, 640, 64, True)])
def test_fused_attention_full_length(vb, B, H, S, dk, masked):
    q0, k0, v0, go = rnd(500, B, H, S, dk), rnd(501, B, H, S, dk), rnd(502, B, H, S, dk), rnd(503, B, H, S, dk)
    mask0 = np.triu(np.full((S, S), -1e9, np.float32), 1)

    def case(T):
        q, k, v = T.from_numpy(q0, True), T.from_numpy(k0, True), T.from_numpy(v0, True)
        o = q.fused_attention(k, v, T.from_numpy(mask0) if masked else None)
        n = go.size
        o.mul(T.from_numpy(go)).reshape([1, n]).matmul(T.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
        return [t.numpy() for t in (o, q.grad(), k.grad(), v.grad())]
    orc.reset_all()
    cpu = case(orc.Tensor)
    vb.zero_gradients(); vb.reset_active_tape()
    gpu = case(vb.Tensor)
    vb.check_errors()
    for g, c, n in zip(gpu, cpu, "out dq dk dv".split()):
        close_and_l2(g, c, "attention S=%d %s" % (S, n))


@pytest.mark.parametrize("B,S,H,dk", [(1, 1024, 4, 64), (2, 768, 2, 64)])
def test_fused_attention_packed_full_length(vb, B, S, H, dk):
    """The packed [B, S, 3D] form the GPT blocks use, causal mask, full sequence length."""
    D = H * dk
    qkv0 = rnd(510, B, S, 3 * D); go = rnd(511, B, S, D)
    mask0 = np.triu(np.full((S, S), -1e9, np.float32), 1)
    orc.reset_all()
    parts = [orc.Tensor.from_numpy(np.ascontiguousarray(qkv0[:, :, i * D:(i + 1) * D].reshape(B, S, H, dk).transpose(0, 2, 1, 3)), True) for i in range(3)]
    o = parts[0].fused_attention(parts[1], parts[2], orc.Tensor.from_numpy(mask0)).transpose(1, 2).reshape([B, S, D])
    n = go.size
    o.mul(orc.Tensor.from_numpy(go)).reshape([1, n]).matmul(orc.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
    want_o = o.numpy()
    want_g = np.concatenate([p.grad().numpy().transpose(0, 2, 1, 3).reshape(B, S, D) for p in parts], axis=2)
    vb.zero_gradients(); vb.reset_active_tape()
    x = vb.Tensor.from_numpy(qkv0, True)
    y = x.fused_attention_packed(H, vb.Tensor.from_numpy(mask0))
    y.mul(vb.Tensor.from_numpy(go)).reshape([1, n]).matmul(vb.Tensor.from_numpy(np.ones((n, 1), np.float32))).reshape([1]).backward()
    vb.check_errors()
    close_and_l2(y.numpy(), want_o, "packed attention S=%d out" % S)
    close_and_l2(x.grad().numpy(), want_g, "packed attention S=%d dqkv" % S)


# ---- one transformer block of full width, full vocabulary, one sequence of 1024 tokens ------------------------------
@pytest.mark.parametrize("name,d,heads,ff", [("config 3 widths", 768, 12, 3072), ("config 5 widths", 1024, 16, 4096)])
def test_gpt_one_block_full_width(vb, name, d, heads, ff):
    V, T = 50304, 1024
    params = ms.gpt_params(V, T, d, 1, ff, seed=5)
    # biases and LayerNorm parameters away from their 0 / 1 initial values, so that every gradient path carries signal
    r = np.random.default_rng(6)
    for i, p in enumerate(params):
        if p.ndim == 1:
            params[i] = (p + r.standard_normal(p.shape) * 0.05).astype(np.float32)
    ids, tg = ms.gpt_batch(V, 1, T, seed=5)
    orc.reset_all(); orc.set_threads(0)
    cm = om.SimpleGPT(params, d, heads, 1)
    _, cl = cm.forward(orc.Tensor.from_numpy(ids), orc.Tensor.from_numpy(tg)); cl.backward()
    gm = vb.SimpleGPT(V, T, d, heads, 1, ff); gm.load(params)
    vb.zero_gradients(); vb.reset_active_tape()
    gl = gm.loss(vb.Tensor.from_numpy(ids), vb.Tensor.from_numpy(tg)); gl.backward()
    vb.check_errors()
    assert_close(gl.numpy(), cl.numpy(), name + " loss")
    for i, (cp, gp) in enumerate(zip(cm.parameters(), gm.parameters())):
        close_and_l2(gp.grad().numpy(), cp.grad().contiguous().numpy(), "%s grad %d %s" % (name, i, tuple(cp.shape)))
    orc.reset_all()


# ---- config 2: LayerNorm -> GELU -> Linear 768 -> 50304 -> cross-entropy on 1024 rows -------------------------------
def test_config2_fused_op_backward_1024_rows(vb):
    x, g, b, W, labels = ms.microbench_inputs(N=1024)
    orc.reset_all(); orc.set_threads(0)
    cx = orc.Tensor.from_numpy(x, True)
    cg, cb, cw = orc.Tensor.from_numpy(g, True), orc.Tensor.from_numpy(b, True), orc.Tensor.from_numpy(W, True)
    cl = cx.layernorm(cg, cb, 1e-5).gelu().matmul(cw.transpose(0, 1)).cross_entropy(orc.Tensor.from_numpy(labels)); cl.backward()
    gm = vb.FusedOpBench(768, 50304); gm.load([g, b, W])
    gx = vb.Tensor.from_numpy(x, True)
    vb.zero_gradients(); vb.reset_active_tape()
    gl = gm.loss(gx, vb.Tensor.from_numpy(labels)); gl.backward()
    vb.check_errors()
    assert_close(gl.numpy(), cl.numpy(), "loss")
    close_and_l2(gx.grad().numpy(), cx.grad().numpy(), "dX")
    gg, gb_, gw = (p.grad().numpy() for p in gm.parameters())
    close_and_l2(gg, cg.grad().numpy(), "dgamma"); close_and_l2(gb_, cb.grad().numpy(), "dbeta")
    close_and_l2(gw, cw.grad().contiguous().numpy(), "dW")
    orc.reset_all()


# ---- config 4: the conv net's three stages at their real channel counts on eight 32x32 images -------------------------
def test_config4_convnet_real_channels(vb):
    ch = (3, 64, 128, 256)
    params = ms.convnet_params(ch, 10); x, labels = ms.convnet_batch(8, 32, 10)
    orc.reset_all(); orc.set_threads(0)
    cm = om.ConvNet(params)
    l = cm.forward(orc.Tensor.from_numpy(x), orc.Tensor.from_numpy(labels)); l.backward()
    gm = vb.ConvNet(ch, 10); gm.load(params)
    vb.zero_gradients(); vb.reset_active_tape()
    gl = gm.loss(vb.Tensor.from_numpy(x), vb.Tensor.from_numpy(labels)); gl.backward()
    vb.check_errors()
    assert_close(gl.numpy(), l.numpy(), "loss")
    for i, (cp, gp) in enumerate(zip(cm.parameters(), gm.parameters())):
        # (a conv bias ahead of a BatchNorm has a gradient that is zero in exact arithmetic: rounding noise on both sides, so
        # only the element-wise bar applies to parameters 1, 5 and 9)
        if i % 4 == 1 and i < 12:
            assert_close(gp.grad().numpy(), cp.grad().contiguous().numpy(), "convnet grad %d" % i, guard=False)
        else:
            close_and_l2(gp.grad().numpy(), cp.grad().contiguous().numpy(), "convnet grad %d %s" % (i, tuple(cp.shape)))
    for s in range(3):
        np.testing.assert_allclose(gm.running(s, 0).numpy(), cm.stages[s]["rm"].numpy(), rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(gm.running(s, 1).numpy(), cm.stages[s]["rv"].numpy(), rtol=1e-4, atol=1e-6)
    orc.reset_all()
