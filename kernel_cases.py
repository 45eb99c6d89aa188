"""Small single-kernel cases of the library's hot kernels, for profiling with ncu and quick timing.

  python kernel_cases.py gemm_fc1      x[8192,768] . W[3072,768]^T   (Linear forward)
  python kernel_cases.py gemm_proj     x[8192,768] . W[768,768]^T    (192 tiles of 128 x 256 for 296 CTA slots)
  python kernel_cases.py gemm_dx       g[8192,3072] . W[3072,768]    (B consumed as a transposed view)
  python kernel_cases.py gemm_dw       g[8192,3072]^T . x[8192,768]  (both operands transposed views, split-K)
  python kernel_cases.py gemm_qk       scores of 96 heads: [1024,64] . [1024,64]^T
  python kernel_cases.py gemm_pv       96 heads: P[1024,1024] . V[1024,64]  (64-wide tiles, 32-wide k-blocks)
  python kernel_cases.py attention     causal attention forward + backward, packed qkv [8,1024,2304], 12 heads
  python kernel_cases.py attention_fwd  the same forward alone, nothing kept for a backward pass (no probabilities written)
  python kernel_cases.py conv_bwd       conv 3x3 (64 -> 128 channels) on [256,64,16,16], forward + backward: implicit GEMMs over the padded NHWC copy
  python kernel_cases.py bn_bwd         fused BatchNorm -> ReLU -> MaxPool on [256,128,16,16], forward + backward
  python kernel_cases.py colsum        bias gradients: column sums of [8192,768] and [8192,3072]
  python kernel_cases.py gelu_bwd      GELU backward over [8192,3072], with the column sums of the result
  python kernel_cases.py layernorm_bwd rows 8192, C 768
  python kernel_cases.py ce_bwd        rows 2048, V 50304
  python kernel_cases.py ce_fused      rows 2048, V 50304: loss and gradient in one in-place pass
  python kernel_cases.py adamw         64 Mi parameters
  python kernel_cases.py adamw8bit     64 Mi parameters, int8 block-wise moments
A second argument gives the repetition count (default 3); `time` instead prints the average device
time per repetition over 20 repetitions (CUDA events through the library's profiling hooks are not
used here: the loop is synchronised on both sides and timed on the host).
Each case holds well under 2 GB on the device.
"""
import sys
import time

import numpy as np

import vearo_b200 as vb


def build(case):
    r = np.random.default_rng(0)
    f = lambda *s: (r.standard_normal(s) * 0.05).astype(np.float32)
    T = vb.Tensor.from_numpy
    if case == "gemm_fc1":
        x, w = T(f(8192, 768)), T(f(3072, 768))
        return lambda: x.linear(w)
    if case == "gemm_proj":
        x, w = T(f(8192, 768)), T(f(768, 768))
        return lambda: x.linear(w)
    if case == "gemm_dx":
        g, w = T(f(8192, 3072)), T(f(3072, 768))
        return lambda: g.matmul(w)
    if case == "gemm_dw":
        g, x = T(f(8192, 3072)), T(f(8192, 768))
        gt = g.transpose(0, 1)
        return lambda: gt.matmul(x)
    if case == "gemm_qk":
        q, k = T(f(8, 12, 1024, 64)), T(f(8, 12, 1024, 64))
        kt = k.transpose(2, 3)
        return lambda: q.matmul(kt)
    if case == "gemm_pv":
        pr, v = T(f(8, 12, 1024, 1024)), T(f(8, 12, 1024, 64))
        return lambda: pr.matmul(v)
    if case == "attention":
        qkv, go = T(f(8, 1024, 2304), True), T(f(8, 1024, 768))
        mask = T(np.triu(np.full((1024, 1024), -1e9, np.float32), 1))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            qkv.fused_attention_packed(12, mask).mul(go).sum(2, False).sum(1, False).sum(0, False).backward()
        return run
    if case == "attention_fwd":
        qkv = T(f(8, 1024, 2304))
        mask = T(np.triu(np.full((1024, 1024), -1e9, np.float32), 1))
        return lambda: qkv.fused_attention_packed(12, mask)
    if case == "conv_bwd":
        x, w, b = T(f(256, 64, 16, 16), True), T(f(128, 64, 3, 3), True), T(f(128), True)
        go = T(f(256, 128, 16, 16))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            x.conv2d(w, b, 1, 1).mul(go).sum(3, False).sum(2, False).sum(1, False).sum(0, False).backward()
        return run
    if case == "bn_bwd":
        x, g, b = T(f(256, 128, 16, 16), True), T(f(128) + 1.0, True), T(f(128), True)
        rm, rv = T(np.zeros(128, np.float32)), T(np.ones(128, np.float32))
        go = T(f(256, 128, 8, 8))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            x.bn_relu_maxpool(g, b, rm, rv, True, 0.1, 1e-5).mul(go).sum(3, False).sum(2, False).sum(1, False).sum(0, False).backward()
        return run
    if case == "colsum":
        a, b = T(f(8192, 768)), T(f(8192, 3072))
        ba, bb = T(f(768), True), T(f(3072), True)

        def run():      # the bias of a broadcast add gets its gradient as a column sum
            vb.zero_gradients(); vb.reset_active_tape()
            a.add(ba).sum(1, False).sum(0, False).backward()
            vb.zero_gradients(); vb.reset_active_tape()
            b.add(bb).sum(1, False).sum(0, False).backward()
        return run
    if case == "gelu_bwd":
        x, g = T(f(8192, 3072), True), T(f(8192, 3072))

        def run():      # the backward kernel also leaves the column sums of its result (the bias gradient of the layer before)
            vb.zero_gradients(); vb.reset_active_tape()
            x.gelu().mul(g).sum(1, False).sum(0, False).backward()
        return run
    if case == "layernorm_bwd":
        x, w, b, g = T(f(8192, 768), True), T(f(768), True), T(f(768), True), T(f(8192, 768))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            x.layernorm(w, b, 1e-5).mul(g).sum(1, False).sum(0, False).backward()
        return run
    if case == "ce_bwd":
        l, t = T(f(2048, 50304), True), T(r.integers(0, 50304, 2048).astype(np.float32))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            l.cross_entropy(t).backward()
        return run
    if case == "ce_fused":
        x, w = T(f(2048, 16), True), T(f(16, 50304))
        t = T(r.integers(0, 50304, 2048).astype(np.float32))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            x.matmul(w).cross_entropy_consuming(t).backward()
        return run
    if case in ("adamw", "adamw8bit"):
        w = T(f(64 << 20), True)
        opt = vb.AdamW([w], 1e-3) if case == "adamw" else vb.AdamW8bit([w], 1e-3)
        g = T(f(64 << 20))

        def run():
            vb.zero_gradients(); vb.reset_active_tape()
            w.mul(g).sum(0, False).backward()
            opt.clip_and_step(1.0)
        return run
    raise SystemExit("unknown case " + case)


def main(case, mode):
    vb.init()
    fn = build(case)
    if mode == "time":
        for _ in range(3):
            fn()
        vb.sync(); t0 = time.perf_counter()
        for _ in range(20):
            fn()
        vb.sync()
        print("%s: %.1f us per call (host clock)" % (case, (time.perf_counter() - t0) / 20 * 1e6))
        # device time of every kernel family (CUDA events around each launcher)
        import ctypes as C
        L = vb.lib()
        vb.vb_check(L.vb_profile_reset()); vb.vb_check(L.vb_profile_enable(1))
        for _ in range(20):
            fn()
        vb.sync(); vb.vb_check(L.vb_profile_enable(0))
        buf = C.create_string_buffer(4096)
        vb.vb_check(L.vb_profile_families(buf, 4096))
        for fam in [f for f in buf.value.decode().split(",") if f]:
            t, n, u = C.c_double(0), C.c_int64(0), C.c_double(0)
            vb.vb_check(L.vb_profile_read(fam.encode(), C.byref(t), C.byref(n), C.byref(u), None))
            if n.value:
                print("  %-28s %4d launches  %9.1f us each (device)" % (fam, n.value, 1e3 * t.value / n.value))
    else:
        for _ in range(int(mode)):
            fn()
        vb.sync()
    vb.check_errors()
    print("ok", case)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else "3")
