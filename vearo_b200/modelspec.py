"""Seeded synthetic parameters and inputs for the five workloads, as NumPy arrays.

The CPU checker of the tests and the CUDA library are fed these same arrays, so parity never depends
on two random generators agreeing; the benchmark draws its synthetic workloads from here too.  Parameter order is the order of the reference's
`parameters()` methods (crates/vearo-nn/src/lib.rs:679-687, 797-806).
"""
import numpy as np


def gpt_params(vocab, T, d, n_layer, ff, seed=0, std=0.02):
    """N(0, std^2) matrices and embeddings, LayerNorm gamma 1 / beta 0, biases 0."""
    r = np.random.default_rng(seed)
    n = lambda *s: (r.standard_normal(s) * std).astype(np.float32)
    ps = [n(vocab, d), n(T, d)]
    for _ in range(n_layer):
        ps += [np.ones(d, np.float32), np.zeros(d, np.float32)]
        for _ in range(4):
            ps += [n(d, d), np.zeros(d, np.float32)]
        ps += [np.ones(d, np.float32), np.zeros(d, np.float32)]
        ps += [n(ff, d), np.zeros(ff, np.float32), n(d, ff), np.zeros(d, np.float32)]
    ps += [np.ones(d, np.float32), np.zeros(d, np.float32), n(vocab, d)]
    return ps


def gpt_batch(vocab, B, T, seed=0):
    """Uniform token ids as f32 (the reference stores ids as f32); targets = next token."""
    r = np.random.default_rng(seed + 1000)
    ids = r.integers(0, vocab, (B, T + 1))
    return ids[:, :-1].astype(np.float32), ids[:, 1:].astype(np.float32)


def mlp_params(sizes=(2, 32, 32, 1), seed=42):
    """Kaiming-uniform: U(-sqrt(6/fan_in), +sqrt(6/fan_in)) weights, zero biases."""
    r = np.random.default_rng(seed)
    ps = []
    for fi, fo in zip(sizes[:-1], sizes[1:]):
        bound = np.sqrt(6.0 / fi)
        ps += [r.uniform(-bound, bound, (fo, fi)).astype(np.float32), np.zeros(fo, np.float32)]
    return ps


def mlp_batch(n=256, seed=42):
    r = np.random.default_rng(seed + 7)
    x = r.uniform(-1, 1, (n, 2)).astype(np.float32)
    y = (np.sin(np.pi * x[:, 0]) + x[:, 1] ** 2).astype(np.float32).reshape(n, 1)
    return x, y


def convnet_params(channels=(3, 64, 128, 256), n_class=10, seed=1):
    r = np.random.default_rng(seed)
    ps = []
    for ci, co in zip(channels[:-1], channels[1:]):
        bound = 1.0 / np.sqrt(ci * 9)
        ps += [r.uniform(-bound, bound, (co, ci, 3, 3)).astype(np.float32), r.uniform(-bound, bound, co).astype(np.float32),
               np.ones(co, np.float32), np.zeros(co, np.float32)]
    bound = 1.0 / np.sqrt(channels[-1])
    ps += [r.uniform(-bound, bound, (n_class, channels[-1])).astype(np.float32), r.uniform(-bound, bound, n_class).astype(np.float32)]
    return ps


def convnet_batch(n=256, hw=32, n_class=10, seed=1):
    r = np.random.default_rng(seed + 11)
    return r.standard_normal((n, 3, hw, hw)).astype(np.float32), r.integers(0, n_class, n).astype(np.float32)


def microbench_inputs(N=8192, C=768, V=50304, seed=0):
    """LayerNorm(gamma 1, beta 0) -> GELU -> Linear C->V -> cross-entropy."""
    r = np.random.default_rng(seed)
    x = r.standard_normal((N, C)).astype(np.float32)
    W = (r.standard_normal((V, C)) * 0.02).astype(np.float32)
    labels = r.integers(0, V, N).astype(np.float32)
    return x, np.ones(C, np.float32), np.zeros(C, np.float32), W, labels
