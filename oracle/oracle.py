"""ctypes front end of the CPU oracle (liboracle.so, built by oracle/build.py).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, from the smoke check and from the
cpu-baseline leg of the benchmark; the shipped package never imports it.

The `Tensor` class mirrors the method names of the reference's `vearo_core::Tensor`
(crates/vearo-core/src/tensor.rs:1365-1970) so that parity tests read like the
reference's own tests.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None

c_i64p = C.POINTER(C.c_int64)
c_f32p = C.POINTER(C.c_float)
c_intp = C.POINTER(C.c_int)


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build as _b
            _b.build()
        _lib = C.CDLL(path)
        _lib.orc_last_error.restype = C.c_char_p
        _lib.orc_numel.restype = C.c_int64
        _lib.orc_clip_grad_norm.restype = C.c_float
        _lib.orc_cosine_lr.restype = C.c_float
        _lib.orc_cosine_lr.argtypes = [C.c_float, C.c_float, C.c_uint32, C.c_uint32, C.c_uint32]
        for name in ("orc_layernorm",):
            getattr(_lib, name).argtypes = [C.c_int, C.c_int, C.c_int, C.c_float]
        _lib.orc_batchnorm.argtypes = [C.c_int] * 6 + [C.c_float, C.c_float]
        _lib.orc_layernorm_backward.argtypes = [C.c_int] * 4 + [C.c_float, c_intp]
        _lib.orc_batchnorm_backward.argtypes = [C.c_int] * 6 + [C.c_float, c_intp]
        _lib.orc_adamw_create.argtypes = [c_intp, C.c_int] + [C.c_float] * 5
        _lib.orc_adamw8bit_create.argtypes = [c_intp, C.c_int] + [C.c_float] * 5
        _lib.orc_opt_state8.argtypes = [C.c_int, C.c_int, C.c_void_p, c_f32p, C.c_void_p, c_f32p]
        _lib.orc_sgd_create.argtypes = [c_intp, C.c_int] + [C.c_float] * 3
        _lib.orc_opt_set_lr.argtypes = [C.c_int, C.c_float]
        _lib.orc_clip_grad_norm.argtypes = [c_intp, C.c_int, C.c_float]
        _lib.orc_block_4x8.argtypes = [c_f32p, c_f32p, c_f32p, C.c_size_t, C.c_size_t]
    return _lib


class OracleError(RuntimeError):
    """Raised where the reference would panic; carries the reference's panic text."""


def _chk(rc):
    if rc == -1:
        raise OracleError(lib().orc_last_error().decode())
    return rc


def _shape_arg(shape):
    arr = (C.c_int64 * max(1, len(shape)))(*shape)
    return arr, len(shape)


class Tensor:
    __slots__ = ("h",)

    def __init__(self, h):
        self.h = _chk(h)

    # -- construction / inspection
    @staticmethod
    def from_numpy(a, requires_grad=False):
        a = np.ascontiguousarray(a, dtype=np.float32)
        sh, r = _shape_arg(a.shape)
        return Tensor(lib().orc_tensor(a.ctypes.data_as(c_f32p), sh, r, int(requires_grad)))

    from_f32 = from_numpy

    @property
    def shape(self):
        out = (C.c_int64 * 8)()
        r = _chk(lib().orc_shape(self.h, out))
        return tuple(out[i] for i in range(r))

    def numpy(self):
        out = np.empty(self.shape, dtype=np.float32)
        _chk(lib().orc_read(self.h, out.ctypes.data_as(c_f32p)))
        return out

    def write(self, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        _chk(lib().orc_write(self.h, a.ctypes.data_as(c_f32p)))

    def set_requires_grad(self, f=True):
        _chk(lib().orc_set_requires_grad(self.h, int(f)))
        return self

    def is_contiguous(self):
        return bool(_chk(lib().orc_is_contiguous(self.h)))

    # -- ops (names as in the reference)
    def add(self, o): return Tensor(lib().orc_binary(0, self.h, o.h))
    def sub(self, o): return Tensor(lib().orc_binary(1, self.h, o.h))
    def mul(self, o): return Tensor(lib().orc_binary(2, self.h, o.h))

    def dropout(self, p, seed):
        """vearo_nn::Dropout::new(p, seed).forward(self) (crates/vearo-nn/src/lib.rs:308-357)."""
        lib().orc_dropout.argtypes = [C.c_int, C.c_float, C.c_uint64]
        return Tensor(_chk(lib().orc_dropout(self.h, p, seed)))
    def div(self, o): return Tensor(lib().orc_binary(3, self.h, o.h))
    def matmul(self, o): return Tensor(lib().orc_matmul(self.h, o.h))
    def relu(self): return Tensor(lib().orc_relu(self.h))
    def gelu(self): return Tensor(lib().orc_gelu(self.h))
    def softmax(self, dim): return Tensor(lib().orc_softmax(self.h, dim))
    def sum(self, dim, keep_dim=False): return Tensor(lib().orc_sum(self.h, dim, int(keep_dim)))
    def mean(self, dim, keep_dim=False): return Tensor(lib().orc_mean(self.h, dim, int(keep_dim)))
    def layernorm(self, w, b, eps): return Tensor(lib().orc_layernorm(self.h, w.h, b.h, eps))
    def embedding(self, w): return Tensor(lib().orc_embedding(self.h, w.h))
    def cross_entropy(self, t): return Tensor(lib().orc_cross_entropy(self.h, t.h))
    def conv2d(self, w, b, stride, padding): return Tensor(lib().orc_conv2d(self.h, w.h, b.h, stride, padding))
    def maxpool2d(self, k, s, p): return Tensor(lib().orc_maxpool2d(self.h, k, s, p))
    def avgpool2d(self, k, s, p): return Tensor(lib().orc_avgpool2d(self.h, k, s, p))

    def batchnorm(self, g, b, rm, rv, training, momentum, eps):
        return Tensor(lib().orc_batchnorm(self.h, g.h, b.h, rm.h, rv.h, int(training), momentum, eps))

    def fused_attention(self, k, v, mask=None):
        return Tensor(lib().orc_fused_attention(self.h, k.h, v.h, -1 if mask is None else mask.h))

    def reshape(self, shape):
        sh, r = _shape_arg(tuple(shape))
        return Tensor(lib().orc_reshape(self.h, sh, r))

    def transpose(self, d0, d1): return Tensor(lib().orc_transpose(self.h, d0, d1))

    def permute(self, axes):
        ax, r = _shape_arg(tuple(axes))
        return Tensor(lib().orc_permute(self.h, ax, r))

    def contiguous(self): return Tensor(lib().orc_contiguous(self.h))

    # -- explicit backward entry points of BackendOps
    def _triple(self, fn, *args):
        out = (C.c_int * 3)()
        _chk(fn(*args, out))
        return Tensor(out[0]), Tensor(out[1]), Tensor(out[2])

    def layernorm_backward(self, w, b, go, eps):
        return self._triple(lib().orc_layernorm_backward, self.h, w.h, b.h, go.h, eps)

    def embedding_backward(self, w, go): return Tensor(lib().orc_embedding_backward(self.h, w.h, go.h))
    def cross_entropy_backward(self, t, go): return Tensor(lib().orc_cross_entropy_backward(self.h, t.h, go.h))

    def conv2d_backward(self, w, go, stride, padding):
        return self._triple(lib().orc_conv2d_backward, self.h, w.h, go.h, stride, padding)

    def maxpool2d_backward(self, go, k, s, p): return Tensor(lib().orc_maxpool2d_backward(self.h, go.h, k, s, p))
    def avgpool2d_backward(self, go, k, s, p): return Tensor(lib().orc_avgpool2d_backward(self.h, go.h, k, s, p))

    def batchnorm_backward(self, g, b, rm, rv, go, training, eps):
        return self._triple(lib().orc_batchnorm_backward, self.h, g.h, rm.h, rv.h, go.h, int(training), eps)

    def fused_attention_backward(self, k, v, mask, go):
        return self._triple(lib().orc_fused_attention_backward, self.h, k.h, v.h, -1 if mask is None else mask.h, go.h)

    def reduce_to(self, shape):
        sh, r = _shape_arg(tuple(shape))
        return Tensor(lib().orc_reduce_to(self.h, sh, r))

    # -- autograd
    def backward(self): _chk(lib().orc_backward(self.h))

    def grad(self):
        h = lib().orc_grad(self.h)
        if h == -2:
            return None
        return Tensor(h)


def _handles(params):
    return (C.c_int * max(1, len(params)))(*[p.h for p in params]), len(params)


class AdamW:
    """vearo_optim::AdamW (crates/vearo-optim/src/lib.rs:61-135)."""

    def __init__(self, params, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        hs, n = _handles(params)
        self.o = _chk(lib().orc_adamw_create(hs, n, lr, beta1, beta2, eps, weight_decay))

    def step(self): _chk(lib().orc_opt_step(self.o))
    def set_lr(self, lr): _chk(lib().orc_opt_set_lr(self.o, lr))


class AdamW8bit:
    """vearo_optim::AdamW8bit (crates/vearo-optim/src/lib.rs:211-303): AdamW whose moments live as int8 with one
    scale per 256 elements, dequantized before and requantized after every step."""

    def __init__(self, params, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        hs, n = _handles(params)
        self.sizes = [int(np.prod(p.shape)) if len(p.shape) else 1 for p in params]
        self.o = _chk(lib().orc_adamw8bit_create(hs, n, lr, beta1, beta2, eps, weight_decay))

    def step(self): _chk(lib().orc_opt_step(self.o))
    def set_lr(self, lr): _chk(lib().orc_opt_set_lr(self.o, lr))

    def state(self, i):
        """(m int8, m scales, v int8, v scales) of parameter i."""
        n = self.sizes[i]; nb = (n + 255) // 256
        m8, v8 = np.zeros(n, np.int8), np.zeros(n, np.int8)
        ms, vs = np.zeros(nb, np.float32), np.zeros(nb, np.float32)
        _chk(lib().orc_opt_state8(self.o, i, m8.ctypes.data, ms.ctypes.data_as(c_f32p), v8.ctypes.data, vs.ctypes.data_as(c_f32p)))
        return m8, ms, v8, vs


class SGD:
    """vearo_optim::SGD (crates/vearo-optim/src/lib.rs:7-58)."""

    def __init__(self, params, lr, momentum=0.0, weight_decay=0.0):
        hs, n = _handles(params)
        self.o = _chk(lib().orc_sgd_create(hs, n, lr, momentum, weight_decay))

    def step(self): _chk(lib().orc_opt_step(self.o))
    def set_lr(self, lr): _chk(lib().orc_opt_set_lr(self.o, lr))


def clip_grad_norm(params, max_norm):
    hs, n = _handles(params)
    norm = float(lib().orc_clip_grad_norm(hs, n, max_norm))
    if norm < 0:
        raise OracleError(lib().orc_last_error().decode())
    return norm


def cosine_lr(base, min_lr, warmup, total, step):
    return float(lib().orc_cosine_lr(base, min_lr, warmup, total, step))


def zero_gradients(): lib().orc_zero_gradients()
def reset_active_tape(): lib().orc_reset_tape()
def reset_all(): lib().orc_reset_all()
def set_training(t): lib().orc_set_training(int(t))


def rng_counter():
    lib().orc_rng_counter.restype = C.c_uint64
    return int(lib().orc_rng_counter())


def set_rng_counter(v):
    lib().orc_set_rng_counter.argtypes = [C.c_uint64]
    lib().orc_set_rng_counter(int(v))
def set_threads(n): lib().orc_set_threads(int(n))
def get_threads(): return int(lib().orc_get_threads())
def set_autograd_enabled(e): lib().orc_set_autograd(int(e))
