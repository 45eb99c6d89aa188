"""vearo_b200 — B200 (sm_100a) training hot path for Vearo: Python driver over the C ABI.

The product is `libvearo_b200.so` (hand-written CUDA kernels, the `vb_*` C ABI declared in
include/vearo_b200.h, and the C++ host mirror of Vearo's Tensor / autograd / nn / optim layers).
This module only loads it and wraps handles; there is no CPU path and no fallback: if the library
is missing, or no B200 is present when a device call is made, it raises.

`Tensor`, `AdamW`, `SGD`, `clip_grad_norm`, `zero_gradients`, `reset_active_tape` carry the names
and argument meaning of the reference's public API (crates/vearo-core/src/tensor.rs,
crates/vearo-optim/src/lib.rs, crates/vearo-autograd/src/lib.rs).
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# VB200_LIB selects another build of the library (the bounds-check build, libvearo_b200_bc.so)
LIB_PATH = os.environ.get("VB200_LIB") or os.path.join(_HERE, "libvearo_b200.so")

c_f32p = C.POINTER(C.c_float)
c_i64p = C.POINTER(C.c_int64)
c_intp = C.POINTER(C.c_int)
VB_MAX_RANK = 8


class VbTensor(C.Structure):
    """`vb_tensor` of include/vearo_b200.h."""
    _fields_ = [("slot", C.c_uint32), ("rank", C.c_int32), ("offset", C.c_int64),
                ("dims", C.c_int64 * VB_MAX_RANK), ("strides", C.c_int64 * VB_MAX_RANK)]

    @staticmethod
    def contiguous(slot, shape, offset=0):
        t = VbTensor()
        t.slot, t.rank, t.offset = slot, len(shape), offset
        s = 1
        for i in range(len(shape) - 1, -1, -1):
            t.dims[i] = shape[i]
            t.strides[i] = s
            s *= shape[i]
        return t

    @property
    def shape(self):
        return tuple(self.dims[i] for i in range(self.rank))


class VearoError(RuntimeError):
    pass


_lib = None
_inited = False


def lib():
    """The loaded shared library; raises if it has not been built (python -m vearo_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise VearoError("libvearo_b200.so is missing: run `python vearo_b200/build.py` (needs nvcc); "
                             "there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        L.vb_last_error.restype = C.c_char_p
        L.vh_last_error.restype = C.c_char_p
        L.vh_cosine_lr.restype = C.c_float
        L.vh_cosine_lr.argtypes = [C.c_float, C.c_float, C.c_uint32, C.c_uint32, C.c_uint32]
        L.vh_layernorm.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float]
        L.vh_batchnorm.argtypes = [C.c_int] * 6 + [C.c_float, C.c_float]
        L.vh_bn_relu_maxpool.argtypes = [C.c_int] * 6 + [C.c_float, C.c_float]
        L.vh_adamw_new.argtypes = [c_intp, C.c_int] + [C.c_float] * 5 + [C.c_int]
        L.vh_sgd_new.argtypes = [c_intp, C.c_int] + [C.c_float] * 3 + [C.c_int]
        L.vh_adamw8bit_new.argtypes = [c_intp, C.c_int] + [C.c_float] * 5 + [C.c_int]
        L.vh_opt_state8.argtypes = [C.c_int, C.c_int, C.c_void_p, c_f32p, C.c_void_p, c_f32p]
        L.vh_opt_set_lr.argtypes = [C.c_int, C.c_float]
        for fn in (L.vh_opt_save_state, L.vh_opt_load_state, L.vh_save_checkpoint, L.vh_load_checkpoint):
            fn.argtypes = [C.c_int, C.c_char_p]
        L.vh_opt_clip_and_step.argtypes = [C.c_int, C.c_float, c_f32p]
        L.vh_clip_grad_norm.argtypes = [c_intp, C.c_int, C.c_float, c_f32p]
        L.vh_gpt_new.argtypes = [C.c_int64] * 6
        L.vh_convnet_new.argtypes = [c_i64p, C.c_int, C.c_int64]
        L.vh_fusedop_new.argtypes = [C.c_int64, C.c_int64]
        L.vh_train_step.argtypes = [C.c_int, C.c_int, c_f32p, c_i64p, C.c_int, C.c_int, c_f32p, c_i64p, C.c_int,
                                    C.c_float, c_f32p, c_f32p]
        L.vh_train_step_resident.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        # vb_* entry points used directly by the C-ABI tests
        L.vb_alloc.argtypes = [C.c_int64, C.c_int, C.POINTER(C.c_uint32)]
        L.vb_write.argtypes = [C.c_uint32, C.c_int64, c_f32p, C.c_int64]
        L.vb_read.argtypes = [C.c_uint32, C.c_int64, c_f32p, C.c_int64]
        L.vb_release.argtypes = [C.c_uint32, c_intp]
        L.vb_retain.argtypes = [C.c_uint32]
        L.vb_scale.argtypes = [C.POINTER(VbTensor), C.c_float, C.POINTER(VbTensor)]
        L.vb_fill.argtypes = [C.POINTER(VbTensor), C.c_float]
        L.vb_layernorm.argtypes = [C.POINTER(VbTensor)] * 3 + [C.c_float, C.POINTER(VbTensor)]
        L.vb_layernorm_backward.argtypes = [C.POINTER(VbTensor)] * 4 + [C.c_float] + [C.POINTER(VbTensor)] * 3
        L.vb_layernorm_backward_accum.argtypes = [C.POINTER(VbTensor)] * 4 + [C.c_float] + [C.POINTER(VbTensor)] * 3
        L.vb_adamw_step.argtypes = [C.POINTER(VbTensor), C.POINTER(VbTensor), C.c_uint32, C.c_uint32, C.c_uint32] + [C.c_float] * 5
        L.vb_sgd_step.argtypes = [C.POINTER(VbTensor), C.POINTER(VbTensor), C.c_uint32] + [C.c_float] * 3
        L.vb_clip_grad_norm.argtypes = [C.POINTER(VbTensor), C.c_int, C.c_float, c_f32p]
        L.vb_batchnorm.argtypes = [C.POINTER(VbTensor)] * 5 + [C.c_int, C.c_float, C.c_float, C.POINTER(VbTensor)]
        L.vb_batchnorm_backward.argtypes = [C.POINTER(VbTensor)] * 6 + [C.c_int, C.c_float] + [C.POINTER(VbTensor)] * 3
        L.vb_memory_stats.argtypes = [c_i64p] * 4
        L.vb_dp_unique_id.argtypes = [C.POINTER(C.c_uint8)]
        L.vb_dp_init.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_uint8)]
        _lib = L
    return _lib


def vb_check(status, what="vb call"):
    if status != 0:
        raise VearoError("%s failed (status %d): %s" % (what, status, lib().vb_last_error().decode()))


def init(device_ordinal=None):
    """vb_init on this process's GPU (LOCAL_RANK by default).  Raises without a B200."""
    global _inited
    if device_ordinal is None:
        device_ordinal = int(os.environ.get("LOCAL_RANK", "0"))
    vb_check(lib().vb_init(device_ordinal), "vb_init")
    _inited = True


def _ensure():
    if not _inited:
        init()


def _chk(rc):
    if rc == -1:
        raise VearoError(lib().vh_last_error().decode())
    return rc


def _shape_arg(shape):
    shape = tuple(int(s) for s in shape)
    return (C.c_int64 * max(1, len(shape)))(*shape), len(shape)


class Tensor:
    """Handle to a device tensor of the C++ host mirror (vearo::Tensor)."""
    __slots__ = ("h",)

    def __init__(self, h):
        self.h = _chk(h)

    def __del__(self):
        try:
            if _lib is not None and self.h >= 0:
                _lib.vh_free(self.h)
        except Exception:
            pass

    @staticmethod
    def from_numpy(a, requires_grad=False):
        _ensure()
        a = np.ascontiguousarray(a, dtype=np.float32)
        sh, r = _shape_arg(a.shape)
        return Tensor(lib().vh_tensor(a.ctypes.data_as(c_f32p), sh, r, int(requires_grad)))

    from_f32 = from_numpy

    @property
    def shape(self):
        out = (C.c_int64 * 8)()
        r = _chk(lib().vh_shape(self.h, out))
        return tuple(out[i] for i in range(r))

    def numpy(self):
        out = np.empty(self.shape, dtype=np.float32)
        _chk(lib().vh_read(self.h, out.ctypes.data_as(c_f32p)))
        return out

    def write(self, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        assert a.shape == self.shape, (a.shape, self.shape)
        _chk(lib().vh_write(self.h, a.ctypes.data_as(c_f32p)))

    def desc(self):
        d = VbTensor()
        _chk(lib().vh_desc(self.h, C.byref(d)))
        return d

    def set_requires_grad(self, f=True):
        _chk(lib().vh_set_requires_grad(self.h, int(f)))
        return self

    def is_contiguous(self): return bool(_chk(lib().vh_is_contiguous(self.h)))

    def add(self, o): return Tensor(lib().vh_binary(0, self.h, o.h))
    def sub(self, o): return Tensor(lib().vh_binary(1, self.h, o.h))
    def mul(self, o): return Tensor(lib().vh_binary(2, self.h, o.h))
    def div(self, o): return Tensor(lib().vh_binary(3, self.h, o.h))
    def matmul(self, o): return Tensor(lib().vh_matmul(self.h, o.h))
    def relu(self): return Tensor(lib().vh_relu(self.h))
    def gelu(self): return Tensor(lib().vh_gelu(self.h))
    def softmax(self, dim): return Tensor(lib().vh_softmax(self.h, dim))
    def sum(self, dim, keep_dim=False): return Tensor(lib().vh_sum(self.h, dim, int(keep_dim)))
    def mean(self, dim, keep_dim=False): return Tensor(lib().vh_mean(self.h, dim, int(keep_dim)))
    def layernorm(self, w, b, eps): return Tensor(lib().vh_layernorm(self.h, w.h, b.h, eps))
    def embedding(self, w): return Tensor(lib().vh_embedding(self.h, w.h))
    def cross_entropy(self, t): return Tensor(lib().vh_cross_entropy(self.h, t.h))

    def dropout(self, p, seed):
        """vearo_nn::Dropout::new(p, seed).forward(self): the reference's mask for (seed, call counter), identity when not training."""
        lib().vh_dropout.argtypes = [C.c_int, C.c_float, C.c_uint64]
        return Tensor(_chk(lib().vh_dropout(self.h, p, seed)))

    def cross_entropy_consuming(self, t):
        """cross_entropy for logits that are needed for nothing else: when the loss will be differentiated, one pass returns
        the loss and leaves the logits' gradient in their place."""
        return Tensor(lib().vh_cross_entropy_consuming(self.h, t.h))
    def conv2d(self, w, b, stride, padding): return Tensor(lib().vh_conv2d(self.h, w.h, b.h, stride, padding))
    def maxpool2d(self, k, s, p): return Tensor(lib().vh_maxpool2d(self.h, k, s, p))
    def avgpool2d(self, k, s, p): return Tensor(lib().vh_avgpool2d(self.h, k, s, p))

    def batchnorm(self, g, b, rm, rv, training, momentum, eps):
        return Tensor(lib().vh_batchnorm(self.h, g.h, b.h, rm.h, rv.h, int(training), momentum, eps))

    def bn_relu_maxpool(self, g, b, rm, rv, training, momentum, eps):
        """batchnorm -> relu -> maxpool2d(2, 2, 0) in one fused op."""
        return Tensor(lib().vh_bn_relu_maxpool(self.h, g.h, b.h, rm.h, rv.h, int(training), momentum, eps))

    def fused_attention(self, k, v, mask=None):
        return Tensor(lib().vh_fused_attention(self.h, k.h, v.h, -1 if mask is None else mask.h))

    def fused_attention_packed(self, n_head, mask=None):
        """self = [B, S, 3*D] with column blocks q | k | v; returns the [B, S, D] context."""
        return Tensor(lib().vh_fused_attention_packed(self.h, int(n_head), -1 if mask is None else mask.h))

    def linear(self, w, b=None): return Tensor(lib().vh_linear(self.h, w.h, -1 if b is None else b.h))

    def linear_gelu(self, w, b=None):
        """self.linear(w, b).gelu() in one device call (the activation comes out of the GEMM's epilogue)."""
        return Tensor(lib().vh_linear_gelu(self.h, w.h, -1 if b is None else b.h))

    def reshape(self, shape):
        sh, r = _shape_arg(shape)
        return Tensor(lib().vh_reshape(self.h, sh, r))

    def transpose(self, d0, d1): return Tensor(lib().vh_transpose(self.h, d0, d1))

    def permute(self, axes):
        ax, r = _shape_arg(axes)
        return Tensor(lib().vh_permute(self.h, ax, r))

    def contiguous(self): return Tensor(lib().vh_contiguous(self.h))

    def backward(self): _chk(lib().vh_backward(self.h))

    def grad(self):
        h = lib().vh_grad(self.h)
        return None if h == -2 else Tensor(h)


def _handles(ts):
    return (C.c_int * max(1, len(ts)))(*[t.h for t in ts]), len(ts)


class _Opt:
    o = -1

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def step(self): _chk(lib().vh_opt_step(self.o))

    def clip_and_step(self, max_norm):
        n = C.c_float(0)
        _chk(lib().vh_opt_clip_and_step(self.o, max_norm, C.byref(n)))
        return n.value

    def set_lr(self, lr): _chk(lib().vh_opt_set_lr(self.o, lr))

    def gradients_registered(self):
        """True when the gradient arena is a buffer registered with the communicator (data parallel, NCCL user buffers)."""
        return bool(_chk(lib().vh_opt_gradients_registered(self.o)))

    def save_state(self, path):
        """m, v (or the velocity) and the step counter, as a `.ve` container."""
        _chk(lib().vh_opt_save_state(self.o, str(path).encode()))

    def load_state(self, path): _chk(lib().vh_opt_load_state(self.o, str(path).encode()))

    def close(self):
        if self.o >= 0:
            lib().vh_opt_free(self.o)
            self.o = -1


class AdamW(_Opt):
    """vearo_optim::AdamW::new(params, lr, beta1, beta2, eps, weight_decay)."""

    def __init__(self, params, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, data_parallel=False):
        hs, n = _handles(params)
        self.params = list(params)
        self.o = _chk(lib().vh_adamw_new(hs, n, lr, beta1, beta2, eps, weight_decay, int(data_parallel)))


class AdamW8bit(_Opt):
    """vearo_optim::AdamW8bit::new(params, lr, beta1, beta2, eps, weight_decay): AdamW whose moments are held as int8
    with one scale per 256 elements (crates/vearo-optim/src/lib.rs:211-303)."""

    def __init__(self, params, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, data_parallel=False):
        hs, n = _handles(params)
        self.params = list(params)
        self.o = _chk(lib().vh_adamw8bit_new(hs, n, lr, beta1, beta2, eps, weight_decay, int(data_parallel)))

    def state(self, i):
        """(m int8, m scales, v int8, v scales) of parameter i, as QuantizedState holds them."""
        n = int(np.prod(self.params[i].shape)) if len(self.params[i].shape) else 1
        nb = (n + 255) // 256
        m8, v8 = np.zeros(n, np.int8), np.zeros(n, np.int8)
        ms, vs = np.zeros(nb, np.float32), np.zeros(nb, np.float32)
        _chk(lib().vh_opt_state8(self.o, i, m8.ctypes.data, ms.ctypes.data_as(c_f32p), v8.ctypes.data, vs.ctypes.data_as(c_f32p)))
        return m8, ms, v8, vs


class SGD(_Opt):
    """vearo_optim::SGD::new(params, lr, momentum, weight_decay)."""

    def __init__(self, params, lr, momentum=0.0, weight_decay=0.0, data_parallel=False):
        hs, n = _handles(params)
        self.params = list(params)
        self.o = _chk(lib().vh_sgd_new(hs, n, lr, momentum, weight_decay, int(data_parallel)))


def clip_grad_norm(params, max_norm):
    hs, n = _handles(params)
    out = C.c_float(0)
    _chk(lib().vh_clip_grad_norm(hs, n, max_norm, C.byref(out)))
    return out.value


def cosine_lr(base, min_lr, warmup, total, step): return float(lib().vh_cosine_lr(base, min_lr, warmup, total, step))
def zero_gradients(): lib().vh_zero_gradients()


def reset_active_tape():
    lib().vh_reset_active_tape()
    del _ckpt_keep[:]          # blocks of tapes that are gone


_CKPT_FN = C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)
_ckpt_keep = []


def checkpoint(x, fn):
    """vearo_autograd::checkpoint(x, f): f(x) runs now without recording (its activations are freed as it goes) and once
    more, recorded, when backward reaches it.  `fn` maps a Tensor to a Tensor."""
    def call(hin, _user):
        try:
            out = fn(Tensor(hin))
            _ckpt_keep.append(out)      # the handle must outlive this call: the library copies the tensor after it returns
            return out.h
        except Exception:               # an exception may not cross the C boundary
            import traceback
            traceback.print_exc()
            return -1
    cb = _CKPT_FN(call)
    _ckpt_keep.append(cb)
    lib().vh_checkpoint.argtypes = [C.c_int, _CKPT_FN, C.c_void_p]
    return Tensor(_chk(lib().vh_checkpoint(x.h, cb, None)))


def is_recomputing(): return bool(lib().vh_is_recomputing())


def rng_counter():
    lib().vh_rng_counter.restype = C.c_uint64
    return int(lib().vh_rng_counter())


def set_rng_counter(v):
    lib().vh_set_rng_counter.argtypes = [C.c_uint64]
    lib().vh_set_rng_counter(int(v))
def set_training(t): lib().vh_set_training(int(t))
def set_autograd_enabled(e): lib().vh_set_autograd_enabled(int(e))
def sync(): vb_check(lib().vb_sync(), "vb_sync")
def check_errors(): vb_check(lib().vb_check_errors(), "vb_check_errors")


def plan_buckets(numels, target_elems):
    """The data-parallel gradient-bucket plan for parameters of the given sizes (host arithmetic, no GPU needed).
    Returns dict(param_offset, bucket_of, buckets=[(offset, numel), ...], total)."""
    n = len(numels)
    arr = (C.c_int64 * max(1, n))(*numels)
    po = (C.c_int64 * max(1, n))(); bo = (C.c_int * max(1, n))()
    boff = (C.c_int64 * max(1, n))(); bnum = (C.c_int64 * max(1, n))(); total = C.c_int64(0)
    nb = _chk(lib().vh_plan_buckets(arr, n, C.c_int64(target_elems), po, bo, boff, bnum, max(1, n), C.byref(total)))
    return dict(param_offset=list(po)[:n], bucket_of=list(bo)[:n], buckets=[(boff[i], bnum[i]) for i in range(nb)], total=total.value)


def memory_stats():
    v = [C.c_int64(0) for _ in range(4)]
    vb_check(lib().vb_memory_stats(*[C.byref(x) for x in v]))
    return dict(live_slots=v[0].value, live_bytes=v[1].value, cached_bytes=v[2].value, peak_bytes=v[3].value)


class Model:
    """A workload graph held by the C++ host mirror (vearo::nn::Model)."""

    def __init__(self, m):
        self.m = _chk(m)
        n = _chk(lib().vh_model_num_params(self.m))
        self._params = [Tensor(lib().vh_model_param(self.m, i)) for i in range(n)]

    def parameters(self): return list(self._params)

    def set_checkpointing(self, on=True):
        """SimpleGPT only: wrap every transformer block in activation checkpointing."""
        _chk(lib().vh_gpt_set_checkpointing(self.m, int(on)))

    def load(self, arrays):
        assert len(arrays) == len(self._params), (len(arrays), len(self._params))
        for p, a in zip(self._params, arrays):
            p.write(a)

    def loss(self, x, y): return Tensor(lib().vh_model_loss(self.m, x.h, y.h))

    def save_checkpoint(self, path):
        """vearo::checkpoint::save_checkpoint(&params, path): the reference's `.ve` weight file."""
        _chk(lib().vh_save_checkpoint(self.m, str(path).encode()))

    def load_checkpoint(self, path): _chk(lib().vh_load_checkpoint(self.m, str(path).encode()))

    def train_step(self, opt, x, y, max_norm=0.0, x_requires_grad=False):
        """One full step from HOST arrays (H2D of inputs and D2H of the loss included)."""
        x = np.ascontiguousarray(x, dtype=np.float32); y = np.ascontiguousarray(y, dtype=np.float32)
        xs, xr = _shape_arg(x.shape); ys, yr = _shape_arg(y.shape)
        loss, norm = C.c_float(0), C.c_float(0)
        _chk(lib().vh_train_step(self.m, opt.o, x.ctypes.data_as(c_f32p), xs, xr, int(x_requires_grad),
                                 y.ctypes.data_as(c_f32p), ys, yr, max_norm, C.byref(loss), C.byref(norm)))
        return loss.value, norm.value

    def train_step_resident(self, opt, x, y, max_norm=0.0):
        """The same step with inputs already on the device; returns the loss tensor (no sync)."""
        return Tensor(lib().vh_train_step_resident(self.m, opt.o, x.h, y.h, max_norm))


def SimpleGPT(vocab, max_seq, n_embd, n_head, n_layer, mlp_dim):
    _ensure()
    return Model(lib().vh_gpt_new(vocab, max_seq, n_embd, n_head, n_layer, mlp_dim))


def MLP(sizes):
    _ensure()
    arr, n = _shape_arg(sizes)
    return Model(lib().vh_mlp_new(arr, n))


def ConvNet(channels=(3, 64, 128, 256), n_class=10):
    _ensure()
    arr, n = _shape_arg(channels)
    m = Model(lib().vh_convnet_new(arr, n, n_class))
    m.running = lambda stage, which: Tensor(lib().vh_convnet_running(m.m, stage, which))
    return m


def FusedOpBench(c, v):
    _ensure()
    return Model(lib().vh_fusedop_new(c, v))
