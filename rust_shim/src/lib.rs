//! `vearo-backend-b200`: `libvearo_b200.so` behind `vearo_core::BackendOps` for `Device::Cuda`.
//!
//! Same shape as `crates/vearo-backend-cuda/src/lib.rs:165-242`: `init()` registers the refcount and
//! memory hooks and one wrapper per `BackendOps` field (`crates/vearo-core/src/tensor.rs:1111-1175`).
//! Every wrapper builds `vb_tensor` descriptors from `shape()` / `strides()` (views are passed as
//! they are: no `contiguous()` round trip through the host), calls the C ABI and adopts the fresh
//! outputs with `Tensor::from_components`.
//!
//! NOT COMPILED: the image this repository was built in has no Rust toolchain.  Written against
//! the reference's vearo-core as read there; a maintainer with cargo should expect to fix small
//! things (visibility of `StorageId` fields, `Shape` constructors) but nothing structural.
#![allow(clippy::missing_panics_doc, clippy::too_many_arguments, clippy::similar_names)]

pub mod ffi;

use ffi::*;
use std::ffi::CStr;
use std::os::raw::c_int;
use std::sync::atomic::{AtomicUsize, Ordering};
use vearo_core::{
    BackendOps, DType, Device, Shape, StorageId, Tensor, register_backend_ops, register_cuda_hooks,
    register_refcount_dec, register_refcount_inc,
};

/// The device ordinal `init_on` was given (the reference hard-codes 0, `lib.rs:20-24`).
static ORDINAL: AtomicUsize = AtomicUsize::new(0);

fn device() -> Device {
    Device::Cuda(ORDINAL.load(Ordering::Relaxed))
}

/// A non-zero status becomes the panic the reference's backends raise, carrying the library's text.
fn check(status: c_int) {
    if status != VB_OK {
        let msg = unsafe { CStr::from_ptr(vb_last_error()) }.to_string_lossy().into_owned();
        panic!("{msg}");
    }
}

/// `Tensor` -> `vb_tensor`: a CUDA `StorageId { shard_idx: 0, slot_idx }` (`lib.rs:64-67`) *is* the slot.
fn desc(t: &Tensor) -> vb_tensor {
    let rank = t.shape().rank();
    assert!(rank <= VB_MAX_RANK, "tensor rank above {VB_MAX_RANK}");
    let mut d = vb_tensor { slot: t.storage_id().slot_idx, rank: rank as i32, ..Default::default() };
    for (i, (&n, &s)) in t.shape().dims().iter().zip(t.strides().dims()).enumerate() {
        d.dims[i] = n as i64;
        d.strides[i] = s as i64;
    }
    d
}

fn opt_desc(t: Option<&Tensor>) -> Option<vb_tensor> {
    t.map(desc)
}

fn ptr_or_null(d: &Option<vb_tensor>) -> *const vb_tensor {
    d.as_ref().map_or(std::ptr::null(), |x| x as *const vb_tensor)
}

/// A fresh output of the library (refcount 1, owned by the caller) as a `Tensor`; strides are taken
/// from the descriptor because the attention entry points return `[B,H,S,dk]` views of `[B,S,H,dk]` buffers.
fn adopt(d: &vb_tensor) -> Tensor {
    let r = d.rank as usize;
    let dims: Vec<usize> = d.dims[..r].iter().map(|&x| x as usize).collect();
    let strides: Vec<usize> = d.strides[..r].iter().map(|&x| x as usize).collect();
    Tensor::from_components(
        StorageId { shard_idx: 0, slot_idx: d.slot },
        Shape::new(dims),
        Shape::new(strides),
        DType::F32,
        device(),
    )
}

fn out() -> vb_tensor {
    vb_tensor::default()
}

// ---- memory and refcount hooks (vearo-core/src/tensor.rs:1328-1363) ---------------------------------

/// `CUDA_ALLOC_HOOK`: zero-filled, as the reference's allocator hands out (`lib.rs:41-112`).
pub fn b200_alloc(numel: usize) -> StorageId {
    let mut slot: vb_slot = 0;
    check(unsafe { vb_alloc(numel as i64, 1, &mut slot) });
    StorageId { shard_idx: 0, slot_idx: slot }
}

/// `CUDA_WRITE_HOOK`
pub fn b200_write(id: StorageId, data: &[f32]) {
    check(unsafe { vb_write(id.slot_idx, 0, data.as_ptr(), data.len() as i64) });
}

/// `CUDA_READ_HOOK`: the whole slot, synchronously (`dtoh_sync_copy`, `lib.rs:124-131`).
pub fn b200_read(id: StorageId) -> Vec<f32> {
    let mut n: i64 = 0;
    check(unsafe { vb_slot_numel(id.slot_idx, &mut n) });
    let mut v = vec![0.0f32; n as usize];
    check(unsafe { vb_read(id.slot_idx, 0, v.as_mut_ptr(), n) });
    // invalid token ids / class labels seen by kernels since the last read surface here, as the CPU backend's panics do
    check(unsafe { vb_check_errors() });
    v
}

/// `REFCOUNT_INC`
pub fn b200_refcount_inc(id: StorageId, dev: Device) {
    if matches!(dev, Device::Cuda(_)) {
        check(unsafe { vb_retain(id.slot_idx) });
    }
}

/// `REFCOUNT_DEC`: true when this was the last owner, so that core fires `DROP_HOOK` (`tensor.rs:56-80`).
pub fn b200_refcount_dec(id: StorageId, dev: Device) -> bool {
    if !matches!(dev, Device::Cuda(_)) {
        return false;
    }
    let mut freed: c_int = 0;
    check(unsafe { vb_release(id.slot_idx, &mut freed) });
    freed != 0
}

// ---- the 26 BackendOps fields ----------------------------------------------------------------------

macro_rules! binary {
    ($name:ident, $f:ident) => {
        pub fn $name(lhs: &Tensor, rhs: &Tensor) -> Tensor {
            let (a, b, mut o) = (desc(lhs), desc(rhs), out());
            check(unsafe { $f(&a, &b, &mut o) });
            adopt(&o)
        }
    };
}
binary!(add, vb_add);
binary!(sub, vb_sub);
binary!(mul, vb_mul);
binary!(div, vb_div);
binary!(matmul, vb_matmul);

pub fn relu(x: &Tensor) -> Tensor {
    let (a, mut o) = (desc(x), out());
    check(unsafe { vb_relu(&a, &mut o) });
    adopt(&o)
}

pub fn gelu(x: &Tensor) -> Tensor {
    let (a, mut o) = (desc(x), out());
    check(unsafe { vb_gelu(&a, &mut o) });
    adopt(&o)
}

pub fn sum(x: &Tensor, dim: usize, keep_dim: bool) -> Tensor {
    let (a, mut o) = (desc(x), out());
    check(unsafe { vb_sum(&a, dim as c_int, c_int::from(keep_dim), &mut o) });
    adopt(&o)
}

pub fn mean(x: &Tensor, dim: usize, keep_dim: bool) -> Tensor {
    let (a, mut o) = (desc(x), out());
    check(unsafe { vb_mean(&a, dim as c_int, c_int::from(keep_dim), &mut o) });
    adopt(&o)
}

pub fn softmax(x: &Tensor, dim: usize) -> Tensor {
    let (a, mut o) = (desc(x), out());
    check(unsafe { vb_softmax(&a, dim as c_int, &mut o) });
    adopt(&o)
}

pub fn layernorm(x: &Tensor, weight: &Tensor, bias: &Tensor, eps: f32) -> Tensor {
    let (a, w, b, mut o) = (desc(x), desc(weight), desc(bias), out());
    check(unsafe { vb_layernorm(&a, &w, &b, eps, &mut o) });
    adopt(&o)
}

pub fn layernorm_backward(x: &Tensor, weight: &Tensor, bias: &Tensor, grad_out: &Tensor, eps: f32) -> (Tensor, Tensor, Tensor) {
    let (a, w, b, g) = (desc(x), desc(weight), desc(bias), desc(grad_out));
    let (mut gx, mut gw, mut gb) = (out(), out(), out());
    check(unsafe { vb_layernorm_backward(&a, &w, &b, &g, eps, &mut gx, &mut gw, &mut gb) });
    (adopt(&gx), adopt(&gw), adopt(&gb))
}

pub fn embedding(ids: &Tensor, weight: &Tensor) -> Tensor {
    let (a, w, mut o) = (desc(ids), desc(weight), out());
    check(unsafe { vb_embedding(&a, &w, &mut o) });
    adopt(&o)
}

pub fn embedding_backward(ids: &Tensor, weight: &Tensor, grad_out: &Tensor) -> Tensor {
    let (a, w, g, mut o) = (desc(ids), desc(weight), desc(grad_out), out());
    check(unsafe { vb_embedding_backward(&a, &w, &g, &mut o) });
    adopt(&o)
}

pub fn cross_entropy(logits: &Tensor, targets: &Tensor) -> Tensor {
    let (l, t, mut o) = (desc(logits), desc(targets), out());
    check(unsafe { vb_cross_entropy(&l, &t, &mut o, std::ptr::null_mut()) });
    adopt(&o)
}

pub fn cross_entropy_backward(logits: &Tensor, targets: &Tensor, grad_out: &Tensor) -> Tensor {
    let (l, t, g, mut o) = (desc(logits), desc(targets), desc(grad_out), out());
    check(unsafe { vb_cross_entropy_backward(&l, &t, &g, std::ptr::null(), &mut o) });
    adopt(&o)
}

pub fn conv2d(input: &Tensor, weight: &Tensor, bias: &Tensor, stride: usize, padding: usize) -> Tensor {
    let (x, w, b, mut o) = (desc(input), desc(weight), desc(bias), out());
    check(unsafe { vb_conv2d(&x, &w, &b, stride as c_int, padding as c_int, &mut o) });
    adopt(&o)
}

pub fn conv2d_backward(input: &Tensor, weight: &Tensor, grad_out: &Tensor, stride: usize, padding: usize) -> (Tensor, Tensor, Tensor) {
    let (x, w, g) = (desc(input), desc(weight), desc(grad_out));
    let (mut gx, mut gw, mut gb) = (out(), out(), out());
    check(unsafe { vb_conv2d_backward(&x, &w, &g, stride as c_int, padding as c_int, &mut gx, &mut gw, &mut gb) });
    (adopt(&gx), adopt(&gw), adopt(&gb))
}

pub fn maxpool2d(input: &Tensor, kernel_size: usize, stride: usize, padding: usize) -> Tensor {
    let (x, mut o) = (desc(input), out());
    check(unsafe { vb_maxpool2d(&x, kernel_size as c_int, stride as c_int, padding as c_int, &mut o) });
    adopt(&o)
}

pub fn maxpool2d_backward(input: &Tensor, grad_out: &Tensor, kernel_size: usize, stride: usize, padding: usize) -> Tensor {
    let (x, g, mut o) = (desc(input), desc(grad_out), out());
    check(unsafe { vb_maxpool2d_backward(&x, &g, kernel_size as c_int, stride as c_int, padding as c_int, &mut o) });
    adopt(&o)
}

pub fn avgpool2d(input: &Tensor, kernel_size: usize, stride: usize, padding: usize) -> Tensor {
    let (x, mut o) = (desc(input), out());
    check(unsafe { vb_avgpool2d(&x, kernel_size as c_int, stride as c_int, padding as c_int, &mut o) });
    adopt(&o)
}

pub fn avgpool2d_backward(input: &Tensor, grad_out: &Tensor, kernel_size: usize, stride: usize, padding: usize) -> Tensor {
    let (x, g, mut o) = (desc(input), desc(grad_out), out());
    check(unsafe { vb_avgpool2d_backward(&x, &g, kernel_size as c_int, stride as c_int, padding as c_int, &mut o) });
    adopt(&o)
}

pub fn batchnorm(x: &Tensor, gamma: &Tensor, beta: &Tensor, running_mean: &Tensor, running_var: &Tensor,
                 training: bool, momentum: f32, eps: f32) -> Tensor {
    let (a, g, b, rm, rv, mut o) = (desc(x), desc(gamma), desc(beta), desc(running_mean), desc(running_var), out());
    // training mode updates running_mean / running_var in place on the device (lib.rs:640-720)
    check(unsafe { vb_batchnorm(&a, &g, &b, &rm, &rv, c_int::from(training), momentum, eps, &mut o) });
    adopt(&o)
}

pub fn batchnorm_backward(x: &Tensor, gamma: &Tensor, beta: &Tensor, running_mean: &Tensor, running_var: &Tensor,
                          grad_out: &Tensor, training: bool, eps: f32) -> (Tensor, Tensor, Tensor) {
    let (a, g, b, rm, rv, go) = (desc(x), desc(gamma), desc(beta), desc(running_mean), desc(running_var), desc(grad_out));
    let (mut gx, mut gg, mut gb) = (out(), out(), out());
    check(unsafe { vb_batchnorm_backward(&a, &g, &b, &rm, &rv, &go, c_int::from(training), eps, &mut gx, &mut gg, &mut gb) });
    (adopt(&gx), adopt(&gg), adopt(&gb))
}

/// Runs on the device (the reference's CUDA backend copies q, k, v to the CPU, `lib.rs:1595-1606`).
pub fn fused_attention(q: &Tensor, k: &Tensor, v: &Tensor, mask: Option<&Tensor>) -> Tensor {
    let (a, b, c, m, mut o) = (desc(q), desc(k), desc(v), opt_desc(mask), out());
    check(unsafe { vb_fused_attention(&a, &b, &c, ptr_or_null(&m), &mut o, std::ptr::null_mut()) });
    adopt(&o)
}

/// `BackendOps` has no slot for the saved probabilities, so the backward call recomputes them
/// (`probs_or_null` = NULL), as the reference's does (`vearo-backend-cpu/src/lib.rs:2480-2630`).
pub fn fused_attention_backward(q: &Tensor, k: &Tensor, v: &Tensor, mask: Option<&Tensor>, grad_out: &Tensor) -> (Tensor, Tensor, Tensor) {
    let (a, b, c, m, g) = (desc(q), desc(k), desc(v), opt_desc(mask), desc(grad_out));
    let (mut dq, mut dk, mut dv) = (out(), out(), out());
    check(unsafe { vb_fused_attention_backward(&a, &b, &c, ptr_or_null(&m), &g, std::ptr::null(), &mut dq, &mut dk, &mut dv) });
    (adopt(&dq), adopt(&dk), adopt(&dv))
}

// ---- entry points for the two changes inside Vearo that the north star names ------------------------------
// (autograd's host-side arms and the optimizers' CUDA branches: see INTEGRATION.md for where they are called from)

/// `relu_grad_mask` + multiply (`vearo-autograd/src/lib.rs:364-374, 537-541`) on the device.
pub fn relu_backward(x: &Tensor, grad_out: &Tensor) -> Tensor {
    let (a, g, mut o) = (desc(x), desc(grad_out), out());
    check(unsafe { vb_relu_backward(&a, &g, &mut o) });
    adopt(&o)
}

/// `gelu_grad_mask` + multiply (`lib.rs:383-403, 542-546`).
pub fn gelu_backward(x: &Tensor, grad_out: &Tensor) -> Tensor {
    let (a, g, mut o) = (desc(x), desc(grad_out), out());
    check(unsafe { vb_gelu_backward(&a, &g, &mut o) });
    adopt(&o)
}

/// The Softmax arm (`lib.rs:547-553`); `x` is the softmax input.
pub fn softmax_backward(x: &Tensor, grad_out: &Tensor, dim: usize) -> Tensor {
    let (a, g, mut o) = (desc(x), desc(grad_out), out());
    check(unsafe { vb_softmax_backward(&a, &g, dim as c_int, &mut o) });
    adopt(&o)
}

/// `reduce_to` (`lib.rs:316-361`) without the device-to-host copy of the gradient.
pub fn reduce_to(grad: &Tensor, target: &Shape) -> Tensor {
    let (g, mut o) = (desc(grad), out());
    let dims: Vec<i64> = target.dims().iter().map(|&d| d as i64).collect();
    check(unsafe { vb_reduce_to(&g, dims.as_ptr(), dims.len() as c_int, &mut o) });
    adopt(&o)
}

/// In-place gradient accumulation (`lib.rs:733-742` allocates a fresh sum).
pub fn accumulate(dst: &Tensor, src: &Tensor) {
    let (d, s) = (desc(dst), desc(src));
    check(unsafe { vb_accumulate(&d, &s) });
}

/// The CUDA branch of `Tensor::adamw_step` (`vearo-core/src/tensor.rs:989-1019`): m and v are device slots
/// (`StorageId`s the optimizer allocates once with `b200_alloc`), nothing crosses to the host.
pub fn adamw_step(param: &Tensor, grad: &Tensor, m: StorageId, v: StorageId, t: u32, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32) {
    let (p, g) = (desc(param), desc(grad));
    check(unsafe { vb_adamw_step(&p, &g, m.slot_idx, v.slot_idx, t, lr, beta1, beta2, eps, weight_decay) });
}

/// The CUDA branch of `Tensor::sgd_step` (`tensor.rs:1073-1092`).
pub fn sgd_step(param: &Tensor, grad: &Tensor, velocity: StorageId, lr: f32, momentum: f32, weight_decay: f32) {
    let (p, g) = (desc(param), desc(grad));
    check(unsafe { vb_sgd_step(&p, &g, velocity.slot_idx, lr, momentum, weight_decay) });
}

/// `clip_grad_norm` (`vearo-optim/src/lib.rs:360-383`) over device gradients; returns the pre-clip norm.
pub fn clip_grad_norm(grads: &[&Tensor], max_norm: f32) -> f32 {
    let ds: Vec<vb_tensor> = grads.iter().map(|g| desc(g)).collect();
    let mut norm = 0.0f32;
    check(unsafe { vb_clip_grad_norm(ds.as_ptr(), ds.len() as c_int, max_norm, &mut norm) });
    norm
}

// ---- init ---------------------------------------------------------------------------------------------

/// `init()` of `vearo-backend-cuda` (`lib.rs:165-242`): hooks, then the op table.  No PTX is loaded:
/// the kernels are sm_100a machine code inside the shared library.
pub fn init() {
    init_on(0);
}

/// The same on a chosen GPU (one process per GPU under data parallelism: rank r calls `init_on(r)`).
pub fn init_on(ordinal: usize) {
    ORDINAL.store(ordinal, Ordering::Relaxed);
    check(unsafe { vb_init(ordinal as c_int) });
    register_refcount_inc(b200_refcount_inc);
    register_refcount_dec(b200_refcount_dec);
    register_cuda_hooks(b200_read, b200_write, b200_alloc);
    register_backend_ops(
        Device::Cuda(ordinal),
        BackendOps {
            add,
            sub,
            mul,
            div,
            matmul,
            sum,
            mean,
            relu,
            gelu,
            softmax,
            layernorm,
            layernorm_backward,
            embedding,
            embedding_backward,
            cross_entropy,
            cross_entropy_backward,
            conv2d,
            conv2d_backward,
            maxpool2d,
            maxpool2d_backward,
            avgpool2d,
            avgpool2d_backward,
            batchnorm,
            batchnorm_backward,
            fused_attention,
            fused_attention_backward,
        },
    );
}
