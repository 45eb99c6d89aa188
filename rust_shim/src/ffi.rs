//! The C ABI of `include/vearo_b200.h`, declaration for declaration.
//! NOT COMPILED here (no Rust toolchain in the build image); kept in step with the header by hand.
#![allow(non_camel_case_types, clippy::too_many_arguments)]
use std::os::raw::{c_char, c_int, c_void};

pub const VB_MAX_RANK: usize = 8;
pub const VB_OK: c_int = 0;
pub const VB_ERR_BAD_INDEX: c_int = 5;

pub type vb_slot = u32;

/// `vb_tensor`: a view of a device slot (element offset, dims and element strides).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct vb_tensor {
    pub slot: vb_slot,
    pub rank: i32,
    pub offset: i64,
    pub dims: [i64; VB_MAX_RANK],
    pub strides: [i64; VB_MAX_RANK],
}

/// `vb_opt_config`
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct vb_opt_config {
    pub kind: i32, // 0 AdamW, 1 SGD, 2 AdamW8bit
    pub lr: f32,
    pub beta1: f32,
    pub beta2: f32,
    pub eps: f32,
    pub weight_decay: f32,
    pub momentum: f32,
}

type T = *const vb_tensor;
type O = *mut vb_tensor;

unsafe extern "C" {
    // context
    pub fn vb_init(device_ordinal: c_int) -> c_int;
    pub fn vb_shutdown() -> c_int;
    pub fn vb_last_error() -> *const c_char;
    pub fn vb_device_ordinal(ordinal: *mut c_int) -> c_int;
    pub fn vb_sync() -> c_int;
    pub fn vb_check_errors() -> c_int;
    pub fn vb_stream(stream: *mut *mut c_void) -> c_int;
    // device memory
    pub fn vb_alloc(numel: i64, zero_fill: c_int, out: *mut vb_slot) -> c_int;
    pub fn vb_retain(slot: vb_slot) -> c_int;
    pub fn vb_release(slot: vb_slot, freed: *mut c_int) -> c_int;
    pub fn vb_write(slot: vb_slot, offset: i64, host: *const f32, numel: i64) -> c_int;
    pub fn vb_read(slot: vb_slot, offset: i64, host: *mut f32, numel: i64) -> c_int;
    pub fn vb_ptr(slot: vb_slot, device_ptr: *mut *mut c_void) -> c_int;
    pub fn vb_slot_numel(slot: vb_slot, numel: *mut i64) -> c_int;
    pub fn vb_memory_stats(live_slots: *mut i64, live_bytes: *mut i64, cached_bytes: *mut i64, peak_bytes: *mut i64) -> c_int;
    pub fn vb_memory_reset_peak() -> c_int;
    // one entry point per BackendOps field
    pub fn vb_add(a: T, b: T, out: O) -> c_int;
    pub fn vb_sub(a: T, b: T, out: O) -> c_int;
    pub fn vb_mul(a: T, b: T, out: O) -> c_int;
    pub fn vb_div(a: T, b: T, out: O) -> c_int;
    pub fn vb_matmul(a: T, b: T, out: O) -> c_int;
    pub fn vb_relu(x: T, out: O) -> c_int;
    pub fn vb_gelu(x: T, out: O) -> c_int;
    pub fn vb_sum(x: T, dim: c_int, keep_dim: c_int, out: O) -> c_int;
    pub fn vb_mean(x: T, dim: c_int, keep_dim: c_int, out: O) -> c_int;
    pub fn vb_softmax(x: T, dim: c_int, out: O) -> c_int;
    pub fn vb_layernorm(x: T, w: T, b: T, eps: f32, out: O) -> c_int;
    pub fn vb_layernorm_backward(x: T, w: T, b: T, grad_out: T, eps: f32, gx: O, gw: O, gb: O) -> c_int;
    pub fn vb_embedding(ids: T, weight: T, out: O) -> c_int;
    pub fn vb_embedding_backward(ids: T, weight: T, grad_out: T, gw: O) -> c_int;
    pub fn vb_cross_entropy(logits: T, targets: T, loss: O, row_stats: O) -> c_int;
    pub fn vb_cross_entropy_fused(logits_inout: T, targets: T, loss: O) -> c_int;
    pub fn vb_cross_entropy_backward(logits: T, targets: T, grad_out: T, row_stats_or_null: T, glogits: O) -> c_int;
    pub fn vb_conv2d(x: T, w: T, bias: T, stride: c_int, padding: c_int, out: O) -> c_int;
    pub fn vb_conv2d_backward(x: T, w: T, grad_out: T, stride: c_int, padding: c_int, gx: O, gw: O, gb: O) -> c_int;
    pub fn vb_maxpool2d(x: T, kernel: c_int, stride: c_int, padding: c_int, out: O) -> c_int;
    pub fn vb_maxpool2d_backward(x: T, grad_out: T, kernel: c_int, stride: c_int, padding: c_int, gx: O) -> c_int;
    pub fn vb_avgpool2d(x: T, kernel: c_int, stride: c_int, padding: c_int, out: O) -> c_int;
    pub fn vb_avgpool2d_backward(x: T, grad_out: T, kernel: c_int, stride: c_int, padding: c_int, gx: O) -> c_int;
    pub fn vb_batchnorm(x: T, gamma: T, beta: T, running_mean: T, running_var: T, training: c_int, momentum: f32, eps: f32, out: O) -> c_int;
    pub fn vb_batchnorm_backward(x: T, gamma: T, beta: T, running_mean: T, running_var: T, grad_out: T, training: c_int, eps: f32,
                                 gx: O, ggamma: O, gbeta: O) -> c_int;
    pub fn vb_bn_relu_maxpool(x: T, gamma: T, beta: T, running_mean: T, running_var: T, training: c_int, momentum: f32, eps: f32,
                              out: O, stats: O) -> c_int;
    pub fn vb_bn_relu_maxpool_backward(x: T, gamma: T, beta: T, stats: T, grad_out: T, training: c_int, gx: O, ggamma: O, gbeta: O) -> c_int;
    pub fn vb_fused_attention(q: T, k: T, v: T, mask_or_null: T, out: O, probs: O) -> c_int;
    pub fn vb_fused_attention_backward(q: T, k: T, v: T, mask_or_null: T, grad_out: T, probs_or_null: T, dq: O, dk: O, dv: O) -> c_int;
    pub fn vb_fused_attention_packed(qkv: T, n_head: c_int, mask_or_null: T, out: O, probs_or_null: O) -> c_int;
    pub fn vb_fused_attention_packed_backward(qkv: T, n_head: c_int, mask_or_null: T, grad_out: T, probs_or_null: T, dqkv: O) -> c_int;
    // backward arms the reference computes on the host for CUDA tensors
    pub fn vb_relu_backward(x: T, grad_out: T, gx: O) -> c_int;
    pub fn vb_gelu_backward(x: T, grad_out: T, gx: O) -> c_int;
    pub fn vb_softmax_backward(x: T, grad_out: T, dim: c_int, gx: O) -> c_int;
    pub fn vb_reduce_to(grad: T, target_dims: *const i64, target_rank: c_int, out: O) -> c_int;
    pub fn vb_accumulate(dst: T, src: T) -> c_int;
    pub fn vb_copy(dst: T, src: T) -> c_int;
    pub fn vb_scale(x: T, alpha: f32, out: O) -> c_int;
    pub fn vb_contiguous(x: T, out: O) -> c_int;
    pub fn vb_fill(dst: T, value: f32) -> c_int;
    pub fn vb_layernorm_backward_noalloc(x: *const f32, w: *const f32, grad_out: *const f32, gx: *mut f32, gw: *mut f32, gb: *mut f32,
                                         rows: i64, c: i64, eps: f32, stream: *mut c_void) -> c_int;
    // fused linear layer (extras)
    pub fn vb_linear(x: T, weight: T, bias_or_null: T, out: O) -> c_int;
    pub fn vb_linear_backward(x: T, weight: T, grad_out: T, gx: O, gw: O, gb: O) -> c_int;
    pub fn vb_linear_gelu(x: T, weight: T, bias_or_null: T, pre: O, act: O) -> c_int;
    pub fn vb_layernorm_backward_accum(x: T, w: T, b: T, grad_out: T, eps: f32, grad_in: T, gw: O, gb: O) -> c_int;
    pub fn vb_linear_backward_into(x: T, weight: T, grad_out: T, gx_or_null: O, gw_into_or_null: T, gb_into_or_null: T) -> c_int;
    // optimizer
    pub fn vb_adamw_step(param: T, grad: T, m: vb_slot, v: vb_slot, t: u32, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32) -> c_int;
    pub fn vb_sgd_step(param: T, grad: T, velocity: vb_slot, lr: f32, momentum: f32, weight_decay: f32) -> c_int;
    pub fn vb_clip_grad_norm(grads: T, n: c_int, max_norm: f32, total_norm: *mut f32) -> c_int;
    pub fn vb_opt_create(cfg: *const vb_opt_config, params: T, grads: T, n: c_int, opt: *mut c_int) -> c_int;
    pub fn vb_opt_destroy(opt: c_int) -> c_int;
    pub fn vb_opt_set_lr(opt: c_int, lr: f32) -> c_int;
    pub fn vb_opt_state(opt: c_int, state: *mut vb_slot, state_numel: *mut i64, step: *mut u32) -> c_int;
    pub fn vb_opt_set_step(opt: c_int, step: u32) -> c_int;
    pub fn vb_opt_state8(opt: c_int, param: c_int, m8: *mut i8, m_scales: *mut f32, v8: *mut i8, v_scales: *mut f32) -> c_int;
    pub fn vb_opt_step(opt: c_int, active: *const u8, max_norm: f32, grad_scale: f32, total_norm: *mut f32) -> c_int;
    // profiling
    pub fn vb_launch_count(count: *mut i64) -> c_int;
    pub fn vb_selftest_wait_timeout(polls: u32, elapsed_ms: *mut f64) -> c_int;
    pub fn vb_tc_launch_count(count: *mut i64) -> c_int;
    pub fn vb_profile_enable(on: c_int) -> c_int;
    pub fn vb_profile_reset() -> c_int;
    pub fn vb_profile_read(family: *const c_char, total_ms: *mut f64, launches: *mut i64, units: *mut f64, dense_units: *mut f64) -> c_int;
    pub fn vb_profile_families(buf: *mut c_char, buflen: c_int) -> c_int;
    // data parallel
    pub fn vb_dp_unique_id(id: *mut u8) -> c_int;
    pub fn vb_dp_init(rank: c_int, world: c_int, id: *const u8) -> c_int;
    pub fn vb_dp_world(rank: *mut c_int, world: *mut c_int) -> c_int;
    pub fn vb_dp_alloc(numel: i64, zero_fill: c_int, out: *mut vb_slot) -> c_int;
    pub fn vb_dp_is_registered(slot: vb_slot, yes: *mut c_int) -> c_int;
    pub fn vb_dp_allreduce(slot: vb_slot, offset: i64, numel: i64) -> c_int;
    pub fn vb_dp_finish(timeout_ms: c_int) -> c_int;
    pub fn vb_dp_wait() -> c_int;
    pub fn vb_dp_shutdown() -> c_int;
}
