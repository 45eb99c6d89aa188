/*
 * vearo_b200 — C ABI of the B200 (sm_100a) training hot path for Vearo.
 *
 * This is the boundary a Vearo backend crate binds through FFI.  It replaces, for
 * `Device::Cuda`, what the reference implements in crates/vearo-backend-cuda/src/lib.rs
 * (device memory, kernel loading, dispatch) and moves onto the device the arithmetic the
 * reference still does on the host for CUDA tensors (gradient reduction, activation masks,
 * optimizer steps).  Citations below are file:line in the reference project.
 *
 * Conventions
 *   - Every function returns a status (VB_OK == 0).  Nothing aborts, nothing throws across
 *     the boundary; vb_last_error() returns the text of the last failure on this thread.
 *   - Storage is a refcounted *slot* (uint32_t, 0 = none), the counterpart of the reference's
 *     `StorageId { shard_idx: 0, slot_idx }` for CUDA tensors
 *     (crates/vearo-backend-cuda/src/lib.rs:26-112).  Views share a slot.
 *   - A tensor crossing the boundary is a `vb_tensor`: slot + element offset + shape + element
 *     strides (rank <= 8, f32 only), i.e. the fields of `vearo_core::Tensor`
 *     (crates/vearo-core/src/tensor.rs:10-18).  Inputs may be strided views; outputs are freshly
 *     allocated, contiguous, refcount 1, and owned by the caller (vb_release when done).
 *   - Token ids and class labels are f32 tensors rounded half away from zero, as in the
 *     reference (crates/vearo-backend-cpu/src/lib.rs:899,1021).  Negative or out-of-range ids do
 *     not fault: they set a device error flag that vb_check_errors() reports.
 *   - One context per process, one compute stream; the API is thread-compatible (the caller
 *     serialises calls), not re-entrant.  All work is asynchronous on the compute stream;
 *     vb_read / vb_sync / vb_check_errors synchronise.
 */
#ifndef VEARO_B200_H
#define VEARO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VB_MAX_RANK 8

enum vb_status {
  VB_OK = 0,
  VB_ERR_INVALID = 1,      /* bad argument: shape mismatch, bad slot, rank, ... */
  VB_ERR_CUDA = 2,         /* a CUDA runtime call failed */
  VB_ERR_NOT_INIT = 3,     /* vb_init has not been called */
  VB_ERR_OOM = 4,          /* device allocation failed */
  VB_ERR_BAD_INDEX = 5,    /* a kernel saw a negative / out-of-range token id or class */
  VB_ERR_COMM = 6,         /* collective library missing or a collective failed */
  VB_ERR_COMM_TIMEOUT = 7, /* a collective did not complete before the host deadline */
  VB_ERR_UNSUPPORTED = 8
};

typedef uint32_t vb_slot;

typedef struct vb_tensor {
  vb_slot slot;
  int32_t rank;
  int64_t offset;                /* element offset of the view inside the slot */
  int64_t dims[VB_MAX_RANK];
  int64_t strides[VB_MAX_RANK];  /* element strides */
} vb_tensor;

/* ---- context ---------------------------------------------------------------------------
 * Replaces `init` / `CudaDevice::new(0)` / `load_ptx` (vearo-backend-cuda/src/lib.rs:165-242):
 * kernels are sm_100a machine code linked into this library, nothing is JIT-compiled and the
 * device ordinal is the caller's, not a hard-coded 0. */
int vb_init(int device_ordinal);
int vb_shutdown(void);
const char* vb_last_error(void);
int vb_device_ordinal(int* ordinal);
int vb_sync(void);
/* Reads and clears the device error flag (invalid ids).  VB_ERR_BAD_INDEX if it was set. */
int vb_check_errors(void);
/* The compute stream as a cudaStream_t, for callers that record their own events on it. */
int vb_stream(void** stream);

/* ---- device memory ---------------------------------------------------------------------
 * Replaces cuda_alloc / cuda_read / cuda_write and the refcount hooks
 * (vearo-backend-cuda/src/lib.rs:41-163; hook types vearo-core/src/tensor.rs:1328-1363). */
int vb_alloc(int64_t numel, int zero_fill, vb_slot* out);
int vb_retain(vb_slot slot);
int vb_release(vb_slot slot, int* freed);         /* *freed = 1 when this was the last owner */
int vb_write(vb_slot slot, int64_t offset, const float* host, int64_t numel);  /* H2D, stream-ordered */
int vb_read(vb_slot slot, int64_t offset, float* host, int64_t numel);         /* D2H, synchronises */
int vb_ptr(vb_slot slot, void** device_ptr);
int vb_slot_numel(vb_slot slot, int64_t* numel);
/* Live slots and bytes held by them / cached by the arena (memory-regression tests, the
 * counterpart of PEAK_CUDA_MEM_BYTES, vearo-backend-cuda/src/lib.rs:35,73-82). */
int vb_memory_stats(int64_t* live_slots, int64_t* live_bytes, int64_t* cached_bytes, int64_t* peak_bytes);
/* Start a new peak measurement from the bytes live now (the reference's peak counter only ever grows). */
int vb_memory_reset_peak(void);

/* ---- forward ops: one per field of `BackendOps` (vearo-core/src/tensor.rs:1111-1175) ---- */
int vb_add(const vb_tensor* a, const vb_tensor* b, vb_tensor* out);   /* vearo-backend-cuda lib.rs:832-899 */
int vb_sub(const vb_tensor* a, const vb_tensor* b, vb_tensor* out);
int vb_mul(const vb_tensor* a, const vb_tensor* b, vb_tensor* out);
int vb_div(const vb_tensor* a, const vb_tensor* b, vb_tensor* out);
/* [..,M,K] x [..,K,N]; leading dims broadcast; transposed / strided operands are consumed in
 * place (vearo-backend-cuda lib.rs:914-1010, vearo-backend-cpu lib.rs:266-417). */
int vb_matmul(const vb_tensor* a, const vb_tensor* b, vb_tensor* out);
int vb_relu(const vb_tensor* x, vb_tensor* out);                      /* lib.rs:1108-1140 */
int vb_gelu(const vb_tensor* x, vb_tensor* out);
int vb_sum(const vb_tensor* x, int dim, int keep_dim, vb_tensor* out);   /* lib.rs:1012-1090 */
int vb_mean(const vb_tensor* x, int dim, int keep_dim, vb_tensor* out);
int vb_softmax(const vb_tensor* x, int dim, vb_tensor* out);             /* lib.rs:1142-1203 */
int vb_layernorm(const vb_tensor* x, const vb_tensor* w, const vb_tensor* b, float eps, vb_tensor* out); /* lib.rs:1205-1261 */
int vb_layernorm_backward(const vb_tensor* x, const vb_tensor* w, const vb_tensor* b, const vb_tensor* grad_out,
                          float eps, vb_tensor* gx, vb_tensor* gw, vb_tensor* gb);                       /* lib.rs:1263-1353 */
int vb_embedding(const vb_tensor* ids, const vb_tensor* weight, vb_tensor* out);                         /* lib.rs:1355-1409 */
int vb_embedding_backward(const vb_tensor* ids, const vb_tensor* weight, const vb_tensor* grad_out, vb_tensor* gw); /* lib.rs:1412-1464 */
/* loss is a shape-[1] tensor: mean over rows.  `row_stats` (may be NULL) receives a [B,2] tensor of
 * per-row (max, sum exp) that vb_cross_entropy_backward can reuse to skip its own first pass. */
int vb_cross_entropy(const vb_tensor* logits, const vb_tensor* targets, vb_tensor* loss, vb_tensor* row_stats); /* lib.rs:1466-1534 */
/* Forward and backward of the loss in one pass (no counterpart in the reference): returns the loss of vb_cross_entropy and
 * overwrites the (contiguous) logits with what vb_cross_entropy_backward returns for an upstream gradient of 1.  For callers that
 * are about to differentiate the loss and need the logits for nothing else; it moves 2 * B * V * 4 bytes instead of 3. */
int vb_cross_entropy_fused(const vb_tensor* logits_inout, const vb_tensor* targets, vb_tensor* loss);
int vb_cross_entropy_backward(const vb_tensor* logits, const vb_tensor* targets, const vb_tensor* grad_out,
                              const vb_tensor* row_stats_or_null, vb_tensor* glogits);                   /* lib.rs:1536-1592 */
int vb_conv2d(const vb_tensor* x, const vb_tensor* w, const vb_tensor* bias, int stride, int padding, vb_tensor* out); /* lib.rs:245-301 */
int vb_conv2d_backward(const vb_tensor* x, const vb_tensor* w, const vb_tensor* grad_out, int stride, int padding,
                       vb_tensor* gx, vb_tensor* gw, vb_tensor* gb);                                     /* lib.rs:334-438 */
int vb_maxpool2d(const vb_tensor* x, int kernel, int stride, int padding, vb_tensor* out);               /* lib.rs:466-505 */
int vb_maxpool2d_backward(const vb_tensor* x, const vb_tensor* grad_out, int kernel, int stride, int padding, vb_tensor* gx); /* lib.rs:507-553 */
int vb_avgpool2d(const vb_tensor* x, int kernel, int stride, int padding, vb_tensor* out);               /* lib.rs:556-595 */
int vb_avgpool2d_backward(const vb_tensor* x, const vb_tensor* grad_out, int kernel, int stride, int padding, vb_tensor* gx); /* lib.rs:597-637 */
/* Training mode updates running_mean / running_var in place (Bessel factor in the running value
 * only), as vearo-backend-cpu lib.rs:2141-2148. */
int vb_batchnorm(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* running_mean,
                 const vb_tensor* running_var, int training, float momentum, float eps, vb_tensor* out); /* lib.rs:640-720 */
int vb_batchnorm_backward(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* running_mean,
                          const vb_tensor* running_var, const vb_tensor* grad_out, int training, float eps,
                          vb_tensor* gx, vb_tensor* ggamma, vb_tensor* gbeta);                           /* lib.rs:722-830 */
/* Fused BatchNorm2d -> ReLU -> MaxPool(2, 2, 0): the composition of vb_batchnorm, vb_relu and vb_maxpool2d(2, 2, 0) and of
 * their backward functions, without the two intermediate tensors.  No single reference function corresponds to it (the
 * reference runs the three ops of vearo-nn's conv blocks one after another; autograd arms lib.rs:537-541, 562-587,
 * 619-627): an extra export for callers that know the pattern.  `stats` ([2, C]: the mean and 1/sqrt(var + eps) the forward
 * normalised with) is produced by the forward and consumed by the backward. */
int vb_bn_relu_maxpool(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* running_mean,
                       const vb_tensor* running_var, int training, float momentum, float eps, vb_tensor* out, vb_tensor* stats);
int vb_bn_relu_maxpool_backward(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* stats,
                                const vb_tensor* grad_out, int training, vb_tensor* gx, vb_tensor* ggamma, vb_tensor* gbeta);
/* q,k,v: [B,H,S,dk] (strided views accepted); mask: NULL or an additive tensor right-aligned to
 * [B,H,S,S] with size-1 dims broadcast; softmax uses 1/(sum + 1e-9) as vearo-backend-cpu
 * lib.rs:2455.  The reference's CUDA backend runs this on the CPU (lib.rs:1594-1636); here it
 * runs on the device.  `probs` (may be NULL) receives the [B,H,S,S] probabilities so that the
 * backward pass need not recompute them.  The results of both calls (out; dq, dk, dv) are the one exception
 * to "outputs are contiguous": they are [B,H,S,dk] views (strides S*H*dk, dk, H*dk, 1) of fresh [B,S,H,dk]
 * buffers, which makes the layer's following transpose(1,2).reshape a view instead of a copy.
 * When the mask is a [S,S] causal mask (0 on/below the diagonal, <= -1e9 above; S a multiple of 128, <= 1024) the
 * triangular structure is exploited; `probs` is then only defined up to the end of each row's 128-wide diagonal tile
 * and must be handed to the backward call together with the same mask.
 * With no mask or the causal mask, head size 64, S >= 128 and 16-byte-aligned operands, the forward is ONE kernel
 * (scores, softmax and the product with V on the SM: the S x S matrix reaches memory only when `probs` is asked
 * for) and the backward fuses dP, the softmax backward and dQ.  The slot `probs` then names is larger than its
 * [B,H,S,S] descriptor says: a [B,H,S,dk] copy of the output follows the probabilities, which the backward kernel
 * reads; treat the tensor as an opaque token between the two calls.  VB200_ATTN_FUSED=0 switches this route off. */
int vb_fused_attention(const vb_tensor* q, const vb_tensor* k, const vb_tensor* v, const vb_tensor* mask_or_null,
                       vb_tensor* out, vb_tensor* probs);
int vb_fused_attention_backward(const vb_tensor* q, const vb_tensor* k, const vb_tensor* v, const vb_tensor* mask_or_null,
                                const vb_tensor* grad_out, const vb_tensor* probs_or_null,
                                vb_tensor* dq, vb_tensor* dk, vb_tensor* dv);
/* The same attention over a packed projection: qkv is a contiguous [B, S, 3*D] tensor whose three column blocks are q, k and
 * v (heads side by side), as one Linear over the stacked q/k/v weights of vearo-nn's MultiHeadAttention (lib.rs:584-621)
 * produces; `out` is the [B, S, D] context and the backward returns a single [B, S, 3*D] gradient.  No reference function
 * corresponds to it: an extra export that saves the three head-split copies and the gradient concatenation. */
int vb_fused_attention_packed(const vb_tensor* qkv, int n_head, const vb_tensor* mask_or_null, vb_tensor* out, vb_tensor* probs_or_null);
int vb_fused_attention_packed_backward(const vb_tensor* qkv, int n_head, const vb_tensor* mask_or_null, const vb_tensor* grad_out,
                                       const vb_tensor* probs_or_null, vb_tensor* dqkv);

/* ---- backward arms the reference computes on the host for CUDA tensors -------------------
 * (vearo-autograd/src/lib.rs: reduce_to 316-361, relu/gelu masks 364-403, softmax arm 547-553,
 * accumulation 733-742).  A drop-in backend adds these as new BackendOps fields. */
int vb_relu_backward(const vb_tensor* x, const vb_tensor* grad_out, vb_tensor* gx);
int vb_gelu_backward(const vb_tensor* x, const vb_tensor* grad_out, vb_tensor* gx);
int vb_softmax_backward(const vb_tensor* x, const vb_tensor* grad_out, int dim, vb_tensor* gx);  /* x = the softmax INPUT */
int vb_reduce_to(const vb_tensor* grad, const int64_t* target_dims, int target_rank, vb_tensor* out);
int vb_accumulate(const vb_tensor* dst, const vb_tensor* src);        /* dst += src in place (dst contiguous) */
int vb_copy(const vb_tensor* dst, const vb_tensor* src);              /* dst = src (dst contiguous view), device side */
int vb_scale(const vb_tensor* x, float alpha, vb_tensor* out);        /* out = x * alpha */
int vb_contiguous(const vb_tensor* x, vb_tensor* out);                /* device-side strided copy; replaces the host
                                                                         round trip of vearo-core tensor.rs:349-368 */
int vb_fill(const vb_tensor* dst, float value);

/* ---- allocation-free LayerNorm backward (no counterpart in the reference) ------------------
 * For callers that cannot allocate device memory where they need this kernel: code running inside a
 * region where the allocator must not be touched, a loop with a fixed memory budget, a plugin that owns
 * nothing but the buffers it was handed.  vb_layernorm_backward takes scratch for the per-CTA partial
 * sums of dgamma / dbeta from the library's arena (and its outputs too); this variant allocates nothing:
 * inputs and outputs are the caller's raw device pointers (contiguous f32, x / grad_out / gx of
 * rows * c elements, w / gw / gb of c elements) and the partial sums go to a fixed 2.4 MB array inside
 * the library image, present on every GPU that loads the library until the process exits.
 *   - Limits: c a multiple of 4 and <= 1024; x, w, grad_out, gx 16-byte aligned.  Anything else is
 *     rejected with VB_ERR_UNSUPPORTED and a message; use vb_layernorm_backward there.
 *   - The first call on each device looks up the array's device address and raises the shared-memory
 *     limit of the two widest kernel instances; make that call before starting any stream capture.
 *     Later calls do no set-up: they only launch kernels.
 *   - All calls share the one array: two calls whose kernels may overlap on the GPU (different
 *     streams) race on it.  Calls on one stream are safe back to back; nothing needs clearing between
 *     them, since every partial row is rewritten in full.
 *   - `stream` is a cudaStream_t (NULL = the default stream).  vb_init is not required. */
int vb_layernorm_backward_noalloc(const float* x, const float* w, const float* grad_out, float* gx, float* gw, float* gb,
                                  int64_t rows, int64_t c, float eps, void* stream);

/* ---- fused linear-layer entry points (extras the binding may ignore) ---------------------
 * y = x . W^T + bias in one GEMM (Linear::forward, vearo-nn/src/lib.rs:120-128), and its
 * backward: gx = gy . W, gw = gy^T . x summed over all leading dims, gb = column sum of gy —
 * the Add / Matmul / Transpose arms plus reduce_to of vearo-autograd/src/lib.rs:460-528.
 * Any output pointer may be NULL to skip it. */
int vb_linear(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* bias_or_null, vb_tensor* out);
int vb_linear_backward(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* grad_out,
                       vb_tensor* gx, vb_tensor* gw, vb_tensor* gb);
/* The same with the weight and bias gradients written into existing tensors (NULL: not wanted) -- a parameter's slice of a flat
 * gradient buffer -- so that no copy follows the GEMM.  No reference counterpart (the reference allocates every gradient). */
int vb_linear_backward_into(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* grad_out, vb_tensor* gx_or_null,
                            const vb_tensor* gw_into_or_null, const vb_tensor* gb_into_or_null);
/* vb_linear followed by GELU (TransformerBlock::forward's fc1 -> gelu, crates/vearo-nn/src/lib.rs:666-675) with both results
 * returned: `pre` = x.W^T + b, which the GELU backward arm needs, and `act` = gelu(pre).  Where the tensor-core kernel takes the
 * product as whole tiles the activation is formed in its epilogue from the values being stored; the results equal
 * vb_linear + vb_gelu bit for bit either way. */
int vb_linear_gelu(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* bias_or_null, vb_tensor* pre, vb_tensor* act);
/* vb_layernorm_backward with the input gradient added to an existing gradient of x in place (grad_in += dx; grad_in contiguous,
 * of x's shape): the accumulation the reference's gradient map does when x has a second consumer, e.g. a residual connection
 * (vearo-autograd/src/lib.rs:733-741), without writing dx out and reading it back. */
int vb_layernorm_backward_accum(const vb_tensor* x, const vb_tensor* w, const vb_tensor* b, const vb_tensor* grad_out, float eps,
                                const vb_tensor* grad_in, vb_tensor* gw, vb_tensor* gb);
/* Bias gradients.  vb_gelu_backward / vb_relu_backward, vb_layernorm_backward and vb_layernorm_backward_accum leave the column
 * sums of the (large, rank >= 2) gradient they write beside it; vb_linear_backward[_into], given that same tensor unchanged as
 * grad_out, copies them as gb instead of summing the columns again.  The sums are dropped as soon as the tensor is written to
 * through this library or released.  VB200_COLSUM_REUSE=0 in the environment switches this off. */

/* ---- optimizer ---------------------------------------------------------------------------
 * Single-tensor steps replace the CUDA branches of Tensor::adamw_step / sgd_step
 * (vearo-core/src/tensor.rs:989-1019, 1073-1092): m, v, velocity live in device slots instead
 * of host Vec<f32> (vearo-optim/src/lib.rs:68-69). */
int vb_adamw_step(const vb_tensor* param, const vb_tensor* grad, vb_slot m, vb_slot v, uint32_t t,
                  float lr, float beta1, float beta2, float eps, float weight_decay);
int vb_sgd_step(const vb_tensor* param, const vb_tensor* grad, vb_slot velocity, float lr, float momentum, float weight_decay);
/* clip_grad_norm (vearo-optim/src/lib.rs:360-383): returns the pre-clip global L2 norm and
 * scales the gradients in place by max_norm/(norm+1e-6) when norm > max_norm. */
int vb_clip_grad_norm(const vb_tensor* grads, int n, float max_norm, float* total_norm);

/* Fused multi-tensor optimizer: one launch updates every parameter; global-norm clipping is
 * folded in (the scale is applied inside the update, the gradients are never rewritten). */
/* VB_OPT_ADAMW8BIT is AdamW8bit (vearo-optim/src/lib.rs:211-303): the moments are held as int8 with one f32 scale per
 * 256 elements of a parameter, dequantized before and requantized after every update (QuantizedState, lib.rs:137-209). */
enum vb_opt_kind { VB_OPT_ADAMW = 0, VB_OPT_SGD = 1, VB_OPT_ADAMW8BIT = 2 };
typedef struct vb_opt_config {
  int32_t kind;
  float lr, beta1, beta2, eps, weight_decay, momentum;
} vb_opt_config;
/* params[i] and grads[i] are contiguous tensors of equal numel; grads are read at each step from
 * the same locations (persistent gradient buffers). */
int vb_opt_create(const vb_opt_config* cfg, const vb_tensor* params, const vb_tensor* grads, int n, int* opt);
int vb_opt_destroy(int opt);
int vb_opt_set_lr(int opt, float lr);
/* Optimizer state for checkpoints: the slot that holds m then v (AdamW) or the velocity (SGD), one flat array in parameter
 * order with every parameter's share rounded up to 4 floats; and the step counter t of AdamW's bias correction
 * (vearo-optim/src/lib.rs:68-70, 105-123 keep them in host Vecs). */
int vb_opt_state(int opt, vb_slot* state, int64_t* state_numel, uint32_t* step);
int vb_opt_set_step(int opt, uint32_t step);
/* Quantized state of parameter `param` of a VB_OPT_ADAMW8BIT optimizer, copied to host memory: numel int8 values and
 * (numel + 255) / 256 scales, for m and for v (the fields of QuantizedState, lib.rs:138-142).  Synchronises.
 * (The slot vb_opt_state returns holds, for this kind, the same bytes: all m values, all v values, then all m scales and all
 * v scales, every parameter's share starting on a 256-element boundary; checkpoints store it as it is.) */
int vb_opt_state8(int opt, int param, int8_t* m8, float* m_scales, int8_t* v8, float* v_scales);
/* active[i] == 0 skips parameter i (no gradient this step; vearo-optim/src/lib.rs:106-108); NULL = all.
 * max_norm <= 0 disables clipping.  grad_scale multiplies every gradient first (1/world for data
 * parallel sums).  *total_norm (may be NULL) receives the pre-clip norm; reading it synchronises. */
int vb_opt_step(int opt, const uint8_t* active, float max_norm, float grad_scale, float* total_norm);

/* ---- kernel profiling (no counterpart in the reference) ------------------------------------
 * When enabled, every launch of a kernel family is bracketed by CUDA events on the compute stream.
 * vb_profile_read synchronises and returns, for `family` ("gemm_tc", "gemm_simt", "layernorm_bwd",
 * "gelu_bwd", "cross_entropy_bwd", "adamw", "attn_softmax", ...): total milliseconds, number of
 * launches, and the summed algorithmic units (bytes for HBM-bound families, flops for GEMMs) -- `units`
 * counts what the launches really moved or issued (a causal attention product skips the tiles above
 * the diagonal), `dense_units` (may be NULL) the same for the dense problem.
 * vb_profile_families writes a comma-separated list of the families seen so far. */
/* Number of kernel-launcher invocations so far (each enqueues at least one kernel of this library). */
int vb_launch_count(int64_t* count);
/* Self-test of the bounded device-side waits: runs one CTA that waits, with a limit of `polls` (1..65536) polls, on a barrier
 * nothing arrives on.  The wait runs out, the kernel raises the wait-timeout bit and returns; the NEXT vb_check_errors reports
 * "a device-side wait ran out" (VB_ERR_BAD_INDEX) and the context stays usable.  elapsed_ms (may be NULL): device time of the kernel. */
int vb_selftest_wait_timeout(uint32_t polls, double* elapsed_ms);
/* Number of launches of the tcgen05 tensor-core GEMM kernel so far. */
int vb_tc_launch_count(int64_t* count);
int vb_profile_enable(int on);
int vb_profile_reset(void);
int vb_profile_read(const char* family, double* total_ms, int64_t* launches, double* units, double* dense_units);
int vb_profile_families(char* buf, int buflen);

/* ---- data parallel -----------------------------------------------------------------------
 * New functionality (the reference is single-device).  One process per GPU; NCCL is loaded at
 * run time.  unique_id is the 128-byte ncclUniqueId produced by vb_dp_unique_id on rank 0 and
 * distributed by the caller. */
int vb_dp_unique_id(uint8_t id[128]);
int vb_dp_init(int rank, int world, const uint8_t id[128]);
int vb_dp_world(int* rank, int* world);
/* A slot for data that will be all-reduced in place (a gradient arena).  With more than one rank the memory comes from NCCL's
 * allocator and is registered with the communicator (the NVLink-switch all-reduce then works on the buffer itself); otherwise,
 * or when the library refuses, an ordinary slot.  Same ownership rules as vb_alloc.  VB200_DP_REGISTER=0 forces ordinary slots.
 * vb_dp_is_registered tells which kind a slot is. */
int vb_dp_alloc(int64_t numel, int zero_fill, vb_slot* out);
int vb_dp_is_registered(vb_slot slot, int* yes);
/* Sum-allreduce `numel` floats at slot+offset on the communication stream, ordered after all
 * work enqueued so far on the compute stream.  Returns immediately. */
int vb_dp_allreduce(vb_slot slot, int64_t offset, int64_t numel);
/* Make the compute stream wait for all allreduces issued so far.
 *   timeout_ms > 0: the host also waits for them, polling for asynchronous NCCL errors, until the deadline (milliseconds):
 *                   VB_ERR_COMM_TIMEOUT / VB_ERR_COMM after aborting the communicator.
 *   timeout_ms = 0: no host-side check.
 *   timeout_ms < 0: deferred check with deadline -timeout_ms: returns at once, so the host can keep enqueuing work; the
 *                   deadline wait for THESE collectives happens at the next vb_dp_finish, vb_dp_wait, vb_sync or vb_read,
 *                   whichever comes first (they have normally completed long before and nothing waits). */
int vb_dp_finish(int timeout_ms);
int vb_dp_wait(void);
int vb_dp_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* VEARO_B200_H */
