// Internal declarations shared by the runtime, the kernels and the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>
#include "../../include/vearo_b200.h"

namespace vb {

using i64 = int64_t;

// Bits of the device error word (reported as VB_ERR_BAD_INDEX by vb_check_errors).
enum : int { ERRBIT_NEG_ID = 1, ERRBIT_OOB_ID = 2, ERRBIT_WAIT_TIMEOUT = 4, ERRBIT_BOUNDS = 8 };

struct Ctx {
  bool ready = false;
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;       // compute stream: every kernel of the library
  cudaStream_t comm_stream = nullptr;  // collectives
  cudaEvent_t ev_compute = nullptr, ev_comm = nullptr;
  int* d_err = nullptr;                // device error word
  float* d_scalars = nullptr;          // small device scratch for scalars (norms, loss partials)
  float* h_pinned = nullptr;           // pinned host mirror for small reads
};
Ctx& ctx();

// Thread-local error text + status helpers.
int set_error(int status, const std::string& msg);
#define VB_CHECK(cond, msg) do { if (!(cond)) return ::vb::set_error(VB_ERR_INVALID, std::string(__func__) + ": " + (msg)); } while (0)
#define VB_CUDA(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) return ::vb::set_error(VB_ERR_CUDA, std::string(__func__) + ": " #expr ": " + cudaGetErrorString(e_)); } while (0)
#define VB_TRY(expr) do { int s_ = (expr); if (s_ != VB_OK) return s_; } while (0)
extern int64_t g_launcher_calls;   // launcher invocations since start (each enqueues one or more kernels)
extern int64_t g_tc_launches;      // launches of the tensor-core GEMM kernel since start (gemm_tc.cu)
#define VB_LAUNCH_CHECK() do { ++::vb::g_launcher_calls; VB_CUDA(cudaGetLastError()); } while (0)

// Slots / arena (runtime.cu).
int slot_alloc(i64 numel, bool zero, vb_slot* out);
int slot_adopt_external(float* p, i64 numel, void (*free_fn)(void*), vb_slot* out);   // a slot over memory that is not the arena's
int slot_ptr(vb_slot s, float** p, i64* numel = nullptr);
int slot_release(vb_slot s, int* freed);
int slot_retain(vb_slot s);
uint64_t slot_serial(vb_slot s);          // changes every time the slot id is handed out again or its contents are overwritten through the ABI
void slot_touch(vb_slot s);               // note that the contents of a slot were overwritten
// Raw cached device scratch, stream-ordered reuse; never shows up in the slot table.
int scratch_alloc(size_t bytes, void** p);
void scratch_free(void* p);

// Tensor-descriptor helpers.
inline i64 numel(const vb_tensor& t) { i64 n = 1; for (int i = 0; i < t.rank; ++i) n *= t.dims[i]; return n; }
inline bool is_contiguous(const vb_tensor& t) {
  i64 s = 1;
  for (int i = t.rank - 1; i >= 0; --i) { if (t.dims[i] != 1 && t.strides[i] != s) return false; s *= t.dims[i]; }
  return true;
}
inline void set_contiguous(vb_tensor& t, int rank, const i64* dims) {
  t.rank = rank; t.offset = 0;
  i64 s = 1;
  for (int i = 0; i < VB_MAX_RANK; ++i) { t.dims[i] = 0; t.strides[i] = 0; }
  for (int i = rank - 1; i >= 0; --i) { t.dims[i] = dims[i]; t.strides[i] = s; s *= dims[i]; }
}
inline bool same_shape(const vb_tensor& a, const vb_tensor& b) {
  if (a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i) if (a.dims[i] != b.dims[i]) return false;
  return true;
}
int tensor_ptr(const vb_tensor* t, float** p);           // slot base + offset, validated
int new_output(vb_tensor* out, int rank, const i64* dims, bool zero = false);  // fresh contiguous slot
// A contiguous device pointer for `t`: the tensor itself when already contiguous, else a strided
// copy into scratch (owned by `Temp`, returned to the arena when it goes out of scope).
struct Temp {
  void* p = nullptr;
  ~Temp() { if (p) scratch_free(p); }
};
int contiguous_ptr(const vb_tensor* t, const float** p, Temp& hold);

// Strided index descriptor passed by value to generic kernels.
struct Strided {
  int rank;
  i64 dims[VB_MAX_RANK];
  i64 sa[VB_MAX_RANK];
  i64 sb[VB_MAX_RANK];
};

// ---- kernel launchers (one family per .cu file); all enqueue on ctx().stream -------------
// elementwise.cu
int launch_binary(int op, const float* a, const float* b, float* out, i64 n);                       // same shape, contiguous
int launch_binary_rowvec(int op, const float* a, const float* b, float* out, i64 n, i64 c, bool b_is_vec); // b (or a) is a length-c vector over the last dim
int launch_binary_scalar(int op, const float* a, const float* b, float* out, i64 n, bool b_is_scalar);
int launch_binary_strided(int op, const float* a, const float* b, float* out, i64 n, const Strided& s);
int launch_unary(int op, const float* x, float* out, i64 n);          // 0 relu 1 gelu
int launch_unary_backward(int op, const float* x, const float* g, float* out, i64 n);  // 0 relu 1 gelu
// the same over [rows, cols] (cols a multiple of 4, 16-byte aligned pointers), also leaving colsum[c] = sum_r out[r, c]
int launch_unary_backward_colsum(int op, const float* x, const float* g, float* out, i64 rows, i64 cols, float* colsum);
int launch_scale(const float* x, float alpha, float* out, i64 n);
int launch_axpy(float* dst, const float* src, i64 n);                 // dst += src
int launch_fill(float* dst, float v, i64 n);
int launch_strided_copy(const float* src, float* dst, i64 n, const Strided& s);   // dst contiguous; s.sa = src strides
// reduce.cu
int launch_sum_axis(const float* x, float* out, i64 outer, i64 d, i64 inner, bool mean);
int launch_colsum(const float* x, float* out, i64 rows, i64 cols, bool accumulate);   // out[c] (+)= sum_r x[r,c]
int launch_colsum_final(const float* part, float* out, i64 cols, int splits);          // out[c] = sum_i part[i, c], in a fixed order
int launch_reduce_general(const float* g, float* out, i64 out_numel, const Strided& kept, const Strided& red, i64 red_count);
int launch_softmax_rows(const float* x, float* out, i64 rows, i64 d);
int launch_softmax_strided(const float* x, float* out, i64 outer, i64 d, i64 inner);
int launch_softmax_backward_rows(const float* x, const float* g, float* out, i64 rows, i64 d);
int launch_softmax_backward_strided(const float* x, const float* g, float* out, i64 outer, i64 d, i64 inner);
// norm.cu
int launch_layernorm(const float* x, const float* w, const float* b, float* out, i64 rows, i64 c, float eps, float* out_lo = nullptr, bool* lo_done = nullptr);
// resid (optional): gx = resid + dx (gx may be resid itself).  out_colsum (optional, c floats): the column sums of what was stored in gx,
// written only where the fast kernel ran (*colsum_done says so).
int launch_layernorm_backward(const float* x, const float* w, const float* g, float* gx, float* gw, float* gb, i64 rows, i64 c, float eps,
                              const float* resid = nullptr, float* out_colsum = nullptr, bool* colsum_done = nullptr);
int launch_batchnorm(const float* x, const float* gamma, const float* beta, float* rm, float* rv, float* out,
                     i64 n, i64 c, i64 hw, bool training, float momentum, float eps);
int launch_batchnorm_backward(const float* x, const float* gamma, const float* rm, const float* rv, const float* g,
                              float* gx, float* gw, float* gb, i64 n, i64 c, i64 hw, bool training, float eps);
// loss.cu
int launch_bn_relu_maxpool(const float* x, const float* gamma, const float* beta, float* rm, float* rv, float* stats, float* out,
                           i64 n, i64 c, i64 h, i64 w, bool training, float momentum, float eps);                       // bn_fused.cu
int launch_bn_relu_maxpool_backward(const float* x, const float* gamma, const float* beta, const float* stats, const float* g,
                                    float* gx, float* gw, float* gb, i64 n, i64 c, i64 h, i64 w, bool training);
int launch_embedding(const float* ids, const float* w, float* out, i64 n, i64 vocab, i64 d);
int launch_embedding_backward(const float* ids, const float* g, float* gw, i64 n, i64 vocab, i64 d);   // gw pre-zeroed
int launch_cross_entropy(const float* logits, const float* targets, float* loss, float* stats, i64 rows, i64 v);
int launch_cross_entropy_fused(float* logits, const float* targets, float* loss, i64 rows, i64 v);
int launch_cross_entropy_backward(const float* logits, const float* targets, const float* gout, const float* stats,
                                  float* gl, i64 rows, i64 v);
// conv.cu
int launch_conv2d(const float* x, const float* w, const float* b, float* out, i64 n, i64 cin, i64 h, i64 wd,
                  i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad);
int launch_conv2d_backward(const float* x, const float* w, const float* g, float* gx, float* gw, float* gb,
                           i64 n, i64 cin, i64 h, i64 wd, i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad);
int launch_maxpool2d(const float* x, float* out, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p);
int launch_maxpool2d_backward(const float* x, const float* g, float* gx, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p);
int launch_avgpool2d(const float* x, float* out, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p);
int launch_avgpool2d_backward(const float* g, float* gx, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p);

// gemm.cu: C[b] = alpha * A[b] . B[b] (+ beta * C[b]) (+ bias[n]); A logical [M,K], B logical [K,N],
// every operand addressed through element strides, two batch levels (b = b1 * nb2 + b2).
// A zero-padded NHWC image batch xp [n, h + 2, w + 2, c] standing in for its unfolded ("im2col") matrix as the B operand of a
// product (3 x 3 window, stride 1, padding 1): cols[(n, y, x), (i, j, ch)] = xp[n, y + i, x + j, ch].
//   mode 1: B = cols[image]^T, i.e. the product is batched over the n images (nb2 = n), N = h * w pixels, K = 9 * c
//   mode 2: B = cols, N = 9 * c taps, K = n * h * w pixels
struct ConvOperand { const float* xp; i64 n, h, w, c; int mode; };
struct GemmArgs {
  const float* A; const float* B; float* C; const float* bias;   // bias: length N or null
  const float* bias_m;                                            // per-row bias: length M or null (output channels of a convolution)
  i64 M, N, K;
  i64 a_rs, a_cs;   // A[m,k] = A[m*a_rs + k*a_cs]
  i64 b_rs, b_cs;   // B[k,n] = B[k*b_rs + n*b_cs]
  i64 c_rs, c_cs;
  i64 nb1, nb2;     // batch counts (>= 1)
  i64 a_b1, a_b2, b_b1, b_b2, c_b1, c_b2;   // batch strides (0 = broadcast)
  float alpha, beta;
  // Triangular structure of attention with a causal mask (square S x S problems, exact zeros above the diagonal):
  //   1  C tiles strictly above the diagonal are neither computed nor written (scores, dP)
  //   2  A[m, k] == 0 for k > m: the k range of a tile stops at its last row (P.V, dS.K)
  //   3  A[m, k] == 0 for k < m (A is a transposed view of such a matrix): the k range starts at the tile's first row (P^T.dO, dS^T.Q)
  // Kernels that do not exploit it compute the full product, which gives the same values.
  int causal;
  // Optional: the TF32 remainders of B (lo = tf32(b - cut_to_tf32(b)), what the tensor-core kernel otherwise computes for every
  // k-block of every tile), laid out exactly like B.  Worth it for an operand used by many tiles and several products (weights).
  const float* B_lo;
  const float* A_lo;      // the same for A (an activation whose producer wrote its remainders)
  // Optional second output: GELU(C) in C's layout, written by the tensor-core kernel's epilogue when it can (*act_fused = 1);
  // otherwise left untouched, and the caller applies the activation itself.
  float* act_out;
  int* act_fused;
  // Optional: B given as an implicit im2col view (then B and its strides are ignored).  Only the tensor-core kernel can read it:
  // *conv_used is set to 1 when it did; otherwise nothing was launched and the caller falls back to an unfolded matrix.
  const ConvOperand* conv;
  int* conv_used;
};
int launch_gemm(const GemmArgs& g);
int launch_tf32_lo(const float* x, float* lo, i64 n);      // gemm_tc.cu: lo[i] as above
int gemm_tc_reset_state();   // gemm_tc.cu: clears kernel-side bookkeeping after a reported device error
inline GemmArgs gemm_args() { GemmArgs g{}; g.nb1 = g.nb2 = 1; g.alpha = 1.0f; g.beta = 0.0f; return g; }

// attention.cu
int launch_attn_softmax(float* s, const float* mask, const i64 mask_strides[4], bool causal, i64 b, i64 h, i64 sq, i64 sk, float scale);
int launch_mask_is_causal(const float* mask, i64 s, i64 row_stride, int* d_flag);   // d_flag <- 0 when some entry breaks the causal pattern
int launch_attn_softmax_backward(const float* p, float* dp_inout, i64 rows, i64 sk, float scale, bool causal, i64 sq);

// attn_fused.cu: attention with the score matrix kept on the SM (head size 64, no mask or the causal mask, S >= 128).
// An operand is a [B,H,S,64] view given by its element strides.
struct AttnOperand { const float* p; i64 sb, sh, ss, sd; };
bool attn_fused_supported(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, i64 B, i64 H, i64 S, i64 dk);
bool attn_fused_operand_ok(const AttnOperand& o, i64 B, i64 H);
// out: rows of 64 floats per head at out + b*o_sb + s*o_ss + h*64; probs: null, or room for B*H*S*(S + 64) floats: the [B,H,S,S]
// probabilities (written up to the end of each row's 128-wide diagonal tile under the causal mask) followed by a [B,H,S,64] copy
// of the output, which is what launch_attn_bwd_dq_fused wants as `saved`
int launch_attn_bwd_dq_fused(const AttnOperand& k, const AttnOperand& v, const AttnOperand& gout, const float* saved, float* ds,
                             float* dq, i64 dq_ss, i64 dq_sb, i64 B, i64 H, i64 S, bool causal, float scale);
int launch_attn_fwd_fused(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, float* out, i64 o_ss, i64 o_sb, float* probs,
                          i64 B, i64 H, i64 S, bool causal, float scale);

// optim.cu
// (8-bit AdamW: m and v point at int8 values, ms and vs at the scales of the chunk's 256-element blocks)
// (lo: where the TF32 remainders of the updated weights go when the weight keeps a lo plane for the tensor-core GEMM, else null)
struct OptChunk { float* w; const float* g; float* m; float* v; int n; int param; float* ms; float* vs; float* lo; };
// abi.cu: the lo plane kept for a weight slot (null if none) and the slot's base address; and the note that the plane was just
// brought up to date with the slot's present contents by the caller
float* lo_plane_base_for(vb_slot weight_slot, float** weight_base);
void lo_plane_mark_current(vb_slot weight_slot);
bool lo_plane_is_current(vb_slot weight_slot);
int dp_wait_pending();                      // data parallel: the host-side deadline check a deferred vb_dp_finish left open (no-op otherwise)
void lo_planes_forget_all();                 // the slot table is being torn down
void lo_plane_on_release(vb_slot slot);      // the slot is gone: so is a lo plane kept for it
// ---- bounds-check build (-DVB200_BOUNDS_CHECK; `python vearo_b200/build.py --bounds-check`) ------------------------------------
// The stand-in for a memory checker on pools where none may run: kernels that compute gather / scatter indices wrap the index in
// VB_BC(index, extent).  In the checked build an index outside [0, extent) sets ERRBIT_BOUNDS in the device error word (reported by
// vb_check_errors as VB_ERR_BAD_INDEX, "a computed index left its tensor") and the access is skipped -- never a trap, never a
// fault; in the normal build the macro is the constant `true` and costs nothing.  Each translation unit keeps its own pointer to
// the error word (no relocatable device code is used); vb_init hands it to every unit through the registrars below.
#ifdef VB200_BOUNDS_CHECK
void bc_register(void (*setter)(int*));          // runtime.cu: remembers a unit's setter; vb_init calls them all
std::vector<void (*)(int*)>& bc_setters();
#ifdef __CUDACC__
static __device__ int* bc_err_word;
static void bc_set_err_word(int* p) { cudaMemcpyToSymbol(bc_err_word, &p, sizeof p); }
namespace { struct BcRegistrar { BcRegistrar() { bc_register(bc_set_err_word); } } bc_registrar_instance; }
__device__ __forceinline__ bool bc_check(long long idx, long long extent) {
  if (idx >= 0 && idx < extent) return true;
  if (bc_err_word) atomicOr(bc_err_word, ERRBIT_BOUNDS);
  return false;
}
#define VB_BC(idx, extent) (::vb::bc_check((long long)(idx), (long long)(extent)))
#endif
#else
#define VB_BC(idx, extent) (true)
#endif

#ifdef __CUDACC__
// tanh(y) = 1 - 2 / (1 + e^(2y)) with the exponential on the special-function unit (2^x, relative error about 2^-22) and an
// approximate division: absolute error of a few 1e-7 over the whole range (exact limits +-1 for large |y|), i.e. the same few
// units in the last place as libm's tanhf for the uses below, at a quarter of its instructions.
__device__ __forceinline__ float tanh_fast(float y) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y * 2.8853900817779268f));      // e^(2y) = 2^(2y log2 e)
  return 1.0f - __fdividef(2.0f, 1.0f + e);
}
// e^x for x <= 0 (softmax numerators) on the special-function unit: 2^(x log2 e).  The product is rounded once (6e-8 relative of
// the argument, i.e. an absolute 1.2e-6 in the exponent at x = -20) and 2^y is good to 2^-22: results within about 1.5e-6
// relative of expf over the range that matters, two orders inside the parity bar; -inf gives 0, underflow flushes to 0.
__device__ __forceinline__ float exp_neg_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}
// GELU, tanh form, with the reference's constants (crates/vearo-backend-cpu/src/lib.rs:458-497)
__device__ __forceinline__ float gelu_value(float v) {
  const float v3 = v * v * v;
  const float inner = 0.79788456f * (v + 0.044715f * v3);
  return 0.5f * v * (1.0f + tanh_fast(inner));
}
// Packed pairs of f32: one instruction drives two lanes of the FP32 pipe (PTX add/mul/fma .f32x2, sm_100).  Each lane rounds as
// the scalar instruction does.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 lo2(const float4& a) { return make_float2(a.x, a.y); }
__device__ __forceinline__ float2 hi2(const float4& a) { return make_float2(a.z, a.w); }
__device__ __forceinline__ float4 cat2(float2 a, float2 b) { return make_float4(a.x, a.y, b.x, b.y); }

// lo part of x when the tensor core takes the raw x as hi (it reads x cut to 10 mantissa bits): the remainder is exact in f32 and
// is rounded to TF32 (nearest, ties away) with integer arithmetic on the bit pattern
__device__ __forceinline__ float tf32_remainder(float x) {
  float d = x - __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  return __uint_as_float((__float_as_uint(d) + 0x1000u) & 0xffffe000u);
}
#endif
int launch_adamw_single(float* w, const float* g, float* m, float* v, i64 n, float lr, float b1, float b2, float eps, float wd,
                        float bc1, float bc2);
int launch_sgd_single(float* w, const float* g, float* vel, i64 n, float lr, float mu, float wd);
int launch_sumsq_chunks(const OptChunk* chunks, int nchunks, const uint8_t* active, float* partials);
int launch_sum_partials(const float* partials, int n, float* out);      // out[0] = sum (single block, fixed order)
int launch_opt_multi(const OptChunk* chunks, int nchunks, const uint8_t* active, int kind, const float* normsq,
                     float max_norm, float grad_scale, float lr, float b1, float b2, float eps, float wd, float mu,
                     float bc1, float bc2, int lo_chunks = 0);     // lo_chunks: how many chunks carry a lo-plane pointer (profiling only)
int launch_scale_inplace_by_clip(float* g, i64 n, const float* normsq, float max_norm);


// prof.cu: optional per-family kernel timing with CUDA events on the compute stream.  Off by
// default (zero cost); the benchmark switches it on for a separate, untimed pass.
struct ProfScope {
  int idx = -1;
  // units: algorithmic bytes or flops this launch really moves / issues; dense_units: the same for the dense problem when the
  // launch skips part of it (causal attention), else 0 (= units)
  ProfScope(const char* family, double units, double dense_units = 0.0);
  ~ProfScope();
};

}  // namespace vb
