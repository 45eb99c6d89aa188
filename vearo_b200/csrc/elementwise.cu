// Elementwise kernels: broadcast binary ops, ReLU / GELU forward and backward, scale, in-place
// accumulate, fill, strided copy.  All are HBM-bound: 128-bit loads and stores on the contiguous
// paths, grids sized in multiples of the SM count, one pass over the data.
//
// Arithmetic follows the reference CPU backend (crates/vearo-backend-cpu/src/lib.rs:160-238,
// 424-497) and the autograd masks (crates/vearo-autograd/src/lib.rs:364-403): same constants,
// full-precision tanhf, x*x*x for the cube.
#include "common.h"

namespace vb {

static constexpr float kSqrt2OverPi = 0.79788456f;
static constexpr float kGeluCoeff = 0.044715f;
static constexpr float kGeluDeriv = 0.134145f;

__device__ __forceinline__ float binop(int op, float a, float b) {
  switch (op) {
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    default: return a / b;
  }
}
__device__ __forceinline__ float relu_f(float v) { return v > 0.0f ? v : 0.0f; }
__device__ __forceinline__ float gelu_f(float v) { return gelu_value(v); }      // (common.h: shared with the GEMM epilogue)
__device__ __forceinline__ float gelu_grad_f(float v) {
  float v3 = v * v * v;
  float inner = kSqrt2OverPi * (v + kGeluCoeff * v3);
  float t = tanh_fast(inner);
  float sech_sq = 1.0f - t * t;
  float inner_deriv = kSqrt2OverPi * (1.0f + kGeluDeriv * v * v);
  return 0.5f * (1.0f + t) + 0.5f * v * sech_sq * inner_deriv;
}

static inline int grid_for(i64 work_items, int block) {
  i64 blocks = (work_items + block - 1) / block;
  i64 cap = (i64)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int OP>
__global__ void k_binary_vec(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ o, i64 n4) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n4; i += (i64)gridDim.x * blockDim.x) {
    float4 x = a[i], y = b[i], r;
    r.x = binop(OP, x.x, y.x); r.y = binop(OP, x.y, y.y); r.z = binop(OP, x.z, y.z); r.w = binop(OP, x.w, y.w);
    o[i] = r;
  }
}
__global__ void k_binary_scalar_tail(int op, const float* a, const float* b, float* o, i64 start, i64 n) {
  i64 i = start + blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i < n) o[i] = binop(op, a[i], b[i]);
}
int launch_binary(int op, const float* a, const float* b, float* o, i64 n) {
  if (n <= 0) return VB_OK;
  ProfScope prof("binary", 3.0 * (double)n * 4.0);
  cudaStream_t st = ctx().stream;
  i64 n4 = (aligned16(a) && aligned16(b) && aligned16(o)) ? n / 4 : 0;
  if (n4) {
    int g = grid_for(n4, 256);
    switch (op) {
      case 0: k_binary_vec<0><<<g, 256, 0, st>>>((const float4*)a, (const float4*)b, (float4*)o, n4); break;
      case 1: k_binary_vec<1><<<g, 256, 0, st>>>((const float4*)a, (const float4*)b, (float4*)o, n4); break;
      case 2: k_binary_vec<2><<<g, 256, 0, st>>>((const float4*)a, (const float4*)b, (float4*)o, n4); break;
      default: k_binary_vec<3><<<g, 256, 0, st>>>((const float4*)a, (const float4*)b, (float4*)o, n4); break;
    }
  }
  i64 rest = n - n4 * 4;
  if (rest) k_binary_scalar_tail<<<(int)((rest + 255) / 256), 256, 0, st>>>(op, a, b, o, n4 * 4, n);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// One operand is a vector over the last dim (bias add and friends), or a single scalar.
__global__ void k_binary_rowvec(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                                i64 n, i64 c, bool b_is_vec) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
    i64 j = i % c;
    o[i] = b_is_vec ? binop(op, a[i], b[j]) : binop(op, a[j], b[i]);
  }
}
int launch_binary_rowvec(int op, const float* a, const float* b, float* o, i64 n, i64 c, bool b_is_vec) {
  if (n <= 0) return VB_OK;
  k_binary_rowvec<<<grid_for(n, 256), 256, 0, ctx().stream>>>(op, a, b, o, n, c, b_is_vec);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void k_binary_scalar(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                                i64 n, bool b_is_scalar) {
  float s = b_is_scalar ? b[0] : a[0];
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x)
    o[i] = b_is_scalar ? binop(op, a[i], s) : binop(op, s, b[i]);
}
int launch_binary_scalar(int op, const float* a, const float* b, float* o, i64 n, bool b_is_scalar) {
  if (n <= 0) return VB_OK;
  k_binary_scalar<<<grid_for(n, 256), 256, 0, ctx().stream>>>(op, a, b, o, n, b_is_scalar);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// General N-d broadcast: the output is walked in row-major order; each operand has its own
// element strides with 0 on broadcast dims.
__global__ void k_binary_strided(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                                 i64 n, Strided s) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
    i64 rem = i, oa = 0, ob = 0;
    for (int d = s.rank - 1; d >= 0; --d) {
      i64 c = rem % s.dims[d]; rem /= s.dims[d];
      oa += c * s.sa[d]; ob += c * s.sb[d];
    }
    o[i] = binop(op, a[oa], b[ob]);
  }
}
int launch_binary_strided(int op, const float* a, const float* b, float* o, i64 n, const Strided& s) {
  if (n <= 0) return VB_OK;
  k_binary_strided<<<grid_for(n, 256), 256, 0, ctx().stream>>>(op, a, b, o, n, s);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

__global__ void k_strided_copy(const float* __restrict__ src, float* __restrict__ dst, i64 n, Strided s) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
    i64 rem = i, off = 0;
    for (int d = s.rank - 1; d >= 0; --d) { i64 c = rem % s.dims[d]; rem /= s.dims[d]; off += c * s.sa[d]; }
    dst[i] = src[off];
  }
}
int launch_strided_copy(const float* src, float* dst, i64 n, const Strided& s) {
  if (n <= 0) return VB_OK;
  ProfScope prof("strided_copy", 2.0 * (double)n * 4.0);
  k_strided_copy<<<grid_for(n, 256), 256, 0, ctx().stream>>>(src, dst, n, s);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// Unary forward (OP 0 relu, 1 gelu) and backward (dx = g * f'(x), the mask then a separate
// multiply as the reference's Relu / Gelu arms do).  12 bytes per element for the backward.
template <int OP, bool BWD>
__global__ void k_unary_vec(const float4* __restrict__ x, const float4* __restrict__ g, float4* __restrict__ o, i64 n4) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n4; i += (i64)gridDim.x * blockDim.x) {
    float4 v = x[i], r;
    if (BWD) {
      float4 gg = g[i];
      if (OP == 0) { r.x = gg.x * (v.x > 0.0f ? 1.0f : 0.0f); r.y = gg.y * (v.y > 0.0f ? 1.0f : 0.0f); r.z = gg.z * (v.z > 0.0f ? 1.0f : 0.0f); r.w = gg.w * (v.w > 0.0f ? 1.0f : 0.0f); }
      else { r.x = gg.x * gelu_grad_f(v.x); r.y = gg.y * gelu_grad_f(v.y); r.z = gg.z * gelu_grad_f(v.z); r.w = gg.w * gelu_grad_f(v.w); }
    } else {
      if (OP == 0) { r.x = relu_f(v.x); r.y = relu_f(v.y); r.z = relu_f(v.z); r.w = relu_f(v.w); }
      else { r.x = gelu_f(v.x); r.y = gelu_f(v.y); r.z = gelu_f(v.z); r.w = gelu_f(v.w); }
    }
    o[i] = r;
  }
}
template <int OP, bool BWD>
__global__ void k_unary_tail(const float* x, const float* g, float* o, i64 start, i64 n) {
  i64 i = start + blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i];
  if (BWD) o[i] = g[i] * (OP == 0 ? (v > 0.0f ? 1.0f : 0.0f) : gelu_grad_f(v));
  else o[i] = OP == 0 ? relu_f(v) : gelu_f(v);
}
template <int OP, bool BWD>
static int unary_impl(const float* x, const float* g, float* o, i64 n) {
  if (n <= 0) return VB_OK;
  ProfScope prof(BWD ? (OP == 0 ? "relu_bwd" : "gelu_bwd") : (OP == 0 ? "relu_fwd" : "gelu_fwd"), (BWD ? 3.0 : 2.0) * (double)n * 4.0);
  cudaStream_t st = ctx().stream;
  i64 n4 = (aligned16(x) && aligned16(o) && (!BWD || aligned16(g))) ? n / 4 : 0;
  if (n4) k_unary_vec<OP, BWD><<<grid_for(n4, 256), 256, 0, st>>>((const float4*)x, (const float4*)g, (float4*)o, n4);
  i64 rest = n - n4 * 4;
  if (rest) k_unary_tail<OP, BWD><<<(int)((rest + 255) / 256), 256, 0, st>>>(x, g, o, n4 * 4, n);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
int launch_unary(int op, const float* x, float* o, i64 n) {
  return op == 0 ? unary_impl<0, false>(x, nullptr, o, n) : unary_impl<1, false>(x, nullptr, o, n);
}
int launch_unary_backward(int op, const float* x, const float* g, float* o, i64 n) {
  return op == 0 ? unary_impl<0, true>(x, g, o, n) : unary_impl<1, true>(x, g, o, n);
}

// The backward of an activation that follows a Linear layer produces that layer's output gradient; the layer's bias gradient is
// the column sum of it.  This variant walks [rows, cols] as bands of whole rows -- a CTA of 256 threads owns a contiguous band, a
// thread the float4 columns t, t + 256, ... (cols <= 4096) with its column sums in registers, four rows in flight -- so that the
// memory stream is as contiguous as the flat kernel's, and leaves one partial row of column sums per band beside the gradient:
// the bias gradient then costs a small ordered sum instead of another pass over the tensor.
template <int OP>
__device__ __forceinline__ float4 unary_grad4(const float4& v, const float4& gg) {
  float4 r;
  if (OP == 0) { r.x = gg.x * (v.x > 0.0f ? 1.0f : 0.0f); r.y = gg.y * (v.y > 0.0f ? 1.0f : 0.0f); r.z = gg.z * (v.z > 0.0f ? 1.0f : 0.0f); r.w = gg.w * (v.w > 0.0f ? 1.0f : 0.0f); }
  else { r.x = gg.x * gelu_grad_f(v.x); r.y = gg.y * gelu_grad_f(v.y); r.z = gg.z * gelu_grad_f(v.z); r.w = gg.w * gelu_grad_f(v.w); }
  return r;
}
template <int OP, int K>
__global__ void __launch_bounds__(256) k_unary_bwd_colsum(const float4* __restrict__ x, const float4* __restrict__ g, float4* __restrict__ o,
                                                          float4* __restrict__ part, i64 rows, int cols4, i64 rows_per_band) {
  const i64 r0 = (i64)blockIdx.x * rows_per_band;
  i64 r1 = r0 + rows_per_band; if (r1 > rows) r1 = rows;
  float2 sa[K], sb[K];
#pragma unroll
  for (int k = 0; k < K; ++k) { sa[k] = make_float2(0.0f, 0.0f); sb[k] = sa[k]; }
  i64 r = r0;
  for (; r + 1 < r1; r += 2) {         // two rows x K columns: 4K loads in flight per thread
    float4 v0[K], v1[K], g0[K], g1[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = k * 256 + threadIdx.x;
      if (c < cols4) { v0[k] = x[r * cols4 + c]; g0[k] = g[r * cols4 + c]; v1[k] = x[(r + 1) * cols4 + c]; g1[k] = g[(r + 1) * cols4 + c]; }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = k * 256 + threadIdx.x;
      if (c < cols4) {
        const float4 d0 = unary_grad4<OP>(v0[k], g0[k]), d1 = unary_grad4<OP>(v1[k], g1[k]);
        o[r * cols4 + c] = d0; o[(r + 1) * cols4 + c] = d1;
        sa[k] = add2(sa[k], lo2(d0)); sb[k] = add2(sb[k], hi2(d0));
        sa[k] = add2(sa[k], lo2(d1)); sb[k] = add2(sb[k], hi2(d1));
      }
    }
  }
  if (r < r1) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = k * 256 + threadIdx.x;
      if (c < cols4) {
        const float4 d = unary_grad4<OP>(x[r * cols4 + c], g[r * cols4 + c]);
        o[r * cols4 + c] = d;
        sa[k] = add2(sa[k], lo2(d)); sb[k] = add2(sb[k], hi2(d));
      }
    }
  }
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = k * 256 + threadIdx.x;
    if (c < cols4) part[(i64)blockIdx.x * cols4 + c] = cat2(sa[k], sb[k]);
  }
}
int launch_unary_backward_colsum(int op, const float* x, const float* g, float* o, i64 rows, i64 cols, float* colsum) {
  if (rows <= 0 || cols <= 0) return VB_OK;
  const int cols4 = (int)(cols / 4), k = (cols4 + 255) / 256;       // the caller keeps cols <= 4096
  i64 bands = (i64)ctx().sm_count * (k == 4 ? 2 : 3);      /* one wave at the registers each instance takes */
  if (bands > rows / 4) bands = rows / 4; if (bands < 1) bands = 1;
  const i64 rpb = (rows + bands - 1) / bands;
  bands = (rows + rpb - 1) / rpb;
  void* part = nullptr;
  VB_TRY(scratch_alloc((size_t)(bands * cols) * sizeof(float), &part));
  int rc = VB_OK;
  {
    ProfScope prof(op == 0 ? "relu_bwd" : "gelu_bwd", 3.0 * (double)rows * (double)cols * 4.0);
    cudaStream_t st = ctx().stream;
#define UBC(OPV, KV) k_unary_bwd_colsum<OPV, KV><<<(unsigned)bands, 256, 0, st>>>((const float4*)x, (const float4*)g, (float4*)o, (float4*)part, rows, cols4, rpb)
    if (op == 0) { switch (k) { case 1: UBC(0, 1); break; case 2: UBC(0, 2); break; case 3: UBC(0, 3); break; default: UBC(0, 4); break; } }
    else { switch (k) { case 1: UBC(1, 1); break; case 2: UBC(1, 2); break; case 3: UBC(1, 3); break; default: UBC(1, 4); break; } }
#undef UBC
    rc = launch_colsum_final((const float*)part, colsum, cols, (int)bands);
  }
  scratch_free(part);
  VB_TRY(rc);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

__global__ void k_scale(const float* __restrict__ x, float alpha, float* __restrict__ o, i64 n) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) o[i] = x[i] * alpha;
}
int launch_scale(const float* x, float alpha, float* o, i64 n) {
  if (n <= 0) return VB_OK;
  k_scale<<<grid_for(n, 256), 256, 0, ctx().stream>>>(x, alpha, o, n);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void k_axpy_vec(float4* __restrict__ d, const float4* __restrict__ s, i64 n4) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n4; i += (i64)gridDim.x * blockDim.x) {
    float4 a = d[i], b = s[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    d[i] = a;
  }
}
__global__ void k_axpy_tail(float* d, const float* s, i64 start, i64 n) {
  i64 i = start + blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i < n) d[i] += s[i];
}
int launch_axpy(float* d, const float* s, i64 n) {
  if (n <= 0) return VB_OK;
  ProfScope prof("accumulate", 3.0 * (double)n * 4.0);
  cudaStream_t st = ctx().stream;
  i64 n4 = (aligned16(d) && aligned16(s)) ? n / 4 : 0;
  if (n4) k_axpy_vec<<<grid_for(n4, 256), 256, 0, st>>>((float4*)d, (const float4*)s, n4);
  i64 rest = n - n4 * 4;
  if (rest) k_axpy_tail<<<(int)((rest + 255) / 256), 256, 0, st>>>(d, s, n4 * 4, n);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void k_fill(float* d, float v, i64 n) {
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) d[i] = v;
}
int launch_fill(float* d, float v, i64 n) {
  if (n <= 0) return VB_OK;
  k_fill<<<grid_for(n, 256), 256, 0, ctx().stream>>>(d, v, n);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
