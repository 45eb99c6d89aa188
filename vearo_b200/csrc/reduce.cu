// Reductions: single-axis sum / mean, column sums (bias gradients and the general `reduce_to`
// of broadcast gradients), softmax forward and backward.
//
// Semantics follow crates/vearo-backend-cpu/src/lib.rs:501-653 (softmax: max with strict >, sum of
// exp(x - max), exp/sum; sum/mean: one division at the end) and crates/vearo-autograd/src/lib.rs:
// 316-361 (reduce_to) and 547-553 (softmax arm: y recomputed from the saved input,
// dx = y * (g - sum(g*y))).  Sums are tree-shaped here, sequential in the reference; the
// difference is within the 1e-4 / 1e-5 parity bound.  No atomics: results are bit-reproducible.
#include "common.h"
#include <cfloat>

namespace vb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions; blockDim.x a multiple of 32, <= 1024.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.0f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : -INFINITY;
  return warp_max(r);
}
static inline int threads_for_row(i64 d) {
  int t = 32;
  while (t < 256 && t * 4 < d) t <<= 1;
  return t;
}

// ---- sum / mean over one axis of [outer, d, inner] -----------------------------------------
__global__ void k_sum_rows(const float* __restrict__ x, float* __restrict__ out, i64 d, float inv) {
  __shared__ float red[32];
  const float* row = x + (i64)blockIdx.x * d;
  float s = 0.0f;
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) s += row[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[blockIdx.x] = inv == 0.0f ? s : s / inv;
}
__global__ void k_sum_inner(const float* __restrict__ x, float* __restrict__ out, i64 outer, i64 d, i64 inner, float inv) {
  i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (idx >= outer * inner) return;
  i64 o = idx / inner, in = idx % inner;
  const float* p = x + o * d * inner + in;
  float s = 0.0f;
  for (i64 j = 0; j < d; ++j) s += p[j * inner];
  out[idx] = inv == 0.0f ? s : s / inv;
}
int launch_sum_axis(const float* x, float* out, i64 outer, i64 d, i64 inner, bool mean) {
  if (outer * inner <= 0) return VB_OK;
  float inv = mean ? (float)d : 0.0f;
  if (inner == 1) k_sum_rows<<<(unsigned)outer, threads_for_row(d), 0, ctx().stream>>>(x, out, d, inv);
  else k_sum_inner<<<(unsigned)((outer * inner + 127) / 128), 128, 0, ctx().stream>>>(x, out, outer, d, inner, inv);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// ---- column sums: out[c] (+)= sum_r x[r, c] -------------------------------------------------
// Stage 1: a 32x8 block sums one 32-column strip over its share of the rows and writes a partial
// row; stage 2 adds the partial rows in a fixed order.  Algorithmic bytes: rows*cols*4 read.
__global__ void k_colsum_partial(const float* __restrict__ x, float* __restrict__ part, i64 rows, i64 cols, i64 rows_per_split) {
  __shared__ float sm[8][33];
  i64 c = (i64)blockIdx.x * 32 + threadIdx.x;
  i64 r0 = (i64)blockIdx.y * rows_per_split;
  i64 r1 = r0 + rows_per_split; if (r1 > rows) r1 = rows;
  float s = 0.0f;
  if (c < cols) for (i64 r = r0 + threadIdx.y; r < r1; r += 8) s += x[r * cols + c];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    part[(i64)blockIdx.y * cols + c] = t;
  }
}
// Adds the partial rows in a fixed order: a 32 x 32 block owns 32 columns, row lane y adds partial rows y, y + 32, ...
// (four loads in flight), then lane 0 adds the 32 sums in lane order.
__global__ void __launch_bounds__(1024) k_colsum_final(const float* __restrict__ part, float* __restrict__ out, i64 cols, int splits, bool accumulate) {
  __shared__ float sm[32][33];
  i64 c = (i64)blockIdx.x * 32 + threadIdx.x;
  float s = 0.0f;
  if (c < cols) {
    int i = threadIdx.y;
    for (; i + 96 < splits; i += 128) {
      float a0 = part[(i64)i * cols + c], a1 = part[(i64)(i + 32) * cols + c], a2 = part[(i64)(i + 64) * cols + c], a3 = part[(i64)(i + 96) * cols + c];
      s += a0; s += a1; s += a2; s += a3;
    }
    for (; i < splits; i += 32) s += part[(i64)i * cols + c];
  }
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += sm[i][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}
// 128-bit variant: a 32 x 8 block owns 128 columns (one float4 per thread and row), four rows in flight per thread.
__global__ void __launch_bounds__(256) k_colsum_partial_vec(const float4* __restrict__ x, float4* __restrict__ part, i64 rows, i64 cols4, i64 rows_per_split) {
  __shared__ float4 sm[8][33];
  i64 c = (i64)blockIdx.x * 32 + threadIdx.x;
  i64 r0 = (i64)blockIdx.y * rows_per_split;
  i64 r1 = r0 + rows_per_split; if (r1 > rows) r1 = rows;
  float4 s = make_float4(0, 0, 0, 0);
  if (c < cols4) {
    i64 r = r0 + threadIdx.y;
    for (; r + 24 < r1; r += 32) {
      float4 a = x[r * cols4 + c], b = x[(r + 8) * cols4 + c], d = x[(r + 16) * cols4 + c], e = x[(r + 24) * cols4 + c];
      s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w;
      s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w;
      s.x += d.x; s.y += d.y; s.z += d.z; s.w += d.w;
      s.x += e.x; s.y += e.y; s.z += e.z; s.w += e.w;
    }
    for (; r < r1; r += 8) { float4 a = x[r * cols4 + c]; s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
  }
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols4) {
    float4 t = make_float4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) { float4 a = sm[i][threadIdx.x]; t.x += a.x; t.y += a.y; t.z += a.z; t.w += a.w; }
    part[(i64)blockIdx.y * cols4 + c] = t;
  }
}
// Whole-row bands (cols <= 4096, a multiple of 4): a CTA of 256 threads sums a contiguous band of rows, a thread the float4
// columns t, t + 256, ... in registers, four rows in flight -- a contiguous memory stream -- and writes one partial row.
template <int K>
__global__ void __launch_bounds__(256) k_colsum_bands(const float4* __restrict__ x, float4* __restrict__ part, i64 rows, int cols4, i64 rows_per_band) {
  const i64 r0 = (i64)blockIdx.x * rows_per_band;
  i64 r1 = r0 + rows_per_band; if (r1 > rows) r1 = rows;
  float4 s[K];
#pragma unroll
  for (int k = 0; k < K; ++k) s[k] = make_float4(0, 0, 0, 0);
  i64 r = r0;
  for (; r + 3 < r1; r += 4) {
    float4 a[K], b[K], c[K], d[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int col = k * 256 + threadIdx.x;
      if (col < cols4) { a[k] = x[r * cols4 + col]; b[k] = x[(r + 1) * cols4 + col]; c[k] = x[(r + 2) * cols4 + col]; d[k] = x[(r + 3) * cols4 + col]; }
    }
#pragma unroll
    for (int k = 0; k < K; ++k)
      if (k * 256 + threadIdx.x < cols4) {
        s[k].x += a[k].x; s[k].y += a[k].y; s[k].z += a[k].z; s[k].w += a[k].w;
        s[k].x += b[k].x; s[k].y += b[k].y; s[k].z += b[k].z; s[k].w += b[k].w;
        s[k].x += c[k].x; s[k].y += c[k].y; s[k].z += c[k].z; s[k].w += c[k].w;
        s[k].x += d[k].x; s[k].y += d[k].y; s[k].z += d[k].z; s[k].w += d[k].w;
      }
  }
  for (; r < r1; ++r)
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int col = k * 256 + threadIdx.x;
      if (col < cols4) { const float4 a = x[r * cols4 + col]; s[k].x += a.x; s[k].y += a.y; s[k].z += a.z; s[k].w += a.w; }
    }
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int col = k * 256 + threadIdx.x;
    if (col < cols4) part[(i64)blockIdx.x * cols4 + col] = s[k];
  }
}
int launch_colsum_final(const float* part, float* out, i64 cols, int splits) {
  if (cols <= 0) return VB_OK;
  k_colsum_final<<<(unsigned)((cols + 31) / 32), dim3(32, 32), 0, ctx().stream>>>(part, out, cols, splits, false);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
int launch_colsum(const float* x, float* out, i64 rows, i64 cols, bool accumulate) {
  if (cols <= 0) return VB_OK;
  ProfScope prof("colsum", (double)rows * (double)cols * 4.0);
  if ((cols & 3) == 0 && cols >= 512 && cols <= 4096 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && rows >= 1024 && !accumulate) {
    const int cols4 = (int)(cols / 4), k = (cols4 + 255) / 256;
    i64 bands = (i64)ctx().sm_count * 2; if (bands > rows / 8) bands = rows / 8;      // one wave whatever the instance
    const i64 rpb = (rows + bands - 1) / bands;
    bands = (rows + rpb - 1) / rpb;
    void* part = nullptr;
    VB_TRY(scratch_alloc((size_t)(bands * cols) * sizeof(float), &part));
    cudaStream_t st = ctx().stream;
    switch (k) {
      case 1: k_colsum_bands<1><<<(unsigned)bands, 256, 0, st>>>((const float4*)x, (float4*)part, rows, cols4, rpb); break;
      case 2: k_colsum_bands<2><<<(unsigned)bands, 256, 0, st>>>((const float4*)x, (float4*)part, rows, cols4, rpb); break;
      case 3: k_colsum_bands<3><<<(unsigned)bands, 256, 0, st>>>((const float4*)x, (float4*)part, rows, cols4, rpb); break;
      default: k_colsum_bands<4><<<(unsigned)bands, 256, 0, st>>>((const float4*)x, (float4*)part, rows, cols4, rpb); break;
    }
    k_colsum_final<<<(unsigned)((cols + 31) / 32), dim3(32, 32), 0, st>>>((const float*)part, out, cols, (int)bands, false);
    scratch_free(part);
    VB_LAUNCH_CHECK();
    return VB_OK;
  }
  if ((cols & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && rows >= 64) {
    i64 cols4 = cols / 4, col_blocks = (cols4 + 31) / 32;
    i64 want = ((i64)ctx().sm_count * 4 + col_blocks - 1) / col_blocks;
    i64 splits = rows / 64; if (splits < 1) splits = 1; if (splits > want) splits = want; if (splits > 65535) splits = 65535;
    i64 rps = (rows + splits - 1) / splits;
    splits = (rows + rps - 1) / rps;
    void* part = nullptr;
    VB_TRY(scratch_alloc((size_t)(splits * cols) * sizeof(float), &part));
    k_colsum_partial_vec<<<dim3((unsigned)col_blocks, (unsigned)splits), dim3(32, 8), 0, ctx().stream>>>((const float4*)x, (float4*)part, rows, cols4, rps);
    k_colsum_final<<<(unsigned)((cols + 31) / 32), dim3(32, 32), 0, ctx().stream>>>((const float*)part, out, cols, (int)splits, accumulate);
    scratch_free(part);
    VB_LAUNCH_CHECK();
    return VB_OK;
  }
  i64 col_blocks = (cols + 31) / 32;
  i64 want = ((i64)ctx().sm_count * 8 + col_blocks - 1) / col_blocks;
  i64 splits = rows / 64; if (splits < 1) splits = 1; if (splits > want) splits = want; if (splits > 65535) splits = 65535;
  i64 rps = (rows + splits - 1) / splits;
  splits = rows > 0 ? (rows + rps - 1) / rps : 1;
  void* part = nullptr;
  VB_TRY(scratch_alloc((size_t)(splits * cols) * sizeof(float), &part));
  dim3 grid((unsigned)col_blocks, (unsigned)splits), block(32, 8);
  k_colsum_partial<<<grid, block, 0, ctx().stream>>>(x, (float*)part, rows, cols, rps);
  k_colsum_final<<<(unsigned)((cols + 31) / 32), dim3(32, 32), 0, ctx().stream>>>((const float*)part, out, cols, (int)splits, accumulate);
  scratch_free(part);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// General broadcast-gradient reduction: one thread per output element walks the reduced index
// space in row-major order (the order reduce_to adds in).
__global__ void k_reduce_general(const float* __restrict__ g, float* __restrict__ out, i64 out_numel, Strided kept, Strided red, i64 red_count, i64 g_numel) {
  i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (idx >= out_numel) return;
  i64 rem = idx, base = 0;
  for (int d = kept.rank - 1; d >= 0; --d) { i64 c = rem % kept.dims[d]; rem /= kept.dims[d]; base += c * kept.sa[d]; }
  float s = 0.0f;
  for (i64 r = 0; r < red_count; ++r) {
    i64 rr = r, off = base;
    for (int d = red.rank - 1; d >= 0; --d) { i64 c = rr % red.dims[d]; rr /= red.dims[d]; off += c * red.sa[d]; }
    if (VB_BC(off, g_numel)) s += g[off];
  }
  out[idx] = s;
}
int launch_reduce_general(const float* g, float* out, i64 out_numel, const Strided& kept, const Strided& red, i64 red_count) {
  if (out_numel <= 0) return VB_OK;
  k_reduce_general<<<(unsigned)((out_numel + 127) / 128), 128, 0, ctx().stream>>>(g, out, out_numel, kept, red, red_count, out_numel * red_count);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// ---- softmax over the last axis: one block per row -------------------------------------------
__global__ void k_softmax_rows(const float* __restrict__ x, float* __restrict__ out, i64 d) {
  __shared__ float red[32];
  const float* row = x + (i64)blockIdx.x * d;
  float* orow = out + (i64)blockIdx.x * d;
  float m = -INFINITY;
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) m = fmaxf(m, row[i]);
  m = block_max(m, red);
  float s = 0.0f;
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) s += expf(row[i] - m);
  s = block_sum(s, red);
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) orow[i] = expf(row[i] - m) / s;
}
int launch_softmax_rows(const float* x, float* out, i64 rows, i64 d) {
  if (rows <= 0 || d <= 0) return VB_OK;
  k_softmax_rows<<<(unsigned)rows, threads_for_row(d), 0, ctx().stream>>>(x, out, d);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void k_softmax_backward_rows(const float* __restrict__ x, const float* __restrict__ g, float* __restrict__ out, i64 d) {
  __shared__ float red[32];
  const float* row = x + (i64)blockIdx.x * d;
  const float* grow = g + (i64)blockIdx.x * d;
  float* orow = out + (i64)blockIdx.x * d;
  float m = -INFINITY;
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) m = fmaxf(m, row[i]);
  m = block_max(m, red);
  float s = 0.0f;
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) s += expf(row[i] - m);
  s = block_sum(s, red);
  float dot = 0.0f;
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) dot += grow[i] * (expf(row[i] - m) / s);
  dot = block_sum(dot, red);
  for (i64 i = threadIdx.x; i < d; i += blockDim.x) { float y = expf(row[i] - m) / s; orow[i] = y * (grow[i] - dot); }
}
int launch_softmax_backward_rows(const float* x, const float* g, float* out, i64 rows, i64 d) {
  if (rows <= 0 || d <= 0) return VB_OK;
  k_softmax_backward_rows<<<(unsigned)rows, threads_for_row(d), 0, ctx().stream>>>(x, g, out, d);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// ---- softmax over an inner axis of [outer, d, inner]: one thread per (outer, inner) ----------
__global__ void k_softmax_strided(const float* __restrict__ x, const float* __restrict__ g, float* __restrict__ out,
                                  i64 outer, i64 d, i64 inner, bool backward) {
  i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (idx >= outer * inner) return;
  i64 base = (idx / inner) * d * inner + idx % inner;
  float m = -INFINITY;
  for (i64 j = 0; j < d; ++j) m = fmaxf(m, x[base + j * inner]);
  float s = 0.0f;
  for (i64 j = 0; j < d; ++j) s += expf(x[base + j * inner] - m);
  if (!backward) {
    for (i64 j = 0; j < d; ++j) out[base + j * inner] = expf(x[base + j * inner] - m) / s;
  } else {
    float dot = 0.0f;
    for (i64 j = 0; j < d; ++j) dot += g[base + j * inner] * (expf(x[base + j * inner] - m) / s);
    for (i64 j = 0; j < d; ++j) { float y = expf(x[base + j * inner] - m) / s; out[base + j * inner] = y * (g[base + j * inner] - dot); }
  }
}
int launch_softmax_strided(const float* x, float* out, i64 outer, i64 d, i64 inner) {
  if (outer * inner <= 0 || d <= 0) return VB_OK;
  k_softmax_strided<<<(unsigned)((outer * inner + 127) / 128), 128, 0, ctx().stream>>>(x, nullptr, out, outer, d, inner, false);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
int launch_softmax_backward_strided(const float* x, const float* g, float* out, i64 outer, i64 d, i64 inner) {
  if (outer * inner <= 0 || d <= 0) return VB_OK;
  k_softmax_strided<<<(unsigned)((outer * inner + 127) / 128), 128, 0, ctx().stream>>>(x, g, out, outer, d, inner, true);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
