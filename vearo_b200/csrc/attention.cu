// Row kernels of scaled-dot-product attention; the matrix products around them run on the GEMM
// kernels (QK^T, PV, and the four backward products), with the score / probability matrices kept
// in HBM ([B,H,S,S] f32; 180 GB of HBM3e makes that the simple choice at S = 1024).
//
// Semantics: crates/vearo-backend-cpu/src/lib.rs:2416-2458 (forward row) and 2573-2591 (backward
// row): score = (q.k) * scale + mask, p = exp(score - max) * (1 / (sum + 1e-9)) — note the 1e-9
// and the reciprocal-multiply, which plain softmax does not have — and
// ds = p * (dp - sum_j dp_j * p_j).  The additive mask is right-aligned to [B,H,Sq,Sk] with
// size-1 dims broadcast (lib.rs:2395-2404, 2430-2442); a [S,S] causal mask stays L2-resident.
//
// Both kernels are HBM-bound: one CTA of 128 threads per row, the row held in registers
// (up to 4096 columns), one read and one write of the matrix.
#include "common.h"
#include <cstdlib>

namespace vb {

__device__ __forceinline__ float a_wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float a_wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float a_bsum(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = a_wsum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  return a_wsum(lane < nw ? red[lane] : 0.0f);
}
__device__ __forceinline__ float a_bmax(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = a_wmax(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  return a_wmax(lane < nw ? red[lane] : -INFINITY);
}

struct MaskStrides { i64 b, h, q, k; };

// s holds scale * (q.k) on entry and the probabilities on exit.
template <int EPT>
__global__ void __launch_bounds__(128) k_attn_softmax(float* __restrict__ s, const float* __restrict__ mask, MaskStrides ms,
                                                      i64 H, i64 sq, i64 sk) {
  __shared__ float red[32];
  i64 row = blockIdx.x;                 // (b * H + h) * sq + i
  i64 i = row % sq, bh = row / sq, h = bh % H, b = bh / H;
  float* r = s + row * sk;
  const float* mrow = mask ? mask + b * ms.b + h * ms.h + i * ms.q : nullptr;
  float v[EPT];
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    i64 j = threadIdx.x + (i64)e * 128;
    if (j < sk) {
      float x = r[j];
      if (mrow) x += mrow[j * ms.k];
      v[e] = x;
      if (x > mx) mx = x;
    } else v[e] = -INFINITY;
  }
  mx = a_bmax(mx, red);
  float sum = 0.0f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    i64 j = threadIdx.x + (i64)e * 128;
    if (j < sk) { v[e] = expf(v[e] - mx); sum += v[e]; }
  }
  sum = a_bsum(sum, red);
  float inv = 1.0f / (sum + 1e-9f);
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    i64 j = threadIdx.x + (i64)e * 128;
    if (j < sk) r[j] = v[e] * inv;
  }
}
// Rows longer than 4096: values are re-read from global memory (L1/L2-hot) instead of registers.
__global__ void __launch_bounds__(256) k_attn_softmax_long(float* __restrict__ s, const float* __restrict__ mask, MaskStrides ms,
                                                           i64 H, i64 sq, i64 sk) {
  __shared__ float red[32];
  i64 row = blockIdx.x;
  i64 i = row % sq, bh = row / sq, h = bh % H, b = bh / H;
  float* r = s + row * sk;
  const float* mrow = mask ? mask + b * ms.b + h * ms.h + i * ms.q : nullptr;
  float mx = -INFINITY;
  for (i64 j = threadIdx.x; j < sk; j += blockDim.x) { float x = r[j]; if (mrow) x += mrow[j * ms.k]; r[j] = x; if (x > mx) mx = x; }
  mx = a_bmax(mx, red);
  float sum = 0.0f;
  for (i64 j = threadIdx.x; j < sk; j += blockDim.x) { float e = expf(r[j] - mx); r[j] = e; sum += e; }
  sum = a_bsum(sum, red);
  float inv = 1.0f / (sum + 1e-9f);
  for (i64 j = threadIdx.x; j < sk; j += blockDim.x) r[j] *= inv;
}

// Warp-per-row variants for rows of up to 1024 columns (a multiple of 4): 128-bit loads and stores, the row lives
// in registers, reductions are warp shuffles only (no block barrier).  V = float4 per lane.
// i_lo, i_cnt: the rows [i_lo, i_lo + i_cnt) of every [sq, sk] matrix are handled by this launch (`rows` = number of matrices).
// Causal launches go by bands of rows, each with the instance whose register array just covers the band's live columns.
template <int V>
__global__ void __launch_bounds__(128, 6) k_attn_softmax_warp(float* __restrict__ s, const float* __restrict__ mask, MaskStrides ms,
                                                           i64 H, i64 sq, i64 sk, i64 rows, int causal, i64 i_lo, i64 i_cnt) {
  const int lane = threadIdx.x & 31;
  // grid: x = groups of four rows of the band, y = matrices (no division on the way to the row's address)
  const i64 ii = (i64)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (ii >= i_cnt) return;
  const i64 i = i_lo + ii;
  for (i64 bh = blockIdx.y; bh < rows; bh += gridDim.y) {
    const i64 row = bh * sq + i;
    float4* r4 = reinterpret_cast<float4*>(s + row * sk);
    const float4* m4 = nullptr;
    if (mask && !causal) { const i64 h = bh % H, b = bh / H; m4 = reinterpret_cast<const float4*>(mask + b * ms.b + h * ms.h + i * ms.q); }
    // causal: columns j > i hold probability 0; they are not read, and zeros are written only up to the end of the
    // 128-row tile that contains row i (what the triangular products that follow can touch)
    const i64 live = causal ? i + 1 : sk;                       // columns [0, live) take part
    const i64 zero_to = causal ? (((i >> 7) + 1) << 7 < sk ? ((i >> 7) + 1) << 7 : sk) : sk;
    float4 v[V];
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      int j4 = e * 32 + lane;
      if (j4 * 4 < live) {
        float4 x = r4[j4];
        if (m4) { float4 m = m4[j4]; x.x += m.x; x.y += m.y; x.z += m.z; x.w += m.w; }
        if (causal) {   // the chunk that straddles the diagonal
          i64 j = (i64)j4 * 4;
          if (j + 1 >= live) x.y = -INFINITY;
          if (j + 2 >= live) x.z = -INFINITY;
          if (j + 3 >= live) x.w = -INFINITY;
        }
        v[e] = x;
        mx = fmaxf(mx, fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w)));
      } else v[e] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    mx = a_wmax(mx);
    float sum = 0.0f;
#pragma unroll
    for (int e = 0; e < V; ++e)
      if ((e * 32 + lane) * 4 < live) {
        v[e].x = expf(v[e].x - mx); v[e].y = expf(v[e].y - mx); v[e].z = expf(v[e].z - mx); v[e].w = expf(v[e].w - mx);
        sum += (v[e].x + v[e].y) + (v[e].z + v[e].w);
      }
    sum = a_wsum(sum);
    float inv = 1.0f / (sum + 1e-9f);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      i64 j = (i64)(e * 32 + lane) * 4;
      if (j < live) r4[e * 32 + lane] = make_float4(v[e].x * inv, v[e].y * inv, v[e].z * inv, v[e].w * inv);
      else if (j < zero_to) r4[e * 32 + lane] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  }
}
template <int V>
__global__ void __launch_bounds__(128) k_attn_softmax_bwd_warp(const float* __restrict__ p, float* __restrict__ dp, i64 sk, float scale, i64 rows,
                                                               int causal, i64 sq, i64 i_lo, i64 i_cnt) {
  const int lane = threadIdx.x & 31;
  const i64 ii = (i64)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (ii >= i_cnt) return;
  const i64 i = i_lo + ii;
  for (i64 bh = blockIdx.y; bh < rows; bh += gridDim.y) {
    const i64 row = bh * sq + i;
    const float4* p4 = reinterpret_cast<const float4*>(p + row * sk);
    float4* d4 = reinterpret_cast<float4*>(dp + row * sk);
    // causal: p is exactly 0 for columns j > i (the forward wrote those zeros inside the diagonal tile), so chunks
    // past the diagonal contribute nothing; dp there was never computed and is overwritten with zeros up to the tile end
    const i64 live = causal ? i + 1 : sk;
    const i64 zero_to = causal ? (((i >> 7) + 1) << 7 < sk ? ((i >> 7) + 1) << 7 : sk) : sk;
    float4 pv[V], dv[V];
    float dot = 0.0f;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      int j4 = e * 32 + lane;
      if (j4 * 4 < live) {
        pv[e] = p4[j4]; dv[e] = d4[j4];
        if (causal) {   // dp entries beyond the diagonal inside this chunk may be unwritten memory: mask them (p is 0 there)
          i64 j = (i64)j4 * 4;
          if (j + 1 >= live) dv[e].y = 0.0f;
          if (j + 2 >= live) dv[e].z = 0.0f;
          if (j + 3 >= live) dv[e].w = 0.0f;
        }
        dot = fmaf(dv[e].x, pv[e].x, dot); dot = fmaf(dv[e].y, pv[e].y, dot); dot = fmaf(dv[e].z, pv[e].z, dot); dot = fmaf(dv[e].w, pv[e].w, dot);
      }
    }
    dot = a_wsum(dot);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      int j4 = e * 32 + lane;
      if (j4 * 4 < live)
        d4[j4] = make_float4((pv[e].x * (dv[e].x - dot)) * scale, (pv[e].y * (dv[e].y - dot)) * scale,
                             (pv[e].z * (dv[e].z - dot)) * scale, (pv[e].w * (dv[e].w - dot)) * scale);
      else if ((i64)j4 * 4 < zero_to) d4[j4] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  }
}
// Elements one [sq, sk] matrix moves under a causal mask: `reads` per live score (columns 0..i of row i) plus `writes` per
// element up to the end of the row's 128-row tile (the zeros the triangular products that follow may touch).
static inline double causal_elems(i64 sq, i64 sk, double reads, double writes) {
  double e = 0.0;
  for (i64 i = 0; i < sq; ++i) {
    i64 live = i + 1 < sk ? i + 1 : sk, z = ((i >> 7) + 1) << 7; if (z > sk) z = sk;
    e += reads * (double)live + writes * (double)z;
  }
  return e;
}
static inline i64 causal_band() { static i64 b = 0; if (!b) { const char* e = getenv("VB200_SOFTMAX_BAND"); b = e ? atoll(e) : 512; if (b < 128) b = 128; } return b; }
static inline bool al16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_attn_softmax(float* s, const float* mask, const i64 mstr[4], bool causal, i64 b, i64 h, i64 sq, i64 sk, float scale) {
  (void)scale;
  i64 rows = b * h * sq;
  if (rows <= 0 || sk <= 0) return VB_OK;
  // bytes really moved: under a causal mask row i reads its i + 1 live scores and writes up to the end of its 128-row tile
  const double dense_bytes = 2.0 * (double)rows * (double)sk * 4.0;
  ProfScope prof("attn_softmax", causal ? (double)(b * h) * causal_elems(sq, sk, 1.0, 1.0) * 4.0 : dense_bytes, dense_bytes);
  MaskStrides ms{0, 0, 0, 0};
  if (mask) ms = MaskStrides{mstr[0], mstr[1], mstr[2], mstr[3]};
  cudaStream_t st = ctx().stream;
  bool mask_vec = !mask || (ms.k == 1 && al16p(mask) && !(ms.b & 3) && !(ms.h & 3) && !(ms.q & 3));
  if (causal && !((sk & 3) == 0 && sk <= 1024 && al16p(s) && sq == sk)) return set_error(VB_ERR_UNSUPPORTED, "causal attention softmax needs square S <= 1024, a multiple of 4");
  if ((sk & 3) == 0 && sk <= 1024 && al16p(s) && (mask_vec || causal)) {
    const i64 mats = b * h;
    // causal: bands of 256 rows, band c with the instance covering its 256 (c + 1) live columns; otherwise one launch over all rows
    const i64 band = causal ? causal_band() : sq;
    for (i64 lo = 0; lo < sq; lo += band) {
      const i64 cnt = sq - lo < band ? sq - lo : band;
      const i64 width = causal ? (lo + cnt < sk ? lo + cnt : sk) : sk;
      const dim3 wg((unsigned)((cnt + 3) / 4), (unsigned)(mats < 65535 ? mats : 65535));
      const int cz = causal ? 1 : 0;
      if (width <= 128) k_attn_softmax_warp<1><<<wg, 128, 0, st>>>(s, mask, ms, h, sq, sk, mats, cz, lo, cnt);
      else if (width <= 256) k_attn_softmax_warp<2><<<wg, 128, 0, st>>>(s, mask, ms, h, sq, sk, mats, cz, lo, cnt);
      else if (width <= 512) k_attn_softmax_warp<4><<<wg, 128, 0, st>>>(s, mask, ms, h, sq, sk, mats, cz, lo, cnt);
      else if (width <= 768) k_attn_softmax_warp<6><<<wg, 128, 0, st>>>(s, mask, ms, h, sq, sk, mats, cz, lo, cnt);
      else k_attn_softmax_warp<8><<<wg, 128, 0, st>>>(s, mask, ms, h, sq, sk, mats, cz, lo, cnt);
    }
    VB_LAUNCH_CHECK();
    return VB_OK;
  }
  unsigned g = (unsigned)rows;
  if (sk <= 128) k_attn_softmax<1><<<g, 128, 0, st>>>(s, mask, ms, h, sq, sk);
  else if (sk <= 256) k_attn_softmax<2><<<g, 128, 0, st>>>(s, mask, ms, h, sq, sk);
  else if (sk <= 512) k_attn_softmax<4><<<g, 128, 0, st>>>(s, mask, ms, h, sq, sk);
  else if (sk <= 1024) k_attn_softmax<8><<<g, 128, 0, st>>>(s, mask, ms, h, sq, sk);
  else if (sk <= 2048) k_attn_softmax<16><<<g, 128, 0, st>>>(s, mask, ms, h, sq, sk);
  else if (sk <= 4096) k_attn_softmax<32><<<g, 128, 0, st>>>(s, mask, ms, h, sq, sk);
  else k_attn_softmax_long<<<g, 256, 0, st>>>(s, mask, ms, h, sq, sk);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// dp holds dO.V^T on entry and scale * p * (dp - sum(dp * p)) on exit.
template <int EPT>
__global__ void __launch_bounds__(128) k_attn_softmax_bwd(const float* __restrict__ p, float* __restrict__ dp, i64 sk, float scale) {
  __shared__ float red[32];
  const float* pr = p + (i64)blockIdx.x * sk;
  float* dr = dp + (i64)blockIdx.x * sk;
  float pv[EPT], dv[EPT];
  float dot = 0.0f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    i64 j = threadIdx.x + (i64)e * 128;
    if (j < sk) { pv[e] = pr[j]; dv[e] = dr[j]; dot = fmaf(dv[e], pv[e], dot); } else { pv[e] = 0.0f; dv[e] = 0.0f; }
  }
  dot = a_bsum(dot, red);
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    i64 j = threadIdx.x + (i64)e * 128;
    if (j < sk) dr[j] = (pv[e] * (dv[e] - dot)) * scale;
  }
}
__global__ void __launch_bounds__(256) k_attn_softmax_bwd_long(const float* __restrict__ p, float* __restrict__ dp, i64 sk, float scale) {
  __shared__ float red[32];
  const float* pr = p + (i64)blockIdx.x * sk;
  float* dr = dp + (i64)blockIdx.x * sk;
  float dot = 0.0f;
  for (i64 j = threadIdx.x; j < sk; j += blockDim.x) dot = fmaf(dr[j], pr[j], dot);
  dot = a_bsum(dot, red);
  for (i64 j = threadIdx.x; j < sk; j += blockDim.x) dr[j] = (pr[j] * (dr[j] - dot)) * scale;
}
int launch_attn_softmax_backward(const float* p, float* dp, i64 rows, i64 sk, float scale, bool causal, i64 sq) {
  if (rows <= 0 || sk <= 0) return VB_OK;
  if (causal && !((sk & 3) == 0 && sk <= 1024 && al16p(p) && al16p(dp) && sq == sk)) return set_error(VB_ERR_UNSUPPORTED, "causal attention softmax needs square S <= 1024, a multiple of 4");
  const double dense_bytes = 3.0 * (double)rows * (double)sk * 4.0;
  ProfScope prof("attn_softmax_bwd", causal ? (double)(rows / sq) * causal_elems(sq, sk, 2.0, 1.0) * 4.0 : dense_bytes, dense_bytes);
  cudaStream_t st = ctx().stream;
  if ((sk & 3) == 0 && sk <= 1024 && al16p(p) && al16p(dp)) {
    const i64 mats = causal ? rows / sq : 1, seq = causal ? sq : rows;      // without a causal mask all rows are alike: one band
    const i64 band = causal ? causal_band() : seq;
    const int cz = causal ? 1 : 0;
    for (i64 lo = 0; lo < seq; lo += band) {
      const i64 cnt = seq - lo < band ? seq - lo : band;
      const i64 width = causal ? (lo + cnt < sk ? lo + cnt : sk) : sk;
      const dim3 wg((unsigned)((cnt + 3) / 4), (unsigned)(mats < 65535 ? mats : 65535));
      if (width <= 128) k_attn_softmax_bwd_warp<1><<<wg, 128, 0, st>>>(p, dp, sk, scale, mats, cz, seq, lo, cnt);
      else if (width <= 256) k_attn_softmax_bwd_warp<2><<<wg, 128, 0, st>>>(p, dp, sk, scale, mats, cz, seq, lo, cnt);
      else if (width <= 512) k_attn_softmax_bwd_warp<4><<<wg, 128, 0, st>>>(p, dp, sk, scale, mats, cz, seq, lo, cnt);
      else if (width <= 768) k_attn_softmax_bwd_warp<6><<<wg, 128, 0, st>>>(p, dp, sk, scale, mats, cz, seq, lo, cnt);
      else k_attn_softmax_bwd_warp<8><<<wg, 128, 0, st>>>(p, dp, sk, scale, mats, cz, seq, lo, cnt);
    }
    VB_LAUNCH_CHECK();
    return VB_OK;
  }
  unsigned g = (unsigned)rows;
  if (sk <= 128) k_attn_softmax_bwd<1><<<g, 128, 0, st>>>(p, dp, sk, scale);
  else if (sk <= 256) k_attn_softmax_bwd<2><<<g, 128, 0, st>>>(p, dp, sk, scale);
  else if (sk <= 512) k_attn_softmax_bwd<4><<<g, 128, 0, st>>>(p, dp, sk, scale);
  else if (sk <= 1024) k_attn_softmax_bwd<8><<<g, 128, 0, st>>>(p, dp, sk, scale);
  else if (sk <= 2048) k_attn_softmax_bwd<16><<<g, 128, 0, st>>>(p, dp, sk, scale);
  else if (sk <= 4096) k_attn_softmax_bwd<32><<<g, 128, 0, st>>>(p, dp, sk, scale);
  else k_attn_softmax_bwd_long<<<g, 256, 0, st>>>(p, dp, sk, scale);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// Does a [S,S] additive mask have the causal pattern for which skipping is exact: 0 on and below the diagonal and
// <= -1e9 above it (exp(score - 1e9 - max) is exactly 0 in f32)?  Clears *d_flag when an entry breaks it.
__global__ void k_mask_is_causal(const float* __restrict__ mask, i64 s, i64 row_stride, int* d_flag) {
  i64 total = s * s;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 i = idx / s, j = idx % s;
    float m = mask[i * row_stride + j];
    bool ok = j <= i ? (m == 0.0f) : (m <= -1e9f);
    if (!ok) *d_flag = 0;
  }
}
int launch_mask_is_causal(const float* mask, i64 s, i64 row_stride, int* d_flag) {
  i64 blocks = (s * s + 255) / 256, cap = (i64)ctx().sm_count * 8; if (blocks > cap) blocks = cap;
  k_mask_is_causal<<<(unsigned)blocks, 256, 0, ctx().stream>>>(mask, s, row_stride, d_flag);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
