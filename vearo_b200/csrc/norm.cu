// LayerNorm and BatchNorm2d, forward and backward.
//
// LayerNorm follows crates/vearo-backend-cpu/src/lib.rs:667-858: two-pass mean / biased variance,
// r = 1/sqrt(var + eps), y = ((x - mean) * r) * w + b;  backward recomputes mean and r per row,
// a = sum(g*w), c = sum(g*w*xhat), dx = (C*g*w - a - xhat*c) * r / C, dw += g*xhat, db += g.
// BatchNorm follows lib.rs:2067-2364 (biased batch variance for normalisation, Bessel factor only
// in the running value, eval mode uses the running statistics).
//
// LayerNorm backward is the HBM-bound kernel of this file: one warp owns a row, reads x and g (and, where the caller accumulates
// into an existing gradient, that gradient) exactly once into registers (128-bit loads), reduces with warp shuffles and does its
// arithmetic on packed pairs of f32.  Each warp keeps running column sums -- dgamma, dbeta and the sum of the rows it stored, which
// is the bias gradient of the Linear layer that produced the normalised tensor's input -- in a strip of shared memory that only
// it touches; one partial row per CTA and sum is then added up in a fixed order.  No atomics, bit-reproducible.
// Algorithmic bytes per call: 3 * rows * C * 4 (read x, read g, write dx), 4 * rows * C * 4 when accumulating.
#include "common.h"

namespace vb {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float bsum(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = wsum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.0f;
  return wsum(r);
}

// ---- LayerNorm, warp-per-row register-resident path (C % 4 == 0, C <= 128 * VPT) ------------
template <int VPT>
__global__ void __launch_bounds__(256) k_ln_fwd_warp(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                                     float* __restrict__ out, i64 rows, int C, float eps, float* __restrict__ out_lo) {
  int lane = threadIdx.x & 31;
  i64 warp = (blockIdx.x * (i64)blockDim.x + threadIdx.x) >> 5;
  i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  float fc = (float)C;
  for (i64 r = warp; r < rows; r += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + r * C);
    float4 v[VPT];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int col = (i * 32 + lane) * 4;
      v[i] = col < C ? xr[i * 32 + lane] : make_float4(0, 0, 0, 0);
      s += v[i].x + v[i].y + v[i].z + v[i].w;
    }
    float mean = wsum(s) / fc;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int col = (i * 32 + lane) * 4;
      if (col < C) { float a = v[i].x - mean, bb = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean; q += a * a + bb * bb + c * c + d * d; }
    }
    float inv = 1.0f / sqrtf(wsum(q) / fc + eps);
    float4* orow = reinterpret_cast<float4*>(out + r * C);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int col = (i * 32 + lane) * 4;
      if (col < C) {
        float4 ww = *reinterpret_cast<const float4*>(w + col), bb = *reinterpret_cast<const float4*>(b + col), o;
        o.x = ((v[i].x - mean) * inv) * ww.x + bb.x; o.y = ((v[i].y - mean) * inv) * ww.y + bb.y;
        o.z = ((v[i].z - mean) * inv) * ww.z + bb.z; o.w = ((v[i].w - mean) * inv) * ww.w + bb.w;
        orow[i * 32 + lane] = o;
        // (the TF32 remainders of the output, for the tensor-core product that will take it as its B operand)
        if (out_lo) reinterpret_cast<float4*>(out_lo + r * C)[i * 32 + lane] = make_float4(tf32_remainder(o.x), tf32_remainder(o.y), tf32_remainder(o.z), tf32_remainder(o.w));
      }
    }
  }
}

// dx = (g w - mean(g w) - x-hat mean(g w x-hat)) r, written as g w r - (a r / C) - x-hat (c r / C) with a = sum(g w), c = sum(g w x-hat).
// NSUMS = 3 also keeps the column sums of the stored rows.  ACCUM: the stored row is resid + dx (gx may be resid).
template <int VPT, bool ACCUM>
__global__ void __launch_bounds__(256, 2) k_ln_bwd_warp(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ g,
                                                        const float* resid, float* gx, float* __restrict__ part,
                                                        i64 rows, int C, float eps, int nsums) {
  extern __shared__ __align__(16) float sm[];   // [warps][3][C]: running column sums of g * x-hat, of g and of the stored rows
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const i64 warp = (i64)blockIdx.x * nw + wid, nwarps = (i64)gridDim.x * nw;
  const float rfc = 1.0f / (float)C;
  const float2 zero2 = make_float2(0.0f, 0.0f);
  const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float4* acc_w = reinterpret_cast<float4*>(sm + (size_t)wid * 3 * C);
  float4* acc_b = acc_w + C / 4;
  float4* acc_o = acc_b + C / 4;
#pragma unroll
  for (int i = 0; i < VPT; ++i)      // a lane only ever touches its own columns of the strip: no synchronisation inside the warp
    if ((i * 32 + lane) * 4 < C) { acc_w[i * 32 + lane] = zero4; acc_b[i * 32 + lane] = zero4; acc_o[i * 32 + lane] = zero4; }
  for (i64 r = warp; r < rows; r += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + r * C);
    const float4* gr = reinterpret_cast<const float4*>(g + r * C);
    float4 v[VPT], gg[VPT], rs[ACCUM ? VPT : 1];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const bool in = (i * 32 + lane) * 4 < C;
      v[i] = in ? xr[i * 32 + lane] : zero4;
      gg[i] = in ? gr[i * 32 + lane] : zero4;
      if (ACCUM) rs[i] = in ? reinterpret_cast<const float4*>(resid + r * C)[i * 32 + lane] : zero4;
    }
    float2 acc = zero2;
#pragma unroll
    for (int i = 0; i < VPT; ++i) acc = add2(acc, add2(lo2(v[i]), hi2(v[i])));
    const float mean = wsum(acc.x + acc.y) * rfc;
    const float2 nmean = make_float2(-mean, -mean);
    acc = zero2;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {                  // v becomes x - mean
      float2 a = add2(lo2(v[i]), nmean), b = add2(hi2(v[i]), nmean);
      if ((i * 32 + lane) * 4 >= C) { a = zero2; b = zero2; }
      acc = fma2(a, a, acc); acc = fma2(b, b, acc);
      v[i] = cat2(a, b);
    }
    const float inv = 1.0f / sqrtf(wsum(acc.x + acc.y) * rfc + eps);
    const float2 inv2 = make_float2(inv, inv);
    float2 s1 = zero2, s2 = zero2;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {                  // v becomes x-hat, gg becomes g * w
      const bool in = (i * 32 + lane) * 4 < C;
      const float4 ww = in ? *reinterpret_cast<const float4*>(w + (i * 32 + lane) * 4) : zero4;
      const float2 xa = mul2(lo2(v[i]), inv2), xb = mul2(hi2(v[i]), inv2);
      const float2 ga = lo2(gg[i]), gb = hi2(gg[i]);
      if (in) {
        const float4 cw = acc_w[i * 32 + lane], cb = acc_b[i * 32 + lane];
        acc_w[i * 32 + lane] = cat2(fma2(ga, xa, lo2(cw)), fma2(gb, xb, hi2(cw)));
        acc_b[i * 32 + lane] = cat2(add2(ga, lo2(cb)), add2(gb, hi2(cb)));
      }
      const float2 pa = mul2(ga, lo2(ww)), pb = mul2(gb, hi2(ww));
      s1 = add2(s1, add2(pa, pb));
      s2 = fma2(pa, xa, s2); s2 = fma2(pb, xb, s2);
      v[i] = cat2(xa, xb); gg[i] = cat2(pa, pb);
    }
    const float t1 = wsum(s1.x + s1.y), t2 = wsum(s2.x + s2.y);
    const float na = -(t1 * inv * rfc), nb = -(t2 * inv * rfc);
    const float2 na2 = make_float2(na, na), nb2 = make_float2(nb, nb);
    float4* orow = reinterpret_cast<float4*>(gx + r * C);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float2 oa = fma2(lo2(gg[i]), inv2, fma2(lo2(v[i]), nb2, na2));
      float2 ob = fma2(hi2(gg[i]), inv2, fma2(hi2(v[i]), nb2, na2));
      if (ACCUM) { oa = add2(oa, lo2(rs[i])); ob = add2(ob, hi2(rs[i])); }
      if ((i * 32 + lane) * 4 < C) {
        orow[i * 32 + lane] = cat2(oa, ob);
        if (nsums == 3) {
          const float4 co = acc_o[i * 32 + lane];
          acc_o[i * 32 + lane] = cat2(add2(oa, lo2(co)), add2(ob, hi2(co)));
        }
      }
    }
  }
  // combine the warps of this CTA in warp order: one partial row per CTA and sum, part[sum][cta][C]
  __syncthreads();
  for (int c = threadIdx.x; c < nsums * C; c += blockDim.x) {
    float t = 0.0f;
    for (int k = 0; k < nw; ++k) t += sm[(size_t)k * 3 * C + c];
    part[((i64)(c / C) * gridDim.x + blockIdx.x) * C + (c % C)] = t;
  }
}

// Second stage of the fast path: add the per-CTA partial rows in a fixed order.  A 32 x 32 block owns 32 columns of one of the
// sums (blockIdx.y); its 32 row lanes each add every 32nd partial row (four loads in flight), then lane 0 adds the 32 sums in
// lane order.  out0 / out1 / out2 take dgamma, dbeta and the column sums of the stored rows.
__global__ void __launch_bounds__(1024) k_ln_partials_sum(const float* __restrict__ part, float* __restrict__ out0, float* __restrict__ out1,
                                                           float* __restrict__ out2, int ctas, int C) {
  __shared__ float sw[32][33];
  const float* p = part + (i64)blockIdx.y * ctas * C;
  float* out = blockIdx.y == 0 ? out0 : (blockIdx.y == 1 ? out1 : out2);
  int c = blockIdx.x * 32 + threadIdx.x;
  float a = 0.0f;
  if (c < C) {
    int i = threadIdx.y;
    for (; i + 96 < ctas; i += 128) {
      float a0 = p[(i64)i * C + c], a1 = p[(i64)(i + 32) * C + c], a2 = p[(i64)(i + 64) * C + c], a3 = p[(i64)(i + 96) * C + c];
      a += a0; a += a1; a += a2; a += a3;
    }
    for (; i < ctas; i += 32) a += p[(i64)i * C + c];
  }
  sw[threadIdx.y][threadIdx.x] = a;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    float ta = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) ta += sw[i][threadIdx.x];
    out[c] = ta;
  }
}

// ---- LayerNorm, generic path (any C): one block per row, rows re-read from L1/L2 ------------
__global__ void k_ln_fwd_block(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                               float* __restrict__ out, float* __restrict__ stats, i64 C, float eps) {
  __shared__ float red[32];
  const float* xr = x + (i64)blockIdx.x * C;
  float fc = (float)C;
  float s = 0.0f;
  for (i64 i = threadIdx.x; i < C; i += blockDim.x) s += xr[i];
  float mean = bsum(s, red) / fc;
  float q = 0.0f;
  for (i64 i = threadIdx.x; i < C; i += blockDim.x) { float d = xr[i] - mean; q += d * d; }
  float inv = 1.0f / sqrtf(bsum(q, red) / fc + eps);
  if (out) for (i64 i = threadIdx.x; i < C; i += blockDim.x) out[(i64)blockIdx.x * C + i] = ((xr[i] - mean) * inv) * w[i] + b[i];
  if (stats && threadIdx.x == 0) { stats[2 * (i64)blockIdx.x] = mean; stats[2 * (i64)blockIdx.x + 1] = inv; }
}
__global__ void k_ln_bwd_block(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ g,
                               const float* __restrict__ stats, float* __restrict__ gx, i64 C) {
  __shared__ float red[32];
  i64 r = blockIdx.x;
  const float* xr = x + r * C; const float* gr = g + r * C;
  float mean = stats[2 * r], inv = stats[2 * r + 1], fc = (float)C;
  float s1 = 0.0f, s2 = 0.0f;
  for (i64 i = threadIdx.x; i < C; i += blockDim.x) { float xh = (xr[i] - mean) * inv, p = gr[i] * w[i]; s1 += p; s2 += p * xh; }
  s1 = bsum(s1, red); s2 = bsum(s2, red);
  for (i64 i = threadIdx.x; i < C; i += blockDim.x) {
    float xh = (xr[i] - mean) * inv;
    gx[r * C + i] = (fc * gr[i] * w[i] - s1 - xh * s2) * inv / fc;
  }
}
__global__ void k_ln_bwd_cols(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ stats,
                              float* __restrict__ gw, float* __restrict__ gb, i64 rows, i64 C) {
  i64 c = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (c >= C) return;
  float a = 0.0f, b = 0.0f;
  for (i64 r = 0; r < rows; ++r) { float gg = g[r * C + c]; a += gg * ((x[r * C + c] - stats[2 * r]) * stats[2 * r + 1]); b += gg; }
  gw[c] = a; gb[c] = b;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
// The shared-memory strip of an instance is [8 warps][3][128 * VPT] floats: past 48 KB from VPT = 5 on.  Raised once per instance.
template <int VPT, bool ACCUM>
static cudaError_t ln_bwd_smem_attr() {
  static cudaError_t rc = cudaFuncSetAttribute(k_ln_bwd_warp<VPT, ACCUM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 128 * VPT * (int)sizeof(float));
  return rc;
}
template <bool ACCUM>
static int ln_bwd_launch(int vpt, unsigned blocks, size_t smem, cudaStream_t st, const float* x, const float* w, const float* g, const float* resid,
                         float* gx, float* part, i64 rows, int c, float eps, int nsums) {
#define LN_BWD(V) case V: \
    if (V >= 5) VB_CUDA((ln_bwd_smem_attr<V, ACCUM>())); \
    k_ln_bwd_warp<V, ACCUM><<<blocks, 256, smem, st>>>(x, w, g, resid, gx, part, rows, c, eps, nsums); break;
  switch (vpt) { LN_BWD(1) LN_BWD(2) LN_BWD(3) LN_BWD(4) LN_BWD(5) LN_BWD(6) LN_BWD(7) LN_BWD(8) }
#undef LN_BWD
  return VB_OK;
}

int launch_layernorm(const float* x, const float* w, const float* b, float* out, i64 rows, i64 c, float eps, float* out_lo, bool* lo_done) {
  if (lo_done) *lo_done = false;
  if (rows <= 0 || c <= 0) return VB_OK;
  cudaStream_t st = ctx().stream;
  bool fast = (c % 4 == 0) && c <= 1024 && al16(x) && al16(w) && al16(b) && al16(out);
  // x read, y written, and y's lo plane written where the caller asked for one
  ProfScope prof("layernorm_fwd", ((fast && out_lo && al16(out_lo)) ? 3.0 : 2.0) * (double)rows * (double)c * 4.0);
  if (fast) {
    int vpt = (int)((c + 127) / 128);
    i64 blocks = (rows + 7) / 8; i64 cap = (i64)ctx().sm_count * 8; if (blocks > cap) blocks = cap;
    float* lo = (out_lo && al16(out_lo)) ? out_lo : nullptr;
#define LN_FWD(V) case V: k_ln_fwd_warp<V><<<(unsigned)blocks, 256, 0, st>>>(x, w, b, out, rows, (int)c, eps, lo); break;
    switch (vpt) { LN_FWD(1) LN_FWD(2) LN_FWD(3) LN_FWD(4) LN_FWD(5) LN_FWD(6) LN_FWD(7) LN_FWD(8) }
#undef LN_FWD
    if (lo && lo_done) *lo_done = true;
  } else {
    int t = 32; while (t < 256 && t * 4 < c) t <<= 1;
    k_ln_fwd_block<<<(unsigned)rows, t, 0, st>>>(x, w, b, out, nullptr, c, eps);
  }
  VB_LAUNCH_CHECK();
  return VB_OK;
}

int launch_layernorm_backward(const float* x, const float* w, const float* g, float* gx, float* gw, float* gb, i64 rows, i64 c, float eps,
                              const float* resid, float* out_colsum, bool* colsum_done) {
  if (colsum_done) *colsum_done = false;
  if (c <= 0) return VB_OK;
  cudaStream_t st = ctx().stream;
  if (rows <= 0) { VB_TRY(launch_fill(gw, 0.0f, c)); return launch_fill(gb, 0.0f, c); }
  bool fast = (c % 4 == 0) && c <= 1024 && al16(x) && al16(w) && al16(g) && al16(gx) && (!resid || al16(resid));
  if (fast) {
    ProfScope prof("layernorm_bwd", (resid ? 4.0 : 3.0) * (double)rows * (double)c * 4.0);
    int vpt = (int)((c + 127) / 128);
    const int warps = 8;
    const int nsums = out_colsum ? 3 : 2;
    i64 blocks = (rows + warps - 1) / warps; i64 cap = (i64)ctx().sm_count * 2; if (blocks > cap) blocks = cap;
    size_t smem = (size_t)warps * 3 * c * sizeof(float);   // 96 KiB at C = 1024
    void* part = nullptr;
    VB_TRY(scratch_alloc((size_t)(nsums * blocks * c) * sizeof(float), &part));
    int rc = resid ? ln_bwd_launch<true>(vpt, (unsigned)blocks, smem, st, x, w, g, resid, gx, (float*)part, rows, (int)c, eps, nsums)
                   : ln_bwd_launch<false>(vpt, (unsigned)blocks, smem, st, x, w, g, nullptr, gx, (float*)part, rows, (int)c, eps, nsums);
    if (rc == VB_OK) {
      k_ln_partials_sum<<<dim3((unsigned)((c + 31) / 32), (unsigned)nsums), dim3(32, 32), 0, st>>>((const float*)part, gw, gb, out_colsum, (int)blocks, (int)c);
      if (colsum_done && out_colsum) *colsum_done = true;
    }
    scratch_free(part);
    VB_TRY(rc);
  } else {
    void* stats = nullptr;
    VB_TRY(scratch_alloc((size_t)(2 * rows) * sizeof(float), &stats));
    float* dx = gx; void* tmp = nullptr;
    if (resid) { int rc = scratch_alloc((size_t)(rows * c) * sizeof(float), &tmp); if (rc != VB_OK) { scratch_free(stats); return rc; } dx = (float*)tmp; }
    {
      ProfScope prof("layernorm_bwd", 3.0 * (double)rows * (double)c * 4.0);
      int t = 32; while (t < 256 && t * 4 < c) t <<= 1;
      k_ln_fwd_block<<<(unsigned)rows, t, 0, st>>>(x, w, w, nullptr, (float*)stats, c, eps);
      k_ln_bwd_block<<<(unsigned)rows, t, 0, st>>>(x, w, g, (const float*)stats, dx, c);
      k_ln_bwd_cols<<<(unsigned)((c + 127) / 128), 128, 0, st>>>(x, g, (const float*)stats, gw, gb, rows, c);
    }
    scratch_free(stats);
    if (resid) {
      int rc = VB_OK;
      if (gx != resid) { cudaError_t e = cudaMemcpyAsync(gx, resid, (size_t)(rows * c) * sizeof(float), cudaMemcpyDeviceToDevice, st); if (e != cudaSuccess) rc = set_error(VB_ERR_CUDA, cudaGetErrorString(e)); }
      if (rc == VB_OK) rc = launch_axpy(gx, dx, rows * c);
      scratch_free(tmp);
      VB_TRY(rc);
    }
  }
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// ---- BatchNorm2d: one CTA per channel, x is [n, c, hw] ---------------------------------------
__global__ void k_bn_fwd(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                         float* __restrict__ rm, float* __restrict__ rv, float* __restrict__ out,
                         i64 n, i64 c, i64 hw, bool training, float momentum, float eps) {
  __shared__ float red[32];
  i64 cc = blockIdx.x;
  i64 cnt = n * hw;
  float m = (float)cnt;
  float mean, var;
  if (training) {
    float s = 0.0f;
    for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) s += x[((i / hw) * c + cc) * hw + i % hw];
    mean = bsum(s, red) / m;
    float q = 0.0f;
    for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) { float d = x[((i / hw) * c + cc) * hw + i % hw] - mean; q += d * d; }
    var = bsum(q, red) / m;
    if (threadIdx.x == 0) {
      float bessel = m > 1.0f ? m / (m - 1.0f) : 1.0f;
      rm[cc] = (1.0f - momentum) * rm[cc] + momentum * mean;
      rv[cc] = (1.0f - momentum) * rv[cc] + momentum * var * bessel;
    }
  } else { mean = rm[cc]; var = rv[cc]; }
  float inv = 1.0f / sqrtf(var + eps), ga = gamma[cc], be = beta[cc];
  for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) {
    i64 idx = ((i / hw) * c + cc) * hw + i % hw;
    out[idx] = ((x[idx] - mean) * inv) * ga + be;
  }
}
int launch_batchnorm(const float* x, const float* gamma, const float* beta, float* rm, float* rv, float* out,
                     i64 n, i64 c, i64 hw, bool training, float momentum, float eps) {
  if (n * c * hw <= 0) return VB_OK;
  k_bn_fwd<<<(unsigned)c, 1024, 0, ctx().stream>>>(x, gamma, beta, rm, rv, out, n, c, hw, training, momentum, eps);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void k_bn_bwd(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ rm, const float* __restrict__ rv,
                         const float* __restrict__ g, float* __restrict__ gx, float* __restrict__ gw, float* __restrict__ gb,
                         i64 n, i64 c, i64 hw, bool training, float eps) {
  __shared__ float red[32];
  i64 cc = blockIdx.x;
  i64 cnt = n * hw;
  float m = (float)cnt;
  float mean, var;
  if (training) {
    float s = 0.0f;
    for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) s += x[((i / hw) * c + cc) * hw + i % hw];
    mean = bsum(s, red) / m;
    float q = 0.0f;
    for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) { float d = x[((i / hw) * c + cc) * hw + i % hw] - mean; q += d * d; }
    var = bsum(q, red) / m;
  } else { mean = rm[cc]; var = rv[cc]; }
  float inv = 1.0f / sqrtf(var + eps);
  float sdy = 0.0f, sdyx = 0.0f;
  for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) {
    i64 idx = ((i / hw) * c + cc) * hw + i % hw;
    float dy = g[idx];
    sdy += dy; sdyx += dy * ((x[idx] - mean) * inv);
  }
  sdy = bsum(sdy, red); sdyx = bsum(sdyx, red);
  if (threadIdx.x == 0) { gb[cc] = sdy; gw[cc] = sdyx; }
  float ga = gamma[cc];
  for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) {
    i64 idx = ((i / hw) * c + cc) * hw + i % hw;
    float dy = g[idx];
    if (training) { float xh = (x[idx] - mean) * inv; gx[idx] = (ga * inv / m) * (m * dy - sdy - xh * sdyx); }
    else gx[idx] = dy * ga * inv;
  }
}
int launch_batchnorm_backward(const float* x, const float* gamma, const float* rm, const float* rv, const float* g,
                              float* gx, float* gw, float* gb, i64 n, i64 c, i64 hw, bool training, float eps) {
  if (c <= 0) return VB_OK;
  if (n * hw <= 0) { VB_TRY(launch_fill(gw, 0.0f, c)); return launch_fill(gb, 0.0f, c); }
  k_bn_bwd<<<(unsigned)c, 1024, 0, ctx().stream>>>(x, gamma, rm, rv, g, gx, gw, gb, n, c, hw, training, eps);
  VB_LAUNCH_CHECK();
  return VB_OK;
}


// ---- LayerNorm backward without any allocation --------------------------------------------------
// Some callers cannot allocate device memory at the point where they need this kernel: code that
// runs inside a region where the allocator is off limits (a framework's capture or replay phase, a
// real-time loop with a fixed memory budget, a plugin that was handed buffers and nothing else).
// The regular entry point takes per-CTA partial sums of dgamma / dbeta from the arena; this variant
// keeps them in a fixed array that is part of the library image instead.  The array is sized for
// C <= 1024 and at most 296 CTAs: 2 * 296 * 1024 floats = 2.4 MB, resident on every GPU that loads
// the library, for as long as the process lives.
namespace {
constexpr int kNoAllocMaxC = 1024;
constexpr int kNoAllocMaxCtas = 296;
static __device__ __align__(256) float g_ln_bwd_noalloc_scratch[2 * kNoAllocMaxCtas * kNoAllocMaxC];

// The array's name is only meaningful in device code; host code needs its device address, looked up
// once per device with that device current.
struct NoAllocDevice { bool ready = false; float* scratch = nullptr; int sm_count = 0; };
NoAllocDevice g_noalloc_dev[64];

__global__ void k_ln_noalloc_finish(const float* __restrict__ part_w, const float* __restrict__ part_b,
                                    float* __restrict__ gw, float* __restrict__ gb, int ctas, int C) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float a = 0.0f, b = 0.0f;
  for (int i = 0; i < ctas; ++i) { a += part_w[(i64)i * C + c]; b += part_b[(i64)i * C + c]; }
  gw[c] = a; gb[c] = b;
}
__global__ void k_ln_noalloc_zero(float* gw, float* gb, int C) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) { gw[c] = 0.0f; gb[c] = 0.0f; }
}
}  // namespace
}  // namespace vb

extern "C" int vb_layernorm_backward_noalloc(const float* x, const float* w, const float* grad_out, float* gx, float* gw, float* gb,
                                             int64_t rows, int64_t c, float eps, void* stream) {
  using namespace vb;
  if (!x || !w || !grad_out || !gx || !gw || !gb) return set_error(VB_ERR_INVALID, "vb_layernorm_backward_noalloc: null pointer");
  if (rows < 0 || c <= 0) return set_error(VB_ERR_INVALID, "vb_layernorm_backward_noalloc: bad shape");
  if (c > kNoAllocMaxC || (c & 3))
    return set_error(VB_ERR_UNSUPPORTED, "vb_layernorm_backward_noalloc: the row length must be a multiple of 4 and at most 1024 "
                                         "(the fixed scratch array is sized for that); use vb_layernorm_backward for other sizes");
  if (!al16(x) || !al16(w) || !al16(grad_out) || !al16(gx))
    return set_error(VB_ERR_UNSUPPORTED, "vb_layernorm_backward_noalloc: x, w, grad_out and gx must be 16-byte aligned");
  int dev = 0;
  VB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(VB_ERR_UNSUPPORTED, "vb_layernorm_backward_noalloc: device ordinal out of range");
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (!d.ready) {   // first call on this device: resolve the array's device address (not capturable; do it before any stream capture)
    float* p = nullptr;
    VB_CUDA(cudaGetSymbolAddress((void**)&p, g_ln_bwd_noalloc_scratch));
    VB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    // rows of more than 512 floats need more than the default 48 KB of shared memory: raise those instances' limit once, here
    VB_CUDA((ln_bwd_smem_attr<5, false>())); VB_CUDA((ln_bwd_smem_attr<6, false>()));
    VB_CUDA((ln_bwd_smem_attr<7, false>())); VB_CUDA((ln_bwd_smem_attr<8, false>()));
    d.scratch = p; d.ready = true;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int C = (int)c;
  if (rows == 0) {
    k_ln_noalloc_zero<<<(C + 255) / 256, 256, 0, st>>>(gw, gb, C);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
  }
  const int warps = 8;
  i64 ctas = (rows + warps - 1) / warps;
  i64 cap = (i64)d.sm_count * 2; if (cap > kNoAllocMaxCtas) cap = kNoAllocMaxCtas;
  if (ctas > cap) ctas = cap;
  // every CTA overwrites its own partial row in full, so nothing in the array needs clearing first
  float* pw = d.scratch; float* pb = d.scratch + (size_t)ctas * C;       // the kernel's layout: [sum][cta][C], two sums here
  size_t smem = (size_t)warps * 3 * C * sizeof(float);
  int vpt = (C + 127) / 128;
#define LN_BWD_NA(V) case V: \
    k_ln_bwd_warp<V, false><<<(unsigned)ctas, warps * 32, smem, st>>>(x, w, grad_out, nullptr, gx, pw, rows, C, eps, 2); break;
  switch (vpt) { LN_BWD_NA(1) LN_BWD_NA(2) LN_BWD_NA(3) LN_BWD_NA(4) LN_BWD_NA(5) LN_BWD_NA(6) LN_BWD_NA(7) LN_BWD_NA(8) }
#undef LN_BWD_NA
  k_ln_noalloc_finish<<<(C + 127) / 128, 128, 0, st>>>(pw, pb, gw, gb, (int)ctas, C);
  VB_CUDA(cudaGetLastError());
  return VB_OK;
}
