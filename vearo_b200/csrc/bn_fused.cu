// Fused BatchNorm2d -> ReLU -> MaxPool(2, 2, 0), forward and backward, for NCHW tensors.
//
// Semantics are the composition of the three reference ops (crates/vearo-backend-cpu/src/lib.rs: batchnorm
// 2067-2364 with biased batch variance and the Bessel-corrected running variance 2141-2148; relu 424-454 and its
// gradient mask x > 0, crates/vearo-autograd/src/lib.rs:364-374; max-pool 1797-1948: the FIRST maximum of a window in
// (i, j) scan order receives the gradient, strict >).  What changes is the traffic: the normalised tensor, the
// rectified tensor and their gradients never exist in memory.
//
//   forward   x is read twice (statistics, apply), the pooled quarter-size output is written once
//   backward  x twice and the pooled gradient twice (channel sums, apply), dx written once
//
// A channel is spread over several CTAs so that 64-256 channels fill 148 SMs.  Channel statistics: every CTA
// computes (count, mean, M2) of its share in two passes over it (the second hits L2), and the shares are merged in a
// fixed order with Chan's formula; the backward's two channel sums are per-CTA partial sums added in CTA order.
// Everything is bit-reproducible (no atomics).
#include "common.h"

namespace vb {
namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __shared__ float bcast;
  if (threadIdx.x == 0) bcast = r;
  __syncthreads();
  return bcast;
}

// grid (c, splits): images [i0, i1) of channel cc.  part[(cc*splits + s)*3 + {0,1,2}] = count, mean, M2.
__global__ void __launch_bounds__(256) k_bn_stats_partial(const float* __restrict__ x, float* __restrict__ part, i64 n, i64 c, i64 hw, i64 imgs_per_split) {
  __shared__ float red[32];
  const i64 cc = blockIdx.x, s = blockIdx.y, splits = gridDim.y;
  i64 i0 = s * imgs_per_split, i1 = i0 + imgs_per_split; if (i1 > n) i1 = n; if (i0 > n) i0 = n;
  const i64 cnt = (i1 - i0) * hw;
  float sum = 0.0f;
  for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) sum += x[((i0 + i / hw) * c + cc) * hw + i % hw];
  sum = block_sum(sum, red);
  const float mean = cnt > 0 ? sum / (float)cnt : 0.0f;
  float q = 0.0f;
  for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) { float d = x[((i0 + i / hw) * c + cc) * hw + i % hw] - mean; q += d * d; }
  q = block_sum(q, red);
  if (threadIdx.x == 0) { float* o = part + (cc * splits + s) * 3; o[0] = (float)cnt; o[1] = mean; o[2] = q; }
}
// One thread per channel: merge the shares in order; stats[cc] = mean, stats[c + cc] = 1/sqrt(var + eps); running statistics.
__global__ void k_bn_stats_final(const float* __restrict__ part, float* __restrict__ stats, float* __restrict__ rm, float* __restrict__ rv,
                                 i64 c, int splits, bool training, float momentum, float eps) {
  i64 cc = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (cc >= c) return;
  float mean, var;
  if (training) {
    float na = 0.0f, ma = 0.0f, qa = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float* o = part + (cc * splits + s) * 3;
      float nb = o[0], mb = o[1], qb = o[2];
      if (nb == 0.0f) continue;
      float nt = na + nb, d = mb - ma;
      ma += d * (nb / nt);
      qa += qb + d * d * (na * nb / nt);
      na = nt;
    }
    mean = ma; var = na > 0.0f ? qa / na : 0.0f;
    float bessel = na > 1.0f ? na / (na - 1.0f) : 1.0f;
    rm[cc] = (1.0f - momentum) * rm[cc] + momentum * mean;
    rv[cc] = (1.0f - momentum) * rv[cc] + momentum * var * bessel;
  } else { mean = rm[cc]; var = rv[cc]; }
  stats[cc] = mean; stats[c + cc] = 1.0f / sqrtf(var + eps);
}
// The four taps of a 2 x 2 window of y = relu(bn(x)) and the index (0..3, scan order) of the first maximum.
struct Window { float xh[4]; float y[4]; int arg; };
__device__ __forceinline__ Window window_of(const float* __restrict__ xp, i64 w, float mean, float inv, float ga, float be) {
  Window r;
  float2 a = *reinterpret_cast<const float2*>(xp), b = *reinterpret_cast<const float2*>(xp + w);
  float v[4] = {a.x, a.y, b.x, b.y};
  float best = 0.0f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    r.xh[t] = (v[t] - mean) * inv;
    float z = r.xh[t] * ga + be;
    r.y[t] = z > 0.0f ? z : 0.0f;
    if (t == 0 || r.y[t] > best) { best = r.y[t]; r.arg = t; }
  }
  return r;
}
__device__ __forceinline__ Window window_of_unaligned(const float* __restrict__ xp, i64 w, float mean, float inv, float ga, float be) {
  Window r;
  float v[4] = {xp[0], xp[1], xp[w], xp[w + 1]};
  float best = 0.0f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    r.xh[t] = (v[t] - mean) * inv;
    float z = r.xh[t] * ga + be;
    r.y[t] = z > 0.0f ? z : 0.0f;
    if (t == 0 || r.y[t] > best) { best = r.y[t]; r.arg = t; }
  }
  return r;
}
// One thread per pooled output.
__global__ void k_bn_relu_pool_fwd(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                   const float* __restrict__ stats, float* __restrict__ out, i64 n, i64 c, i64 h, i64 w, i64 oh, i64 ow, bool even_w) {
  i64 total = n * c * oh * ow;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 ox = idx % ow, oy = (idx / ow) % oh, cc = (idx / (ow * oh)) % c, nn = idx / (ow * oh * c);
    const float* xp = x + ((nn * c + cc) * h + 2 * oy) * w + 2 * ox;
    Window wd = even_w ? window_of(xp, w, stats[cc], stats[c + cc], gamma[cc], beta[cc]) : window_of_unaligned(xp, w, stats[cc], stats[c + cc], gamma[cc], beta[cc]);
    out[idx] = wd.y[wd.arg];
  }
}
// grid (c, splits): channel sums of dy and dy * xhat over the windows of images [i0, i1), dy being the pooled gradient
// routed to the first maximum and masked by the rectifier.  part[(cc*splits + s)*2 + {0,1}].
__global__ void __launch_bounds__(256) k_bn_pool_bwd_partial(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                             const float* __restrict__ stats, const float* __restrict__ g, float* __restrict__ part,
                                                             i64 n, i64 c, i64 h, i64 w, i64 oh, i64 ow, i64 imgs_per_split, bool even_w) {
  __shared__ float red[32];
  const i64 cc = blockIdx.x, s = blockIdx.y, splits = gridDim.y;
  i64 i0 = s * imgs_per_split, i1 = i0 + imgs_per_split; if (i1 > n) i1 = n; if (i0 > n) i0 = n;
  const i64 ohw = oh * ow, cnt = (i1 - i0) * ohw;
  const float mean = stats[cc], inv = stats[c + cc], ga = gamma[cc], be = beta[cc];
  float sdy = 0.0f, sdyx = 0.0f;
  for (i64 i = threadIdx.x; i < cnt; i += blockDim.x) {
    i64 nn = i0 + i / ohw, p = i % ohw, oy = p / ow, ox = p % ow;
    const float* xp = x + ((nn * c + cc) * h + 2 * oy) * w + 2 * ox;
    Window wd = even_w ? window_of(xp, w, mean, inv, ga, be) : window_of_unaligned(xp, w, mean, inv, ga, be);
    if (wd.y[wd.arg] > 0.0f) { float dy = g[(nn * c + cc) * ohw + p]; sdy += dy; sdyx += dy * wd.xh[wd.arg]; }
  }
  sdy = block_sum(sdy, red); sdyx = block_sum(sdyx, red);
  if (threadIdx.x == 0) { part[(cc * splits + s) * 2] = sdy; part[(cc * splits + s) * 2 + 1] = sdyx; }
}
__global__ void k_bn_pool_bwd_final(const float* __restrict__ part, float* __restrict__ gw, float* __restrict__ gb, i64 c, int splits) {
  i64 cc = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (cc >= c) return;
  float a = 0.0f, b = 0.0f;
  for (int s = 0; s < splits; ++s) { a += part[(cc * splits + s) * 2]; b += part[(cc * splits + s) * 2 + 1]; }
  gb[cc] = a; gw[cc] = b;
}
// One thread per 2 x 2 block of the input (blocks cut by an odd height or width included: their elements belong to no
// window and only carry the batch-statistics terms of the gradient).
__global__ void k_bn_pool_bwd_apply(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                    const float* __restrict__ stats, const float* __restrict__ g, const float* __restrict__ gw, const float* __restrict__ gb,
                                    float* __restrict__ gx, i64 n, i64 c, i64 h, i64 w, i64 oh, i64 ow, bool training) {
  const i64 bh = (h + 1) / 2, bw = (w + 1) / 2;
  i64 total = n * c * bh * bw;
  const float m = (float)(n * h * w);
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 bx = idx % bw, by = (idx / bw) % bh, cc = (idx / (bw * bh)) % c, nn = idx / (bw * bh * c);
    const float mean = stats[cc], inv = stats[c + cc], ga = gamma[cc], be = beta[cc];
    const float sdy = gb[cc], sdyx = gw[cc];
    const i64 base = ((nn * c + cc) * h + 2 * by) * w + 2 * bx;
    const bool full = by < oh && bx < ow;      // a pooling window (2*by+1 < h and 2*bx+1 < w follow from oh, ow)
    int arg = -1; float gv = 0.0f;
    if (full) {
      Window wd = window_of_unaligned(x + base, w, mean, inv, ga, be);
      if (wd.y[wd.arg] > 0.0f) { arg = wd.arg; gv = g[((nn * c + cc) * oh + by) * ow + bx]; }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      i64 yy = 2 * by + (t >> 1), xx = 2 * bx + (t & 1);
      if (yy >= h || xx >= w) continue;
      i64 e = base + (t >> 1) * w + (t & 1);
      float dy = t == arg ? gv : 0.0f;
      if (training) { float xh = (x[e] - mean) * inv; gx[e] = (ga * inv / m) * (m * dy - sdy - xh * sdyx); }
      else gx[e] = dy * ga * inv;
    }
  }
}

i64 pick_splits(i64 c, i64 n) {
  i64 want = ((i64)ctx().sm_count * 4 + c - 1) / c;
  if (want > n) want = n;
  if (want < 1) want = 1;
  return want;
}

}  // namespace

// stats: [2, c] (mean, 1/sqrt(var + eps)), written here and read by the backward.
int launch_bn_relu_maxpool(const float* x, const float* gamma, const float* beta, float* rm, float* rv, float* stats, float* out,
                           i64 n, i64 c, i64 h, i64 w, bool training, float momentum, float eps) {
  if (n * c * h * w <= 0) return VB_OK;
  cudaStream_t st = ctx().stream;
  const i64 oh = h / 2, ow = w / 2;
  i64 splits = pick_splits(c, n), ips = (n + splits - 1) / splits;
  splits = (n + ips - 1) / ips;
  Temp part;
  {
    ProfScope prof("bn_stats", (double)(n * c * h * w) * 4.0);
    if (training) {
      VB_TRY(scratch_alloc((size_t)(c * splits * 3) * sizeof(float), &part.p));
      k_bn_stats_partial<<<dim3((unsigned)c, (unsigned)splits), 256, 0, st>>>(x, (float*)part.p, n, c, h * w, ips);
    }
    k_bn_stats_final<<<(unsigned)((c + 127) / 128), 128, 0, st>>>((const float*)part.p, stats, rm, rv, c, (int)splits, training, momentum, eps);
    VB_LAUNCH_CHECK();
  }
  i64 total = n * c * oh * ow;
  if (total > 0) {
    ProfScope prof("bn_relu_pool_fwd", (double)(n * c * h * w) * 4.0 + (double)total * 4.0);
    i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32; if (blocks > cap) blocks = cap;
    k_bn_relu_pool_fwd<<<(unsigned)blocks, 256, 0, st>>>(x, gamma, beta, stats, out, n, c, h, w, oh, ow, (w & 1) == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0);
    VB_LAUNCH_CHECK();
  }
  return VB_OK;
}

int launch_bn_relu_maxpool_backward(const float* x, const float* gamma, const float* beta, const float* stats, const float* g,
                                    float* gx, float* gw, float* gb, i64 n, i64 c, i64 h, i64 w, bool training) {
  if (c <= 0) return VB_OK;
  if (n * h * w <= 0) { VB_TRY(launch_fill(gw, 0.0f, c)); return launch_fill(gb, 0.0f, c); }
  cudaStream_t st = ctx().stream;
  const i64 oh = h / 2, ow = w / 2;
  i64 splits = pick_splits(c, n), ips = (n + splits - 1) / splits;
  splits = (n + ips - 1) / ips;
  Temp part;
  VB_TRY(scratch_alloc((size_t)(c * splits * 2) * sizeof(float), &part.p));
  const bool even_w = (w & 1) == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0;
  {
    ProfScope prof("bn_relu_pool_bwd_sums", (double)(n * c * h * w) * 4.0 + (double)(n * c * oh * ow) * 4.0);
    k_bn_pool_bwd_partial<<<dim3((unsigned)c, (unsigned)splits), 256, 0, st>>>(x, gamma, beta, stats, g, (float*)part.p, n, c, h, w, oh, ow, ips, even_w);
    k_bn_pool_bwd_final<<<(unsigned)((c + 127) / 128), 128, 0, st>>>((const float*)part.p, gw, gb, c, (int)splits);
    VB_LAUNCH_CHECK();
  }
  {
    ProfScope prof("bn_relu_pool_bwd_apply", 2.0 * (double)(n * c * h * w) * 4.0 + (double)(n * c * oh * ow) * 4.0);
    i64 total = n * c * ((h + 1) / 2) * ((w + 1) / 2);
    i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32; if (blocks > cap) blocks = cap;
    k_bn_pool_bwd_apply<<<(unsigned)blocks, 256, 0, st>>>(x, gamma, beta, stats, g, gw, gb, gx, n, c, h, w, oh, ow, training);
    VB_LAUNCH_CHECK();
  }
  return VB_OK;
}

}  // namespace vb
