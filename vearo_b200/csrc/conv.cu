// Direct NCHW convolution (forward, and the three backward products) and 2-D pooling.
//
// Semantics: crates/vearo-backend-cpu/src/lib.rs:1474-2058.  Forward: each output starts at the
// bias and accumulates taps in (c, i, j) order with fused multiply-adds, the order of the CPU
// backend; padded taps contribute nothing.  Max-pool keeps the FIRST maximum in (i, j) scan order
// (strict >) and never selects a padded tap; average-pool divides by the number of valid taps.
// All kernels are gather formulations: no atomics, bit-reproducible.
#include "common.h"

namespace vb {

__global__ void k_conv2d_fwd(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float* __restrict__ out,
                             i64 n, i64 cin, i64 h, i64 wd, i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad) {
  i64 total = n * cout * oh * ow;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 xo = idx % ow, y = (idx / ow) % oh, co = (idx / (ow * oh)) % cout, nn = idx / (ow * oh * cout);
    float acc = b[co];
    for (i64 c = 0; c < cin; ++c)
      for (i64 i = 0; i < kh; ++i) {
        i64 ih = y * stride + i - pad;
        if (ih < 0 || ih >= h) continue;
        for (i64 j = 0; j < kw; ++j) {
          i64 iw = xo * stride + j - pad;
          if (iw < 0 || iw >= wd) continue;
          acc = fmaf(w[((co * cin + c) * kh + i) * kw + j], x[((nn * cin + c) * h + ih) * wd + iw], acc);
        }
      }
    out[idx] = acc;
  }
}
int launch_conv2d(const float* x, const float* w, const float* b, float* out, i64 n, i64 cin, i64 h, i64 wd,
                  i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad) {
  i64 total = n * cout * oh * ow;
  if (total <= 0) return VB_OK;
  i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32; if (blocks > cap) blocks = cap;
  k_conv2d_fwd<<<(unsigned)blocks, 256, 0, ctx().stream>>>(x, w, b, out, n, cin, h, wd, cout, kh, kw, oh, ow, stride, pad);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

__device__ __forceinline__ float bsum_c(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}
// db[co] = sum over n, y, x of g
__global__ void k_conv2d_bwd_bias(const float* __restrict__ g, float* __restrict__ gb, i64 n, i64 cout, i64 ohw) {
  __shared__ float red[32];
  i64 co = blockIdx.x;
  float s = 0.0f;
  for (i64 i = threadIdx.x; i < n * ohw; i += blockDim.x) s += g[((i / ohw) * cout + co) * ohw + i % ohw];
  s = bsum_c(s, red);
  if (threadIdx.x == 0) gb[co] = s;
}
// dW[co,c,i,j] = sum over n, y, x of g[n,co,y,x] * x_pad[n,c,y*s+i,x*s+j]; one CTA per weight.
__global__ void k_conv2d_bwd_weight(const float* __restrict__ x, const float* __restrict__ g, float* __restrict__ gw,
                                    i64 n, i64 cin, i64 h, i64 wd, i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad) {
  __shared__ float red[32];
  i64 widx = blockIdx.x;
  i64 j = widx % kw, i = (widx / kw) % kh, c = (widx / (kw * kh)) % cin, co = widx / (kw * kh * cin);
  i64 ohw = oh * ow;
  float s = 0.0f;
  for (i64 t = threadIdx.x; t < n * ohw; t += blockDim.x) {
    i64 nn = t / ohw, y = (t % ohw) / ow, xo = t % ow;
    i64 ih = y * stride + i - pad, iw = xo * stride + j - pad;
    if (ih < 0 || ih >= h || iw < 0 || iw >= wd) continue;
    s = fmaf(g[(nn * cout + co) * ohw + y * ow + xo], x[((nn * cin + c) * h + ih) * wd + iw], s);
  }
  s = bsum_c(s, red);
  if (threadIdx.x == 0) gw[widx] = s;
}
// dX[n,c,ih,iw] = sum over co, i, j of g[n,co,y,x] * w[co,c,i,j] with y*s + i - pad = ih, x*s + j - pad = iw
__global__ void k_conv2d_bwd_input(const float* __restrict__ w, const float* __restrict__ g, float* __restrict__ gx,
                                   i64 n, i64 cin, i64 h, i64 wd, i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad) {
  i64 total = n * cin * h * wd;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 iw = idx % wd, ih = (idx / wd) % h, c = (idx / (wd * h)) % cin, nn = idx / (wd * h * cin);
    float acc = 0.0f;
    for (i64 co = 0; co < cout; ++co)
      for (i64 i = 0; i < kh; ++i) {
        i64 ty = ih + pad - i;
        if (ty < 0 || ty % stride) continue;
        i64 y = ty / stride; if (y >= oh) continue;
        for (i64 j = 0; j < kw; ++j) {
          i64 tx = iw + pad - j;
          if (tx < 0 || tx % stride) continue;
          i64 xo = tx / stride; if (xo >= ow) continue;
          acc = fmaf(g[((nn * cout + co) * oh + y) * ow + xo], w[((co * cin + c) * kh + i) * kw + j], acc);
        }
      }
    gx[idx] = acc;
  }
}
int launch_conv2d_backward(const float* x, const float* w, const float* g, float* gx, float* gw, float* gb,
                           i64 n, i64 cin, i64 h, i64 wd, i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad) {
  cudaStream_t st = ctx().stream;
  if (cout > 0) k_conv2d_bwd_bias<<<(unsigned)cout, 256, 0, st>>>(g, gb, n, cout, oh * ow);
  i64 nw = cout * cin * kh * kw;
  if (nw > 0) k_conv2d_bwd_weight<<<(unsigned)nw, 256, 0, st>>>(x, g, gw, n, cin, h, wd, cout, kh, kw, oh, ow, stride, pad);
  i64 total = n * cin * h * wd;
  if (total > 0) {
    i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32; if (blocks > cap) blocks = cap;
    k_conv2d_bwd_input<<<(unsigned)blocks, 256, 0, st>>>(w, g, gx, n, cin, h, wd, cout, kh, kw, oh, ow, stride, pad);
  }
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// ---- pooling ---------------------------------------------------------------------------------
__global__ void k_maxpool_fwd(const float* __restrict__ x, float* __restrict__ out, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  i64 total = nc * oh * ow;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 xo = idx % ow, y = (idx / ow) % oh, c = idx / (ow * oh);
    float best = -INFINITY;
    for (i64 i = 0; i < k; ++i) {
      i64 ih = y * s + i - p; if (ih < 0 || ih >= h) continue;
      for (i64 j = 0; j < k; ++j) {
        i64 iw = xo * s + j - p; if (iw < 0 || iw >= w) continue;
        float v = x[(c * h + ih) * w + iw];
        if (v > best) best = v;
      }
    }
    out[idx] = best;
  }
}
// Gather form of the backward: an input element collects g from every window whose first maximum it is.
__global__ void k_maxpool_bwd(const float* __restrict__ x, const float* __restrict__ g, float* __restrict__ gx,
                              i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  i64 total = nc * h * w;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 iw0 = idx % w, ih0 = (idx / w) % h, c = idx / (w * h);
    float acc = 0.0f;
    // windows (y, xo) that cover (ih0, iw0), visited in (y, xo) order
    i64 y_lo = ih0 + p - k + 1; y_lo = y_lo <= 0 ? 0 : (y_lo + s - 1) / s;
    i64 x_lo = iw0 + p - k + 1; x_lo = x_lo <= 0 ? 0 : (x_lo + s - 1) / s;
    for (i64 y = y_lo; y < oh && y * s <= ih0 + p; ++y)
      for (i64 xo = x_lo; xo < ow && xo * s <= iw0 + p; ++xo) {
        float best = -INFINITY; i64 bi = -1;
        for (i64 i = 0; i < k; ++i) {
          i64 ih = y * s + i - p; if (ih < 0 || ih >= h) continue;
          for (i64 j = 0; j < k; ++j) {
            i64 iw = xo * s + j - p; if (iw < 0 || iw >= w) continue;
            float v = x[(c * h + ih) * w + iw];
            if (v > best) { best = v; bi = ih * w + iw; }
          }
        }
        if (bi == ih0 * w + iw0) acc += g[(c * oh + y) * ow + xo];
      }
    gx[idx] = acc;
  }
}
__global__ void k_avgpool_fwd(const float* __restrict__ x, float* __restrict__ out, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  i64 total = nc * oh * ow;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 xo = idx % ow, y = (idx / ow) % oh, c = idx / (ow * oh);
    float sum = 0.0f; int cnt = 0;
    for (i64 i = 0; i < k; ++i) {
      i64 ih = y * s + i - p; if (ih < 0 || ih >= h) continue;
      for (i64 j = 0; j < k; ++j) {
        i64 iw = xo * s + j - p; if (iw < 0 || iw >= w) continue;
        sum += x[(c * h + ih) * w + iw]; ++cnt;
      }
    }
    out[idx] = sum / (float)cnt;
  }
}
__device__ __forceinline__ int valid_taps(i64 o, i64 s, i64 p, i64 k, i64 lim) {
  int cnt = 0;
  for (i64 i = 0; i < k; ++i) { i64 v = o * s + i - p; if (v >= 0 && v < lim) ++cnt; }
  return cnt;
}
__global__ void k_avgpool_bwd(const float* __restrict__ g, float* __restrict__ gx, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  i64 total = nc * h * w;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 iw0 = idx % w, ih0 = (idx / w) % h, c = idx / (w * h);
    float acc = 0.0f;
    i64 y_lo = ih0 + p - k + 1; y_lo = y_lo <= 0 ? 0 : (y_lo + s - 1) / s;
    i64 x_lo = iw0 + p - k + 1; x_lo = x_lo <= 0 ? 0 : (x_lo + s - 1) / s;
    for (i64 y = y_lo; y < oh && y * s <= ih0 + p; ++y)
      for (i64 xo = x_lo; xo < ow && xo * s <= iw0 + p; ++xo) {
        int cnt = valid_taps(y, s, p, k, h) * valid_taps(xo, s, p, k, w);
        acc += g[(c * oh + y) * ow + xo] / (float)cnt;
      }
    gx[idx] = acc;
  }
}
static inline unsigned pool_grid(i64 total) {
  i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32;
  if (blocks > cap) blocks = cap; if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}
int launch_maxpool2d(const float* x, float* out, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  if (nc * oh * ow <= 0) return VB_OK;
  k_maxpool_fwd<<<pool_grid(nc * oh * ow), 256, 0, ctx().stream>>>(x, out, nc, h, w, oh, ow, k, s, p);
  VB_LAUNCH_CHECK(); return VB_OK;
}
int launch_maxpool2d_backward(const float* x, const float* g, float* gx, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  if (nc * h * w <= 0) return VB_OK;
  k_maxpool_bwd<<<pool_grid(nc * h * w), 256, 0, ctx().stream>>>(x, g, gx, nc, h, w, oh, ow, k, s, p);
  VB_LAUNCH_CHECK(); return VB_OK;
}
int launch_avgpool2d(const float* x, float* out, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  if (nc * oh * ow <= 0) return VB_OK;
  k_avgpool_fwd<<<pool_grid(nc * oh * ow), 256, 0, ctx().stream>>>(x, out, nc, h, w, oh, ow, k, s, p);
  VB_LAUNCH_CHECK(); return VB_OK;
}
int launch_avgpool2d_backward(const float* g, float* gx, i64 nc, i64 h, i64 w, i64 oh, i64 ow, i64 k, i64 s, i64 p) {
  if (nc * h * w <= 0) return VB_OK;
  k_avgpool_bwd<<<pool_grid(nc * h * w), 256, 0, ctx().stream>>>(g, gx, nc, h, w, oh, ow, k, s, p);
  VB_LAUNCH_CHECK(); return VB_OK;
}

}  // namespace vb
