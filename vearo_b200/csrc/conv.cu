// Direct NCHW convolution (forward, and the three backward products) and 2-D pooling.
//
// Semantics: crates/vearo-backend-cpu/src/lib.rs:1474-2058.  Forward: each output starts at the
// bias and accumulates taps in (c, i, j) order with fused multiply-adds, the order of the CPU
// backend; padded taps contribute nothing.  Max-pool keeps the FIRST maximum in (i, j) scan order
// (strict >) and never selects a padded tap; average-pool divides by the number of valid taps.
// All kernels are gather formulations: no atomics, bit-reproducible.
//
// 3 x 3, stride-1, padding-1 convolutions over a multiple of 32 channels are IMPLICIT GEMMs on the tensor cores: the input
// (or, for the input gradient, the output gradient) is copied once into a zero-padded channels-last buffer [N, H+2, W+2, C],
// and the unfolded matrix cols[(n,y,x), (i,j,c)] = xp[n, y+i, x+j, c] is never written: because a tap row's (j, c) entries
// are contiguous in that buffer, the whole matrix is one 5-D tensor map over it, and the GEMM's TMA boxes are its tiles.
//   forward         out[n] [Cout, HW]   = Wr [Cout, 9 Cin] . cols[n]^T           (Wr = weights in (i, j, c) order)
//   input gradient  dX[n]  [Cin, HW]    = Wf [Cin, 9 Cout] . cols_g[n]^T         (cols_g over the padded gradient, Wf = flipped, transposed weights)
//   weight gradient dWr    [Cout, 9 Cin] = g^T [Cout, N HW] . cols                (K = all pixels of all images)
// NCHW stays at the interface: results land in NCHW straight from the GEMM epilogue (dW through a reorder of 9 Cin columns).
// Other convolutions with enough work unfold explicitly: the padded input windows are written into a
// [N*OH*OW, Cin*KH*KW] matrix (rows padded to a multiple of 4 floats) and the three products become GEMMs of the
// FP32-accurate tcgen05 kernel -- forward  out[n] = W . cols[n]^T + b  (batched over images, written straight in
// NCHW with a per-row bias), input gradient  dcols[n] = g[n]^T . W  folded back by a gather, weight gradient
// dW = g^T . cols  as one long-K product over all images (g transposed to [N*OH*OW, Cout] first).  Summation order
// differs from the direct kernels; results agree with them to FP32 rounding.
#include "common.h"
#include <cstdlib>

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
// ---- unfold / fold and the GEMM formulation ---------------------------------------------------------------------
// cols[(n, y, x), (c, i, j)] = x_pad[n, c, y*s + i - p, x*s + j - p]; row length kp >= cin*kh*kw (a multiple of 4), the tail
// is zero.  One thread writes four consecutive taps of a row (one 16-byte store); index arithmetic in 32 bits.
__global__ void k_im2col(const float* __restrict__ x, float* __restrict__ cols, int n, int cin, int h, int wd, int kh, int kw,
                         int oh, int ow, int stride, int pad, int kc, int kp) {
  const int kq = kp >> 2, khw = kh * kw;
  const i64 total = (i64)n * oh * ow * kq;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const int q = (int)(idx % kq); const i64 r = idx / kq;
    const int xo = (int)(r % ow); const i64 r2 = r / ow;
    const int y = (int)(r2 % oh), nn = (int)(r2 / oh);
    float v[4];
    int k = q * 4, c = k / khw, rem = k - c * khw, i = rem / kw, j = rem - i * kw;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float e = 0.0f;
      if (k < kc) {
        int ih = y * stride + i - pad, iw = xo * stride + j - pad;
        if (ih >= 0 && ih < h && iw >= 0 && iw < wd && VB_BC((((i64)nn * cin + c) * h + ih) * wd + iw, (i64)n * cin * h * wd)) e = x[(((i64)nn * cin + c) * h + ih) * wd + iw];
      }
      v[t] = e;
      ++k; if (++j == kw) { j = 0; if (++i == kh) { i = 0; ++c; } }
    }
    reinterpret_cast<float4*>(cols)[idx] = make_float4(v[0], v[1], v[2], v[3]);
  }
}
// dX[n, c, ih, iw] = sum over taps (i, j), in that order, of dcols[(n, y, x), (c, i, j)] with y*s + i - p = ih, x*s + j - p = iw.
__global__ void k_col2im(const float* __restrict__ dcols, float* __restrict__ gx, int n, int cin, int h, int wd, int kh, int kw,
                         int oh, int ow, int stride, int pad, int kp) {
  const i64 total = (i64)n * cin * h * wd;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const int iw = (int)(idx % wd); const i64 r1 = idx / wd;
    const int ih = (int)(r1 % h); const i64 r2 = r1 / h;
    const int c = (int)(r2 % cin), nn = (int)(r2 / cin);
    float acc = 0.0f;
    for (int i = 0; i < kh; ++i) {
      int ty = ih + pad - i;
      if (ty < 0 || ty % stride) continue;
      int y = ty / stride; if (y >= oh) continue;
      for (int j = 0; j < kw; ++j) {
        int tx = iw + pad - j;
        if (tx < 0 || tx % stride) continue;
        int xo = tx / stride; if (xo >= ow) continue;
        if (VB_BC((((i64)nn * oh + y) * ow + xo) * kp + (c * kh + i) * kw + j, (i64)n * oh * ow * kp)) acc += dcols[(((i64)nn * oh + y) * ow + xo) * kp + (c * kh + i) * kw + j];
      }
    }
    gx[idx] = acc;
  }
}
// g [n, cout, ohw] -> gt [n*ohw, cout] (32 x 32 tiles through shared memory)
__global__ void k_nchw_to_rows(const float* __restrict__ g, float* __restrict__ gt, i64 cout, i64 ohw) {
  __shared__ float tile[32][33];
  const float* src = g + (i64)blockIdx.z * cout * ohw;
  float* dst = gt + (i64)blockIdx.z * ohw * cout;
  i64 p0 = (i64)blockIdx.x * 32, c0 = (i64)blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    i64 c = c0 + i, pp = p0 + threadIdx.x;
    tile[i][threadIdx.x] = (c < cout && pp < ohw) ? src[c * ohw + pp] : 0.0f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    i64 pp = p0 + i, c = c0 + threadIdx.x;
    if (pp < ohw && c < cout) dst[pp * cout + c] = tile[threadIdx.x][i];
  }
}
// dst [rows, cols] <- src [rows, ld] (the first `cols` entries of every row)
__global__ void k_copy_cols(const float* __restrict__ src, float* __restrict__ dst, i64 rows, i64 cols, i64 ld) {
  i64 total = rows * cols;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x)
    dst[idx] = src[(idx / cols) * ld + idx % cols];
}
// Row length of the unfolded matrix: the taps rounded up to 4 floats, and to 32 when there are fewer than 32 taps
// (the tensor-core GEMM wants at least 32 columns on either side of a product).
static i64 unfolded_row(i64 kc) { return kc < 32 ? 32 : ((kc + 3) & ~i64(3)); }
static bool conv_as_gemm(i64 n, i64 cin, i64 cout, i64 kh, i64 kw, i64 oh, i64 ow) {
  static int off = -1;
  if (off < 0) { const char* e = getenv("VB200_CONV_DIRECT"); off = (e && e[0] == '1') ? 1 : 0; }
  if (off) return false;
  double macs = (double)n * (double)oh * (double)ow * (double)cin * (double)kh * (double)kw * (double)cout;
  return macs >= 2.0e6 && n <= 60000 && (i64)oh * ow < 0x7fffffffLL && cin * kh * kw < (1 << 24);
}
// x [n, c, h, w] -> xp [n, h + 2, w + 2, c], border zero.  One CTA per padded row: the [c, w] slab of an image row goes
// through shared memory so that both the reads (along x) and the writes (along c) are contiguous.
__global__ void __launch_bounds__(256) k_nchw_to_padded_nhwc(const float* __restrict__ x, float* __restrict__ xp, int c, int h, int w) {
  extern __shared__ float tile[];                  // [w][c + 1]
  const int yp = blockIdx.x, n = blockIdx.y;
  float* row = xp + ((i64)n * (h + 2) + yp) * (i64)(w + 2) * c;
  const int total = (w + 2) * c;
  if (yp == 0 || yp == h + 1) { for (int i = threadIdx.x; i < total; i += blockDim.x) row[i] = 0.0f; return; }
  const float* src = x + (i64)n * c * h * w + (i64)(yp - 1) * w;
  for (int i = threadIdx.x; i < c * w; i += blockDim.x) { const int cc = i / w, xx = i - cc * w; tile[xx * (c + 1) + cc] = src[(i64)cc * h * w + xx]; }
  __syncthreads();
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int xx = i / c, cc = i - xx * c;
    if (VB_BC((xx == 0 || xx == w + 1) ? 0 : (xx - 1) * (c + 1) + cc, w * (c + 1))) row[i] = (xx == 0 || xx == w + 1) ? 0.0f : tile[(xx - 1) * (c + 1) + cc];
  }
}
// Weights [cout, cin, 3, 3] -> wr [cout, (i, j, c)] (forward / weight-gradient order) and back; -> wf [cin, (i, j, co)] with the
// window flipped (the input gradient is the correlation of the padded output gradient with the flipped weights).
__global__ void k_weights_to_taps(const float* __restrict__ w, float* __restrict__ wr, int cout, int cin, int flip_transpose) {
  const int total = cout * cin * 9;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int j = idx % 3, i = (idx / 3) % 3, c = (idx / 9) % cin, co = idx / (9 * cin);
    const i64 dst = !flip_transpose ? (i64)co * 9 * cin + (i * 3 + j) * cin + c : (i64)c * 9 * cout + ((2 - i) * 3 + (2 - j)) * cout + co;
    if (VB_BC(dst, total)) wr[dst] = w[idx];
  }
}
__global__ void k_taps_to_weights(const float* __restrict__ wr, float* __restrict__ w, int cout, int cin) {
  const int total = cout * cin * 9;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int j = idx % 3, i = (idx / 3) % 3, c = (idx / 9) % cin, co = idx / (9 * cin);
    w[idx] = wr[(i64)co * 9 * cin + (i * 3 + j) * cin + c];
  }
}
static bool conv_implicit_ok(i64 n, i64 c, i64 h, i64 wd, i64 kh, i64 kw, i64 stride, i64 pad) {
  static int off = -1;
  if (off < 0) { const char* e = getenv("VB200_CONV_IMPLICIT"); off = (e && e[0] == '0') ? 1 : 0; }
  return !off && kh == 3 && kw == 3 && stride == 1 && pad == 1 && c % 32 == 0 && c <= 1024 && wd <= 128 && (wd & (wd - 1)) == 0 && wd >= 4 &&
         (h * wd) % 32 == 0 && n >= 1 && n <= 60000 && (size_t)wd * (c + 1) * sizeof(float) <= 48 * 1024;
}
static int to_padded_nhwc(const float* x, float* xp, i64 n, i64 c, i64 h, i64 wd) {
  ProfScope prof("conv_nhwc", ((double)n * c * h * wd + (double)n * (h + 2) * (wd + 2) * c) * 4.0);
  k_nchw_to_padded_nhwc<<<dim3((unsigned)(h + 2), (unsigned)n), 256, (size_t)wd * (c + 1) * sizeof(float), ctx().stream>>>(x, xp, (int)c, (int)h, (int)wd);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
// out[n] [m, hw] = taps [m, 9 c] . cols(xp)[n]^T (+ bias per row m): the forward product, and the input gradient with the roles
// of the channel counts swapped.  *used = 0 when the tensor-core kernel declined (nothing was written).
static int implicit_product(const float* taps, const float* xp, const float* bias_m, float* out, i64 n, i64 m, i64 c, i64 h, i64 wd, int* used) {
  ConvOperand cv{xp, n, h, wd, c, 1};
  GemmArgs g = gemm_args();
  g.A = taps; g.M = m; g.K = 9 * c; g.a_rs = 9 * c; g.a_cs = 1;
  g.N = h * wd; g.C = out; g.c_rs = h * wd; g.c_cs = 1;
  g.nb1 = 1; g.nb2 = n; g.a_b2 = 0; g.c_b2 = m * h * wd;
  g.bias_m = bias_m;
  g.conv = &cv; g.conv_used = used;
  return launch_gemm(g);
}
static int unfold(const float* x, float* cols, i64 n, i64 cin, i64 h, i64 wd, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad, i64 kc, i64 kp) {
  ProfScope prof("conv_unfold", ((double)n * cin * h * wd + (double)n * oh * ow * kp) * 4.0);
  i64 total = n * oh * ow * (kp / 4);
  i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32; if (blocks > cap) blocks = cap;
  k_im2col<<<(unsigned)blocks, 256, 0, ctx().stream>>>(x, cols, (int)n, (int)cin, (int)h, (int)wd, (int)kh, (int)kw, (int)oh, (int)ow, (int)stride, (int)pad, (int)kc, (int)kp);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

int launch_conv2d(const float* x, const float* w, const float* b, float* out, i64 n, i64 cin, i64 h, i64 wd,
                  i64 cout, i64 kh, i64 kw, i64 oh, i64 ow, i64 stride, i64 pad) {
  i64 total = n * cout * oh * ow;
  if (total <= 0) return VB_OK;
  if (conv_as_gemm(n, cin, cout, kh, kw, oh, ow) && conv_implicit_ok(n, cin, h, wd, kh, kw, stride, pad) && cout >= 32) {
    Temp xp, wr;
    VB_TRY(scratch_alloc((size_t)(n * (h + 2) * (wd + 2) * cin) * sizeof(float), &xp.p));
    VB_TRY(scratch_alloc((size_t)(cout * 9 * cin) * sizeof(float), &wr.p));
    VB_TRY(to_padded_nhwc(x, (float*)xp.p, n, cin, h, wd));
    k_weights_to_taps<<<(unsigned)((cout * cin * 9 + 255) / 256), 256, 0, ctx().stream>>>(w, (float*)wr.p, (int)cout, (int)cin, 0);
    VB_LAUNCH_CHECK();
    int used = 0;
    VB_TRY(implicit_product((const float*)wr.p, (const float*)xp.p, b, out, n, cout, cin, h, wd, &used));
    if (used) return VB_OK;
  }
  if (conv_as_gemm(n, cin, cout, kh, kw, oh, ow)) {
    const i64 kc = cin * kh * kw, kp = unfolded_row(kc), ohw = oh * ow;
    Temp cols;
    VB_TRY(scratch_alloc((size_t)(n * ohw * kp) * sizeof(float), &cols.p));
    VB_TRY(unfold(x, (float*)cols.p, n, cin, h, wd, kh, kw, oh, ow, stride, pad, kc, kp));
    GemmArgs g = gemm_args();            // out[img] [cout, ohw] = W [cout, kc] . cols[img]^T [kc, ohw] + b[cout]
    g.A = w; g.M = cout; g.K = kc; g.a_rs = kc; g.a_cs = 1;
    g.B = (const float*)cols.p; g.N = ohw; g.b_rs = 1; g.b_cs = kp;
    g.C = out; g.c_rs = ohw; g.c_cs = 1;
    g.nb1 = 1; g.nb2 = n; g.a_b2 = 0; g.b_b2 = ohw * kp; g.c_b2 = cout * ohw;
    g.bias_m = b;
    return launch_gemm(g);
  }
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
  // implicit forms: the weight gradient over the padded input, the input gradient over the padded output gradient
  bool dw_done = false, dx_done = false;
  if (n * cout * oh * ow > 0 && cin > 0 && conv_as_gemm(n, cin, cout, kh, kw, oh, ow) && cout % 32 == 0) {
    const i64 ohw = oh * ow, rows = n * ohw;
    if (conv_implicit_ok(n, cin, h, wd, kh, kw, stride, pad)) {
      Temp xp, gt, dwr;
      VB_TRY(scratch_alloc((size_t)(n * (h + 2) * (wd + 2) * cin) * sizeof(float), &xp.p));
      VB_TRY(scratch_alloc((size_t)(rows * cout) * sizeof(float), &gt.p));
      VB_TRY(scratch_alloc((size_t)(cout * 9 * cin) * sizeof(float), &dwr.p));
      VB_TRY(to_padded_nhwc(x, (float*)xp.p, n, cin, h, wd));
      {
        ProfScope prof("conv_nhwc", 2.0 * (double)rows * cout * 4.0);
        dim3 grid((unsigned)((ohw + 31) / 32), (unsigned)((cout + 31) / 32), (unsigned)n), block(32, 8);
        k_nchw_to_rows<<<grid, block, 0, st>>>(g, (float*)gt.p, cout, ohw);
        VB_LAUNCH_CHECK();
      }
      ConvOperand cv{(const float*)xp.p, n, h, wd, cin, 2};
      int used = 0;
      GemmArgs a = gemm_args();          // dWr [cout, 9 cin] = g^T [cout, rows] . cols [rows, 9 cin]
      a.A = (const float*)gt.p; a.M = cout; a.K = rows; a.a_rs = 1; a.a_cs = cout;
      a.N = 9 * cin; a.C = (float*)dwr.p; a.c_rs = 9 * cin; a.c_cs = 1;
      a.conv = &cv; a.conv_used = &used;
      VB_TRY(launch_gemm(a));
      if (used) {
        k_taps_to_weights<<<(unsigned)((cout * cin * 9 + 255) / 256), 256, 0, st>>>((const float*)dwr.p, gw, (int)cout, (int)cin);
        VB_LAUNCH_CHECK();
        VB_TRY(launch_colsum((const float*)gt.p, gb, rows, cout, false));
        dw_done = true;
      }
    }
    if (gx && conv_implicit_ok(n, cout, h, wd, kh, kw, stride, pad) && cin >= 32) {
      Temp gp, wf;
      VB_TRY(scratch_alloc((size_t)(n * (h + 2) * (wd + 2) * cout) * sizeof(float), &gp.p));
      VB_TRY(scratch_alloc((size_t)(cin * 9 * cout) * sizeof(float), &wf.p));
      VB_TRY(to_padded_nhwc(g, (float*)gp.p, n, cout, h, wd));
      k_weights_to_taps<<<(unsigned)((cout * cin * 9 + 255) / 256), 256, 0, st>>>(w, (float*)wf.p, (int)cout, (int)cin, 1);
      VB_LAUNCH_CHECK();
      int used = 0;
      VB_TRY(implicit_product((const float*)wf.p, (const float*)gp.p, nullptr, gx, n, cin, cout, h, wd, &used));
      dx_done = used != 0;
    }
    if (dw_done && (dx_done || !gx)) return VB_OK;
  }
  if (n * cout * oh * ow > 0 && cin > 0 && conv_as_gemm(n, cin, cout, kh, kw, oh, ow)) {
    const i64 kc = cin * kh * kw, kp = unfolded_row(kc), ohw = oh * ow, rows = n * ohw;
    Temp cols, gt;
    VB_TRY(scratch_alloc((size_t)(rows * kp) * sizeof(float), &cols.p));
    VB_TRY(scratch_alloc((size_t)(rows * cout) * sizeof(float), &gt.p));
    {
      ProfScope prof("conv_unfold", 2.0 * (double)rows * cout * 4.0);
      dim3 grid((unsigned)((ohw + 31) / 32), (unsigned)((cout + 31) / 32), (unsigned)n), block(32, 8);
      k_nchw_to_rows<<<grid, block, 0, st>>>(g, (float*)gt.p, cout, ohw);
      VB_LAUNCH_CHECK();
    }
    // db = column sums of g^T; dW [cout, kc] = g^T^T [cout, rows] . cols [rows, kc]
    if (!dw_done) {
    VB_TRY(launch_colsum((const float*)gt.p, gb, rows, cout, false));
    VB_TRY(unfold(x, (float*)cols.p, n, cin, h, wd, kh, kw, oh, ow, stride, pad, kc, kp));
    GemmArgs a = gemm_args();
    a.A = (const float*)gt.p; a.M = cout; a.K = rows; a.a_rs = 1; a.a_cs = cout;
    a.B = (const float*)cols.p; a.N = kc; a.b_rs = kp; a.b_cs = 1;
    a.C = gw; a.c_rs = kc; a.c_cs = 1;
    if (kc < 32) {          // all 32 (zero-padded) columns into scratch, then the real ones out
      Temp wide;
      VB_TRY(scratch_alloc((size_t)(cout * kp) * sizeof(float), &wide.p));
      a.N = kp; a.C = (float*)wide.p; a.c_rs = kp;
      VB_TRY(launch_gemm(a));
      k_copy_cols<<<(unsigned)((cout * kc + 255) / 256), 256, 0, st>>>((const float*)wide.p, gw, cout, kc, kp);
      VB_LAUNCH_CHECK();
    } else {
      VB_TRY(launch_gemm(a));
    }
    }
    if (gx && !dx_done) {
      // dcols[img] [ohw, kc] = g[img]^T [ohw, cout] . W [cout, kc], over the same scratch as cols; then folded back
      GemmArgs d = gemm_args();
      d.A = g; d.M = ohw; d.K = cout; d.a_rs = 1; d.a_cs = ohw;
      d.B = w; d.N = kc; d.b_rs = kc; d.b_cs = 1;
      d.C = (float*)cols.p; d.c_rs = kp; d.c_cs = 1;
      d.nb1 = 1; d.nb2 = n; d.a_b2 = cout * ohw; d.b_b2 = 0; d.c_b2 = ohw * kp;
      VB_TRY(launch_gemm(d));
      ProfScope prof("conv_fold", ((double)rows * kc + (double)n * cin * h * wd) * 4.0);
      i64 total = n * cin * h * wd;
      i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 32; if (blocks > cap) blocks = cap;
      k_col2im<<<(unsigned)blocks, 256, 0, st>>>((const float*)cols.p, gx, (int)n, (int)cin, (int)h, (int)wd, (int)kh, (int)kw, (int)oh, (int)ow, (int)stride, (int)pad, (int)kp);
      VB_LAUNCH_CHECK();
    }
    return VB_OK;
  }
  if (cout > 0) k_conv2d_bwd_bias<<<(unsigned)cout, 256, 0, st>>>(g, gb, n, cout, oh * ow);
  i64 nw = cout * cin * kh * kw;
  if (nw > 0) k_conv2d_bwd_weight<<<(unsigned)nw, 256, 0, st>>>(x, g, gw, n, cin, h, wd, cout, kh, kw, oh, ow, stride, pad);
  i64 total = n * cin * h * wd;
  if (total > 0 && gx) {
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
        if (!VB_BC((c * h + ih) * w + iw, nc * h * w)) continue;
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
