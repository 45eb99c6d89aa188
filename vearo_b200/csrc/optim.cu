// Optimizer kernels: AdamW, SGD with momentum, global-norm gradient clipping.
//
// Arithmetic follows crates/vearo-core/src/tensor.rs:972-985 (AdamW: moments, bias-corrected
// estimates, then `w -= lr*wd*w` and only then `w -= lr*m_hat/(sqrt(v_hat)+eps)`), :1062-1069
// (SGD: g += wd*w when wd != 0; vel = mu*vel + g; w -= lr*vel) and
// crates/vearo-optim/src/lib.rs:360-383 (clip: norm = sqrt(sum g^2); if norm > max,
// g *= max/(norm + 1e-6)).  The reference runs these loops on the host even for CUDA tensors.
//
// The multi-tensor kernel updates every parameter of a model in one launch: a table of chunks
// (at most 16384 elements each, never spanning two tensors) lives in device memory, one CTA per
// chunk, 128-bit loads and stores.  Algorithmic bytes per element: AdamW 28 (read g, w, m, v;
// write w, m, v), SGD 20.  The clip scale is computed in-kernel from the device-resident sum of
// squares, so clipping costs one extra read of the gradients and no rewrite.
#include "common.h"

namespace vb {

struct Hyper { float lr, b1, b2, eps, wd, mu, bc1, bc2; };

__device__ __forceinline__ void adamw_elem(float& w, float g, float& m, float& v, const Hyper& h) {
  m = h.b1 * m + (1.0f - h.b1) * g;
  v = h.b2 * v + (1.0f - h.b2) * g * g;
  float mh = m / h.bc1, vh = v / h.bc2;
  w -= h.lr * h.wd * w;
  w -= h.lr * mh / (sqrtf(vh) + h.eps);
}
__device__ __forceinline__ void sgd_elem(float& w, float g, float& vel, const Hyper& h) {
  if (h.wd != 0.0f) g += h.wd * w;
  vel = h.mu * vel + g;
  w -= h.lr * vel;
}
__device__ __forceinline__ float clip_scale(const float* normsq, float max_norm, float grad_scale) {
  if (!(max_norm > 0.0f)) return grad_scale;
  float norm = sqrtf(normsq[0]) * fabsf(grad_scale);
  return norm > max_norm ? grad_scale * (max_norm / (norm + 1e-6f)) : grad_scale;
}

template <int KIND>
__device__ __forceinline__ void update_range(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                             int n, float gs, const Hyper& h, float* __restrict__ lo = nullptr) {
  bool vec = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
               (KIND == 0 ? reinterpret_cast<uintptr_t>(v) : 0)) & 15) == 0;
  int n4 = vec ? n / 4 : 0;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    float4 ww = reinterpret_cast<float4*>(w)[i], gg = reinterpret_cast<const float4*>(g)[i], mm = reinterpret_cast<float4*>(m)[i];
    gg.x *= gs; gg.y *= gs; gg.z *= gs; gg.w *= gs;
    if (KIND == 0) {
      float4 vv = reinterpret_cast<float4*>(v)[i];
      adamw_elem(ww.x, gg.x, mm.x, vv.x, h); adamw_elem(ww.y, gg.y, mm.y, vv.y, h);
      adamw_elem(ww.z, gg.z, mm.z, vv.z, h); adamw_elem(ww.w, gg.w, mm.w, vv.w, h);
      reinterpret_cast<float4*>(v)[i] = vv;
    } else {
      sgd_elem(ww.x, gg.x, mm.x, h); sgd_elem(ww.y, gg.y, mm.y, h); sgd_elem(ww.z, gg.z, mm.z, h); sgd_elem(ww.w, gg.w, mm.w, h);
    }
    reinterpret_cast<float4*>(w)[i] = ww; reinterpret_cast<float4*>(m)[i] = mm;
    if (lo) reinterpret_cast<float4*>(lo)[i] = make_float4(tf32_remainder(ww.x), tf32_remainder(ww.y), tf32_remainder(ww.z), tf32_remainder(ww.w));
  }
  for (int i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
    float ww = w[i], gg = g[i] * gs, mm = m[i];
    if (KIND == 0) { float vv = v[i]; adamw_elem(ww, gg, mm, vv, h); v[i] = vv; } else sgd_elem(ww, gg, mm, h);
    w[i] = ww; m[i] = mm;
    if (lo) lo[i] = tf32_remainder(ww);
  }
}

// ---- AdamW with 8-bit block-wise state (crates/vearo-optim/src/lib.rs:137-303) ----------------------------------
// m and v live as int8 with one f32 scale per 256 elements of a parameter (scale = block maximum / 127).  A step
// dequantizes (q * scale), applies the AdamW update above, and requantizes: q = round-half-away(x * (127 / max)),
// clamped to [-127, 127]; a block whose maximum is 0 stores zeros and scale 0.  One warp per block: lane l owns
// elements 4l..4l+3 and 128+4l..128+4l+3, the block maximum is a warp shuffle, nothing is staged.  Algorithmic bytes
// per element: 16 (read g, w, m, v; write w, m, v) + 16 per block of scales, against 28 for the f32 state.
// The arithmetic is written with explicit single-rounding intrinsics (no fused multiply-add): an update that differs
// in the last bit from the reference's can land on the other side of a rounding boundary of the quantizer.
__device__ __forceinline__ void adamw_elem_exact(float& w, float g, float& m, float& v, const Hyper& h) {
  m = __fadd_rn(__fmul_rn(h.b1, m), __fmul_rn(__fsub_rn(1.0f, h.b1), g));
  v = __fadd_rn(__fmul_rn(h.b2, v), __fmul_rn(__fmul_rn(__fsub_rn(1.0f, h.b2), g), g));
  const float mh = __fdiv_rn(m, h.bc1), vh = __fdiv_rn(v, h.bc2);
  w = __fsub_rn(w, __fmul_rn(__fmul_rn(h.lr, h.wd), w));
  w = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, mh), __fadd_rn(__fsqrt_rn(vh), h.eps)));
}
__device__ __forceinline__ float wmax32(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ int quant8(float x, float inv) {
  float q = roundf(__fmul_rn(x, inv));
  q = fminf(fmaxf(q, -127.0f), 127.0f);
  return (int)q;
}
__global__ void __launch_bounds__(256, 4) k_opt_adamw8(const OptChunk* __restrict__ chunks, const uint8_t* __restrict__ active,
                                                    const float* __restrict__ normsq, float max_norm, float grad_scale, Hyper h) {
  const OptChunk c = chunks[blockIdx.x];
  if (active && !active[c.param]) return;
  const float gs = clip_scale(normsq, max_norm, grad_scale);
  int8_t* __restrict__ m8 = reinterpret_cast<int8_t*>(c.m);
  int8_t* __restrict__ v8 = reinterpret_cast<int8_t*>(c.v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (c.n + 255) >> 8;
  const bool vec = ((reinterpret_cast<uintptr_t>(c.w) | reinterpret_cast<uintptr_t>(c.g)) & 15) == 0;
  for (int b = warp; b < nblk; b += 8) {
    const int base = b << 8, cnt = c.n - base < 256 ? c.n - base : 256;
    const float sm = c.ms[b], sv = c.vs[b];
    float w[8], m[8], v[8];
    bool ok[8];
    if (vec && cnt == 256) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int e = base + hf * 128 + lane * 4;
        const float4 ww = *reinterpret_cast<const float4*>(c.w + e), gg = *reinterpret_cast<const float4*>(c.g + e);
        const char4 mq = *reinterpret_cast<const char4*>(m8 + e), vq = *reinterpret_cast<const char4*>(v8 + e);
        const float wv[4] = {ww.x, ww.y, ww.z, ww.w}, gv[4] = {gg.x, gg.y, gg.z, gg.w};
        const signed char mv[4] = {mq.x, mq.y, mq.z, mq.w}, vv[4] = {vq.x, vq.y, vq.z, vq.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int k = hf * 4 + t;
          w[k] = wv[t]; m[k] = __fmul_rn((float)mv[t], sm); v[k] = __fmul_rn((float)vv[t], sv); ok[k] = true;
          adamw_elem_exact(w[k], __fmul_rn(gv[t], gs), m[k], v[k], h);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int o = (k >> 2) * 128 + lane * 4 + (k & 3);
        ok[k] = o < cnt;
        w[k] = 0.0f; m[k] = 0.0f; v[k] = 0.0f;
        if (ok[k]) {
          w[k] = c.w[base + o]; m[k] = __fmul_rn((float)m8[base + o], sm); v[k] = __fmul_rn((float)v8[base + o], sv);
          adamw_elem_exact(w[k], __fmul_rn(c.g[base + o], gs), m[k], v[k], h);
        }
      }
    }
    float mx_m = 0.0f, mx_v = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) if (ok[k]) { mx_m = fmaxf(mx_m, fabsf(m[k])); mx_v = fmaxf(mx_v, fabsf(v[k])); }
    mx_m = wmax32(mx_m); mx_v = wmax32(mx_v);
    const float inv_m = mx_m > 0.0f ? __fdiv_rn(127.0f, mx_m) : 0.0f, inv_v = mx_v > 0.0f ? __fdiv_rn(127.0f, mx_v) : 0.0f;
    int qm[8], qv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { qm[k] = mx_m > 0.0f ? quant8(m[k], inv_m) : 0; qv[k] = mx_v > 0.0f ? quant8(v[k], inv_v) : 0; }
    if (vec && cnt == 256) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int e = base + hf * 128 + lane * 4;
        *reinterpret_cast<float4*>(c.w + e) = make_float4(w[hf * 4], w[hf * 4 + 1], w[hf * 4 + 2], w[hf * 4 + 3]);
        if (c.lo) *reinterpret_cast<float4*>(c.lo + e) = make_float4(tf32_remainder(w[hf * 4]), tf32_remainder(w[hf * 4 + 1]), tf32_remainder(w[hf * 4 + 2]), tf32_remainder(w[hf * 4 + 3]));
        *reinterpret_cast<char4*>(m8 + e) = make_char4((signed char)qm[hf * 4], (signed char)qm[hf * 4 + 1], (signed char)qm[hf * 4 + 2], (signed char)qm[hf * 4 + 3]);
        *reinterpret_cast<char4*>(v8 + e) = make_char4((signed char)qv[hf * 4], (signed char)qv[hf * 4 + 1], (signed char)qv[hf * 4 + 2], (signed char)qv[hf * 4 + 3]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int o = (k >> 2) * 128 + lane * 4 + (k & 3);
        if (ok[k]) { c.w[base + o] = w[k]; m8[base + o] = (int8_t)qm[k]; v8[base + o] = (int8_t)qv[k]; if (c.lo) c.lo[base + o] = tf32_remainder(w[k]); }
      }
    }
    if (lane == 0) { c.ms[b] = __fdiv_rn(mx_m, 127.0f); c.vs[b] = __fdiv_rn(mx_v, 127.0f); }
  }
}

template <int KIND>
__global__ void __launch_bounds__(256) k_opt_multi(const OptChunk* __restrict__ chunks, const uint8_t* __restrict__ active,
                                                   const float* __restrict__ normsq, float max_norm, float grad_scale, Hyper h) {
  OptChunk c = chunks[blockIdx.x];
  if (active && !active[c.param]) return;
  float gs = clip_scale(normsq, max_norm, grad_scale);
  update_range<KIND>(c.w, c.g, c.m, c.v, c.n, gs, h, c.lo);
}
int launch_opt_multi(const OptChunk* chunks, int nchunks, const uint8_t* active, int kind, const float* normsq,
                     float max_norm, float grad_scale, float lr, float b1, float b2, float eps, float wd, float mu,
                     float bc1, float bc2, int lo_chunks) {
  if (nchunks <= 0) return VB_OK;
  // bytes per parameter: g, w, m, v read and w, m, v written (AdamW); +4 where the chunk also rewrites the weight's lo plane
  ProfScope prof(kind == VB_OPT_ADAMW ? "adamw" : (kind == VB_OPT_ADAMW8BIT ? "adamw8bit" : "sgd"),
                 (kind == VB_OPT_ADAMW ? 28.0 : (kind == VB_OPT_ADAMW8BIT ? 16.0625 : 20.0)) * 16384.0 * (double)nchunks + 4.0 * 16384.0 * (double)lo_chunks);
  Hyper h{lr, b1, b2, eps, wd, mu, bc1, bc2};
  if (kind == VB_OPT_ADAMW8BIT) k_opt_adamw8<<<nchunks, 256, 0, ctx().stream>>>(chunks, active, normsq, max_norm, grad_scale, h);
  else if (kind == VB_OPT_ADAMW) k_opt_multi<0><<<nchunks, 256, 0, ctx().stream>>>(chunks, active, normsq, max_norm, grad_scale, h);
  else k_opt_multi<1><<<nchunks, 256, 0, ctx().stream>>>(chunks, active, normsq, max_norm, grad_scale, h);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// Single-tensor entry points (one call per parameter, as AdamW::step / SGD::step loop).
template <int KIND>
__global__ void __launch_bounds__(256) k_opt_single(float* w, const float* g, float* m, float* v, i64 n, Hyper h) {
  i64 per = 16384;
  i64 start = (i64)blockIdx.x * per;
  i64 cnt = n - start; if (cnt > per) cnt = per;
  if (cnt > 0) update_range<KIND>(w + start, g + start, m + start, KIND == 0 ? v + start : nullptr, (int)cnt, 1.0f, h);
}
int launch_adamw_single(float* w, const float* g, float* m, float* v, i64 n, float lr, float b1, float b2, float eps, float wd,
                        float bc1, float bc2) {
  if (n <= 0) return VB_OK;
  Hyper h{lr, b1, b2, eps, wd, 0.0f, bc1, bc2};
  k_opt_single<0><<<(unsigned)((n + 16383) / 16384), 256, 0, ctx().stream>>>(w, g, m, v, n, h);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
int launch_sgd_single(float* w, const float* g, float* vel, i64 n, float lr, float mu, float wd) {
  if (n <= 0) return VB_OK;
  Hyper h{lr, 0, 0, 0, wd, mu, 1, 1};
  k_opt_single<1><<<(unsigned)((n + 16383) / 16384), 256, 0, ctx().stream>>>(w, g, vel, nullptr, n, h);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// Sum of squares: one partial per chunk, then a single CTA adds the partials in index order.
__global__ void __launch_bounds__(256) k_sumsq_chunks(const OptChunk* __restrict__ chunks, const uint8_t* __restrict__ active, float* __restrict__ partials) {
  __shared__ float red[8];
  OptChunk c = chunks[blockIdx.x];
  float s = 0.0f;
  if (!active || active[c.param]) {
    const float* g = c.g;
    int n4 = (reinterpret_cast<uintptr_t>(g) & 15) == 0 ? c.n / 4 : 0;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) { float4 x = reinterpret_cast<const float4*>(g)[i]; s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w; }
    for (int i = n4 * 4 + threadIdx.x; i < c.n; i += blockDim.x) s += g[i] * g[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.0f; for (int i = 0; i < 8; ++i) t += red[i]; partials[blockIdx.x] = t; }
}
int launch_sumsq_chunks(const OptChunk* chunks, int nchunks, const uint8_t* active, float* partials) {
  if (nchunks <= 0) return VB_OK;
  ProfScope prof("grad_sumsq", 4.0 * 16384.0 * (double)nchunks);
  k_sumsq_chunks<<<nchunks, 256, 0, ctx().stream>>>(chunks, active, partials);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void __launch_bounds__(1024) k_sum_partials(const float* __restrict__ partials, int n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) out[0] = t;
  }
}
int launch_sum_partials(const float* partials, int n, float* out) {
  k_sum_partials<<<1, 1024, 0, ctx().stream>>>(partials, n, out);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
__global__ void k_scale_by_clip(float* g, i64 n, const float* normsq, float max_norm) {
  float norm = sqrtf(normsq[0]);
  if (!(norm > max_norm)) return;
  float sc = max_norm / (norm + 1e-6f);
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) g[i] = g[i] * sc;
}
int launch_scale_inplace_by_clip(float* g, i64 n, const float* normsq, float max_norm) {
  if (n <= 0) return VB_OK;
  i64 blocks = (n + 255) / 256, cap = (i64)ctx().sm_count * 16; if (blocks > cap) blocks = cap;
  k_scale_by_clip<<<(unsigned)blocks, 256, 0, ctx().stream>>>(g, n, normsq, max_norm);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
