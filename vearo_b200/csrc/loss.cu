// Embedding lookup and softmax cross-entropy, forward and backward.
//
// Semantics: crates/vearo-backend-cpu/src/lib.rs:862-1127.  Ids and classes are f32, rounded half
// away from zero; a negative or out-of-range value sets a bit in the device error word (the CPU
// backend panics there, lib.rs:893-905, 1015-1027) and the row is skipped.
//
// Cross-entropy at V = 50304 is the largest HBM-bound kernel of a GPT step.  Forward: one CTA per
// row reads the row once (128-bit loads) keeping an online (max, sum exp) pair, writes the row's
// (max, sum) and its loss term; a single-block kernel then adds the row terms in a fixed order.
// Backward with the saved row statistics is one read and one write of the logits:
// algorithmic bytes 2 * rows * V * 4.  Without statistics it first redoes the forward pass.
#include "common.h"

namespace vb {

__device__ __forceinline__ float wsum2(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// id = round-half-away(v); returns -1 after flagging when invalid.
__device__ __forceinline__ i64 checked_id(float v, i64 bound, int* err) {
  if (!(v >= 0.0f)) { atomicOr(err, ERRBIT_NEG_ID); return -1; }
  i64 id = (i64)roundf(v);
  if (id >= bound) { atomicOr(err, ERRBIT_OOB_ID); return -1; }
  return id;
}

// ---- embedding: one warp per token row -----------------------------------------------------
__global__ void k_embedding(const float* __restrict__ ids, const float* __restrict__ w, float* __restrict__ out,
                            i64 n, i64 vocab, i64 d, int* err) {
  int lane = threadIdx.x & 31;
  i64 warp = (blockIdx.x * (i64)blockDim.x + threadIdx.x) >> 5;
  i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 i = warp; i < n; i += nwarps) {
    i64 t = checked_id(ids[i], vocab, err);
    float* o = out + i * d;
    if (t < 0) { for (i64 j = lane; j < d; j += 32) o[j] = 0.0f; continue; }
    const float* src = w + t * d;
    if ((d & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(o)) & 15) == 0) {
      for (i64 j = lane; j < d / 4; j += 32) reinterpret_cast<float4*>(o)[j] = reinterpret_cast<const float4*>(src)[j];
    } else for (i64 j = lane; j < d; j += 32) o[j] = src[j];
  }
}
int launch_embedding(const float* ids, const float* w, float* out, i64 n, i64 vocab, i64 d) {
  if (n <= 0 || d <= 0) return VB_OK;
  i64 blocks = (n + 7) / 8, cap = (i64)ctx().sm_count * 8; if (blocks > cap) blocks = cap;
  k_embedding<<<(unsigned)blocks, 256, 0, ctx().stream>>>(ids, w, out, n, vocab, d, ctx().d_err);
  VB_LAUNCH_CHECK();
  return VB_OK;
}
// Fallback backward (D > 1024 or unaligned): gw[id] += g[i] with float atomics; the order of additions into one row
// is then not fixed.  gw must be zero on entry (both paths are given a zeroed buffer).
__global__ void k_embedding_backward(const float* __restrict__ ids, const float* __restrict__ g, float* __restrict__ gw,
                                     i64 n, i64 vocab, i64 d, int* err) {
  int lane = threadIdx.x & 31;
  i64 warp = (blockIdx.x * (i64)blockDim.x + threadIdx.x) >> 5;
  i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 i = warp; i < n; i += nwarps) {
    i64 t = checked_id(ids[i], vocab, err);
    if (t < 0) continue;
    const float* src = g + i * d;
    float* dst = gw + t * d;
    for (i64 j = lane; j < d; j += 32) atomicAdd(dst + j, src[j]);
  }
}
// Deterministic backward for D <= 1024 (a multiple of 4).  The table gradient is zero-filled first; then one warp per
// token position scans the token ids (staged in shared memory, 8192 at a time).  The warp of the FIRST position that
// names a row owns that row: it adds the gradient rows of all positions naming it in increasing position — the order of
// the CPU backend (lib.rs:948-976) — in registers and writes the row once.  Warps of later duplicates stop at their first
// earlier hit.  No atomics: bit-reproducible, and bit-identical to a sequential sum.
constexpr int kEmbChunk = 8192;
template <int V4>
__global__ void __launch_bounds__(256) k_embedding_backward_tokens(const float* __restrict__ ids, const float* __restrict__ g, float* __restrict__ gw,
                                                                   i64 n, i64 vocab, int d, int* err) {
  __shared__ int sids[kEmbChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 tok = (i64)blockIdx.x * 8 + warp;
  int my = -1;
  if (tok < n) {
    float v = ids[tok];
    if (!(v >= 0.0f)) { if (lane == 0) atomicOr(err, ERRBIT_NEG_ID); }
    else { i64 t = (i64)roundf(v); if (t >= vocab) { if (lane == 0) atomicOr(err, ERRBIT_OOB_ID); } else my = (int)t; }
  }
  bool owner = my >= 0;
  float4 acc[V4];
#pragma unroll
  for (int v = 0; v < V4; ++v) acc[v] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (i64 c0 = 0; c0 < n; c0 += kEmbChunk) {      // uniform per block: the barriers are safe
    int cn = (int)(n - c0 < kEmbChunk ? n - c0 : kEmbChunk);
    __syncthreads();
    for (int i = threadIdx.x; i < cn; i += blockDim.x) {
      float v = ids[c0 + i];
      int id = -1;
      if (v >= 0.0f) { i64 t = (i64)roundf(v); if (t < vocab) id = (int)t; }
      sids[i] = id;
    }
    __syncthreads();
    if (!owner) continue;
    for (int base = 0; base < cn; base += 32) {
      int id = base + lane < cn ? sids[base + lane] : -1;
      unsigned hit = __ballot_sync(0xffffffffu, id == my);
      if (!hit) continue;
      const i64 j0 = c0 + base;
      if (j0 < tok) {       // positions before this one in the word
        unsigned before = tok - j0 >= 32 ? 0xffffffffu : ((1u << (unsigned)(tok - j0)) - 1u);
        if (hit & before) { owner = false; break; }
      }
      while (hit) {
        int b = __ffs(hit) - 1; hit &= hit - 1;
        const float4* src = reinterpret_cast<const float4*>(g + (j0 + b) * d);
#pragma unroll
        for (int v = 0; v < V4; ++v)
          if ((v * 32 + lane) * 4 < d) { float4 x = src[v * 32 + lane]; acc[v].x += x.x; acc[v].y += x.y; acc[v].z += x.z; acc[v].w += x.w; }
      }
    }
  }
  if (owner) {
    float4* dst = reinterpret_cast<float4*>(gw + (i64)my * d);
#pragma unroll
    for (int v = 0; v < V4; ++v) if ((v * 32 + lane) * 4 < d) dst[v * 32 + lane] = acc[v];
  }
}
// The same result when there are more token positions than table rows (the scan above is quadratic in the positions):
// one warp owns a row of the table, scans the token ids
// (staged in shared memory, 8192 at a time) and adds the gradient rows that hit it in increasing token position —
// the order of the CPU backend (lib.rs:948-976) — keeping the row in registers; every row is written exactly once
// (zeros where no token hit), so no pre-zeroing and no atomics: bit-reproducible, and bit-identical to a sequential sum.
template <int V4>
__global__ void __launch_bounds__(256) k_embedding_backward_rows(const float* __restrict__ ids, const float* __restrict__ g, float* __restrict__ gw,
                                                                 i64 n, i64 vocab, int d, int* err) {
  __shared__ int sids[kEmbChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 rows_per_pass = (i64)gridDim.x * 8;
  for (i64 row0 = (i64)blockIdx.x * 8; row0 < vocab; row0 += rows_per_pass) {     // uniform per block: barriers below are safe
    const i64 row = row0 + warp;
    float4 acc[V4];
#pragma unroll
    for (int v = 0; v < V4; ++v) acc[v] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (i64 c0 = 0; c0 < n; c0 += kEmbChunk) {
      int cn = (int)(n - c0 < kEmbChunk ? n - c0 : kEmbChunk);
      __syncthreads();
      for (int i = threadIdx.x; i < cn; i += blockDim.x) {
        float v = ids[c0 + i];
        int id = -1;
        if (!(v >= 0.0f)) { if (row0 == 0) atomicOr(err, ERRBIT_NEG_ID); }
        else { i64 t = (i64)roundf(v); if (t >= vocab) { if (row0 == 0) atomicOr(err, ERRBIT_OOB_ID); } else id = (int)t; }
        sids[i] = id;
      }
      __syncthreads();
      if (row < vocab) {
        for (int base = 0; base < cn; base += 32) {
          int id = base + lane < cn ? sids[base + lane] : -1;
          unsigned hit = __ballot_sync(0xffffffffu, id == (int)row);
          while (hit) {
            int b = __ffs(hit) - 1; hit &= hit - 1;
            const float4* src = reinterpret_cast<const float4*>(g + (c0 + base + b) * d);
#pragma unroll
            for (int v = 0; v < V4; ++v)
              if ((v * 32 + lane) * 4 < d) { float4 x = src[v * 32 + lane]; acc[v].x += x.x; acc[v].y += x.y; acc[v].z += x.z; acc[v].w += x.w; }
          }
        }
      }
    }
    if (row < vocab) {
      float4* dst = reinterpret_cast<float4*>(gw + row * d);
#pragma unroll
      for (int v = 0; v < V4; ++v) if ((v * 32 + lane) * 4 < d) dst[v * 32 + lane] = acc[v];
    }
  }
}
int launch_embedding_backward(const float* ids, const float* g, float* gw, i64 n, i64 vocab, i64 d) {
  if (n <= 0 || d <= 0) return VB_OK;
  if ((d & 3) == 0 && d <= 1024 && vocab < 0x7fffffff && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(gw)) & 15) == 0) {
    ProfScope prof("embedding_bwd", ((double)n * (double)d + (double)vocab * (double)d) * 4.0);
    int v4 = (int)((d + 127) / 128);
    if (n <= vocab) {
      VB_CUDA(cudaMemsetAsync(gw, 0, (size_t)(vocab * d) * sizeof(float), ctx().stream));
      i64 blocks = (n + 7) / 8;
#define EMB(V) case V: k_embedding_backward_tokens<V><<<(unsigned)blocks, 256, 0, ctx().stream>>>(ids, g, gw, n, vocab, (int)d, ctx().d_err); break;
      switch (v4) { EMB(1) EMB(2) EMB(3) EMB(4) EMB(5) EMB(6) EMB(7) EMB(8) }
#undef EMB
    } else {
      i64 blocks = (vocab + 7) / 8, cap = (i64)ctx().sm_count * 8; if (blocks > cap) blocks = cap;
#define EMB(V) case V: k_embedding_backward_rows<V><<<(unsigned)blocks, 256, 0, ctx().stream>>>(ids, g, gw, n, vocab, (int)d, ctx().d_err); break;
      switch (v4) { EMB(1) EMB(2) EMB(3) EMB(4) EMB(5) EMB(6) EMB(7) EMB(8) }
#undef EMB
    }
    VB_LAUNCH_CHECK();
    return VB_OK;
  }
  ProfScope prof("embedding_bwd", 2.0 * (double)n * (double)d * 4.0);
  i64 blocks = (n + 7) / 8, cap = (i64)ctx().sm_count * 8; if (blocks > cap) blocks = cap;
  k_embedding_backward<<<(unsigned)blocks, 256, 0, ctx().stream>>>(ids, g, gw, n, vocab, d, ctx().d_err);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// ---- cross-entropy ---------------------------------------------------------------------------
// Online (max, sum): folding a value or another pair keeps sum = sum exp(x - max).
__device__ __forceinline__ void online_add(float& m, float& s, float x) {
  if (x > m) { s = s * exp_neg_fast(m - x) + 1.0f; m = x; }
  else s += exp_neg_fast(x - m);
}
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  if (m2 > m) { s = s * exp_neg_fast(m - m2) + s2; m = m2; }
  else if (m2 != -INFINITY) s += s2 * exp_neg_fast(m2 - m);
}
__device__ void row_max_sum(const float* __restrict__ row, i64 v, float& m_out, float& s_out, float* red) {
  float m = -INFINITY, s = 0.0f;
  if ((v & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    for (i64 i = threadIdx.x; i < v / 4; i += blockDim.x) {
      float4 x = r4[i];
      float lm = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
      float ls = exp_neg_fast(x.x - lm) + exp_neg_fast(x.y - lm) + exp_neg_fast(x.z - lm) + exp_neg_fast(x.w - lm);
      online_merge(m, s, lm, ls);
    }
  } else for (i64 i = threadIdx.x; i < v; i += blockDim.x) online_add(m, s, row[i]);
  // warp, then block combine
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { red[wid] = m; red[32 + wid] = s; }
  __syncthreads();
  m = lane < nw ? red[lane] : -INFINITY; s = lane < nw ? red[32 + lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  m_out = m; s_out = s;
}
__global__ void k_ce_rows(const float* __restrict__ logits, const float* __restrict__ targets, float* __restrict__ row_loss,
                          float* __restrict__ stats, i64 v, int* err) {
  __shared__ float red[64];
  i64 r = blockIdx.x;
  const float* row = logits + r * v;
  float m, s;
  row_max_sum(row, v, m, s, red);
  if (threadIdx.x == 0) {
    i64 cls = checked_id(targets[r], v, err);
    row_loss[r] = cls < 0 ? 0.0f : -(row[cls] - m - logf(s));
    if (stats) { stats[2 * r] = m; stats[2 * r + 1] = s; }
  }
}
// loss = (sum of row terms, increasing row order within each thread, fixed tree after) / rows
__global__ void k_ce_mean(const float* __restrict__ row_loss, float* __restrict__ loss, i64 rows) {
  __shared__ float red[32];
  float s = 0.0f;
  for (i64 i = threadIdx.x; i < rows; i += blockDim.x) s += row_loss[i];
  s = wsum2(s);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) red[wid] = s;
  __syncthreads();
  if (wid == 0) {
    float t = lane < (blockDim.x >> 5) ? red[lane] : 0.0f;
    t = wsum2(t);
    if (lane == 0) loss[0] = t / (float)rows;
  }
}
int launch_cross_entropy(const float* logits, const float* targets, float* loss, float* stats, i64 rows, i64 v) {
  void* rl = nullptr;
  VB_TRY(scratch_alloc((size_t)rows * sizeof(float), &rl));
  ProfScope prof("cross_entropy_fwd", (double)rows * (double)v * 4.0);
  int threads = v >= 8192 ? 512 : (v >= 1024 ? 256 : 64);
  k_ce_rows<<<(unsigned)rows, threads, 0, ctx().stream>>>(logits, targets, (float*)rl, stats, v, ctx().d_err);
  k_ce_mean<<<1, 1024, 0, ctx().stream>>>((const float*)rl, loss, rows);
  scratch_free(rl);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// dl[b,c] = g * (exp(l - max)/sum - 1[c == class]) / B, evaluated in that order (lib.rs:1116-1123).
template <bool HAVE_STATS>
__global__ void k_ce_backward(const float* __restrict__ logits, const float* __restrict__ targets, const float* __restrict__ gout,
                              const float* __restrict__ stats, float* __restrict__ gl, i64 rows, i64 v, int* err) {
  __shared__ float red[64];
  i64 r = blockIdx.x;
  const float* row = logits + r * v;
  float* orow = gl + r * v;
  float m, s;
  if (HAVE_STATS) { m = stats[2 * r]; s = stats[2 * r + 1]; }
  else row_max_sum(row, v, m, s, red);
  float g = gout[0], fb = (float)rows;
  i64 cls = checked_id(targets[r], v, err);
  if ((v & 3) == 0 && ((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(orow)) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    float4* o4 = reinterpret_cast<float4*>(orow);
    for (i64 i = threadIdx.x; i < v / 4; i += blockDim.x) {
      float4 x = r4[i], o;
      i64 c = i * 4;
      o.x = g * (exp_neg_fast(x.x - m) / s - (c == cls ? 1.0f : 0.0f)) / fb;
      o.y = g * (exp_neg_fast(x.y - m) / s - (c + 1 == cls ? 1.0f : 0.0f)) / fb;
      o.z = g * (exp_neg_fast(x.z - m) / s - (c + 2 == cls ? 1.0f : 0.0f)) / fb;
      o.w = g * (exp_neg_fast(x.w - m) / s - (c + 3 == cls ? 1.0f : 0.0f)) / fb;
      o4[i] = o;
    }
  } else {
    for (i64 c = threadIdx.x; c < v; c += blockDim.x) orow[c] = g * (exp_neg_fast(row[c] - m) / s - (c == cls ? 1.0f : 0.0f)) / fb;
  }
}
// Forward and backward in one pass over the logits, in place: the row's (max, sum) pass is followed, while the row is still in
// L2, by the pass that overwrites it with d loss / d logits for an upstream gradient of 1 (the value a loss gets from
// backward()); the row's loss term comes out of the first pass.  Algorithmic bytes 2 * rows * V * 4 for both directions
// together -- what the backward alone moves otherwise.
__global__ void k_ce_fused(float* __restrict__ logits, const float* __restrict__ targets, float* __restrict__ row_loss, i64 rows, i64 v, int* err) {
  __shared__ float red[64];
  __shared__ i64 s_cls;
  const i64 r = blockIdx.x;
  float* row = logits + r * v;
  float m, s;
  row_max_sum(row, v, m, s, red);
  if (threadIdx.x == 0) {
    const i64 cls = checked_id(targets[r], v, err);
    row_loss[r] = cls < 0 ? 0.0f : -(row[cls] - m - logf(s));
    s_cls = cls;
  }
  __syncthreads();      // the loss term has read row[cls] before anyone overwrites it
  const i64 cls = s_cls;
  // (softmax - onehot) / rows with the two divisions as multiplications by reciprocals formed once per row: a correctly rounded
  // division costs several times a multiplication and this pass is short of issue slots, not of bandwidth (results move by an ulp)
  const float inv_s = 1.0f / s, inv_fb = 1.0f / (float)rows;
  if ((v & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    float4* r4 = reinterpret_cast<float4*>(row);
    const i64 cq = cls >= 0 ? cls / 4 : -1;
    for (i64 i = threadIdx.x; i < v / 4; i += blockDim.x) {
      const float4 x = r4[i];
      float4 o;
      o.x = exp_neg_fast(x.x - m) * inv_s; o.y = exp_neg_fast(x.y - m) * inv_s; o.z = exp_neg_fast(x.z - m) * inv_s; o.w = exp_neg_fast(x.w - m) * inv_s;
      if (i == cq) reinterpret_cast<float*>(&o)[cls & 3] -= 1.0f;
      o.x *= inv_fb; o.y *= inv_fb; o.z *= inv_fb; o.w *= inv_fb;
      r4[i] = o;
    }
  } else {
    for (i64 c = threadIdx.x; c < v; c += blockDim.x) row[c] = (exp_neg_fast(row[c] - m) * inv_s - (c == cls ? 1.0f : 0.0f)) * inv_fb;
  }
}
int launch_cross_entropy_fused(float* logits, const float* targets, float* loss, i64 rows, i64 v) {
  void* rl = nullptr;
  VB_TRY(scratch_alloc((size_t)rows * sizeof(float), &rl));
  ProfScope prof("cross_entropy_fused", 2.0 * (double)rows * (double)v * 4.0);
  // long rows: 1024 threads per row, so that at most two rows per SM are in flight and the second pass finds its row in L2
  // (with 512 threads and four rows per SM the row came from HBM again: 759 MB read for 412 MB of logits)
  int threads = v >= 32768 ? 1024 : (v >= 8192 ? 512 : (v >= 1024 ? 256 : 64));
  k_ce_fused<<<(unsigned)rows, threads, 0, ctx().stream>>>(logits, targets, (float*)rl, rows, v, ctx().d_err);
  k_ce_mean<<<1, 1024, 0, ctx().stream>>>((const float*)rl, loss, rows);
  scratch_free(rl);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

int launch_cross_entropy_backward(const float* logits, const float* targets, const float* gout, const float* stats,
                                  float* gl, i64 rows, i64 v) {
  if (rows <= 0 || v <= 0) return VB_OK;
  ProfScope prof("cross_entropy_bwd", (stats ? 2.0 : 3.0) * (double)rows * (double)v * 4.0);
  int threads = v >= 8192 ? 512 : (v >= 1024 ? 256 : 64);
  if (stats) k_ce_backward<true><<<(unsigned)rows, threads, 0, ctx().stream>>>(logits, targets, gout, stats, gl, rows, v, ctx().d_err);
  else k_ce_backward<false><<<(unsigned)rows, threads, 0, ctx().stream>>>(logits, targets, gout, stats, gl, rows, v, ctx().d_err);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
