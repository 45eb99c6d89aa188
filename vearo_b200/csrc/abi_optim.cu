// Optimizer entry points of the C ABI (host side of optim.cu).
//
// vb_adamw_step / vb_sgd_step are per-tensor, the shape of Tensor::adamw_step / sgd_step
// (crates/vearo-core/src/tensor.rs:931-1096).  vb_opt_* is the fused multi-tensor form: the
// chunk table is built once and stays in device memory; a step is three launches (sum of squares
// per chunk, sum of partials, update) or one when clipping is off.
#include "common.h"
#include <cmath>
#include <memory>

using namespace vb;

namespace {
// f32::powi as the reference's bias corrections use it (tensor.rs:972-973): repeated squaring.
float powi(float a, int n) {
  float r = 1.0f;
  while (true) { if (n & 1) r *= a; n /= 2; if (n == 0) break; a *= a; }
  return r;
}
constexpr int kChunk = 16384;

struct Opt {
  vb_opt_config cfg;
  uint32_t t = 0;
  int nparams = 0, nchunks = 0;
  vb_slot state = 0;           // m then v (AdamW) or velocity (SGD), flat
  void* d_chunks = nullptr;    // OptChunk[nchunks]
  void* d_partials = nullptr;  // float[nchunks]
  void* d_active = nullptr;    // uint8[nparams]
  std::vector<vb_slot> retained;
  std::vector<OptChunk> h_chunks;          // host copy of the chunk table (re-uploaded when a weight gains or loses its lo plane)
  std::vector<float*> lo_base;             // per parameter: the lo plane its chunks write to (null: none)
  // 8-bit AdamW: byte offset of every parameter's share of the int8 planes, their common length, and the parameter sizes
  std::vector<i64> off8, numel8; i64 total8 = 0;
};
std::vector<std::unique_ptr<Opt>>& g_opts = *new std::vector<std::unique_ptr<Opt>>();
}  // namespace

extern "C" {

int vb_adamw_step(const vb_tensor* param, const vb_tensor* grad, vb_slot m, vb_slot v, uint32_t t,
                  float lr, float beta1, float beta2, float eps, float weight_decay) {
  VB_CHECK(same_shape(*param, *grad), "adamw_step shapes must match");
  VB_CHECK(is_contiguous(*param), "adamw_step self must be contiguous");
  VB_CHECK(is_contiguous(*grad), "adamw_step grad must be contiguous");
  VB_CHECK(t >= 1, "adamw_step expects t >= 1");
  float *pw, *pg, *pm, *pv; i64 nm, nv;
  VB_TRY(tensor_ptr(param, &pw)); VB_TRY(tensor_ptr(grad, &pg));
  VB_TRY(slot_ptr(m, &pm, &nm)); VB_TRY(slot_ptr(v, &pv, &nv));
  i64 n = numel(*param);
  VB_CHECK(nm == n, "Momentum vector m must match parameter length");
  VB_CHECK(nv == n, "Variance vector v must match parameter length");
  float bc1 = 1.0f - powi(beta1, (int)t), bc2 = 1.0f - powi(beta2, (int)t);
  slot_touch(param->slot);
  return launch_adamw_single(pw, pg, pm, pv, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2);
}
int vb_sgd_step(const vb_tensor* param, const vb_tensor* grad, vb_slot velocity, float lr, float momentum, float weight_decay) {
  VB_CHECK(same_shape(*param, *grad), "sgd_step shapes must match");
  VB_CHECK(is_contiguous(*param), "sgd_step self must be contiguous");
  VB_CHECK(is_contiguous(*grad), "sgd_step grad must be contiguous");
  float *pw, *pg, *pv; i64 nv;
  VB_TRY(tensor_ptr(param, &pw)); VB_TRY(tensor_ptr(grad, &pg)); VB_TRY(slot_ptr(velocity, &pv, &nv));
  VB_CHECK(nv == numel(*param), "Velocity vector must match parameter length");
  slot_touch(param->slot);
  return launch_sgd_single(pw, pg, pv, numel(*param), lr, momentum, weight_decay);
}

int vb_clip_grad_norm(const vb_tensor* grads, int n, float max_norm, float* total_norm) {
  VB_CHECK(n >= 0, "negative count");
  std::vector<OptChunk> chunks;
  for (int i = 0; i < n; ++i) {
    VB_CHECK(is_contiguous(grads[i]), "clip_grad_norm expects contiguous grads");
    float* p; VB_TRY(tensor_ptr(&grads[i], &p));
    i64 cnt = numel(grads[i]);
    for (i64 o = 0; o < cnt; o += kChunk) chunks.push_back(OptChunk{nullptr, p + o, nullptr, nullptr, (int)(cnt - o < kChunk ? cnt - o : kChunk), i});
  }
  float* d_norm = ctx().d_scalars;   // [0]
  if (chunks.empty()) { if (total_norm) *total_norm = 0.0f; return VB_OK; }
  void *d_ch = nullptr, *d_pa = nullptr;
  VB_TRY(scratch_alloc(chunks.size() * sizeof(OptChunk), &d_ch));
  int rc = scratch_alloc(chunks.size() * sizeof(float), &d_pa);
  if (rc == VB_OK) {
    cudaError_t e = cudaMemcpyAsync(d_ch, chunks.data(), chunks.size() * sizeof(OptChunk), cudaMemcpyHostToDevice, ctx().stream);
    if (e != cudaSuccess) rc = set_error(VB_ERR_CUDA, cudaGetErrorString(e));
    // pageable source: the copy has been staged before the call returns, `chunks` may go away
  }
  if (rc == VB_OK) rc = launch_sumsq_chunks((const OptChunk*)d_ch, (int)chunks.size(), nullptr, (float*)d_pa);
  if (rc == VB_OK) rc = launch_sum_partials((const float*)d_pa, (int)chunks.size(), d_norm);
  for (int i = 0; rc == VB_OK && i < n; ++i) {
    float* p; tensor_ptr(&grads[i], &p);
    slot_touch(grads[i].slot);          // scaled in place: a lo plane or a cached verdict about the old contents is void
    rc = launch_scale_inplace_by_clip(p, numel(grads[i]), d_norm, max_norm);
  }
  float h = 0.0f;
  if (rc == VB_OK) {
    cudaError_t e = cudaMemcpyAsync(&h, d_norm, sizeof(float), cudaMemcpyDeviceToHost, ctx().stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx().stream);
    if (e != cudaSuccess) rc = set_error(VB_ERR_CUDA, cudaGetErrorString(e));
  }
  if (d_ch) scratch_free(d_ch);
  if (d_pa) scratch_free(d_pa);
  if (rc == VB_OK && total_norm) *total_norm = sqrtf(h);
  return rc;
}

int vb_opt_create(const vb_opt_config* cfg, const vb_tensor* params, const vb_tensor* grads, int n, int* opt) {
  VB_CHECK(cfg && opt && n >= 0, "bad arguments");
  VB_CHECK(cfg->kind == VB_OPT_ADAMW || cfg->kind == VB_OPT_SGD || cfg->kind == VB_OPT_ADAMW8BIT, "unknown optimizer kind");
  const bool q8 = cfg->kind == VB_OPT_ADAMW8BIT;
  auto o = std::make_unique<Opt>();
  o->cfg = *cfg; o->nparams = n;
  i64 total = 0;
  for (int i = 0; i < n; ++i) {
    VB_CHECK(is_contiguous(params[i]) && is_contiguous(grads[i]), "optimizer tensors must be contiguous");
    VB_CHECK(numel(params[i]) == numel(grads[i]), "param / grad sizes differ");
    if (q8) { o->off8.push_back(total); o->numel8.push_back(numel(params[i])); total += (numel(params[i]) + 255) & ~i64(255); }   // whole blocks of 256
    else total += (numel(params[i]) + 3) & ~i64(3);   // keep every tensor's state 16-byte aligned
  }
  int planes = cfg->kind == VB_OPT_SGD ? 1 : 2;
  // 8-bit: two planes of `total` bytes, then two planes of total / 256 scales -- counted in floats for the slot
  const i64 state_floats = q8 ? total / 2 + 2 * (total / 256) : total * planes;
  o->total8 = q8 ? total : 0;
  VB_TRY(slot_alloc(state_floats > 0 ? state_floats : 1, true, &o->state));
  float* st; VB_TRY(slot_ptr(o->state, &st));
  int8_t* st8 = reinterpret_cast<int8_t*>(st);
  float* scales8 = st + total / 2;
  std::vector<OptChunk> chunks;
  i64 off = 0;
  for (int i = 0; i < n; ++i) {
    float *pw, *pg; VB_TRY(tensor_ptr(&params[i], &pw)); VB_TRY(tensor_ptr(&grads[i], &pg));
    i64 cnt = numel(params[i]);
    for (i64 c = 0; c < cnt; c += kChunk) {
      OptChunk ch; ch.w = pw + c; ch.g = pg + c; ch.ms = ch.vs = nullptr; ch.lo = nullptr;
      if (q8) {
        ch.m = reinterpret_cast<float*>(st8 + off + c); ch.v = reinterpret_cast<float*>(st8 + total + off + c);
        ch.ms = scales8 + (off + c) / 256; ch.vs = scales8 + total / 256 + (off + c) / 256;
      } else { ch.m = st + off + c; ch.v = planes == 2 ? st + total + off + c : nullptr; }
      ch.n = (int)(cnt - c < kChunk ? cnt - c : kChunk); ch.param = i;
      chunks.push_back(ch);
    }
    off += q8 ? ((cnt + 255) & ~i64(255)) : ((cnt + 3) & ~i64(3));
    VB_TRY(slot_retain(params[i].slot)); o->retained.push_back(params[i].slot);
    VB_TRY(slot_retain(grads[i].slot)); o->retained.push_back(grads[i].slot);
  }
  o->nchunks = (int)chunks.size();
  o->h_chunks = chunks; o->lo_base.assign((size_t)n, nullptr);
  VB_TRY(scratch_alloc((chunks.size() + 1) * sizeof(OptChunk), &o->d_chunks));
  VB_TRY(scratch_alloc((chunks.size() + 1) * sizeof(float), &o->d_partials));
  VB_TRY(scratch_alloc((size_t)n + 16, &o->d_active));
  if (!chunks.empty()) VB_CUDA(cudaMemcpyAsync(o->d_chunks, chunks.data(), chunks.size() * sizeof(OptChunk), cudaMemcpyHostToDevice, ctx().stream));
  VB_CUDA(cudaStreamSynchronize(ctx().stream));
  g_opts.push_back(std::move(o));
  *opt = (int)g_opts.size() - 1;
  return VB_OK;
}
static int get_opt(int id, Opt** o) {
  if (id < 0 || id >= (int)g_opts.size() || !g_opts[id]) return set_error(VB_ERR_INVALID, "bad optimizer handle");
  *o = g_opts[id].get();
  return VB_OK;
}
int vb_opt_destroy(int id) {
  Opt* o; VB_TRY(get_opt(id, &o));
  for (vb_slot s : o->retained) slot_release(s, nullptr);
  slot_release(o->state, nullptr);
  scratch_free(o->d_chunks); scratch_free(o->d_partials); scratch_free(o->d_active);
  g_opts[id].reset();
  return VB_OK;
}
int vb_opt_state(int id, vb_slot* state, int64_t* state_numel, uint32_t* step) {
  Opt* o; VB_TRY(get_opt(id, &o));
  if (state) *state = o->state;
  if (state_numel) { float* p; VB_TRY(slot_ptr(o->state, &p, state_numel)); }
  if (step) *step = o->t;
  return VB_OK;
}
int vb_opt_state8(int id, int param, int8_t* m8, float* m_scales, int8_t* v8, float* v_scales) {
  Opt* o; VB_TRY(get_opt(id, &o));
  VB_CHECK(o->cfg.kind == VB_OPT_ADAMW8BIT, "not an 8-bit optimizer");
  VB_CHECK(param >= 0 && param < o->nparams && m8 && m_scales && v8 && v_scales, "bad arguments");
  float* st; VB_TRY(slot_ptr(o->state, &st));
  const int8_t* st8 = reinterpret_cast<const int8_t*>(st);
  const float* sc = st + o->total8 / 2;
  const i64 off = o->off8[param], n = o->numel8[param], nb = (n + 255) / 256;
  cudaStream_t s = ctx().stream;
  if (n > 0) {
    VB_CUDA(cudaMemcpyAsync(m8, st8 + off, (size_t)n, cudaMemcpyDeviceToHost, s));
    VB_CUDA(cudaMemcpyAsync(v8, st8 + o->total8 + off, (size_t)n, cudaMemcpyDeviceToHost, s));
    VB_CUDA(cudaMemcpyAsync(m_scales, sc + off / 256, (size_t)nb * sizeof(float), cudaMemcpyDeviceToHost, s));
    VB_CUDA(cudaMemcpyAsync(v_scales, sc + o->total8 / 256 + off / 256, (size_t)nb * sizeof(float), cudaMemcpyDeviceToHost, s));
  }
  VB_CUDA(cudaStreamSynchronize(s));
  return VB_OK;
}
int vb_opt_set_step(int id, uint32_t step) { Opt* o; VB_TRY(get_opt(id, &o)); o->t = step; return VB_OK; }
int vb_opt_set_lr(int id, float lr) { Opt* o; VB_TRY(get_opt(id, &o)); o->cfg.lr = lr; return VB_OK; }

int vb_opt_step(int id, const uint8_t* active, float max_norm, float grad_scale, float* total_norm) {
  Opt* o; VB_TRY(get_opt(id, &o));
  const vb_opt_config& c = o->cfg;
  if (c.kind != VB_OPT_SGD) o->t += 1;
  const uint8_t* d_active = nullptr;
  if (active && o->nparams > 0) {
    VB_CUDA(cudaMemcpyAsync(o->d_active, active, (size_t)o->nparams, cudaMemcpyHostToDevice, ctx().stream));
    d_active = (const uint8_t*)o->d_active;
  }
  float* d_normsq = ctx().d_scalars + 1;
  bool need_norm = max_norm > 0.0f || total_norm;
  if (need_norm && o->nchunks > 0) {
    VB_TRY(launch_sumsq_chunks((const OptChunk*)o->d_chunks, o->nchunks, d_active, (float*)o->d_partials));
    VB_TRY(launch_sum_partials((const float*)o->d_partials, o->nchunks, d_normsq));
  }
  // weights that keep a lo plane for the tensor-core GEMM get it rewritten by the update itself
  {
    bool changed = false;
    std::vector<float*> wbase((size_t)o->nparams, nullptr);
    for (int i = 0; i < o->nparams; ++i) {
      float* lb = lo_plane_base_for(o->retained[2 * (size_t)i], &wbase[i]);
      if (lb != o->lo_base[i]) { o->lo_base[i] = lb; changed = true; }
    }
    if (changed && o->nchunks > 0) {
      for (OptChunk& ch : o->h_chunks) ch.lo = o->lo_base[ch.param] ? o->lo_base[ch.param] + (ch.w - wbase[ch.param]) : nullptr;
      VB_CUDA(cudaMemcpyAsync(o->d_chunks, o->h_chunks.data(), o->h_chunks.size() * sizeof(OptChunk), cudaMemcpyHostToDevice, ctx().stream));
    }
  }
  float bc1 = 1.0f, bc2 = 1.0f;
  if (c.kind != VB_OPT_SGD) { bc1 = 1.0f - powi(c.beta1, (int)o->t); bc2 = 1.0f - powi(c.beta2, (int)o->t); }
  int lo_chunks = 0;
  for (const OptChunk& ch : o->h_chunks) if (ch.lo) ++lo_chunks;
  VB_TRY(launch_opt_multi((const OptChunk*)o->d_chunks, o->nchunks, d_active, c.kind, d_normsq, max_norm, grad_scale,
                          c.lr, c.beta1, c.beta2, c.eps, c.weight_decay, c.momentum, bc1, bc2, lo_chunks));
  // the updated parameters' contents changed; a lo plane that was current before stays so (the kernel rewrote the updated part)
  {
    std::vector<uint8_t> was((size_t)o->nparams, 0);
    for (int i = 0; i < o->nparams; ++i) was[i] = o->lo_base[i] && lo_plane_is_current(o->retained[2 * (size_t)i]);
    for (int i = 0; i < o->nparams; ++i) if (!(active && !active[i])) slot_touch(o->retained[2 * (size_t)i]);
    for (int i = 0; i < o->nparams; ++i) if (was[i]) lo_plane_mark_current(o->retained[2 * (size_t)i]);
  }
  if (total_norm) {
    float h = 0.0f;
    if (o->nchunks > 0) {
      VB_CUDA(cudaMemcpyAsync(&h, d_normsq, sizeof(float), cudaMemcpyDeviceToHost, ctx().stream));
      VB_CUDA(cudaStreamSynchronize(ctx().stream));
    }
    *total_norm = sqrtf(h) * fabsf(grad_scale);
  }
  return VB_OK;
}

}  // extern "C"
