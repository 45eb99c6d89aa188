// Plain-C handles over the C++ host mirror, for drivers written in another language (the Python
// tests and the benchmark).  Pure plumbing: each function forwards to one method of
// vearo::Tensor / autograd / nn / optim and converts exceptions into a status + message.
#include "vearo_host.h"
#include <cstring>
#include <memory>

using namespace vearo;

namespace {
thread_local std::string t_msg;
// never destroyed: at process exit the device context may already be gone
std::vector<std::unique_ptr<Tensor>>& g_t = *new std::vector<std::unique_ptr<Tensor>>();
std::vector<int>& g_free = *new std::vector<int>();
std::vector<std::unique_ptr<nn::Model>>& g_models = *new std::vector<std::unique_ptr<nn::Model>>();
std::vector<std::unique_ptr<optim::Optimizer>>& g_opts = *new std::vector<std::unique_ptr<optim::Optimizer>>();

int put(const Tensor& t) {
  if (!g_free.empty()) { int h = g_free.back(); g_free.pop_back(); g_t[h].reset(new Tensor(t)); return h; }
  g_t.emplace_back(new Tensor(t));
  return (int)g_t.size() - 1;
}
Tensor& at(int h) {
  if (h < 0 || h >= (int)g_t.size() || !g_t[h]) throw Error("bad tensor handle");
  return *g_t[h];
}
nn::Model& model(int m) { if (m < 0 || m >= (int)g_models.size() || !g_models[m]) throw Error("bad model handle"); return *g_models[m]; }
optim::Optimizer& opt(int o) { if (o < 0 || o >= (int)g_opts.size() || !g_opts[o]) throw Error("bad optimizer handle"); return *g_opts[o]; }
}  // namespace

#define VH_TRY(...) try { __VA_ARGS__; } catch (const std::exception& e) { t_msg = e.what(); return -1; }

extern "C" {
const char* vh_last_error() { return t_msg.c_str(); }

int vh_tensor(const float* data, const int64_t* shape, int rank, int requires_grad) {
  VH_TRY(Tensor t = Tensor::from_f32(data, std::vector<i64>(shape, shape + rank)); t.set_requires_grad(requires_grad != 0); return put(t));
}
int vh_free(int h) { VH_TRY(at(h); g_t[h].reset(); g_free.push_back(h); return 0); }
int vh_rank(int h) { VH_TRY(return at(h).rank()); }
int vh_shape(int h, int64_t* out) { VH_TRY(Tensor& t = at(h); for (int i = 0; i < t.rank(); ++i) out[i] = t.desc().dims[i]; return t.rank()); }
int vh_read(int h, float* out) { VH_TRY(std::vector<float> v = at(h).to_vec_f32(); if (!v.empty()) std::memcpy(out, v.data(), v.size() * sizeof(float)); return 0); }
int vh_write(int h, const float* in) { VH_TRY(at(h).write_f32(in); return 0); }
int vh_set_requires_grad(int h, int f) { VH_TRY(at(h).set_requires_grad(f != 0); return 0); }
int vh_is_contiguous(int h) { VH_TRY(return at(h).is_contiguous() ? 1 : 0); }
int vh_desc(int h, vb_tensor* out) { VH_TRY(*out = at(h).desc(); return 0); }

int vh_binary(int op, int a, int b) {
  VH_TRY(Tensor& x = at(a); Tensor& y = at(b);
         return put(op == 0 ? x.add(y) : op == 1 ? x.sub(y) : op == 2 ? x.mul(y) : x.div(y)));
}
int vh_matmul(int a, int b) { VH_TRY(return put(at(a).matmul(at(b)))); }
int vh_relu(int a) { VH_TRY(return put(at(a).relu())); }
int vh_gelu(int a) { VH_TRY(return put(at(a).gelu())); }
int vh_softmax(int a, int dim) { VH_TRY(return put(at(a).softmax(dim))); }
int vh_sum(int a, int dim, int keep) { VH_TRY(return put(at(a).sum(dim, keep != 0))); }
int vh_mean(int a, int dim, int keep) { VH_TRY(return put(at(a).mean(dim, keep != 0))); }
int vh_layernorm(int x, int w, int b, float eps) { VH_TRY(return put(at(x).layernorm(at(w), at(b), eps))); }
int vh_embedding(int ids, int w) { VH_TRY(return put(at(ids).embedding(at(w)))); }
int vh_cross_entropy(int l, int t) { VH_TRY(return put(at(l).cross_entropy(at(t)))); }
int vh_cross_entropy_consuming(int l, int t) { VH_TRY(return put(at(l).cross_entropy_consuming(at(t)))); }
int vh_conv2d(int x, int w, int b, int stride, int pad) { VH_TRY(return put(at(x).conv2d(at(w), at(b), stride, pad))); }
int vh_maxpool2d(int x, int k, int s, int p) { VH_TRY(return put(at(x).maxpool2d(k, s, p))); }
int vh_avgpool2d(int x, int k, int s, int p) { VH_TRY(return put(at(x).avgpool2d(k, s, p))); }
int vh_fused_attention_packed(int qkv, int n_head, int mask) { VH_TRY(return put(at(qkv).fused_attention_packed(n_head, mask >= 0 ? &at(mask) : nullptr))); }
int vh_bn_relu_maxpool(int x, int g, int b, int rm, int rv, int training, float mom, float eps) {
  VH_TRY(return put(at(x).bn_relu_maxpool(at(g), at(b), at(rm), at(rv), training != 0, mom, eps)));
}
int vh_batchnorm(int x, int g, int b, int rm, int rv, int training, float mom, float eps) {
  VH_TRY(return put(at(x).batchnorm(at(g), at(b), at(rm), at(rv), training != 0, mom, eps)));
}
int vh_fused_attention(int q, int k, int v, int mask) { VH_TRY(return put(at(q).fused_attention(at(k), at(v), mask >= 0 ? &at(mask) : nullptr))); }
int vh_linear(int x, int w, int b) { VH_TRY(return put(at(x).linear(at(w), b >= 0 ? &at(b) : nullptr))); }
int vh_linear_gelu(int x, int w, int b) { VH_TRY(return put(at(x).linear_gelu(at(w), b >= 0 ? &at(b) : nullptr))); }
int vh_reshape(int a, const int64_t* shape, int rank) { VH_TRY(return put(at(a).reshape(std::vector<i64>(shape, shape + rank)))); }
int vh_transpose(int a, int d0, int d1) { VH_TRY(return put(at(a).transpose(d0, d1))); }
int vh_permute(int a, const int64_t* axes, int rank) { VH_TRY(return put(at(a).permute(std::vector<i64>(axes, axes + rank)))); }
int vh_contiguous(int a) { VH_TRY(return put(at(a).contiguous())); }

int vh_backward(int h) { VH_TRY(at(h).backward(); return 0); }
int vh_grad(int h) { VH_TRY(Tensor g; if (!at(h).grad(&g)) return -2; return put(g)); }
void vh_zero_gradients() { autograd::zero_gradients(); }
void vh_reset_active_tape() { autograd::reset_active_tape(); }
void vh_set_training(int t) { autograd::set_training(t != 0); }
void vh_set_autograd_enabled(int e) { autograd::set_enabled(e != 0); }

// ---- models ----
int vh_gpt_new(int64_t vocab, int64_t max_seq, int64_t d, int64_t heads, int64_t layers, int64_t ff) {
  VH_TRY(g_models.emplace_back(new nn::SimpleGPT(vocab, max_seq, d, heads, layers, ff)); return (int)g_models.size() - 1);
}
int vh_mlp_new(const int64_t* sizes, int n) { VH_TRY(g_models.emplace_back(new nn::MLP(std::vector<i64>(sizes, sizes + n))); return (int)g_models.size() - 1); }
int vh_convnet_new(const int64_t* channels, int n, int64_t n_class) {
  VH_TRY(g_models.emplace_back(new nn::ConvNet(std::vector<i64>(channels, channels + n), n_class)); return (int)g_models.size() - 1);
}
int vh_fusedop_new(int64_t c, int64_t v) { VH_TRY(g_models.emplace_back(new nn::FusedOpBench(c, v)); return (int)g_models.size() - 1); }
int vh_model_free(int m) { VH_TRY(model(m); g_models[m].reset(); return 0); }
int vh_model_num_params(int m) { VH_TRY(return (int)model(m).parameters().size()); }
int vh_model_param(int m, int i) { VH_TRY(std::vector<Tensor> p = model(m).parameters(); if (i < 0 || i >= (int)p.size()) throw Error("parameter index out of range"); return put(p[i])); }
int vh_model_loss(int m, int x, int y) { VH_TRY(return put(model(m).loss(at(x), at(y)))); }
// ConvNet running statistics (stage s: 0 = running_mean, 1 = running_var)
int vh_convnet_running(int m, int stage, int which) {
  VH_TRY(nn::ConvNet* c = dynamic_cast<nn::ConvNet*>(&model(m)); if (!c) throw Error("not a ConvNet");
         if (stage < 0 || stage >= (int)c->stages.size()) throw Error("stage out of range");
         return put(which == 0 ? c->stages[stage].rm : c->stages[stage].rv));
}

// Activation checkpointing.  vh_checkpoint: `fn(x_handle, user)` returns the handle of the block's output (or a negative value on
// failure); it is called once now, without recording, and once more during backward.  The caller keeps `fn` and `user` alive until then.
int vh_checkpoint(int x, int (*fn)(int, void*), void* user) {
  VH_TRY(Tensor out = autograd::checkpoint(at(x), [fn, user](const Tensor& in) {
           int hin = put(in);
           int hout = fn(hin, user);
           if (hout < 0) throw Error("checkpoint callback failed");
           return at(hout);
         });
         return put(out));
}
int vh_dropout(int x, float p, uint64_t seed) { VH_TRY(return put(nn::Dropout(p, seed).forward(at(x)))); }
uint64_t vh_rng_counter() { return autograd::rng_counter(); }
void vh_set_rng_counter(uint64_t v) { autograd::set_rng_counter(v); }
int vh_is_recomputing() { return autograd::is_recomputing() ? 1 : 0; }
int vh_gpt_set_checkpointing(int m, int on) {
  VH_TRY(nn::SimpleGPT* g = dynamic_cast<nn::SimpleGPT*>(&model(m)); if (!g) throw Error("not a SimpleGPT"); g->checkpoint_blocks = on != 0; return 0);
}

// ---- optimizers ----
static int make_opt(const vb_opt_config& cfg, const int* params, int n, int dp) {
  std::vector<Tensor> ps; for (int i = 0; i < n; ++i) ps.push_back(at(params[i]));
  g_opts.emplace_back(new optim::Optimizer(cfg, ps, dp != 0));
  return (int)g_opts.size() - 1;
}
int vh_adamw_new(const int* params, int n, float lr, float b1, float b2, float eps, float wd, int data_parallel) {
  VH_TRY(vb_opt_config c{VB_OPT_ADAMW, lr, b1, b2, eps, wd, 0.0f}; return make_opt(c, params, n, data_parallel));
}
// AdamW8bit::new (vearo-optim/src/lib.rs:225-253): block-wise int8 moments, blocks of 256
int vh_adamw8bit_new(const int* params, int n, float lr, float b1, float b2, float eps, float wd, int data_parallel) {
  VH_TRY(vb_opt_config c{VB_OPT_ADAMW8BIT, lr, b1, b2, eps, wd, 0.0f}; return make_opt(c, params, n, data_parallel));
}
int vh_opt_state8(int o, int param, int8_t* m8, float* ms, int8_t* v8, float* vs) {
  VH_TRY(if (vb_opt_state8(opt(o).handle(), param, m8, ms, v8, vs) != 0) throw Error(vb_last_error()); return 0);
}
int vh_sgd_new(const int* params, int n, float lr, float momentum, float wd, int data_parallel) {
  VH_TRY(vb_opt_config c{VB_OPT_SGD, lr, 0.0f, 0.0f, 0.0f, wd, momentum}; return make_opt(c, params, n, data_parallel));
}
int vh_opt_free(int o) { VH_TRY(opt(o); g_opts[o].reset(); return 0); }
int vh_opt_step(int o) { VH_TRY(opt(o).step(); return 0); }
int vh_opt_clip_and_step(int o, float max_norm, float* norm) { VH_TRY(float n = opt(o).clip_and_step(max_norm); if (norm) *norm = n; return 0); }
int vh_opt_save_state(int o, const char* path) { VH_TRY(opt(o).save_state(path); return 0); }
int vh_opt_load_state(int o, const char* path) { VH_TRY(opt(o).load_state(path); return 0); }
int vh_save_checkpoint(int m, const char* path) { VH_TRY(checkpoint::save_checkpoint(model(m).parameters(), path); return 0); }
int vh_load_checkpoint(int m, const char* path) { VH_TRY(checkpoint::load_checkpoint(model(m).parameters(), path); return 0); }
int vh_opt_handle(int o) { VH_TRY(return opt(o).handle()); }       // the library's vb_opt_* handle of this optimizer
int vh_opt_gradients_registered(int o) { VH_TRY(return opt(o).gradients_registered() ? 1 : 0); }
int vh_opt_set_lr(int o, float lr) { VH_TRY(opt(o).set_lr(lr); return 0); }
int vh_clip_grad_norm(const int* params, int n, float max_norm, float* norm) {
  VH_TRY(std::vector<Tensor> ps; for (int i = 0; i < n; ++i) ps.push_back(at(params[i])); *norm = optim::clip_grad_norm(ps, max_norm); return 0);
}
float vh_cosine_lr(float base, float min_lr, uint32_t warmup, uint32_t total, uint32_t step) { return optim::cosine_lr(base, min_lr, warmup, total, step); }

// Gradient-bucket plan (host arithmetic only, usable without a device): fills param_offset[n], bucket_of[n],
// and up to `max_buckets` entries of bucket_offset / bucket_numel; returns the number of buckets.
int vh_plan_buckets(const int64_t* numels, int n, int64_t target_elems, int64_t* param_offset, int* bucket_of,
                    int64_t* bucket_offset, int64_t* bucket_numel, int max_buckets, int64_t* total) {
  VH_TRY(optim::BucketPlan bp = optim::plan_buckets(std::vector<i64>(numels, numels + n), target_elems);
         if ((int)bp.bucket_offset.size() > max_buckets) throw Error("too many buckets for the caller's arrays");
         for (int i = 0; i < n; ++i) { param_offset[i] = bp.param_offset[i]; bucket_of[i] = bp.bucket_of[i]; }
         for (size_t b = 0; b < bp.bucket_offset.size(); ++b) { bucket_offset[b] = bp.bucket_offset[b]; bucket_numel[b] = bp.bucket_numel[b]; }
         if (total) *total = bp.total;
         return (int)bp.bucket_offset.size());
}

// One whole training step from HOST buffers: upload inputs, zero_gradients, reset tape, forward,
// backward (gradient exchange overlapped when data parallel), clip + optimizer step, read the loss.
// x / y are flat f32 arrays with the given shapes.  max_norm <= 0: no clipping.
int vh_train_step(int m, int o, const float* x, const int64_t* xshape, int xrank, int x_requires_grad,
                  const float* y, const int64_t* yshape, int yrank, float max_norm, float* loss, float* grad_norm) {
  VH_TRY(
    autograd::zero_gradients(); autograd::reset_active_tape();
    Tensor tx = Tensor::from_f32(x, std::vector<i64>(xshape, xshape + xrank));
    tx.set_requires_grad(x_requires_grad != 0);
    Tensor ty = Tensor::from_f32(y, std::vector<i64>(yshape, yshape + yrank));
    Tensor l = model(m).loss(tx, ty);
    l.backward();
    float n = 0.0f;
    if (max_norm > 0.0f) n = opt(o).clip_and_step(max_norm); else opt(o).step();
    std::vector<float> lv = l.to_vec_f32();
    if (loss) *loss = lv[0];
    if (grad_norm) *grad_norm = n;
    return 0);
}
// The same step with inputs already resident on the device (handles), loss left on the device.
int vh_train_step_resident(int m, int o, int x, int y, float max_norm) {
  VH_TRY(
    autograd::zero_gradients(); autograd::reset_active_tape();
    Tensor l = model(m).loss(at(x), at(y));
    l.backward();
    if (max_norm > 0.0f) opt(o).clip_and_step(max_norm, false); else opt(o).step();
    return put(l));
}
}
