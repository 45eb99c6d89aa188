// Layers, the five workload graphs, and the optimizers, above the C ABI.
//
// Layers follow crates/vearo-nn/src/lib.rs: Linear (63-137), LayerNorm (510-543),
// MultiHeadAttention (546-633), TransformerBlock pre-LN (636-688), SimpleGPT (691-808).  Where the
// reference emits `transpose -> matmul -> add` for a Linear, this host layer issues one fused
// `linear` op (a GEMM with a bias epilogue and a single backward node); the unfused ops stay
// available on Tensor for arbitrary graphs.  Parameters are created zero-filled / unit-filled and
// are meant to be overwritten by the caller (tests and benchmarks upload seeded arrays), in the
// order of the reference's `parameters()` methods.
//
// Optimizers follow crates/vearo-optim/src/lib.rs: AdamW::step (105-123), SGD::step (33-46),
// clip_grad_norm (360-383), CosineSchedule::lr_at (336-348) — with state on the device and one
// fused launch for all parameters.
#include "vearo_host.h"
#include <cstdlib>
#include <cmath>
#include <cstdio>
#include <cstring>

namespace vearo {
namespace nn {

static Tensor filled(const std::vector<i64>& shape, float v) {
  i64 n = 1; for (i64 d : shape) n *= d;
  std::vector<float> h((size_t)n, v);
  Tensor t = Tensor::from_f32(h.data(), shape);
  t.set_requires_grad(true);
  return t;
}
Tensor Dropout::forward(const Tensor& x) const {
  if (p <= 0.0f || !autograd::is_training()) return x;
  const float scale = 1.0f / (1.0f - p);
  const uint64_t call = autograd::next_rng_counter();
  uint64_t st = seed ^ (call * 0x9E3779B97F4A7C15ull);
  if (st == 0) st = 0x123456789ABCDEF0ull;               // SimpleRng::new, lib.rs:22-30
  std::vector<float> mask((size_t)x.numel());
  for (float& m : mask) {
    st ^= st << 13; st ^= st >> 7; st ^= st << 17;       // next_u64, lib.rs:33-40
    const float u = (float)st / (float)UINT64_MAX;       // next_f32, lib.rs:43-45
    m = u >= p ? scale : 0.0f;
  }
  return x.mul(Tensor::from_f32(mask.data(), x.shape()));
}
static Tensor param_zeros(const std::vector<i64>& shape) { Tensor t = Tensor::zeros(shape); t.set_requires_grad(true); return t; }

Linear::Linear(i64 in, i64 out, bool b) : has_bias(b) {
  if (in <= 0) throw Error("in_features must be greater than 0");
  weight = param_zeros({out, in});
  if (b) bias = param_zeros({out});
}
Tensor Linear::forward(const Tensor& x) const { return x.linear(weight, has_bias ? &bias : nullptr); }
void Linear::parameters(std::vector<Tensor>& out) const { out.push_back(weight); if (has_bias) out.push_back(bias); }

LayerNorm::LayerNorm(i64 dim, float e) : eps(e) { weight = filled({dim}, 1.0f); bias = filled({dim}, 0.0f); }

static Tensor row_block(const Tensor& base, i64 first, i64 rows) {     // rows [first, first + rows) of a contiguous tensor, as a parameter view
  vb_tensor d = base.desc();
  d.dims[0] = rows; d.offset += first * d.strides[0];
  Tensor t = Tensor::view_of(base, d);
  t.set_requires_grad(true);
  return t;
}
MultiHeadAttention::MultiHeadAttention(i64 d, i64 h) : o(d, d, true), n_head(h), n_embd(d) {
  if (d % h != 0) throw Error("n_embd must be divisible by n_head");
  w_qkv = Tensor::zeros({3 * d, d}); b_qkv = Tensor::zeros({3 * d});
  Linear* proj[3] = {&q, &k, &v};
  for (int i = 0; i < 3; ++i) { proj[i]->has_bias = true; proj[i]->weight = row_block(w_qkv, i * d, d); proj[i]->bias = row_block(b_qkv, i * d, d); }
}
// MultiHeadAttention::forward (lib.rs:584-621): q, k, v projections, head split, attention, head merge, output
// projection -- with the three projections as one GEMM over the stacked weights.
Tensor MultiHeadAttention::forward(const Tensor& x, const Tensor* mask) const {
  if (x.rank() != 3) throw Error("MultiHeadAttention expects [B, T, D]");
  Tensor w = Tensor::pack_rows(q.weight, k.weight, v.weight), bias = Tensor::pack_rows(q.bias, k.bias, v.bias);
  Tensor qkv = x.linear(w, &bias);                               // [B, T, 3*D]
  return o.forward(qkv.fused_attention_packed(n_head, mask));
}
void MultiHeadAttention::parameters(std::vector<Tensor>& out) const { q.parameters(out); k.parameters(out); v.parameters(out); o.parameters(out); }

TransformerBlock::TransformerBlock(i64 d, i64 h, i64 ff) : ln1(d), ln2(d), attn(d, h), fc1(d, ff, true), fc2(ff, d, true) {}
Tensor TransformerBlock::forward(const Tensor& x, const Tensor* mask) const {
  Tensor x1 = x.add(attn.forward(ln1.forward(x), mask));
  return x1.add(fc2.forward(ln2.forward(x1).linear_gelu(fc1.weight, fc1.has_bias ? &fc1.bias : nullptr)));
}
void TransformerBlock::parameters(std::vector<Tensor>& out) const {
  ln1.parameters(out); attn.parameters(out); ln2.parameters(out); fc1.parameters(out); fc2.parameters(out);
}

SimpleGPT::SimpleGPT(i64 vocab, i64 max_seq, i64 d, i64 h, i64 n_layer, i64 ff) : ln_f(d), lm_head(d, vocab, false), n_embd(d) {
  tok = param_zeros({vocab, d}); pos = param_zeros({max_seq, d});
  for (i64 i = 0; i < n_layer; ++i) blocks.emplace_back(d, h, ff);
}
std::vector<Tensor> SimpleGPT::parameters() const {
  std::vector<Tensor> p = {tok, pos};
  for (const auto& b : blocks) b.parameters(p);
  ln_f.parameters(p); lm_head.parameters(p);
  return p;
}
// SimpleGPT::forward (lib.rs:741-793).  The reference rebuilds the position ids and the causal
// mask on the CPU device at every call; here they are uploaded once per (B, S) and reused.
Tensor SimpleGPT::loss(const Tensor& ids, const Tensor& targets) {
  std::vector<i64> s = ids.shape();
  i64 b = s[0], t = s[1];
  if (b != cached_b_ || t != cached_s_) {
    std::vector<float> pd((size_t)(b * t)), md((size_t)(t * t), 0.0f);
    for (i64 r = 0; r < b; ++r) for (i64 c = 0; c < t; ++c) pd[r * t + c] = (float)c;
    for (i64 r = 0; r < t; ++r) for (i64 c = r + 1; c < t; ++c) md[r * t + c] = -1e9f;
    pos_ids_ = Tensor::from_f32(pd.data(), {b, t});
    mask_ = Tensor::from_f32(md.data(), {t, t});
    cached_b_ = b; cached_s_ = t;
  }
  Tensor h = ids.embedding(tok).add(pos_ids_.embedding(pos));
  for (const auto& blk : blocks) {
    if (checkpoint_blocks) { const TransformerBlock* bp = &blk; Tensor m = mask_; h = autograd::checkpoint(h, [bp, m](const Tensor& in) { return bp->forward(in, &m); }); }
    else h = blk.forward(h, &mask_);
  }
  Tensor logits = lm_head.forward(ln_f.forward(h).reshape({b * t, n_embd}));
  return logits.cross_entropy_consuming(targets.reshape({b * t}));
}

MLP::MLP(const std::vector<i64>& sizes) { for (size_t i = 0; i + 1 < sizes.size(); ++i) layers.emplace_back(sizes[i], sizes[i + 1], true); }
std::vector<Tensor> MLP::parameters() const { std::vector<Tensor> p; for (const auto& l : layers) l.parameters(p); return p; }
Tensor MLP::forward(const Tensor& x) const {
  Tensor h = x;
  for (size_t i = 0; i < layers.size(); ++i) { h = layers[i].forward(h); if (i + 1 < layers.size()) h = h.relu(); }
  return h;
}
Tensor MLP::loss(const Tensor& x, const Tensor& y) { Tensor diff = forward(x).sub(y); return diff.mul(diff).mean(0, false); }

ConvNet::ConvNet(const std::vector<i64>& ch, i64 n_class) : fc(ch.back(), n_class, true) {
  for (size_t i = 0; i + 1 < ch.size(); ++i) {
    Stage st;
    st.w = param_zeros({ch[i + 1], ch[i], 3, 3}); st.b = param_zeros({ch[i + 1]});
    st.gamma = filled({ch[i + 1]}, 1.0f); st.beta = filled({ch[i + 1]}, 0.0f);
    std::vector<float> ones((size_t)ch[i + 1], 1.0f);
    st.rm = Tensor::zeros({ch[i + 1]}); st.rv = Tensor::from_f32(ones.data(), {ch[i + 1]});
    stages.push_back(st);
  }
}
std::vector<Tensor> ConvNet::parameters() const {
  std::vector<Tensor> p;
  for (const auto& s : stages) { p.push_back(s.w); p.push_back(s.b); p.push_back(s.gamma); p.push_back(s.beta); }
  fc.parameters(p);
  return p;
}
Tensor ConvNet::loss(const Tensor& x, const Tensor& labels) {
  Tensor h = x;
  for (const auto& s : stages)
    h = h.conv2d(s.w, s.b, 1, 1).bn_relu_maxpool(s.gamma, s.beta, s.rm, s.rv, autograd::is_training(), momentum, eps);   // = batchnorm -> relu -> maxpool2d(2, 2, 0)
  std::vector<i64> sh = h.shape();
  h = h.avgpool2d((int)sh[2], (int)sh[2], 0).reshape({sh[0], sh[1]});
  return fc.forward(h).cross_entropy(labels);
}

FusedOpBench::FusedOpBench(i64 c, i64 v) : ln(c), head(c, v, false) {}
std::vector<Tensor> FusedOpBench::parameters() const { std::vector<Tensor> p; ln.parameters(p); head.parameters(p); return p; }
Tensor FusedOpBench::loss(const Tensor& x, const Tensor& labels) { return head.forward(ln.forward(x).gelu()).cross_entropy(labels); }

}  // namespace nn

namespace optim {

BucketPlan plan_buckets(const std::vector<i64>& numels, i64 target_elems) {
  BucketPlan bp;
  for (i64 n : numels) { bp.param_offset.push_back(bp.total); bp.total += (n + 3) & ~i64(3); }
  bp.bucket_of.assign(numels.size(), 0);
  i64 end = bp.total; int cnt = 0;
  for (int i = (int)numels.size() - 1; i >= 0; --i) {
    i64 acc = end - bp.param_offset[i]; ++cnt;
    bp.bucket_of[i] = (int)bp.bucket_offset.size();
    if (acc >= target_elems || i == 0) {
      bp.bucket_offset.push_back(bp.param_offset[i]); bp.bucket_numel.push_back(acc); bp.bucket_nparams.push_back(cnt);
      end = bp.param_offset[i]; cnt = 0;
    }
  }
  return bp;
}

Optimizer::Optimizer(const vb_opt_config& cfg, const std::vector<Tensor>& params, bool data_parallel) : cfg_(cfg), params_(params), dp_(data_parallel) {
  // one flat gradient arena, parameters in registration order, every view 16-byte aligned
  std::vector<i64> numels;
  for (const Tensor& p : params_) {
    if (!p.is_contiguous()) throw Error("optimizer parameters must be contiguous");
    numels.push_back(p.numel());
  }
  // gradient buckets of at least 128 MiB (VB200_DP_BUCKET_MB overrides the size): with 8 GPUs on NVSwitch every all-reduce kernel
  // holds 24 SMs while it runs, and few long ones cost the GEMMs beside them less than many short ones (GPT-small step at 8 GPUs:
  // 46.5 ms with 8 MiB buckets, 46.4 with 32, 45.7 with 128)
  i64 bucket_mb = 128;
  if (const char* e = std::getenv("VB200_DP_BUCKET_MB")) { const long v = std::atol(e); if (v >= 1 && v <= 4096) bucket_mb = v; }
  BucketPlan bp = plan_buckets(numels, (bucket_mb << 20) / 4);
  const i64 total = bp.total;
  const std::vector<i64>& offs = bp.param_offset;
  arena_ = dp_ ? Tensor::zeros_for_collectives({total > 0 ? total : 1}) : Tensor::zeros({total > 0 ? total : 1});
  std::vector<vb_tensor> pd, gd;
  for (size_t i = 0; i < params_.size(); ++i) {
    vb_tensor d = params_[i].desc(); d.slot = arena_.slot(); d.offset = offs[i];
    i64 s = 1; for (int k = d.rank - 1; k >= 0; --k) { d.strides[k] = s; s *= d.dims[k]; }
    sinks_.push_back(Tensor::view_of(arena_, d));
    pd.push_back(params_[i].desc()); gd.push_back(d);
  }
  check(vb_opt_create(&cfg_, pd.data(), gd.data(), (int)params_.size(), &opt_), "opt_create");
  int rank = 0;
  check(vb_dp_world(&rank, &world_), "dp_world");
  if (!dp_) world_ = 1;
  // buckets: contiguous arena ranges of at least the bucket size (see plan_buckets)
  bucket_of_ = bp.bucket_of;
  for (size_t b = 0; b < bp.bucket_offset.size(); ++b) buckets_.push_back(Bucket{bp.bucket_offset[b], bp.bucket_numel[b], bp.bucket_nparams[b], bp.bucket_nparams[b]});
  ready_.assign(params_.size(), 0);
  autograd::register_grad_sinks(params_, sinks_, &Optimizer::on_ready, this);
}
Optimizer::~Optimizer() {
  autograd::clear_grad_sinks(this);
  if (opt_ >= 0) vb_opt_destroy(opt_);
}
// VB200_DP_OVERLAP=0: every bucket is reduced after the backward pass instead of as soon as it is complete (A/B switch).
static bool dp_overlap() {
  static const bool on = [] { const char* e = std::getenv("VB200_DP_OVERLAP"); return !(e && e[0] == '0'); }();
  return on;
}
void Optimizer::on_ready(int idx, void* self) {
  Optimizer* o = (Optimizer*)self;
  if (idx < 0) {      // a further contribution to parameter -1 - idx was added to its sink after the first was published
    if (o->world_ > 1) throw Error("a parameter that gets gradient from several checkpointed regions is not supported under data parallel: its bucket may already have been reduced");
    return;
  }
  if (o->ready_[idx]) {
    // a second backward pass before step(): on one GPU the sink is simply overwritten, as the reference's gradient map is; under
    // data parallel the bucket holding it has been reduced already and would not be reduced again
    if (o->world_ > 1) throw Error("backward() ran twice before the optimizer step: not supported under data parallel (the first pass's gradients were already reduced)");
    return;
  }
  o->ready_[idx] = 1;
  if (o->world_ <= 1) return;
  Bucket& b = o->buckets_[o->bucket_of_[idx]];
  if (--b.pending == 0 && dp_overlap()) check(vb_dp_allreduce(o->arena_.slot(), b.offset, b.numel), "dp_allreduce");
}
// Host deadline for the step's collectives, in milliseconds: VB200_DP_TIMEOUT_MS, 30 s by default.
static int collective_timeout_ms() {
  static int ms = -1;
  if (ms < 0) { const char* e = std::getenv("VB200_DP_TIMEOUT_MS"); ms = (e && std::atoi(e) > 0) ? std::atoi(e) : 30000; }
  return ms;
}
// Buckets with a parameter that received no gradient this step are still reduced (every rank must
// issue the same collectives): their stale ranges are zeroed first.
// deferred: the host does not wait for the collectives here (their deadline is checked at the next step's, or at the next
// read-back / synchronisation through the library) -- for callers that read nothing back from this step.
void Optimizer::finish_reduce(bool deferred) {
  if (world_ > 1) {
    for (size_t i = 0; i < params_.size(); ++i)
      if (!ready_[i]) {
        check(vb_fill(&sinks_[i].desc(), 0.0f), "fill");
        Bucket& b = buckets_[bucket_of_[i]];
        if (--b.pending == 0 && dp_overlap()) check(vb_dp_allreduce(arena_.slot(), b.offset, b.numel), "dp_allreduce");
      }
    if (!dp_overlap()) for (Bucket& b : buckets_) check(vb_dp_allreduce(arena_.slot(), b.offset, b.numel), "dp_allreduce");
    check(vb_dp_finish(deferred ? -collective_timeout_ms() : collective_timeout_ms()), "dp_finish");
    for (Bucket& b : buckets_) b.pending = b.nparams;
  }
}
// Which parameters the update touches: on one GPU those that received a gradient this step (vearo-optim/src/lib.rs:106-108 skips the
// others); under data parallel ALL of them -- a parameter may have received gradient on some ranks only, every rank holds the same
// reduced sum after finish_reduce (zero-filled where nothing was produced locally), and replicas must apply the same update.
void Optimizer::step() {
  finish_reduce(true);
  check(vb_opt_step(opt_, world_ > 1 ? nullptr : ready_.data(), 0.0f, 1.0f / (float)world_, nullptr), "opt_step");
  std::fill(ready_.begin(), ready_.end(), 0);
}
float Optimizer::clip_and_step(float max_norm, bool read_norm) {
  finish_reduce(!read_norm);
  float norm = 0.0f;
  check(vb_opt_step(opt_, world_ > 1 ? nullptr : ready_.data(), max_norm, 1.0f / (float)world_, read_norm ? &norm : nullptr), "opt_step");
  std::fill(ready_.begin(), ready_.end(), 0);
  return norm;
}
void Optimizer::set_lr(float lr) { cfg_.lr = lr; check(vb_opt_set_lr(opt_, lr), "opt_set_lr"); }

float clip_grad_norm(const std::vector<Tensor>& params, float max_norm) {
  std::vector<vb_tensor> gd;
  std::vector<Tensor> hold;
  for (const Tensor& p : params) {
    Tensor g;
    if (!p.grad(&g)) continue;
    if (!g.is_contiguous()) throw Error("clip_grad_norm expects contiguous grads");
    hold.push_back(g); gd.push_back(g.desc());
  }
  float norm = 0.0f;
  check(vb_clip_grad_norm(gd.data(), (int)gd.size(), max_norm, &norm), "clip_grad_norm");
  return norm;
}
float cosine_lr(float base, float min_lr, uint32_t warmup, uint32_t total, uint32_t step) {
  if (step < warmup) return base * ((float)step + 1.0f) / ((float)warmup + 1.0f);
  if (step > total) return min_lr;
  uint32_t denom = total > warmup ? total - warmup : 0; if (denom < 1) denom = 1;
  float progress = (float)(step - warmup) / (float)denom;
  float coeff = 0.5f * (1.0f + std::cos(3.14159265358979323846f * progress));
  return min_lr + coeff * (base - min_lr);
}

}  // namespace optim
// ---- `.ve` checkpoints ----------------------------------------------------------------------------------------
namespace checkpoint {
namespace {
struct File {
  FILE* f;
  File(const std::string& path, const char* mode) : f(std::fopen(path.c_str(), mode)) { if (!f) throw Error("cannot open " + path); }
  ~File() { if (f) std::fclose(f); }
};
void put_u32(FILE* f, uint64_t v) {
  if (v > 0xffffffffull) throw Error("value does not fit the checkpoint format's u32 field");
  uint32_t x = (uint32_t)v; unsigned char b[4] = {(unsigned char)x, (unsigned char)(x >> 8), (unsigned char)(x >> 16), (unsigned char)(x >> 24)};
  if (std::fwrite(b, 1, 4, f) != 4) throw Error("checkpoint write failed");
}
uint32_t get_u32(FILE* f) {
  unsigned char b[4];
  if (std::fread(b, 1, 4, f) != 4) throw Error("failed to fill whole buffer");       // std::io::ErrorKind::UnexpectedEof
  return (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
}
}  // namespace
void write_container(const std::vector<HostTensor>& ts, const std::string& path) {
  File fl(path, "wb");
  put_u32(fl.f, ts.size());
  for (const HostTensor& t : ts) {
    put_u32(fl.f, t.dims.size());
    for (i64 d : t.dims) put_u32(fl.f, (uint64_t)d);
    put_u32(fl.f, t.data.size());
    // f32 little endian: the byte order of every machine this library runs on
    if (!t.data.empty() && std::fwrite(t.data.data(), sizeof(float), t.data.size(), fl.f) != t.data.size()) throw Error("checkpoint write failed");
  }
  if (std::fflush(fl.f) != 0) throw Error("checkpoint write failed");
}
// Bytes left in the file from the current position (so that a length field is never trusted beyond what the file can hold).
static uint64_t bytes_left(FILE* f) {
  long here = std::ftell(f);
  if (here < 0 || std::fseek(f, 0, SEEK_END) != 0) throw Error("checkpoint read failed");
  long end = std::ftell(f);
  if (end < here || std::fseek(f, here, SEEK_SET) != 0) throw Error("checkpoint read failed");
  return (uint64_t)(end - here);
}
// One tensor record; `expect` (may be null) is the shape it must have, checked before any of its data is read.
static HostTensor read_record(FILE* f, const std::vector<i64>* expect) {
  HostTensor t;
  const uint32_t rank = get_u32(f);
  if (rank > 8 || (uint64_t)rank * 4 > bytes_left(f)) throw Error("checkpoint is damaged: tensor rank " + std::to_string(rank));
  t.dims.resize(rank);
  for (i64& d : t.dims) d = get_u32(f);
  if (expect && t.dims != *expect) throw Error("Checkpoint shape does not match parameter shape");
  const uint32_t n = get_u32(f);
  uint64_t prod = 1;
  for (i64 d : t.dims) { prod *= (uint64_t)d; if (prod > 0xffffffffull) break; }
  if (prod != n) throw Error("Checkpoint shape does not match parameter shape");        // (the reference's copy_from_slice panics on this)
  if ((uint64_t)n * 4 > bytes_left(f)) throw Error("failed to fill whole buffer");
  t.data.resize(n);
  if (n && std::fread(t.data.data(), sizeof(float), n, f) != n) throw Error("failed to fill whole buffer");
  return t;
}
std::vector<HostTensor> read_container(const std::string& path) {
  File fl(path, "rb");
  const uint32_t count = get_u32(fl.f);
  if ((uint64_t)count * 8 > bytes_left(fl.f)) throw Error("checkpoint is damaged: tensor count " + std::to_string(count));      // a record is at least 8 bytes
  std::vector<HostTensor> ts;
  ts.reserve(count);
  for (uint32_t i = 0; i < count; ++i) ts.push_back(read_record(fl.f, nullptr));
  return ts;
}
void save_checkpoint(const std::vector<Tensor>& params, const std::string& path) {
  std::vector<HostTensor> ts;
  for (const Tensor& p : params) ts.push_back(HostTensor{p.shape(), p.to_vec_f32()});
  write_container(ts, path);
}
// As crates/vearo/src/checkpoint.rs:42-86: the count is compared first, then every tensor's shape before its data is read
// (nothing is written to a parameter until its own record has been validated; earlier parameters keep what was loaded).
void load_checkpoint(const std::vector<Tensor>& params, const std::string& path) {
  File fl(path, "rb");
  if (get_u32(fl.f) != params.size()) throw Error("Checkpoint tensor count does not match model parameter count");
  for (const Tensor& p : params) {
    const std::vector<i64> shape = p.shape();
    HostTensor t = read_record(fl.f, &shape);
    p.write_f32(t.data.data());
  }
}
}  // namespace checkpoint

namespace optim {
// State file: tensor 0 = [6] exact small integers held as f32 -- the step counter t as two 16-bit halves (low, high) and the
// per-call randomness counter (vearo-core/src/tensor.rs:1240-1285) as four 16-bit parts, low first; tensor 1 = the flat state
// array.  (Files written before the counter was added hold tensor 0 = [t] as one f32; they still load.)
void Optimizer::save_state(const std::string& path) const {
  vb_slot st; int64_t n = 0; uint32_t t = 0;
  check(vb_opt_state(opt_, &st, &n, &t), "opt_state");
  const uint64_t rng = autograd::rng_counter();
  checkpoint::HostTensor head{{6}, {(float)(t & 0xffffu), (float)(t >> 16), (float)(rng & 0xffffu), (float)((rng >> 16) & 0xffffu),
                                    (float)((rng >> 32) & 0xffffu), (float)((rng >> 48) & 0xffffu)}};
  checkpoint::HostTensor state{{n}, std::vector<float>((size_t)n)};
  if (n) check(vb_read(st, 0, state.data.data(), n), "read optimizer state");
  checkpoint::write_container({head, state}, path);
}
void Optimizer::load_state(const std::string& path) {
  std::vector<checkpoint::HostTensor> ts = checkpoint::read_container(path);
  vb_slot st; int64_t n = 0;
  check(vb_opt_state(opt_, &st, &n, nullptr), "opt_state");
  if (ts.size() != 2 || (ts[0].data.size() != 1 && ts[0].data.size() != 6) || (int64_t)ts[1].data.size() != n)
    throw Error("optimizer state file does not match this optimizer");
  if (n) check(vb_write(st, 0, ts[1].data.data(), n), "write optimizer state");
  const std::vector<float>& h = ts[0].data;
  if (h.size() == 1) { check(vb_opt_set_step(opt_, (uint32_t)h[0]), "opt_set_step"); return; }
  check(vb_opt_set_step(opt_, (uint32_t)h[0] | ((uint32_t)h[1] << 16)), "opt_set_step");
  autograd::set_rng_counter((uint64_t)h[2] | ((uint64_t)h[3] << 16) | ((uint64_t)h[4] << 32) | ((uint64_t)h[5] << 48));
}
}  // namespace optim

}  // namespace vearo
