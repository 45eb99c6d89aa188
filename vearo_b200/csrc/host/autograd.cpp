// Tensor dispatch + record, the tape, and the backward walk.
//
// Mirrors crates/vearo-core/src/tensor.rs:1365-1970 (each op: run the backend, then record when
// autograd is on and an input requires grad) and crates/vearo-autograd/src/lib.rs:129-197 (tape,
// generation-tagged node tokens, lazily created leaf nodes) and :429-792 (backward_impl: reverse
// walk, one arm per op, `existing + new` accumulation, gradients published for leaves only).
//
// What differs from the reference, by design: every arm stays on the device (the reference
// downloads gradients for reduce_to and builds ReLU / GELU masks on the host, lib.rs:316-403);
// op attributes are plain fields, not formatted strings; the tape is moved, not cloned; a
// gradient whose storage nobody else holds is accumulated in place; node gradients and saved
// activations are dropped as soon as the walk has passed them; and a leaf's gradient is
// published the moment its last contribution has arrived (its earliest consumer on the tape),
// which is what allows gradient exchange to overlap the rest of the walk.
#include "vearo_host.h"
#include <functional>
#include <algorithm>
#include <cmath>
#include <unordered_map>

namespace vearo {

void check(int status, const char* what) {
  if (status != VB_OK) throw Error(std::string(what) + ": " + vb_last_error());
}
Storage::~Storage() { if (slot) vb_release(slot, nullptr); }

// ---- Tensor basics ---------------------------------------------------------------------------
static vb_tensor contiguous_desc(const std::vector<i64>& shape) {
  if (shape.size() > VB_MAX_RANK) throw Error("rank > 8 is not supported");
  vb_tensor t{}; t.rank = (int)shape.size();
  i64 s = 1;
  for (int i = t.rank - 1; i >= 0; --i) { t.dims[i] = shape[i]; t.strides[i] = s; s *= shape[i]; }
  return t;
}
Tensor Tensor::adopt(const vb_tensor& t) { Tensor r; r.st_ = std::make_shared<Storage>(t.slot); r.d_ = t; return r; }
Tensor Tensor::view_of(const Tensor& base, const vb_tensor& d) { Tensor r; r.st_ = base.st_; r.d_ = d; r.d_.slot = base.d_.slot; return r; }
Tensor Tensor::zeros(const std::vector<i64>& shape) {
  vb_tensor t = contiguous_desc(shape);
  i64 n = 1; for (i64 d : shape) n *= d;
  check(vb_alloc(n, 1, &t.slot), "alloc");
  return adopt(t);
}
Tensor Tensor::zeros_for_collectives(const std::vector<i64>& shape) {
  vb_tensor t = contiguous_desc(shape);
  i64 n = 1; for (i64 d : shape) n *= d;
  check(vb_dp_alloc(n, 1, &t.slot), "dp_alloc");
  return adopt(t);
}
Tensor Tensor::from_f32(const float* data, const std::vector<i64>& shape) {
  vb_tensor t = contiguous_desc(shape);
  i64 n = 1; for (i64 d : shape) n *= d;
  check(vb_alloc(n, 0, &t.slot), "alloc");
  Tensor r = adopt(t);
  if (n) check(vb_write(t.slot, 0, data, n), "write");
  return r;
}
bool Tensor::is_contiguous() const {
  i64 s = 1;
  for (int i = d_.rank - 1; i >= 0; --i) { if (d_.dims[i] != 1 && d_.strides[i] != s) return false; s *= d_.dims[i]; }
  return true;
}
Tensor Tensor::contiguous() const {
  if (is_contiguous()) return *this;
  vb_tensor o; check(vb_contiguous(&d_, &o), "contiguous");
  Tensor r = adopt(o);
  r.meta_->requires_grad = meta_->requires_grad; r.meta_->node = meta_->node;
  return r;
}
std::vector<float> Tensor::to_vec_f32() const {
  Tensor c = contiguous();
  std::vector<float> v((size_t)numel());
  if (!v.empty()) check(vb_read(c.d_.slot, c.d_.offset, v.data(), (i64)v.size()), "read");
  return v;
}
void Tensor::write_f32(const float* data) const {
  if (!is_contiguous()) throw Error("write_f32 needs a contiguous tensor");
  if (numel()) check(vb_write(d_.slot, d_.offset, data, numel()), "write");
}

// ---- tape ------------------------------------------------------------------------------------
namespace {
enum class Op { Add, Sub, Mul, Div, Matmul, Reshape, Transpose, Permute, Relu, Gelu, Softmax, LayerNorm, Embedding,
                CrossEntropy, Sum, Mean, Conv2d, MaxPool2d, AvgPool2d, BatchNorm, FusedAttention, Linear, BnReluPool, PackRows, FusedAttentionPacked, Checkpoint, Leaf };
struct Node {
  int id = 0; Op op = Op::Leaf;
  std::vector<int> inputs;
  std::vector<Tensor> saved;
  i64 a0 = 0, a1 = 0, a2 = 0; float f0 = 0.0f;
  std::vector<i64> axes;
  Tensor extra;             // attention probabilities / cross-entropy row statistics
  Tensor leaf;              // for Leaf nodes: the tensor itself
  std::function<Tensor(const Tensor&)> fn;      // Checkpoint nodes: the block to run again during backward
  uint64_t rng = 0;                             // Checkpoint nodes: the per-call randomness counter when the block first ran
};
struct Tape { std::vector<Node> nodes; uint32_t generation = 0; };
thread_local Tape t_tape;
thread_local bool t_enabled = true, t_training = true, t_recomputing = false;
thread_local uint64_t t_rng_counter = 0;        // per-call randomness counter (vearo-core/src/tensor.rs:1240-1285)
// A leaf is identified by where it lives: slot and offset (several parameters may be views of one slot).
using LeafKey = uint64_t;
inline LeafKey leaf_key(const Tensor& t) { return ((uint64_t)t.slot() << 40) ^ (uint64_t)t.desc().offset; }
thread_local std::unordered_map<LeafKey, Tensor> t_grads;

// Gradient sinks of every live optimizer (several may coexist, each over its own parameters; a parameter given to two
// optimizers belongs to the one registered last).
struct SinkEntry { Tensor sink; int idx = 0; void (*on_ready)(int, void*) = nullptr; void* user = nullptr; };
struct Sinks { std::unordered_map<uint64_t, SinkEntry> index; };      // leaf_key -> sink, index within its optimizer, callback
thread_local Sinks t_sinks;

i64 pack(uint32_t gen, uint32_t idx) { return ((i64)gen << 32) | idx; }
int live_index(const Tensor& t) {
  i64 tok = t.node_id();
  if (tok < 0 || (uint32_t)(tok >> 32) != t_tape.generation) return -1;
  return (int)(tok & 0xffffffff);
}
// Tape::push (lib.rs:151-189)
Node& push(Op op, const std::vector<const Tensor*>& ins, Tensor& out) {
  std::vector<int> ids;
  for (const Tensor* in : ins) {
    int live = live_index(*in);
    if (live >= 0) ids.push_back(live);
    else if (in->requires_grad()) {
      Node leaf; leaf.id = (int)t_tape.nodes.size(); leaf.op = Op::Leaf; leaf.leaf = *in;
      in->set_node_id(pack(t_tape.generation, (uint32_t)leaf.id));
      ids.push_back(leaf.id);
      t_tape.nodes.push_back(std::move(leaf));
    } else ids.push_back(-1);
  }
  Node n; n.id = (int)t_tape.nodes.size(); n.op = op; n.inputs = ids;
  for (const Tensor* in : ins) n.saved.push_back(*in);
  out.set_node_id(pack(t_tape.generation, (uint32_t)n.id));
  t_tape.nodes.push_back(std::move(n));
  return t_tape.nodes.back();
}
Node* record(Op op, const std::vector<const Tensor*>& ins, Tensor& out) {
  if (!t_enabled) return nullptr;
  bool any = false;
  for (const Tensor* t : ins) any = any || t->requires_grad();
  if (!any) return nullptr;
  out.set_requires_grad(true);
  return &push(op, ins, out);
}
}  // namespace

namespace autograd {
void set_enabled(bool e) { t_enabled = e; }
bool is_enabled() { return t_enabled; }
void set_training(bool t) { t_training = t; }
bool is_training() { return t_training; }
void reset_active_tape() { t_tape.nodes.clear(); t_tape.generation++; }
void zero_gradients() { t_grads.clear(); }
size_t tape_len() { return t_tape.nodes.size(); }
void register_grad_sinks(const std::vector<Tensor>& params, const std::vector<Tensor>& sinks, void (*on_ready)(int, void*), void* user) {
  for (size_t i = 0; i < params.size(); ++i) t_sinks.index[leaf_key(params[i])] = SinkEntry{sinks[i], (int)i, on_ready, user};
}
void clear_grad_sinks(void* user) {
  for (auto it = t_sinks.index.begin(); it != t_sinks.index.end();) { if (it->second.user == user) it = t_sinks.index.erase(it); else ++it; }
}
}  // namespace autograd

// ---- ops ---------------------------------------------------------------------------------------
#define VB_OUT1(call, what) vb_tensor o_; check(call, what); Tensor out = Tensor::adopt(o_)
Tensor Tensor::add(const Tensor& o) const { VB_OUT1(vb_add(&d_, &o.d_, &o_), "add"); record(Op::Add, {this, &o}, out); return out; }
Tensor Tensor::sub(const Tensor& o) const { VB_OUT1(vb_sub(&d_, &o.d_, &o_), "sub"); record(Op::Sub, {this, &o}, out); return out; }
Tensor Tensor::mul(const Tensor& o) const { VB_OUT1(vb_mul(&d_, &o.d_, &o_), "mul"); record(Op::Mul, {this, &o}, out); return out; }
Tensor Tensor::div(const Tensor& o) const { VB_OUT1(vb_div(&d_, &o.d_, &o_), "div"); record(Op::Div, {this, &o}, out); return out; }
Tensor Tensor::matmul(const Tensor& o) const { VB_OUT1(vb_matmul(&d_, &o.d_, &o_), "matmul"); record(Op::Matmul, {this, &o}, out); return out; }
Tensor Tensor::relu() const { VB_OUT1(vb_relu(&d_, &o_), "relu"); record(Op::Relu, {this}, out); return out; }
Tensor Tensor::gelu() const { VB_OUT1(vb_gelu(&d_, &o_), "gelu"); record(Op::Gelu, {this}, out); return out; }
Tensor Tensor::sum(int dim, bool keep) const {
  VB_OUT1(vb_sum(&d_, dim, keep, &o_), "sum");
  if (Node* n = record(Op::Sum, {this}, out)) { n->a0 = dim; n->a1 = keep; }
  return out;
}
Tensor Tensor::mean(int dim, bool keep) const {
  VB_OUT1(vb_mean(&d_, dim, keep, &o_), "mean");
  if (Node* n = record(Op::Mean, {this}, out)) { n->a0 = dim; n->a1 = keep; }
  return out;
}
Tensor Tensor::softmax(int dim) const {
  VB_OUT1(vb_softmax(&d_, dim, &o_), "softmax");
  if (Node* n = record(Op::Softmax, {this}, out)) n->a0 = dim;
  return out;
}
Tensor Tensor::layernorm(const Tensor& w, const Tensor& b, float eps) const {
  VB_OUT1(vb_layernorm(&d_, &w.d_, &b.d_, eps, &o_), "layernorm");
  if (Node* n = record(Op::LayerNorm, {this, &w, &b}, out)) n->f0 = eps;
  return out;
}
Tensor Tensor::embedding(const Tensor& weight) const {
  VB_OUT1(vb_embedding(&d_, &weight.d_, &o_), "embedding");
  record(Op::Embedding, {this, &weight}, out);
  return out;
}
Tensor Tensor::cross_entropy(const Tensor& targets) const {
  bool rec = t_enabled && (requires_grad() || targets.requires_grad());
  vb_tensor o_, st_;
  check(vb_cross_entropy(&d_, &targets.d_, &o_, rec ? &st_ : nullptr), "cross_entropy");
  Tensor out = Tensor::adopt(o_);
  Tensor stats; if (rec) stats = Tensor::adopt(st_);
  if (Node* n = record(Op::CrossEntropy, {this, &targets}, out)) n->extra = stats;
  return out;
}
// cross_entropy for a caller that gives the logits up: when the loss is going to be differentiated and nobody else holds the
// logits, one pass computes the loss and leaves d loss / d logits (for a unit upstream gradient) in their place.
Tensor Tensor::cross_entropy_consuming(const Tensor& targets) const {
  const bool fuse = t_enabled && requires_grad() && !targets.requires_grad() && is_contiguous() && live_index(*this) >= 0;
  if (!fuse) return cross_entropy(targets);
  vb_tensor o_;
  check(vb_cross_entropy_fused(&d_, &targets.d_, &o_), "cross_entropy_fused");
  Tensor out = Tensor::adopt(o_);
  if (Node* n = record(Op::CrossEntropy, {this, &targets}, out)) n->a1 = 1;      // saved[0] now holds the gradient
  return out;
}
Tensor Tensor::conv2d(const Tensor& w, const Tensor& b, int stride, int padding) const {
  VB_OUT1(vb_conv2d(&d_, &w.d_, &b.d_, stride, padding, &o_), "conv2d");
  if (Node* n = record(Op::Conv2d, {this, &w, &b}, out)) { n->a0 = stride; n->a1 = padding; }
  return out;
}
Tensor Tensor::maxpool2d(int k, int s, int p) const {
  VB_OUT1(vb_maxpool2d(&d_, k, s, p, &o_), "maxpool2d");
  if (Node* n = record(Op::MaxPool2d, {this}, out)) { n->a0 = k; n->a1 = s; n->a2 = p; }
  return out;
}
Tensor Tensor::avgpool2d(int k, int s, int p) const {
  VB_OUT1(vb_avgpool2d(&d_, k, s, p, &o_), "avgpool2d");
  if (Node* n = record(Op::AvgPool2d, {this}, out)) { n->a0 = k; n->a1 = s; n->a2 = p; }
  return out;
}
Tensor Tensor::batchnorm(const Tensor& gamma, const Tensor& beta, const Tensor& rm, const Tensor& rv, bool training, float momentum, float eps) const {
  // under recomputation (a checkpointed block run again during backward) the running statistics must not advance a second time
  // (vearo-nn/src/lib.rs:437-454 passes detached copies); momentum 0 leaves them bit-for-bit as they are
  if (t_recomputing) momentum = 0.0f;
  VB_OUT1(vb_batchnorm(&d_, &gamma.d_, &beta.d_, &rm.d_, &rv.d_, training, momentum, eps, &o_), "batchnorm");
  if (Node* n = record(Op::BatchNorm, {this, &gamma, &beta, &rm, &rv}, out)) { n->a0 = training; n->f0 = eps; }
  return out;
}
Tensor Tensor::bn_relu_maxpool(const Tensor& gamma, const Tensor& beta, const Tensor& rm, const Tensor& rv, bool training, float momentum, float eps) const {
  vb_tensor o_, s_;
  if (t_recomputing) momentum = 0.0f;
  check(vb_bn_relu_maxpool(&d_, &gamma.d_, &beta.d_, &rm.d_, &rv.d_, training, momentum, eps, &o_, &s_), "bn_relu_maxpool");
  Tensor out = Tensor::adopt(o_), stats = Tensor::adopt(s_);
  if (Node* n = record(Op::BnReluPool, {this, &gamma, &beta}, out)) { n->a0 = training; n->extra = stats; }
  return out;
}
Tensor Tensor::fused_attention(const Tensor& k, const Tensor& v, const Tensor* mask) const {
  std::vector<const Tensor*> ins = {this, &k, &v};
  if (mask) ins.push_back(mask);
  bool rec = false;
  if (t_enabled) for (const Tensor* t : ins) rec = rec || t->requires_grad();
  vb_tensor o_, p_;
  check(vb_fused_attention(&d_, &k.d_, &v.d_, mask ? &mask->d_ : nullptr, &o_, rec ? &p_ : nullptr), "fused_attention");
  Tensor out = Tensor::adopt(o_);
  Tensor probs; if (rec) probs = Tensor::adopt(p_);
  if (Node* n = record(Op::FusedAttention, ins, out)) n->extra = probs;
  return out;
}
Tensor Tensor::fused_attention_packed(i64 n_head, const Tensor* mask) const {
  std::vector<const Tensor*> ins = {this};
  if (mask) ins.push_back(mask);
  const bool rec = t_enabled && requires_grad();
  vb_tensor o_, p_;
  check(vb_fused_attention_packed(&d_, (int)n_head, mask ? &mask->d_ : nullptr, &o_, rec ? &p_ : nullptr), "fused_attention_packed");
  Tensor out = Tensor::adopt(o_);
  Tensor probs; if (rec) probs = Tensor::adopt(p_);
  if (Node* n = record(Op::FusedAttentionPacked, ins, out)) { n->extra = probs; n->a0 = n_head; }
  return out;
}
Tensor Tensor::pack_rows(const Tensor& a, const Tensor& b, const Tensor& c) {
  const vb_tensor &da = a.d_, &db = b.d_, &dc = c.d_;
  bool ok = a.defined() && da.rank >= 1 && da.slot == db.slot && da.slot == dc.slot && a.is_contiguous() && b.is_contiguous() && c.is_contiguous() &&
            da.rank == db.rank && da.rank == dc.rank && db.offset == da.offset + a.numel() && dc.offset == db.offset + b.numel();
  for (int i = 1; ok && i < da.rank; ++i) ok = da.dims[i] == db.dims[i] && da.dims[i] == dc.dims[i];
  if (!ok) throw Error("pack_rows needs three contiguous views that follow one another in one storage");
  vb_tensor d = da;
  d.dims[0] = da.dims[0] + db.dims[0] + dc.dims[0];
  Tensor out = view_of(a, d);
  if (Node* n = record(Op::PackRows, {&a, &b, &c}, out)) { n->a0 = da.dims[0]; n->a1 = db.dims[0]; n->a2 = dc.dims[0]; }
  return out;
}
Tensor Tensor::linear(const Tensor& weight, const Tensor* bias) const {
  VB_OUT1(vb_linear(&d_, &weight.d_, bias ? &bias->d_ : nullptr, &o_), "linear");
  std::vector<const Tensor*> ins = {this, &weight};
  if (bias) ins.push_back(bias);
  record(Op::Linear, ins, out);
  return out;
}
// linear followed by gelu: one device call, two tape nodes (exactly what x.linear(w, b).gelu() records)
Tensor Tensor::linear_gelu(const Tensor& weight, const Tensor* bias) const {
  vb_tensor pre_{}, act_{};
  check(vb_linear_gelu(&d_, &weight.d_, bias ? &bias->d_ : nullptr, &pre_, &act_), "linear_gelu");
  Tensor pre = Tensor::adopt(pre_), act = Tensor::adopt(act_);
  std::vector<const Tensor*> ins = {this, &weight};
  if (bias) ins.push_back(bias);
  record(Op::Linear, ins, pre);
  record(Op::Gelu, {&pre}, act);
  return act;
}
// reshape / transpose / permute: views (tensor.rs:493-642); reshape of a strided view copies first.
Tensor Tensor::reshape(const std::vector<i64>& shape) const {
  i64 n = 1; for (i64 d : shape) n *= d;
  if (n != numel()) throw Error("Reshape numel must match");
  Tensor c = contiguous();
  vb_tensor d = contiguous_desc(shape); d.offset = c.d_.offset;
  Tensor out = view_of(c, d);
  out.meta_->requires_grad = c.requires_grad(); out.meta_->node = c.node_id();
  if (t_enabled && requires_grad()) { out.set_requires_grad(true); push(Op::Reshape, {this}, out); }
  return out;
}
Tensor Tensor::transpose(int d0, int d1) const {
  if (d0 < 0 || d1 < 0 || d0 >= d_.rank || d1 >= d_.rank) throw Error("transpose dims out of bounds");
  vb_tensor d = d_;
  std::swap(d.dims[d0], d.dims[d1]); std::swap(d.strides[d0], d.strides[d1]);
  Tensor out = view_of(*this, d);
  out.meta_->requires_grad = requires_grad(); out.meta_->node = node_id();
  if (t_enabled && requires_grad()) { Node& n = push(Op::Transpose, {this}, out); n.a0 = d0; n.a1 = d1; }
  return out;
}
Tensor Tensor::permute(const std::vector<i64>& axes) const {
  if ((int)axes.size() != d_.rank) throw Error("permute needs one axis per dim");
  vb_tensor d = d_;
  for (int i = 0; i < d_.rank; ++i) { d.dims[i] = d_.dims[axes[i]]; d.strides[i] = d_.strides[axes[i]]; }
  Tensor out = view_of(*this, d);
  out.meta_->requires_grad = requires_grad(); out.meta_->node = node_id();
  if (t_enabled && requires_grad()) { Node& n = push(Op::Permute, {this}, out); n.axes = axes; }
  return out;
}

// ---- backward ----------------------------------------------------------------------------------
namespace {
Tensor reduce_to(const Tensor& g, const std::vector<i64>& target) {
  if (g.shape() == target) return g;
  vb_tensor o; check(vb_reduce_to(&g.desc(), target.data(), (int)target.size(), &o), "reduce_to");
  return Tensor::adopt(o);
}
Tensor scaled(const Tensor& g, float a) { vb_tensor o; check(vb_scale(&g.desc(), a, &o), "scale"); return Tensor::adopt(o); }
// expand_reduce_grad (lib.rs:410-425): zeros of the input shape + the (re-inserted) reduced gradient
Tensor expand_reduce_grad(const Tensor& go, const std::vector<i64>& in_shape, int dim, bool keep) {
  Tensor gk = go;
  if (!keep) { std::vector<i64> d = go.shape(); d.insert(d.begin() + dim, 1); gk = go.reshape(d); }
  return Tensor::zeros(in_shape).add(gk);
}
struct Restore { ~Restore() { t_enabled = true; } };

// Where a nested (checkpoint) backward delivers the gradient of the block's input instead of publishing it as a leaf gradient.
struct NestedInput { bool active = false; LeafKey key = 0; Tensor* gx = nullptr; };

void publish_leaf(const Node& leaf, Tensor& grad, const NestedInput& nested) {
  LeafKey key = leaf_key(leaf.leaf);
  if (nested.active && key == nested.key) {
    *nested.gx = nested.gx->defined() ? nested.gx->add(grad) : grad;
    return;
  }
  auto it = t_sinks.index.find(key);
  auto have = t_grads.find(key);
  if (have != t_grads.end()) {
    // a second contribution within one backward pass (a parameter used by several checkpointed blocks, or inside and outside
    // one): summed, as the reference merges its checkpoint gradients (lib.rs:717-726, 781-791)
    Tensor& ex = have->second;
    if (ex.is_contiguous() && ex.shape() == grad.shape() && (it != t_sinks.index.end() || ex.storage_unique()))
      check(vb_accumulate(&ex.desc(), &grad.desc()), "accumulate");
    else ex = ex.add(grad);
    if (it != t_sinks.index.end() && it->second.on_ready) it->second.on_ready(-1 - it->second.idx, it->second.user);
    return;
  }
  if (it != t_sinks.index.end()) {
    const Tensor& sink = it->second.sink;
    if (sink.numel() != grad.numel()) throw Error("gradient sink size mismatch");
    const bool in_place = grad.slot() == sink.slot() && grad.desc().offset == sink.desc().offset;      // the producer wrote into the sink
    if (!in_place) check(vb_copy(&sink.desc(), &grad.desc()), "copy into gradient buffer");
    t_grads[key] = sink;
    if (it->second.on_ready) it->second.on_ready(it->second.idx, it->second.user);
  } else t_grads[key] = grad;
}
}  // namespace

namespace { void run_backward(const Tensor& y, const Tensor& seed, const NestedInput& nested); }

void Tensor::backward() const {
  if (numel() != 1) throw Error("backward can only be called on scalar tensors");
  t_enabled = false;
  Restore restore;
  if (live_index(*this) < 0) return;
  float one = 1.0f;
  Tensor seed = Tensor::from_f32(&one, shape());
  t_grads.clear();
  run_backward(*this, seed, NestedInput{});
  t_tape.generation++;
}

namespace {
// backward_impl (vearo-autograd/src/lib.rs:429-792) over the nodes recorded since the last reset; `seed` is the gradient of y.
// Called once per Tensor::backward, and once more, on a tape of its own, for every checkpointed block met on the way.
void run_backward(const Tensor& y, const Tensor& seed, const NestedInput& nested) {
  int out_idx = live_index(y);
  if (out_idx < 0) return;
  std::vector<Node> nodes = std::move(t_tape.nodes);
  t_tape.nodes.clear();
  const int N = (int)nodes.size();
  // earliest consumer of every node: once the walk has processed it, that node's gradient is final
  std::vector<int> first_use(N, N);
  for (const Node& n : nodes) for (int in : n.inputs) if (in >= 0 && n.id < first_use[in]) first_use[in] = n.id;
  std::vector<Tensor> gm(N);
  gm[out_idx] = seed;
  for (int ni = N - 1; ni >= 0; --ni) {
    Node& node = nodes[ni];
    if (!gm[ni].defined()) { node.saved.clear(); node.extra = Tensor(); continue; }
    if (node.op == Op::Leaf) continue;
    Tensor go = std::move(gm[ni]); gm[ni] = Tensor();
    const std::vector<Tensor>& sv = node.saved;
    std::vector<Tensor> gin;
    switch (node.op) {
      case Op::Add: gin = {reduce_to(go, sv[0].shape()), reduce_to(go, sv[1].shape())}; break;
      case Op::Sub: gin = {reduce_to(go, sv[0].shape()), reduce_to(scaled(go, -1.0f), sv[1].shape())}; break;
      case Op::Mul: gin = {reduce_to(go.mul(sv[1]), sv[0].shape()), reduce_to(go.mul(sv[0]), sv[1].shape())}; break;
      case Op::Div: {
        Tensor gl = go.div(sv[1]);
        Tensor gr = scaled(go, -1.0f).mul(sv[0]).div(sv[1].mul(sv[1]));
        gin = {reduce_to(gl, sv[0].shape()), reduce_to(gr, sv[1].shape())}; break;
      }
      case Op::Matmul: {
        Tensor lt = sv[0].transpose(sv[0].rank() - 2, sv[0].rank() - 1);
        Tensor rt = sv[1].transpose(sv[1].rank() - 2, sv[1].rank() - 1);
        gin = {reduce_to(go.matmul(rt), sv[0].shape()), reduce_to(lt.matmul(go), sv[1].shape())}; break;
      }
      case Op::Reshape: gin = {go.reshape(sv[0].shape())}; break;
      case Op::Transpose: gin = {go.transpose((int)node.a0, (int)node.a1)}; break;
      case Op::Permute: { std::vector<i64> inv(node.axes.size()); for (size_t i = 0; i < node.axes.size(); ++i) inv[node.axes[i]] = (i64)i; gin = {go.permute(inv)}; break; }
      case Op::Relu: { vb_tensor o; check(vb_relu_backward(&sv[0].desc(), &go.desc(), &o), "relu_backward"); gin = {Tensor::adopt(o)}; break; }
      case Op::Gelu: { vb_tensor o; check(vb_gelu_backward(&sv[0].desc(), &go.desc(), &o), "gelu_backward"); gin = {Tensor::adopt(o)}; break; }
      case Op::Softmax: { vb_tensor o; check(vb_softmax_backward(&sv[0].desc(), &go.desc(), (int)node.a0, &o), "softmax_backward"); gin = {Tensor::adopt(o)}; break; }
      case Op::LayerNorm: {
        vb_tensor gx, gw, gb;
        // x already holds a gradient from another consumer (a residual connection) in storage nobody else reads: dx is added to it
        // by the kernel that forms it, instead of being written out and accumulated afterwards
        const int xid = node.inputs[0];
        if (xid >= 0 && gm[xid].defined() && gm[xid].storage_unique() && gm[xid].is_contiguous() && gm[xid].shape() == sv[0].shape()) {
          check(vb_layernorm_backward_accum(&sv[0].desc(), &sv[1].desc(), &sv[2].desc(), &go.desc(), node.f0, &gm[xid].desc(), &gw, &gb), "layernorm_backward");
          gin = {Tensor(), Tensor::adopt(gw), Tensor::adopt(gb)}; break;
        }
        check(vb_layernorm_backward(&sv[0].desc(), &sv[1].desc(), &sv[2].desc(), &go.desc(), node.f0, &gx, &gw, &gb), "layernorm_backward");
        gin = {Tensor::adopt(gx), Tensor::adopt(gw), Tensor::adopt(gb)}; break;
      }
      case Op::BatchNorm: {
        vb_tensor gx, gw, gb;
        check(vb_batchnorm_backward(&sv[0].desc(), &sv[1].desc(), &sv[2].desc(), &sv[3].desc(), &sv[4].desc(), &go.desc(),
                                    (int)node.a0, node.f0, &gx, &gw, &gb), "batchnorm_backward");
        gin = {Tensor::adopt(gx), Tensor::adopt(gw), Tensor::adopt(gb), Tensor(), Tensor()}; break;
      }
      case Op::BnReluPool: {
        vb_tensor gx, gw, gb;
        check(vb_bn_relu_maxpool_backward(&sv[0].desc(), &sv[1].desc(), &sv[2].desc(), &node.extra.desc(), &go.desc(), (int)node.a0, &gx, &gw, &gb), "bn_relu_maxpool_backward");
        gin = {Tensor::adopt(gx), Tensor::adopt(gw), Tensor::adopt(gb)}; break;
      }
      case Op::Embedding: { vb_tensor o; check(vb_embedding_backward(&sv[0].desc(), &sv[1].desc(), &go.desc(), &o), "embedding_backward"); gin = {Tensor(), Tensor::adopt(o)}; break; }
      case Op::CrossEntropy: {
        if (node.a1) {      // fused forward: the gradient for a unit seed is already in place of the logits
          const bool unit_seed = !nested.active && ni == out_idx;
          gin = {unit_seed ? sv[0] : sv[0].mul(go), Tensor()};
          break;
        }
        vb_tensor o;
        check(vb_cross_entropy_backward(&sv[0].desc(), &sv[1].desc(), &go.desc(), node.extra.defined() ? &node.extra.desc() : nullptr, &o), "cross_entropy_backward");
        gin = {Tensor::adopt(o), Tensor()}; break;
      }
      case Op::FusedAttention: {
        vb_tensor dq, dk, dv;
        check(vb_fused_attention_backward(&sv[0].desc(), &sv[1].desc(), &sv[2].desc(), sv.size() > 3 ? &sv[3].desc() : nullptr, &go.desc(),
                                          node.extra.defined() ? &node.extra.desc() : nullptr, &dq, &dk, &dv), "fused_attention_backward");
        gin = {Tensor::adopt(dq), Tensor::adopt(dk), Tensor::adopt(dv)};
        if (sv.size() > 3) gin.push_back(Tensor());
        break;
      }
      case Op::FusedAttentionPacked: {
        vb_tensor dqkv;
        check(vb_fused_attention_packed_backward(&sv[0].desc(), (int)node.a0, sv.size() > 1 ? &sv[1].desc() : nullptr, &go.desc(),
                                                 node.extra.defined() ? &node.extra.desc() : nullptr, &dqkv), "fused_attention_packed_backward");
        gin = {Tensor::adopt(dqkv)};
        if (sv.size() > 1) gin.push_back(Tensor());
        break;
      }
      case Op::PackRows: {      // row blocks of the gradient, as views
        i64 rows[3] = {node.a0, node.a1, node.a2}, at = 0;
        for (int i = 0; i < 3; ++i) {
          vb_tensor d = go.desc();
          d.dims[0] = rows[i]; d.offset += at * d.strides[0];
          gin.push_back(Tensor::view_of(go, d));
          at += rows[i];
        }
        break;
      }
      case Op::Conv2d: {
        vb_tensor gi, gw, gb;
        const bool need_x = node.inputs[0] >= 0;       // the first layer's input takes no gradient
        check(vb_conv2d_backward(&sv[0].desc(), &sv[1].desc(), &go.desc(), (int)node.a0, (int)node.a1, need_x ? &gi : nullptr, &gw, &gb), "conv2d_backward");
        gin = {need_x ? Tensor::adopt(gi) : Tensor(), Tensor::adopt(gw), Tensor::adopt(gb)}; break;
      }
      case Op::MaxPool2d: { vb_tensor o; check(vb_maxpool2d_backward(&sv[0].desc(), &go.desc(), (int)node.a0, (int)node.a1, (int)node.a2, &o), "maxpool2d_backward"); gin = {Tensor::adopt(o)}; break; }
      case Op::AvgPool2d: { vb_tensor o; check(vb_avgpool2d_backward(&sv[0].desc(), &go.desc(), (int)node.a0, (int)node.a1, (int)node.a2, &o), "avgpool2d_backward"); gin = {Tensor::adopt(o)}; break; }
      case Op::Sum: gin = {expand_reduce_grad(go, sv[0].shape(), (int)node.a0, node.a1 != 0)}; break;
      case Op::Mean: {
        Tensor e = expand_reduce_grad(go, sv[0].shape(), (int)node.a0, node.a1 != 0);
        gin = {scaled(e, 1.0f / (float)sv[0].shape()[node.a0])}; break;
      }
      case Op::Linear: {
        bool need_x = node.inputs[0] >= 0, need_w = node.inputs[1] >= 0, need_b = sv.size() > 2 && node.inputs[2] >= 0;
        // A parameter that gets its whole gradient from this node and owns a slice of the flat gradient buffer: the products
        // write straight into the slice (no fresh tensor, no copy when the leaf is published).
        auto sink_of = [&](int id) -> const Tensor* {
          if (id < 0 || nodes[id].op != Op::Leaf || first_use[id] != ni || gm[id].defined()) return nullptr;
          auto it = t_sinks.index.find(leaf_key(nodes[id].leaf));
          if (it == t_sinks.index.end()) return nullptr;
          if (t_grads.count(leaf_key(nodes[id].leaf))) return nullptr;      // already holds a contribution of this pass: must be added to
          const Tensor& s = it->second.sink;
          return (s.is_contiguous() && s.numel() == nodes[id].leaf.numel()) ? &s : nullptr;
        };
        const Tensor* ws = need_w ? sink_of(node.inputs[1]) : nullptr;
        const Tensor* bs = need_b ? sink_of(node.inputs[2]) : nullptr;
        vb_tensor gx, gw, gb;
        if (ws || bs) {
          check(vb_linear_backward_into(&sv[0].desc(), &sv[1].desc(), &go.desc(), need_x ? &gx : nullptr, ws ? &ws->desc() : nullptr, bs ? &bs->desc() : nullptr), "linear_backward");
          if ((need_w && !ws) || (need_b && !bs))      // the other gradient the ordinary way
            check(vb_linear_backward(&sv[0].desc(), &sv[1].desc(), &go.desc(), nullptr, (need_w && !ws) ? &gw : nullptr, (need_b && !bs) ? &gb : nullptr), "linear_backward");
        } else {
          check(vb_linear_backward(&sv[0].desc(), &sv[1].desc(), &go.desc(), need_x ? &gx : nullptr, need_w ? &gw : nullptr, need_b ? &gb : nullptr), "linear_backward");
        }
        gin = {need_x ? Tensor::adopt(gx) : Tensor(), !need_w ? Tensor() : (ws ? *ws : Tensor::adopt(gw))};
        if (sv.size() > 2) gin.push_back(!need_b ? Tensor() : (bs ? *bs : Tensor::adopt(gb)));
        break;
      }
      case Op::Checkpoint: {
        // Run the block again, recording this time, and walk its tape with `go` as the seed (lib.rs:649-730).  Stateful
        // layers see is_recomputing() and leave their state alone; parameter gradients are published from the inner walk.
        const Tensor x = sv[0];
        const i64 x_token = x.node_id();
        t_tape.nodes.clear(); t_tape.generation++;
        // rewind the randomness counter to where the block first ran: a dropout inside draws the same mask again (lib.rs:680-690)
        const uint64_t saved_counter = t_rng_counter;
        t_rng_counter = node.rng;
        t_enabled = true; t_recomputing = true;
        Tensor y_new;
        try { y_new = node.fn(x); } catch (...) { t_enabled = false; t_recomputing = false; t_rng_counter = saved_counter; throw; }
        t_enabled = false; t_recomputing = false;
        t_rng_counter = saved_counter;
        Tensor gx;
        NestedInput inner; inner.active = true; inner.key = leaf_key(x); inner.gx = &gx;
        run_backward(y_new, go, inner);
        t_tape.nodes.clear(); t_tape.generation++;
        x.set_node_id(x_token);
        gin = {gx};
        node.fn = nullptr;
        break;
      }
      case Op::Leaf: break;
    }
    go = Tensor();
    for (size_t i = 0; i < node.inputs.size(); ++i) {
      int id = node.inputs[i];
      if (id < 0 || !gin[i].defined()) continue;
      if (!gm[id].defined()) gm[id] = gin[i];
      else if (gm[id].storage_unique() && gm[id].is_contiguous() && gm[id].shape() == gin[i].shape())
        check(vb_accumulate(&gm[id].desc(), &gin[i].desc()), "accumulate");          // existing += new
      else gm[id] = gm[id].add(gin[i]);                                              // existing + new (lib.rs:736-737)
    }
    gin.clear();
    // leaves whose last contribution this was: publish now
    for (int id : node.inputs)
      if (id >= 0 && nodes[id].op == Op::Leaf && first_use[id] == ni && gm[id].defined()) { publish_leaf(nodes[id], gm[id], nested); gm[id] = Tensor(); }
    node.saved.clear(); node.extra = Tensor();
  }
}
}  // namespace

namespace autograd {
// checkpoint (vearo-autograd/src/lib.rs:897-959): run the block without recording -- its activations are freed as it goes -- keep
// only the input, and record one node that re-runs the block when the backward walk reaches it.
Tensor checkpoint(const Tensor& x, std::function<Tensor(const Tensor&)> f) {
  const bool was = t_enabled;
  const uint64_t rng_at_entry = t_rng_counter;
  t_enabled = false;
  Tensor out;
  try { out = f(x); } catch (...) { t_enabled = was; throw; }
  t_enabled = was;
  if (was && (x.requires_grad() || out.requires_grad())) {
    out.set_requires_grad(true);
    Node& n = push(Op::Checkpoint, {&x}, out);
    n.fn = std::move(f);
    n.rng = rng_at_entry;
  }
  return out;
}
bool is_recomputing() { return t_recomputing; }
uint64_t rng_counter() { return t_rng_counter; }
void set_rng_counter(uint64_t v) { t_rng_counter = v; }
uint64_t next_rng_counter() { return t_rng_counter++; }
}  // namespace autograd

bool Tensor::grad(Tensor* out) const {
  auto it = t_grads.find(leaf_key(*this));
  if (it == t_grads.end()) return false;
  *out = it->second;
  return true;
}

}  // namespace vearo
