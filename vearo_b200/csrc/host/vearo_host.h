// Host side above the C ABI: the C++ mirror of the reference's Rust host layers for the training
// hot path — `Tensor` with its dispatch + record methods (crates/vearo-core/src/tensor.rs), the
// autograd tape and backward walk (crates/vearo-autograd/src/lib.rs), the layers that emit the
// five workload graphs (crates/vearo-nn/src/lib.rs) and the optimizers (crates/vearo-optim/src/lib.rs).
// Same names, argument meaning and error behaviour (a Rust panic becomes a C++ exception carrying
// the same text).  Everything below talks to the device only through include/vearo_b200.h.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../../include/vearo_b200.h"

namespace vearo {

using i64 = int64_t;

struct Error : std::runtime_error { using std::runtime_error::runtime_error; };
void check(int status, const char* what);   // throws Error with vb_last_error() text

// One owner of a device slot; the last owner to go releases it (the REFCOUNT_INC / REFCOUNT_DEC
// protocol of vearo-core/src/tensor.rs:20-80 collapsed into a shared_ptr).
struct Storage {
  vb_slot slot;
  explicit Storage(vb_slot s) : slot(s) {}
  ~Storage();
  Storage(const Storage&) = delete;
  Storage& operator=(const Storage&) = delete;
};

struct Meta { bool requires_grad = false; i64 node = -1; };

class Tensor {
 public:
  Tensor() = default;
  static Tensor from_f32(const float* data, const std::vector<i64>& shape);   // H2D upload
  static Tensor zeros(const std::vector<i64>& shape);
  static Tensor zeros_for_collectives(const std::vector<i64>& shape);          // vb_dp_alloc: registered with the communicator where possible
  static Tensor adopt(const vb_tensor& t);                                     // takes ownership of a fresh output
  static Tensor view_of(const Tensor& base, const vb_tensor& d);               // shares storage

  bool defined() const { return (bool)st_; }
  const vb_tensor& desc() const { return d_; }
  std::vector<i64> shape() const { return std::vector<i64>(d_.dims, d_.dims + d_.rank); }
  int rank() const { return d_.rank; }
  i64 numel() const { i64 n = 1; for (int i = 0; i < d_.rank; ++i) n *= d_.dims[i]; return n; }
  bool is_contiguous() const;
  std::vector<float> to_vec_f32() const;                  // contiguous D2H copy
  void write_f32(const float* data) const;                // overwrite (contiguous tensors)
  bool requires_grad() const { return meta_->requires_grad; }
  void set_requires_grad(bool f) const { meta_->requires_grad = f; }
  i64 node_id() const { return meta_->node; }
  void set_node_id(i64 n) const { meta_->node = n; }
  bool storage_unique() const { return st_.use_count() == 1; }
  vb_slot slot() const { return d_.slot; }

  // ops: dispatch to the device library, then record on the tape (tensor.rs:1365-1970)
  Tensor add(const Tensor& o) const; Tensor sub(const Tensor& o) const;
  Tensor mul(const Tensor& o) const; Tensor div(const Tensor& o) const;
  Tensor matmul(const Tensor& o) const;
  Tensor relu() const; Tensor gelu() const;
  Tensor sum(int dim, bool keep_dim) const; Tensor mean(int dim, bool keep_dim) const;
  Tensor softmax(int dim) const;
  Tensor layernorm(const Tensor& w, const Tensor& b, float eps) const;
  Tensor embedding(const Tensor& weight) const;             // self = ids
  Tensor cross_entropy(const Tensor& targets) const;        // self = logits
  Tensor conv2d(const Tensor& w, const Tensor& b, int stride, int padding) const;
  Tensor maxpool2d(int k, int s, int p) const; Tensor avgpool2d(int k, int s, int p) const;
  Tensor batchnorm(const Tensor& gamma, const Tensor& beta, const Tensor& rm, const Tensor& rv, bool training, float momentum, float eps) const;
  // batchnorm -> relu -> maxpool2d(2, 2, 0) as one op (one tape node, one fused backward)
  Tensor bn_relu_maxpool(const Tensor& gamma, const Tensor& beta, const Tensor& rm, const Tensor& rv, bool training, float momentum, float eps) const;
  Tensor fused_attention(const Tensor& k, const Tensor& v, const Tensor* mask) const;
  // self = packed projection [B, S, 3*D] (column blocks q | k | v): context [B, S, D]; one backward node returning [B, S, 3*D]
  Tensor fused_attention_packed(i64 n_head, const Tensor* mask) const;
  // a, b, c: views that lie one after another along dim 0 of one storage (same trailing shape); the view that spans the three.
  // Recorded on the tape: its gradient is handed back to a, b and c as row blocks.
  static Tensor pack_rows(const Tensor& a, const Tensor& b, const Tensor& c);
  Tensor linear(const Tensor& weight, const Tensor* bias) const;   // fused x.W^T + b
  Tensor linear_gelu(const Tensor& weight, const Tensor* bias) const;   // linear(...).gelu() with the activation formed in the GEMM's epilogue
  Tensor reshape(const std::vector<i64>& shape) const;
  Tensor transpose(int d0, int d1) const;
  Tensor permute(const std::vector<i64>& axes) const;
  Tensor contiguous() const;

  // cross_entropy that may overwrite the logits (self) with their gradient; use where the logits are needed for nothing else
  Tensor cross_entropy_consuming(const Tensor& targets) const;
  void backward() const;                // tensor.rs:703-714
  bool grad(Tensor* out) const;         // tensor.rs:716-725; false when no gradient is held

 private:
  std::shared_ptr<Storage> st_;
  std::shared_ptr<Meta> meta_ = std::make_shared<Meta>();
  vb_tensor d_{};
};

// ---- autograd (vearo-autograd/src/lib.rs) ----------------------------------------------------
namespace autograd {
void set_enabled(bool e); bool is_enabled();
void set_training(bool t); bool is_training();
void reset_active_tape();      // lib.rs:831
void zero_gradients();         // lib.rs:836
size_t tape_len();
// Activation checkpointing (lib.rs:897-959): runs f(x) without recording and keeps only x; the backward walk runs f again,
// recording, and differentiates that.  While it does, is_recomputing() is true and stateful layers leave their state alone.
Tensor checkpoint(const Tensor& x, std::function<Tensor(const Tensor&)> f);
bool is_recomputing();
// Per-call randomness counter (vearo-core/src/tensor.rs:1240-1285): random layers derive their draw from it instead of holding
// state, and checkpoint() rewinds it for the recomputation.
uint64_t rng_counter(); void set_rng_counter(uint64_t v); uint64_t next_rng_counter();
// Persistent gradient buffers: when a leaf with a registered sink gets its final gradient, the
// gradient is written into the sink (a view of a flat arena) instead of a fresh tensor, and
// `on_ready(index)` fires — which is what lets the data-parallel reducer start a bucket's
// allreduce while the backward pass is still running.
void register_grad_sinks(const std::vector<Tensor>& params, const std::vector<Tensor>& sinks, void (*on_ready)(int, void*), void* user);
void clear_grad_sinks(void* user);   // removes the sinks `user` registered
}  // namespace autograd

// ---- optimizers (vearo-optim/src/lib.rs) -----------------------------------------------------
namespace optim {
// Fused multi-tensor optimizer over persistent gradient buffers; `step()` has the semantics of
// AdamW::step / SGD::step (parameters without a gradient this step are skipped, t still advances).
class Optimizer {
 public:
  Optimizer(const vb_opt_config& cfg, const std::vector<Tensor>& params, bool data_parallel);
  ~Optimizer();
  void step();                                 // no clipping
  float clip_and_step(float max_norm, bool read_norm = true);   // clip_grad_norm + step fused; returns the pre-clip norm (0 when not read)
  void set_lr(float lr); float lr() const { return cfg_.lr; }
  const std::vector<Tensor>& params() const { return params_; }
  const std::vector<Tensor>& grads() const { return sinks_; }
  // Optimizer state as a `.ve` container (see checkpoint::): tensor 0 = the AdamW step counter t and the per-call randomness
  // counter, as exact 16-bit parts; tensor 1 = the flat state array (m then v, or the velocity).  Loading restores all
  // three.  The reference's optimizers have no save of their own.
  void save_state(const std::string& path) const;
  void load_state(const std::string& path);
  int handle() const { return opt_; }          // the library's optimizer handle (vb_opt_*)
  bool gradients_registered() const { int yes = 0; vb_dp_is_registered(arena_.slot(), &yes); return yes != 0; }   // the gradient arena is a buffer registered with the communicator
 private:
  void finish_reduce(bool deferred = false);
  static void on_ready(int idx, void* self);
  vb_opt_config cfg_;
  std::vector<Tensor> params_, sinks_;
  Tensor arena_;
  int opt_ = -1;
  bool dp_ = false;
  // data-parallel bucketing over the flat gradient arena
  struct Bucket { i64 offset, numel; int pending, nparams; };
  std::vector<Bucket> buckets_;
  std::vector<int> bucket_of_;
  std::vector<uint8_t> ready_;
  int world_ = 1;
};
// Gradient-bucket plan for data parallel: parameters are laid out in a flat arena in registration order
// (each rounded up to 4 floats); buckets are contiguous arena ranges of at least `target_elems`, cut from
// the END of the arena backwards, because gradients become final in roughly reverse parameter order.
// Pure host arithmetic (no device needed); every rank computes the same plan from the same shapes.
struct BucketPlan { std::vector<i64> param_offset, bucket_offset, bucket_numel; std::vector<int> bucket_of, bucket_nparams; i64 total = 0; };
BucketPlan plan_buckets(const std::vector<i64>& numels, i64 target_elems);
// Reference-shaped free function: clip_grad_norm(params, max_norm) -> pre-clip norm (lib.rs:360-383).
float clip_grad_norm(const std::vector<Tensor>& params, float max_norm);
float cosine_lr(float base_lr, float min_lr, uint32_t warmup, uint32_t total, uint32_t step);   // lib.rs:336-348
}  // namespace optim

// ---- `.ve` weight checkpoints (crates/vearo/src/checkpoint.rs:10-88) ---------------------------
// File: u32 tensor count; per tensor u32 rank, u32 dims..., u32 element count, f32 data; little endian.
namespace checkpoint {
void save_checkpoint(const std::vector<Tensor>& params, const std::string& path);
void load_checkpoint(const std::vector<Tensor>& params, const std::string& path);   // count / shape mismatches throw with the reference's messages
// the container itself, on host arrays
struct HostTensor { std::vector<i64> dims; std::vector<float> data; };
void write_container(const std::vector<HostTensor>& ts, const std::string& path);
std::vector<HostTensor> read_container(const std::string& path);
}  // namespace checkpoint

// ---- layers and the five workload graphs (vearo-nn/src/lib.rs) -------------------------------
namespace nn {
// Dropout (vearo-nn/src/lib.rs:308-357): the mask is a pure function of (seed, call counter) drawn from the reference's xorshift64
// generator on the host, as the reference does for every device, uploaded and multiplied in.  Identity when p <= 0 or not training.
struct Dropout {
  float p = 0.0f; uint64_t seed = 0;
  Dropout() = default;
  Dropout(float p_, uint64_t seed_) : p(p_), seed(seed_) {}
  Tensor forward(const Tensor& x) const;
};
struct Linear {
  Tensor weight, bias; bool has_bias = false;
  Linear() = default;
  Linear(i64 in, i64 out, bool bias);
  Tensor forward(const Tensor& x) const;
  void parameters(std::vector<Tensor>& out) const;
};
struct LayerNorm {
  Tensor weight, bias; float eps = 1e-5f;
  LayerNorm() = default;
  explicit LayerNorm(i64 dim, float eps = 1e-5f);
  Tensor forward(const Tensor& x) const { return x.layernorm(weight, bias, eps); }
  void parameters(std::vector<Tensor>& out) const { out.push_back(weight); out.push_back(bias); }
};
// The q, k and v projections are separate parameters, as in the reference, but their storage is one [3*D, D] weight
// block and one [3*D] bias block: the forward runs ONE GEMM for the three projections and the attention op reads its
// packed output in place; the backward mirrors it (one GEMM for dX over K = 3*D, one for the stacked weight gradient).
struct MultiHeadAttention {
  Linear q, k, v, o; i64 n_head = 1, n_embd = 1;
  Tensor w_qkv, b_qkv;        // the blocks that q/k/v .weight and .bias are views of
  MultiHeadAttention() = default;
  MultiHeadAttention(i64 n_embd, i64 n_head);
  Tensor forward(const Tensor& x, const Tensor* mask) const;
  void parameters(std::vector<Tensor>& out) const;
};
struct TransformerBlock {
  LayerNorm ln1, ln2; MultiHeadAttention attn; Linear fc1, fc2;
  TransformerBlock() = default;
  TransformerBlock(i64 n_embd, i64 n_head, i64 mlp_dim);
  Tensor forward(const Tensor& x, const Tensor* mask) const;
  void parameters(std::vector<Tensor>& out) const;
};
struct Model {
  virtual ~Model() = default;
  virtual std::vector<Tensor> parameters() const = 0;
  // inputs -> scalar loss
  virtual Tensor loss(const Tensor& x, const Tensor& y) = 0;
};
struct SimpleGPT : Model {
  Tensor tok, pos; std::vector<TransformerBlock> blocks; LayerNorm ln_f; Linear lm_head; i64 n_embd;
  Tensor pos_ids_, mask_; i64 cached_b_ = -1, cached_s_ = -1;     // built on the device once per shape
  bool checkpoint_blocks = false;     // wrap every transformer block in autograd::checkpoint (activations of one block live at a time)
  SimpleGPT(i64 vocab, i64 max_seq, i64 n_embd, i64 n_head, i64 n_layer, i64 mlp_dim);
  std::vector<Tensor> parameters() const override;
  Tensor loss(const Tensor& ids, const Tensor& targets) override;
};
struct MLP : Model {
  std::vector<Linear> layers;
  explicit MLP(const std::vector<i64>& sizes);
  std::vector<Tensor> parameters() const override;
  Tensor forward(const Tensor& x) const;
  Tensor loss(const Tensor& x, const Tensor& y) override;   // mean((f(x)-y)^2) over dim 0
};
struct ConvNet : Model {
  struct Stage { Tensor w, b, gamma, beta, rm, rv; };
  std::vector<Stage> stages; Linear fc; float momentum = 0.1f, eps = 1e-5f;
  ConvNet(const std::vector<i64>& channels, i64 n_class);
  std::vector<Tensor> parameters() const override;
  Tensor loss(const Tensor& x, const Tensor& labels) override;
};
// LayerNorm -> GELU -> Linear (no bias) -> cross-entropy, with x itself requiring a gradient.
struct FusedOpBench : Model {
  LayerNorm ln; Linear head;
  FusedOpBench(i64 c, i64 v);
  std::vector<Tensor> parameters() const override;
  Tensor loss(const Tensor& x, const Tensor& labels) override;
};
}  // namespace nn

}  // namespace vearo
