// CPU oracle: a plain C++ restatement of the reference's CPU backend, autograd
// backward arms and optimizers.  TEST INFRASTRUCTURE ONLY: nothing in the shipped
// library links, loads or calls this file.  It exists so that the CUDA path can be
// compared against the arithmetic the reference defines, and so that a CPU baseline
// can be timed next to the GPU numbers.
//
// Every function cites the reference file:line it follows (paths are relative to the
// reference project root).  Loop orders, accumulation orders and the places where the
// reference uses a fused multiply-add (`mul_add`) are kept; everything else is plain
// IEEE f32.  Build with -ffp-contract=off so the compiler fuses nothing on its own.
//
// Pinning: checked against the reference's own known-answer tests and NumPy fixtures
// (tests/test_oracle_*.py) and, for the matmul micro-kernel, bit-for-bit against the
// reference's assembly kernel compiled from its own source (oracle/_ref).
//
// What is deliberately not restated: the arena/mutex traffic and per-element heap
// allocations of the reference (`flat_to_coord`), which cost time but change no value.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>
#include <immintrin.h>

namespace orc {

using i64 = int64_t;
using Buf = std::shared_ptr<std::vector<float>>;

static std::string g_err;
[[noreturn]] static void fail(const std::string& m) { throw std::runtime_error(m); }

static int g_threads = 0;  // 0 = hardware_concurrency (std::thread::available_parallelism)
static int n_threads() {
  int t = g_threads > 0 ? g_threads : (int)std::thread::hardware_concurrency();
  return t < 1 ? 1 : t;
}

// ---------------------------------------------------------------------------------
// Tensor: storage + shape + strides (vearo-core/src/tensor.rs:10-18).  Views share the
// buffer.  `node` is the tape token (generation << 32 | index), -1 when absent.
// ---------------------------------------------------------------------------------
struct Tensor {
  Buf buf;
  std::vector<i64> shape, strides;
  mutable i64 node = -1;
  mutable bool requires_grad = false;

  i64 numel() const { i64 n = 1; for (i64 d : shape) n *= d; return n; }
  int rank() const { return (int)shape.size(); }
  bool is_contiguous() const {
    i64 s = 1;
    for (int i = rank() - 1; i >= 0; --i) {
      if (shape[i] != 1 && strides[i] != s) return false;
      s *= shape[i];
    }
    return true;
  }
};

static std::vector<i64> contiguous_strides(const std::vector<i64>& shape) {
  std::vector<i64> st(shape.size());
  i64 s = 1;
  for (int i = (int)shape.size() - 1; i >= 0; --i) { st[i] = s; s *= shape[i]; }
  return st;
}

static Tensor make(const std::vector<i64>& shape) {
  Tensor t;
  t.shape = shape;
  t.strides = contiguous_strides(shape);
  t.buf = std::make_shared<std::vector<float>>((size_t)t.numel(), 0.0f);
  return t;
}
static Tensor from_data(const float* d, const std::vector<i64>& shape) {
  Tensor t = make(shape);
  if (t.numel()) std::memcpy(t.buf->data(), d, sizeof(float) * (size_t)t.numel());
  return t;
}
static Tensor scalar1(float v) { return from_data(&v, {1}); }

// Offset of a coordinate given as the trailing `rank` entries of an output coordinate;
// size-1 dims contribute 0 (vearo-core/src/shape.rs:271-282).
static inline i64 bc_offset(const i64* coord, int coord_rank, const Tensor& t) {
  i64 off = 0;
  int r = t.rank();
  for (int d = 0; d < r; ++d) {
    i64 c = coord[coord_rank - r + d];
    if (t.shape[d] != 1) off += c * t.strides[d];
  }
  return off;
}

// Row-major odometer (vearo-core/src/shape.rs NdIterator).
struct NdIter {
  std::vector<i64> shape, coord;
  explicit NdIter(const std::vector<i64>& s) : shape(s), coord(s.size(), 0) {}
  bool step() {
    for (int d = (int)shape.size() - 1; d >= 0; --d) {
      if (++coord[d] < shape[d]) return true;
      coord[d] = 0;
    }
    return false;
  }
};

// Materialise a view in row-major order (vearo-core/src/tensor.rs:345-368).
static Tensor contiguous(const Tensor& t) {
  if (t.is_contiguous()) return t;
  Tensor o = make(t.shape);
  o.node = t.node; o.requires_grad = t.requires_grad;
  if (!t.numel()) return o;
  NdIter it(t.shape);
  float* dst = o.buf->data();
  const float* src = t.buf->data();
  i64 i = 0;
  int r = t.rank();
  do {
    i64 off = 0;
    for (int d = 0; d < r; ++d) off += it.coord[d] * t.strides[d];
    dst[i++] = src[off];
  } while (it.step());
  return o;
}
static const float* cdata(const Tensor& t) { return t.buf->data(); }

static std::vector<i64> broadcast_shape(const std::vector<i64>& a, const std::vector<i64>& b) {
  // NumPy rules, right aligned (vearo-core/src/shape.rs:91-124).
  size_t r = std::max(a.size(), b.size());
  std::vector<i64> o(r);
  for (size_t i = 0; i < r; ++i) {
    i64 da = i < r - a.size() ? 1 : a[i - (r - a.size())];
    i64 db = i < r - b.size() ? 1 : b[i - (r - b.size())];
    if (da == db || da == 1 || db == 1) o[i] = (da == 1 ? db : da);
    else fail("Shapes are not broadcastable");
  }
  return o;
}

// ---------------------------------------------------------------------------------
// Tape (vearo-autograd/src/lib.rs:15-197).
// ---------------------------------------------------------------------------------
enum Op { ADD, SUB, MUL, DIV, MATMUL, RESHAPE, TRANSPOSE, PERMUTE, RELU, GELU, SOFTMAX, LAYERNORM,
          EMBEDDING, CROSS_ENTROPY, SUM, MEAN, CONV2D, MAXPOOL2D, AVGPOOL2D, BATCHNORM,
          FUSED_ATTENTION, LEAF };

struct Node {
  int id; Op op;
  std::vector<int> inputs;          // node index or -1
  std::vector<Tensor> saved;
  i64 a0 = 0, a1 = 0, a2 = 0;        // integer attributes (dims, stride, padding, kernel, flags)
  float f0 = 0;                     // eps
  std::vector<i64> axes;
};
struct Tape { std::vector<Node> nodes; uint32_t generation = 0; };
static Tape g_tape;
static bool g_autograd = true;
static bool g_training = true;
// GRADIENTS keyed by storage (vearo-autograd/src/lib.rs:207).
static std::unordered_map<const void*, Tensor> g_grads;

static i64 pack(uint32_t gen, uint32_t idx) { return ((i64)gen << 32) | idx; }

// Tape::push (vearo-autograd/src/lib.rs:151-189).
static Node& tape_push(Op op, const std::vector<const Tensor*>& ins, Tensor& out) {
  std::vector<int> ids;
  for (const Tensor* in : ins) {
    int live = -1;
    if (in->node >= 0 && (uint32_t)(in->node >> 32) == g_tape.generation) live = (int)(in->node & 0xffffffff);
    if (live >= 0) ids.push_back(live);
    else if (in->requires_grad) {
      int leaf = (int)g_tape.nodes.size();
      Node n; n.id = leaf; n.op = LEAF;
      g_tape.nodes.push_back(n);
      in->node = pack(g_tape.generation, (uint32_t)leaf);
      ids.push_back(leaf);
    } else ids.push_back(-1);
  }
  Node n; n.id = (int)g_tape.nodes.size(); n.op = op; n.inputs = ids;
  for (const Tensor* in : ins) n.saved.push_back(*in);
  g_tape.nodes.push_back(n);
  out.node = pack(g_tape.generation, (uint32_t)n.id);
  return g_tape.nodes.back();
}
static bool want_record(const std::vector<const Tensor*>& ins) {
  if (!g_autograd) return false;
  for (const Tensor* t : ins) if (t->requires_grad) return true;
  return false;
}
// Dispatch + record as the Tensor::<op> methods do (vearo-core/src/tensor.rs:1365-1970).
static Node* record(Op op, const std::vector<const Tensor*>& ins, Tensor& out) {
  if (!want_record(ins)) return nullptr;
  out.requires_grad = true;
  return &tape_push(op, ins, out);
}

// ---------------------------------------------------------------------------------
// Raw (unrecorded) backend ops: vearo-backend-cpu/src/lib.rs.
// ---------------------------------------------------------------------------------
// elementwise_op, lib.rs:160-202
template <class F> static Tensor raw_binary(const Tensor& l, const Tensor& r, F op) {
  std::vector<i64> os = broadcast_shape(l.shape, r.shape);
  Tensor o = make(os);
  i64 n = o.numel();
  if (!n) return o;
  float* od = o.buf->data();
  const float* ld = cdata(l); const float* rd = cdata(r);
  if (l.is_contiguous() && r.is_contiguous() && l.shape == r.shape) {
    for (i64 i = 0; i < n; ++i) od[i] = op(ld[i], rd[i]);
  } else {
    NdIter it(os);
    int R = (int)os.size();
    i64 i = 0;
    do {
      od[i++] = op(ld[bc_offset(it.coord.data(), R, l)], rd[bc_offset(it.coord.data(), R, r)]);
    } while (it.step());
  }
  return o;
}
static Tensor raw_add(const Tensor& a, const Tensor& b) { return raw_binary(a, b, [](float x, float y) { return x + y; }); }
static Tensor raw_sub(const Tensor& a, const Tensor& b) { return raw_binary(a, b, [](float x, float y) { return x - y; }); }
static Tensor raw_mul(const Tensor& a, const Tensor& b) { return raw_binary(a, b, [](float x, float y) { return x * y; }); }
static Tensor raw_div(const Tensor& a, const Tensor& b) { return raw_binary(a, b, [](float x, float y) { return x / y; }); }

// The 4x8 AVX2/FMA block of src/asm/x86_64/matmul.s:13-98: four rows of A against eight
// columns of B, accumulators start at zero, one fused multiply-add per k in increasing k.
static inline void block_4x8(float* out, const float* lhs, const float* rhs, size_t k_l, size_t n) {
  __m256 c0 = _mm256_setzero_ps(), c1 = c0, c2 = c0, c3 = c0;
  const float* a0 = lhs; const float* a1 = lhs + k_l; const float* a2 = a1 + k_l; const float* a3 = a2 + k_l;
  for (size_t k = 0; k < k_l; ++k) {
    __m256 b = _mm256_loadu_ps(rhs);
    c0 = _mm256_fmadd_ps(_mm256_broadcast_ss(a0 + k), b, c0);
    c1 = _mm256_fmadd_ps(_mm256_broadcast_ss(a1 + k), b, c1);
    c2 = _mm256_fmadd_ps(_mm256_broadcast_ss(a2 + k), b, c2);
    c3 = _mm256_fmadd_ps(_mm256_broadcast_ss(a3 + k), b, c3);
    rhs += n;
  }
  _mm256_storeu_ps(out, c0); _mm256_storeu_ps(out + n, c1);
  _mm256_storeu_ps(out + 2 * n, c2); _mm256_storeu_ps(out + 3 * n, c3);
}

// matmul, lib.rs:266-417: operands made contiguous, leading dims broadcast, output rows
// split evenly over threads (400-413); full 4-row groups use the 4x8 block for full 8-column
// groups and a scalar fused chain for the column tail (344-368); other rows take the one-row
// path, k outer, n inner (383-393).  Every output is the same chain: fma over increasing k.
static Tensor raw_matmul(const Tensor& lhs, const Tensor& rhs) {
  int rl = lhs.rank(), rr = rhs.rank();
  if (rl < 2 || rr < 2) fail("Matmul requires rank >= 2");
  i64 m = lhs.shape[rl - 2], k_l = lhs.shape[rl - 1], k_r = rhs.shape[rr - 2], n = rhs.shape[rr - 1];
  if (k_l != k_r) fail("Incompatible dimensions for matmul");
  std::vector<i64> bl(lhs.shape.begin(), lhs.shape.end() - 2), br(rhs.shape.begin(), rhs.shape.end() - 2);
  std::vector<i64> ob = broadcast_shape(bl, br);
  std::vector<i64> os = ob; os.push_back(m); os.push_back(n);
  Tensor out = make(os);
  if (!out.numel()) return out;
  Tensor lc = contiguous(lhs), rc = contiguous(rhs);
  const float* ld = cdata(lc); const float* rd = cdata(rc);
  float* od = out.buf->data();
  Tensor lb; lb.shape = bl; lb.strides.assign(lc.strides.begin(), lc.strides.end() - 2);
  Tensor rb; rb.shape = br; rb.strides.assign(rc.strides.begin(), rc.strides.end() - 2);
  i64 nbatch = 1; for (i64 d : ob) nbatch *= d;
  i64 total_rows = nbatch * m;
  int obr = (int)ob.size();

  auto compute = [&](i64 start_row, i64 end_row) {
    i64 row = start_row;
    std::vector<i64> bc(obr > 0 ? obr : 1, 0);
    while (row < end_row) {
      i64 r_m = row % m, batch = row / m;
      i64 rem = batch;
      for (int i = obr - 1; i >= 0; --i) { bc[i] = rem % ob[i]; rem /= ob[i]; }
      i64 off_l = bc_offset(bc.data(), obr, lb), off_r = bc_offset(bc.data(), obr, rb);
      if (r_m + 4 <= m && row + 4 <= end_row) {
        i64 nb = n / 8;
        for (i64 b = 0; b < nb; ++b)
          block_4x8(od + row * n + b * 8, ld + off_l + r_m * k_l, rd + off_r + b * 8, (size_t)k_l, (size_t)n);
        for (i64 c = nb * 8; c < n; ++c)
          for (int ro = 0; ro < 4; ++ro) {
            float sum = 0.0f;
            for (i64 k = 0; k < k_l; ++k) sum = std::fmaf(ld[off_l + (r_m + ro) * k_l + k], rd[off_r + k * n + c], sum);
            od[(row + ro) * n + c] = sum;
          }
        row += 4;
      } else {
        float* rs = od + row * n;
        for (i64 k = 0; k < k_l; ++k) {
          float lv = ld[off_l + r_m * k_l + k];
          const float* rrow = rd + off_r + k * n;
          for (i64 c = 0; c < n; ++c) rs[c] = std::fmaf(lv, rrow[c], rs[c]);
        }
        row += 1;
      }
    }
  };
  int threads = n_threads();
  i64 rpt = (total_rows + threads - 1) / threads;
  if (threads <= 1 || total_rows < 2) compute(0, total_rows);
  else {
    std::vector<std::thread> th;
    for (i64 s = 0; s < total_rows; s += rpt) th.emplace_back(compute, s, std::min(total_rows, s + rpt));
    for (auto& t : th) t.join();
  }
  return out;
}

template <class F> static Tensor raw_unary(const Tensor& x, F f) {
  Tensor xc = contiguous(x);
  Tensor o = make(x.shape);
  const float* xd = cdata(xc); float* od = o.buf->data();
  for (i64 i = 0, n = o.numel(); i < n; ++i) od[i] = f(xd[i]);
  return o;
}
// relu, lib.rs:424-454
static Tensor raw_relu(const Tensor& x) { return raw_unary(x, [](float v) { return v > 0.0f ? v : 0.0f; }); }
static constexpr float SQRT_2_OVER_PI = 0.79788456f, GELU_COEFF = 0.044715f, GELU_DERIV = 0.134145f;
// gelu (tanh form), lib.rs:458-497
static Tensor raw_gelu(const Tensor& x) {
  return raw_unary(x, [](float v) {
    float v3 = v * v * v;
    float inner = SQRT_2_OVER_PI * (v + GELU_COEFF * v3);
    return 0.5f * v * (1.0f + std::tanh(inner));
  });
}
// relu_grad_mask / gelu_grad_mask, vearo-autograd/src/lib.rs:364-403
static Tensor relu_grad_mask(const Tensor& x) { return raw_unary(x, [](float v) { return v > 0.0f ? 1.0f : 0.0f; }); }
static Tensor gelu_grad_mask(const Tensor& x) {
  return raw_unary(x, [](float v) {
    float v3 = v * v * v;
    float inner = SQRT_2_OVER_PI * (v + GELU_COEFF * v3);
    float t = std::tanh(inner);
    float sech_sq = 1.0f - t * t;
    float inner_deriv = SQRT_2_OVER_PI * (1.0f + GELU_DERIV * v * v);
    return 0.5f * (1.0f + t) + 0.5f * v * sech_sq * inner_deriv;
  });
}

// softmax, lib.rs:501-563: per slice max (strict >), sum of exp in index order, exp/sum.
static Tensor raw_softmax(const Tensor& x, int dim) {
  if (dim >= x.rank()) fail("Softmax dim out of range");
  Tensor o = make(x.shape);
  if (!o.numel()) return o;
  const float* xd = cdata(x); float* od = o.buf->data();
  std::vector<i64> red = x.shape; red[dim] = 1;
  i64 dn = x.shape[dim];
  NdIter it(red);
  int R = x.rank();
  do {
    i64 base = 0, obase = 0;
    for (int d = 0; d < R; ++d) { base += it.coord[d] * x.strides[d]; obase += it.coord[d] * o.strides[d]; }
    float mx = -INFINITY;
    for (i64 j = 0; j < dn; ++j) { float v = xd[base + j * x.strides[dim]]; if (v > mx) mx = v; }
    float se = 0.0f;
    for (i64 j = 0; j < dn; ++j) se += std::exp(xd[base + j * x.strides[dim]] - mx);
    for (i64 j = 0; j < dn; ++j) od[obase + j * o.strides[dim]] = std::exp(xd[base + j * x.strides[dim]] - mx) / se;
  } while (it.step());
  return o;
}

// reduce_sum_data / sum / mean, lib.rs:566-653: contributions arrive in increasing index
// along the reduced axis; mean divides once at the end.
static Tensor raw_sum(const Tensor& x, int dim, bool keep, bool mean) {
  if (dim >= x.rank()) fail("Reduction dim out of range");
  std::vector<i64> os = x.shape;
  if (keep) os[dim] = 1; else os.erase(os.begin() + dim);
  Tensor o = make(os);
  float* od = o.buf->data();
  if (x.numel()) {
    const float* xd = cdata(x);
    NdIter it(x.shape);
    int R = x.rank();
    do {
      i64 in_off = 0, idx = 0, stride = 1;
      for (int d = 0; d < R; ++d) in_off += it.coord[d] * x.strides[d];
      for (int d = R - 1; d >= 0; --d) {
        if (d == dim) continue;
        idx += it.coord[d] * stride; stride *= x.shape[d];
      }
      od[idx] += xd[in_off];
    } while (it.step());
  }
  if (mean) { float c = (float)x.shape[dim]; for (i64 i = 0, n = o.numel(); i < n; ++i) od[i] /= c; }
  return o;
}

// layernorm, lib.rs:667-740
static Tensor raw_layernorm(const Tensor& x, const Tensor& w, const Tensor& b, float eps) {
  Tensor o = make(x.shape);
  if (!o.numel()) return o;
  i64 C = x.shape.back();
  if (w.rank() != 1 || b.rank() != 1 || w.shape[0] != C || b.shape[0] != C) fail("LayerNorm weight/bias must be rank 1 of norm_dim");
  Tensor xc = contiguous(x), wc = contiguous(w), bc = contiguous(b);
  const float* xd = cdata(xc); const float* wd = cdata(wc); const float* bd = cdata(bc);
  float* od = o.buf->data();
  i64 rows = o.numel() / C;
  for (i64 r = 0; r < rows; ++r) {
    const float* xr = xd + r * C;
    float sum = 0.0f; for (i64 i = 0; i < C; ++i) sum += xr[i];
    float mean = sum / (float)C;
    float sq = 0.0f; for (i64 i = 0; i < C; ++i) { float d = xr[i] - mean; sq += d * d; }
    float var = sq / (float)C;
    float inv = 1.0f / std::sqrt(var + eps);
    for (i64 i = 0; i < C; ++i) { float xh = (xr[i] - mean) * inv; od[r * C + i] = xh * wd[i] + bd[i]; }
  }
  return o;
}
// layernorm_backward, lib.rs:745-858
static void raw_layernorm_backward(const Tensor& x, const Tensor& w, const Tensor& b, const Tensor& go, float eps,
                                   Tensor& gx, Tensor& gw, Tensor& gb) {
  gx = make(x.shape); gw = make(w.shape); gb = make(b.shape);
  if (!x.numel()) return;
  i64 C = x.shape.back();
  Tensor xc = contiguous(x), wc = contiguous(w), gc = contiguous(go);
  const float* xd = cdata(xc); const float* wd = cdata(wc); const float* gd = cdata(gc);
  float* gxd = gx.buf->data(); float* gwd = gw.buf->data(); float* gbd = gb.buf->data();
  i64 rows = x.numel() / C;
  for (i64 r = 0; r < rows; ++r) {
    const float* xr = xd + r * C; const float* gr = gd + r * C;
    float sum = 0.0f; for (i64 i = 0; i < C; ++i) sum += xr[i];
    float mean = sum / (float)C;
    float sq = 0.0f; for (i64 i = 0; i < C; ++i) { float d = xr[i] - mean; sq += d * d; }
    float var = sq / (float)C;
    float inv = 1.0f / std::sqrt(var + eps);
    float s1 = 0.0f, s2 = 0.0f;
    for (i64 i = 0; i < C; ++i) {
      float xh = (xr[i] - mean) * inv;
      float wv = wd[i], g = gr[i];
      s1 += g * wv;
      s2 += g * wv * xh;
      gwd[i] += g * xh;
      gbd[i] += g;
    }
    for (i64 i = 0; i < C; ++i) {
      float xh = (xr[i] - mean) * inv;
      float t1 = (float)C * gr[i] * wd[i];
      float t3 = xh * s2;
      gxd[r * C + i] = (t1 - s1 - t3) * inv / (float)C;
    }
  }
}

static i64 checked_id(float v, i64 bound, const char* neg, const char* oob) {
  if (!(v >= 0.0f)) fail(neg);
  i64 id = (i64)std::round(v);  // half away from zero, as f32::round
  if (id >= bound) fail(oob);
  return id;
}
// embedding, lib.rs:862-918
static Tensor raw_embedding(const Tensor& idx, const Tensor& w) {
  if (w.rank() != 2) fail("Weight must be rank 2 (vocab_size, embedding_dim)");
  i64 V = w.shape[0], D = w.shape[1];
  std::vector<i64> os = idx.shape; os.push_back(D);
  Tensor o = make(os);
  if (!idx.numel()) return o;
  Tensor ic = contiguous(idx), wc = contiguous(w);
  const float* id = cdata(ic); const float* wd = cdata(wc); float* od = o.buf->data();
  for (i64 i = 0, n = idx.numel(); i < n; ++i) {
    i64 t = checked_id(id[i], V, "Token ID cannot be negative", "Token ID out of vocabulary bound");
    std::memcpy(od + i * D, wd + t * D, sizeof(float) * (size_t)D);
  }
  return o;
}
// embedding_backward, lib.rs:923-980: rows added in increasing token position.
static Tensor raw_embedding_backward(const Tensor& idx, const Tensor& w, const Tensor& go) {
  i64 V = w.shape[0], D = w.shape[1];
  Tensor gw = make(w.shape);
  Tensor ic = contiguous(idx), gc = contiguous(go);
  const float* id = cdata(ic); const float* gd = cdata(gc); float* o = gw.buf->data();
  for (i64 i = 0, n = idx.numel(); i < n; ++i) {
    i64 t = checked_id(id[i], V, "Token ID cannot be negative", "Token ID out of vocabulary bound");
    for (i64 d = 0; d < D; ++d) o[t * D + d] += gd[i * D + d];
  }
  return gw;
}

// cross_entropy, lib.rs:984-1051: mean over rows of -(l[t] - max - ln(sum exp)).
static Tensor raw_cross_entropy(const Tensor& logits, const Tensor& targets) {
  if (logits.rank() != 2 || targets.rank() != 1) fail("Logits must be rank 2 and targets rank 1");
  i64 B = logits.shape[0], V = logits.shape[1];
  if (B <= 0) fail("Batch size must be greater than 0");
  if (targets.shape[0] != B) fail("Targets shape must match batch size");
  Tensor lc = contiguous(logits), tc = contiguous(targets);
  const float* ld = cdata(lc); const float* td = cdata(tc);
  float loss_sum = 0.0f;
  for (i64 b = 0; b < B; ++b) {
    i64 cls = checked_id(td[b], V, "Target class cannot be negative", "Target class out of vocab bounds");
    const float* row = ld + b * V;
    float mx = -INFINITY; for (i64 c = 0; c < V; ++c) if (row[c] > mx) mx = row[c];
    float se = 0.0f; for (i64 c = 0; c < V; ++c) se += std::exp(row[c] - mx);
    float lsm = row[cls] - mx - std::log(se);
    loss_sum -= lsm;
  }
  return scalar1(loss_sum / (float)B);
}
// cross_entropy_backward, lib.rs:1055-1127
static Tensor raw_cross_entropy_backward(const Tensor& logits, const Tensor& targets, const Tensor& go) {
  i64 B = logits.shape[0], V = logits.shape[1];
  if (go.numel() != 1) fail("grad_out must be a scalar");
  Tensor lc = contiguous(logits), tc = contiguous(targets), gc = contiguous(go);
  const float* ld = cdata(lc); const float* td = cdata(tc);
  float g = cdata(gc)[0];
  Tensor gl = make(logits.shape);
  float* o = gl.buf->data();
  for (i64 b = 0; b < B; ++b) {
    i64 cls = checked_id(td[b], V, "Target class cannot be negative", "Target class out of vocab bounds");
    const float* row = ld + b * V;
    float mx = -INFINITY; for (i64 c = 0; c < V; ++c) if (row[c] > mx) mx = row[c];
    float se = 0.0f; for (i64 c = 0; c < V; ++c) se += std::exp(row[c] - mx);
    for (i64 c = 0; c < V; ++c) {
      float p = std::exp(row[c] - mx) / se;
      float ind = c == cls ? 1.0f : 0.0f;
      o[b * V + c] = g * (p - ind) / (float)B;
    }
  }
  return gl;
}

template <class F> static void parallel_tasks(i64 total, F f) {
  int threads = n_threads();
  i64 per = (total + threads - 1) / threads;
  std::vector<std::thread> th;
  for (int t = 0; t < threads; ++t) {
    i64 s = t * per, e = std::min(total, s + per);
    if (s >= e) continue;
    th.emplace_back([=] { f(s, e); });
  }
  for (auto& t : th) t.join();
}
static std::vector<float> pad_input(const float* x, i64 n, i64 cin, i64 h, i64 w, i64 p) {
  i64 hp = h + 2 * p, wp = w + 2 * p;
  std::vector<float> xp((size_t)(n * cin * hp * wp), 0.0f);
  for (i64 a = 0; a < n * cin; ++a)
    for (i64 ih = 0; ih < h; ++ih)
      std::memcpy(&xp[(a * hp + ih + p) * wp + p], x + (a * h + ih) * w, sizeof(float) * (size_t)w);
  return xp;
}
// conv2d (direct, zero-padded copy), lib.rs:1474-1582: output starts at the bias, taps arrive
// in (c, i, j) order with fma; a weight equal to 0.0 is skipped (1551).
static Tensor raw_conv2d(const Tensor& input, const Tensor& weight, const Tensor& bias, i64 stride, i64 pad) {
  Tensor ic = contiguous(input), wc = contiguous(weight), bc = contiguous(bias);
  i64 n = ic.shape[0], cin = ic.shape[1], h = ic.shape[2], w = ic.shape[3];
  i64 cout = wc.shape[0], kh = wc.shape[2], kw = wc.shape[3];
  if (wc.shape[1] != cin) fail("conv2d channel mismatch");
  i64 oh = (h + 2 * pad - kh) / stride + 1, ow = (w + 2 * pad - kw) / stride + 1;
  Tensor out = make({n, cout, oh, ow});
  if (!out.numel()) return out;
  i64 hp = h + 2 * pad, wp = w + 2 * pad;
  std::vector<float> xp = pad_input(cdata(ic), n, cin, h, w, pad);
  const float* wt = cdata(wc); const float* b = cdata(bc); float* od = out.buf->data();
  parallel_tasks(n * cout, [&](i64 s, i64 e) {
    for (i64 task = s; task < e; ++task) {
      i64 nn = task / cout, co = task % cout;
      i64 oo = (nn * cout + co) * oh * ow;
      std::fill(od + oo, od + oo + oh * ow, b[co]);
      for (i64 c = 0; c < cin; ++c)
        for (i64 i = 0; i < kh; ++i)
          for (i64 j = 0; j < kw; ++j) {
            float wv = wt[((co * cin + c) * kh + i) * kw + j];
            if (wv == 0.0f) continue;
            for (i64 y = 0; y < oh; ++y) {
              const float* xr = &xp[((nn * cin + c) * hp + y * stride + i) * wp + j];
              float* dr = od + oo + y * ow;
              for (i64 xo = 0; xo < ow; ++xo) dr[xo] = std::fmaf(wv, xr[xo * stride], dr[xo]);
            }
          }
    }
  });
  return out;
}
// conv2d_backward, lib.rs:1597-1793
static void raw_conv2d_backward(const Tensor& input, const Tensor& weight, const Tensor& go_, i64 stride, i64 pad,
                                Tensor& gi, Tensor& gw, Tensor& gb) {
  Tensor ic = contiguous(input), wc = contiguous(weight), gc = contiguous(go_);
  i64 n = ic.shape[0], cin = ic.shape[1], h = ic.shape[2], w = ic.shape[3];
  i64 cout = wc.shape[0], kh = wc.shape[2], kw = wc.shape[3];
  i64 oh = gc.shape[2], ow = gc.shape[3];
  gi = make(ic.shape); gw = make(wc.shape); gb = make({cout});
  const float* wt = cdata(wc); const float* go = cdata(gc);
  float* gid = gi.buf->data(); float* gwd = gw.buf->data(); float* gbd = gb.buf->data();
  parallel_tasks(cout, [&](i64 s, i64 e) {      // bias: n outer, pixels inner (1642-1651)
    for (i64 co = s; co < e; ++co) {
      float sum = 0.0f;
      for (i64 b = 0; b < n; ++b) { const float* p = go + (b * cout + co) * oh * ow; for (i64 i = 0; i < oh * ow; ++i) sum += p[i]; }
      gbd[co] = sum;
    }
  });
  i64 hp = h + 2 * pad, wp = w + 2 * pad;
  std::vector<float> xp = pad_input(cdata(ic), n, cin, h, w, pad);
  parallel_tasks(cout * cin, [&](i64 s, i64 e) {  // weight: n -> y -> x with fma (1687-1718)
    for (i64 task = s; task < e; ++task) {
      i64 co = task / cin, c = task % cin;
      for (i64 i = 0; i < kh; ++i)
        for (i64 j = 0; j < kw; ++j) {
          float acc = 0.0f;
          for (i64 nn = 0; nn < n; ++nn)
            for (i64 y = 0; y < oh; ++y) {
              const float* xr = &xp[((nn * cin + c) * hp + y * stride + i) * wp + j];
              const float* gr = go + ((nn * cout + co) * oh + y) * ow;
              for (i64 xo = 0; xo < ow; ++xo) acc = std::fmaf(gr[xo], xr[xo * stride], acc);
            }
          gwd[((co * cin + c) * kh + i) * kw + j] = acc;
        }
    }
  });
  std::vector<float> gip((size_t)(n * cin * hp * wp), 0.0f);
  parallel_tasks(n * cin, [&](i64 s, i64 e) {    // input: scatter in (co, i, j, y, x) order (1743-1776)
    for (i64 task = s; task < e; ++task) {
      i64 nn = task / cin, c = task % cin;
      for (i64 co = 0; co < cout; ++co)
        for (i64 i = 0; i < kh; ++i)
          for (i64 j = 0; j < kw; ++j) {
            float wv = wt[((co * cin + c) * kh + i) * kw + j];
            if (wv == 0.0f) continue;
            for (i64 y = 0; y < oh; ++y) {
              float* dr = &gip[((nn * cin + c) * hp + y * stride + i) * wp + j];
              const float* gr = go + ((nn * cout + co) * oh + y) * ow;
              for (i64 xo = 0; xo < ow; ++xo) dr[xo * stride] = std::fmaf(gr[xo], wv, dr[xo * stride]);
            }
          }
    }
  });
  for (i64 a = 0; a < n * cin; ++a)
    for (i64 ih = 0; ih < h; ++ih)
      std::memcpy(gid + (a * h + ih) * w, &gip[(a * hp + ih + pad) * wp + pad], sizeof(float) * (size_t)w);
}

// maxpool2d, lib.rs:1797-1865 (first maximum wins: strict >, padded taps never selected)
static Tensor raw_maxpool2d(const Tensor& input, i64 k, i64 s, i64 p) {
  Tensor ic = contiguous(input);
  i64 n = ic.shape[0], c = ic.shape[1], h = ic.shape[2], w = ic.shape[3];
  i64 oh = (h + 2 * p - k) / s + 1, ow = (w + 2 * p - k) / s + 1;
  Tensor out = make({n, c, oh, ow});
  if (!out.numel()) return out;
  const float* x = cdata(ic); float* od = out.buf->data();
  parallel_tasks(n * c, [&](i64 a, i64 b) {
    for (i64 nc = a; nc < b; ++nc)
      for (i64 y = 0; y < oh; ++y)
        for (i64 xo = 0; xo < ow; ++xo) {
          float best = -INFINITY;
          for (i64 i = 0; i < k; ++i) {
            i64 ih = y * s + i; if (ih < p || ih >= h + p) continue; ih -= p;
            for (i64 j = 0; j < k; ++j) {
              i64 iw = xo * s + j; if (iw < p || iw >= w + p) continue; iw -= p;
              float v = x[nc * h * w + ih * w + iw];
              if (v > best) best = v;
            }
          }
          od[nc * oh * ow + y * ow + xo] = best;
        }
  });
  return out;
}
// maxpool2d_backward, lib.rs:1870-1948
static Tensor raw_maxpool2d_backward(const Tensor& input, const Tensor& go_, i64 k, i64 s, i64 p) {
  Tensor ic = contiguous(input), gc = contiguous(go_);
  i64 n = ic.shape[0], c = ic.shape[1], h = ic.shape[2], w = ic.shape[3];
  i64 oh = gc.shape[2], ow = gc.shape[3];
  Tensor gi = make(ic.shape);
  const float* x = cdata(ic); const float* go = cdata(gc); float* g = gi.buf->data();
  parallel_tasks(n * c, [&](i64 a, i64 b) {
    for (i64 nc = a; nc < b; ++nc)
      for (i64 y = 0; y < oh; ++y)
        for (i64 xo = 0; xo < ow; ++xo) {
          float best = -INFINITY; i64 bi = -1;
          for (i64 i = 0; i < k; ++i) {
            i64 ih = y * s + i; if (ih < p || ih >= h + p) continue; ih -= p;
            for (i64 j = 0; j < k; ++j) {
              i64 iw = xo * s + j; if (iw < p || iw >= w + p) continue; iw -= p;
              float v = x[nc * h * w + ih * w + iw];
              if (v > best) { best = v; bi = ih * w + iw; }
            }
          }
          if (bi >= 0) g[nc * h * w + bi] += go[nc * oh * ow + y * ow + xo];
        }
  });
  return gi;
}
// avgpool2d / avgpool2d_backward, lib.rs:1952-2058 (mean over valid taps only)
static Tensor raw_avgpool2d(const Tensor& input, i64 k, i64 s, i64 p) {
  Tensor ic = contiguous(input);
  i64 n = ic.shape[0], c = ic.shape[1], h = ic.shape[2], w = ic.shape[3];
  i64 oh = (h + 2 * p - k) / s + 1, ow = (w + 2 * p - k) / s + 1;
  Tensor out = make({n, c, oh, ow});
  if (!out.numel()) return out;
  const float* x = cdata(ic); float* od = out.buf->data();
  for (i64 nc = 0; nc < n * c; ++nc)
    for (i64 y = 0; y < oh; ++y)
      for (i64 xo = 0; xo < ow; ++xo) {
        float sum = 0.0f; i64 cnt = 0;
        for (i64 i = 0; i < k; ++i) {
          i64 ih = y * s + i; if (ih < p || ih >= h + p) continue; ih -= p;
          for (i64 j = 0; j < k; ++j) {
            i64 iw = xo * s + j; if (iw < p || iw >= w + p) continue; iw -= p;
            sum += x[nc * h * w + ih * w + iw]; ++cnt;
          }
        }
        od[nc * oh * ow + y * ow + xo] = sum / (float)cnt;
      }
  return out;
}
static Tensor raw_avgpool2d_backward(const Tensor& input, const Tensor& go_, i64 k, i64 s, i64 p) {
  Tensor gc = contiguous(go_);
  i64 n = input.shape[0], c = input.shape[1], h = input.shape[2], w = input.shape[3];
  i64 oh = gc.shape[2], ow = gc.shape[3];
  Tensor gi = make(input.shape);
  const float* go = cdata(gc); float* g = gi.buf->data();
  for (i64 nc = 0; nc < n * c; ++nc)
    for (i64 y = 0; y < oh; ++y)
      for (i64 xo = 0; xo < ow; ++xo) {
        i64 cnt = 0;
        for (i64 i = 0; i < k; ++i) {
          i64 ih = y * s + i; if (ih < p || ih >= h + p) continue;
          for (i64 j = 0; j < k; ++j) { i64 iw = xo * s + j; if (iw >= p && iw < w + p) ++cnt; }
        }
        float gv = go[nc * oh * ow + y * ow + xo] / (float)cnt;
        for (i64 i = 0; i < k; ++i) {
          i64 ih = y * s + i; if (ih < p || ih >= h + p) continue; ih -= p;
          for (i64 j = 0; j < k; ++j) {
            i64 iw = xo * s + j; if (iw < p || iw >= w + p) continue; iw -= p;
            g[nc * h * w + ih * w + iw] += gv;
          }
        }
      }
  return gi;
}

// batchnorm, lib.rs:2067-2194.  Training mode writes the running statistics in place.
static Tensor raw_batchnorm(const Tensor& x, const Tensor& gamma, const Tensor& beta, const Tensor& rm, const Tensor& rv,
                            bool training, float momentum, float eps) {
  Tensor xc = contiguous(x);
  if (xc.rank() != 4) fail("BatchNorm2d input must be rank 4 (N, C, H, W)");
  i64 n = xc.shape[0], c = xc.shape[1], h = xc.shape[2], w = xc.shape[3];
  float m = (float)(n * h * w);
  if (gamma.rank() != 1 || beta.rank() != 1 || gamma.shape[0] != c || beta.shape[0] != c) fail("Gamma/Beta dim must match channels C");
  Tensor out = make(x.shape);
  if (!out.numel()) return out;
  const float* xd = cdata(xc); const float* gd = cdata(gamma); const float* bd = cdata(beta);
  float* od = out.buf->data();
  float* rmd = rm.buf->data(); float* rvd = rv.buf->data();
  i64 hw = h * w;
  for (i64 cc = 0; cc < c; ++cc) {
    float mean, var;
    if (training) {
      float sum = 0.0f;
      for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) sum += xd[(nn * c + cc) * hw + i];
      mean = sum / m;
      float sq = 0.0f;
      for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) { float d = xd[(nn * c + cc) * hw + i] - mean; sq += d * d; }
      var = sq / m;
      float bessel = m > 1.0f ? m / (m - 1.0f) : 1.0f;
      float nrm = (1.0f - momentum) * rmd[cc] + momentum * mean;
      float nrv = (1.0f - momentum) * rvd[cc] + momentum * var * bessel;
      rmd[cc] = nrm; rvd[cc] = nrv;
    } else { mean = rmd[cc]; var = rvd[cc]; }
    float inv = 1.0f / std::sqrt(var + eps);
    for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) {
      i64 idx = (nn * c + cc) * hw + i;
      float xh = (xd[idx] - mean) * inv;
      od[idx] = xh * gd[cc] + bd[cc];
    }
  }
  return out;
}
// batchnorm_backward, lib.rs:2204-2364
static void raw_batchnorm_backward(const Tensor& x, const Tensor& gamma, const Tensor& rm, const Tensor& rv, const Tensor& go_,
                                   bool training, float eps, Tensor& gx, Tensor& gw, Tensor& gb) {
  Tensor xc = contiguous(x), gc = contiguous(go_);
  i64 n = xc.shape[0], c = xc.shape[1], h = xc.shape[2], w = xc.shape[3];
  float m = (float)(n * h * w);
  gx = make(x.shape); gw = make(gamma.shape); gb = make(gamma.shape);
  if (!x.numel()) return;
  const float* xd = cdata(xc); const float* gd = cdata(gamma); const float* go = cdata(gc);
  float* gxd = gx.buf->data(); float* gwd = gw.buf->data(); float* gbd = gb.buf->data();
  i64 hw = h * w;
  for (i64 cc = 0; cc < c; ++cc) {
    float mean, var;
    if (training) {
      float sum = 0.0f;
      for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) sum += xd[(nn * c + cc) * hw + i];
      mean = sum / m;
      float sq = 0.0f;
      for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) { float d = xd[(nn * c + cc) * hw + i] - mean; sq += d * d; }
      var = sq / m;
    } else { mean = cdata(rm)[cc]; var = cdata(rv)[cc]; }
    float inv = 1.0f / std::sqrt(var + eps);
    float sdy = 0.0f, sdyx = 0.0f;
    for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) {
      i64 idx = (nn * c + cc) * hw + i;
      float dy = go[idx]; float xh = (xd[idx] - mean) * inv;
      sdy += dy; sdyx += dy * xh;
    }
    gbd[cc] = sdy; gwd[cc] = sdyx;
    for (i64 nn = 0; nn < n; ++nn) for (i64 i = 0; i < hw; ++i) {
      i64 idx = (nn * c + cc) * hw + i;
      float dy = go[idx];
      if (training) {
        float xh = (xd[idx] - mean) * inv;
        gxd[idx] = (gd[cc] * inv / m) * (m * dy - sdy - xh * sdyx);
      } else gxd[idx] = dy * gd[cc] * inv;
    }
  }
}

// Attention probabilities of one query row, shared by forward and backward
// (lib.rs:2416-2458 and 2529-2571): fused dot over d, scale, + mask (right-aligned to rank 4,
// size-1 dims broadcast), max, exp, then multiply by 1/(sum + 1e-9).
struct MaskView { const float* d = nullptr; i64 s[4] = {1, 1, 1, 1}; };
static MaskView mask_view(const Tensor* mask, Tensor& hold) {
  MaskView mv;
  if (!mask) return mv;
  hold = contiguous(*mask);
  mv.d = cdata(hold);
  int r = hold.rank();
  for (int i = 0; i < r && i < 4; ++i) mv.s[4 - r + i] = hold.shape[i];
  return mv;
}
static void attn_row(const float* q_row, const float* kd, i64 s, i64 dk, float scale, const MaskView& mv, i64 b, i64 h, i64 i,
                     std::vector<float>& scores) {
  float mx = -INFINITY;
  for (i64 j = 0; j < s; ++j) {
    const float* kr = kd + j * dk;
    float dot = 0.0f;
    for (i64 d = 0; d < dk; ++d) dot = std::fmaf(q_row[d], kr[d], dot);
    dot *= scale;
    if (mv.d) {
      i64 mb = mv.s[0] == 1 ? 0 : b, mh = mv.s[1] == 1 ? 0 : h, ms = mv.s[2] == 1 ? 0 : i, mc = mv.s[3] == 1 ? 0 : j;
      dot += mv.d[mb * (mv.s[1] * mv.s[2] * mv.s[3]) + mh * (mv.s[2] * mv.s[3]) + ms * mv.s[3] + mc];
    }
    scores[j] = dot;
    if (dot > mx) mx = dot;
  }
  float se = 0.0f;
  for (i64 j = 0; j < s; ++j) { scores[j] = std::exp(scores[j] - mx); se += scores[j]; }
  float inv = 1.0f / (se + 1e-9f);
  for (i64 j = 0; j < s; ++j) scores[j] *= inv;
}
// fused_attention, lib.rs:2368-2476
static Tensor raw_fused_attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* mask) {
  if (q.rank() != 4 || k.shape != q.shape || v.shape != q.shape) fail("fused_attention expects q,k,v of equal shape [B,H,S,dk]");
  i64 B = q.shape[0], H = q.shape[1], S = q.shape[2], dk = q.shape[3];
  Tensor qc = contiguous(q), kc = contiguous(k), vc = contiguous(v), mh;
  MaskView mv = mask_view(mask, mh);
  float scale = 1.0f / std::sqrt((float)dk);
  Tensor out = make(q.shape);
  float* od = out.buf->data();
  std::vector<float> sc((size_t)S);
  for (i64 b = 0; b < B; ++b) for (i64 h = 0; h < H; ++h) {
    i64 off = (b * H + h) * S * dk;
    for (i64 i = 0; i < S; ++i) {
      attn_row(cdata(qc) + off + i * dk, cdata(kc) + off, S, dk, scale, mv, b, h, i, sc);
      for (i64 d = 0; d < dk; ++d) {
        float sum = 0.0f;
        for (i64 j = 0; j < S; ++j) sum = std::fmaf(sc[j], cdata(vc)[off + j * dk + d], sum);
        od[off + i * dk + d] = sum;
      }
    }
  }
  return out;
}
// fused_attention_backward, lib.rs:2480-2630
static void raw_fused_attention_backward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* mask, const Tensor& go_,
                                         Tensor& dq, Tensor& dk_, Tensor& dv) {
  i64 B = q.shape[0], H = q.shape[1], S = q.shape[2], dk = q.shape[3];
  Tensor qc = contiguous(q), kc = contiguous(k), vc = contiguous(v), gc = contiguous(go_), mh;
  MaskView mv = mask_view(mask, mh);
  float scale = 1.0f / std::sqrt((float)dk);
  dq = make(q.shape); dk_ = make(q.shape); dv = make(q.shape);
  float* dqd = dq.buf->data(); float* dkd = dk_.buf->data(); float* dvd = dv.buf->data();
  std::vector<float> sc((size_t)S), dp((size_t)S), ds((size_t)S);
  for (i64 b = 0; b < B; ++b) for (i64 h = 0; h < H; ++h) {
    i64 off = (b * H + h) * S * dk;
    const float* kd = cdata(kc) + off; const float* vd = cdata(vc) + off;
    for (i64 i = 0; i < S; ++i) {
      const float* qr = cdata(qc) + off + i * dk; const float* gr = cdata(gc) + off + i * dk;
      attn_row(qr, kd, S, dk, scale, mv, b, h, i, sc);
      for (i64 j = 0; j < S; ++j) { float s = 0.0f; for (i64 d = 0; d < dk; ++d) s = std::fmaf(gr[d], vd[j * dk + d], s); dp[j] = s; }
      float sdp = 0.0f; for (i64 j = 0; j < S; ++j) sdp = std::fmaf(dp[j], sc[j], sdp);
      for (i64 j = 0; j < S; ++j) ds[j] = sc[j] * (dp[j] - sdp);
      for (i64 d = 0; d < dk; ++d) { float s = 0.0f; for (i64 j = 0; j < S; ++j) s = std::fmaf(ds[j], kd[j * dk + d], s); dqd[off + i * dk + d] = s * scale; }
      for (i64 j = 0; j < S; ++j) { float p = sc[j]; float* o = dvd + off + j * dk; for (i64 d = 0; d < dk; ++d) o[d] = std::fmaf(p, gr[d], o[d]); }
      for (i64 j = 0; j < S; ++j) { float dsj = ds[j] * scale; float* o = dkd + off + j * dk; for (i64 d = 0; d < dk; ++d) o[d] = std::fmaf(dsj, qr[d], o[d]); }
    }
  }
}

// ---------------------------------------------------------------------------------
// Recorded ops (dispatch methods of vearo-core/src/tensor.rs) and views.
// ---------------------------------------------------------------------------------
static Tensor op_binary(Op op, const Tensor& a, const Tensor& b) {
  Tensor o = op == ADD ? raw_add(a, b) : op == SUB ? raw_sub(a, b) : op == MUL ? raw_mul(a, b) : raw_div(a, b);
  record(op, {&a, &b}, o);
  return o;
}
static Tensor op_matmul(const Tensor& a, const Tensor& b) { Tensor o = raw_matmul(a, b); record(MATMUL, {&a, &b}, o); return o; }
static Tensor op_relu(const Tensor& a) { Tensor o = raw_relu(a); record(RELU, {&a}, o); return o; }
static Tensor op_gelu(const Tensor& a) { Tensor o = raw_gelu(a); record(GELU, {&a}, o); return o; }
static Tensor op_softmax(const Tensor& a, int dim) { Tensor o = raw_softmax(a, dim); if (Node* n = record(SOFTMAX, {&a}, o)) n->a0 = dim; return o; }
static Tensor op_sum(const Tensor& a, int dim, bool keep, bool mean) {
  Tensor o = raw_sum(a, dim, keep, mean);
  if (Node* n = record(mean ? MEAN : SUM, {&a}, o)) { n->a0 = dim; n->a1 = keep; }
  return o;
}
static Tensor op_layernorm(const Tensor& x, const Tensor& w, const Tensor& b, float eps) {
  Tensor o = raw_layernorm(x, w, b, eps);
  if (Node* n = record(LAYERNORM, {&x, &w, &b}, o)) n->f0 = eps;
  return o;
}
static Tensor op_embedding(const Tensor& idx, const Tensor& w) { Tensor o = raw_embedding(idx, w); record(EMBEDDING, {&idx, &w}, o); return o; }
static Tensor op_cross_entropy(const Tensor& l, const Tensor& t) { Tensor o = raw_cross_entropy(l, t); record(CROSS_ENTROPY, {&l, &t}, o); return o; }
static Tensor op_conv2d(const Tensor& x, const Tensor& w, const Tensor& b, i64 s, i64 p) {
  Tensor o = raw_conv2d(x, w, b, s, p);
  if (Node* n = record(CONV2D, {&x, &w, &b}, o)) { n->a0 = s; n->a1 = p; }
  return o;
}
static Tensor op_maxpool2d(const Tensor& x, i64 k, i64 s, i64 p) { Tensor o = raw_maxpool2d(x, k, s, p); if (Node* n = record(MAXPOOL2D, {&x}, o)) { n->a0 = k; n->a1 = s; n->a2 = p; } return o; }
static Tensor op_avgpool2d(const Tensor& x, i64 k, i64 s, i64 p) { Tensor o = raw_avgpool2d(x, k, s, p); if (Node* n = record(AVGPOOL2D, {&x}, o)) { n->a0 = k; n->a1 = s; n->a2 = p; } return o; }
static Tensor op_batchnorm(const Tensor& x, const Tensor& g, const Tensor& b, const Tensor& rm, const Tensor& rv, bool training, float mom, float eps) {
  Tensor o = raw_batchnorm(x, g, b, rm, rv, training, mom, eps);
  if (Node* n = record(BATCHNORM, {&x, &g, &b, &rm, &rv}, o)) { n->a0 = training; n->f0 = eps; }
  return o;
}
static Tensor op_fused_attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* mask) {
  Tensor o = raw_fused_attention(q, k, v, mask);
  std::vector<const Tensor*> ins = {&q, &k, &v};
  if (mask) ins.push_back(mask);
  record(FUSED_ATTENTION, ins, o);
  return o;
}
// reshape / transpose / permute, vearo-core/src/tensor.rs:493-642
static Tensor op_reshape(const Tensor& a, const std::vector<i64>& shape) {
  i64 n = 1; for (i64 d : shape) n *= d;
  if (n != a.numel()) fail("Reshape numel must match");
  Tensor c = contiguous(a);
  Tensor o; o.buf = c.buf; o.shape = shape; o.strides = contiguous_strides(shape);
  o.node = c.node; o.requires_grad = c.requires_grad;
  if (g_autograd && a.requires_grad) { o.requires_grad = true; tape_push(RESHAPE, {&a}, o); }
  return o;
}
static Tensor op_transpose(const Tensor& a, int d0, int d1) {
  Tensor o = a; o.node = a.node;
  std::swap(o.shape[d0], o.shape[d1]); std::swap(o.strides[d0], o.strides[d1]);
  if (g_autograd && a.requires_grad) { o.requires_grad = true; Node& n = tape_push(TRANSPOSE, {&a}, o); n.a0 = d0; n.a1 = d1; }
  return o;
}
static Tensor op_permute(const Tensor& a, const std::vector<i64>& axes) {
  Tensor o = a;
  for (size_t i = 0; i < axes.size(); ++i) { o.shape[i] = a.shape[axes[i]]; o.strides[i] = a.strides[axes[i]]; }
  if (g_autograd && a.requires_grad) { o.requires_grad = true; Node& n = tape_push(PERMUTE, {&a}, o); n.axes = axes; }
  return o;
}

// reduce_to, vearo-autograd/src/lib.rs:316-361
static Tensor reduce_to(const Tensor& grad, const std::vector<i64>& target) {
  if (grad.shape == target) return grad;
  Tensor out = make(target);
  if (!grad.numel()) return out;
  Tensor gc = contiguous(grad);
  const float* gd = cdata(gc); float* od = out.buf->data();
  int gr = grad.rank(), tr = (int)target.size();
  if (gr < tr) fail("Grad rank must be >= target rank");
  NdIter it(grad.shape);
  i64 i = 0;
  do {
    i64 idx = 0, stride = 1;
    for (int d = tr - 1; d >= 0; --d) {
      i64 c = it.coord[gr - tr + d];
      idx += (target[d] == 1 ? 0 : c) * stride;
      stride *= target[d];
    }
    od[idx] += gd[i++];
  } while (it.step());
  return out;
}
// expand_reduce_grad, vearo-autograd/src/lib.rs:410-425
static Tensor expand_reduce_grad(const Tensor& go, const std::vector<i64>& in_shape, int dim, bool keep) {
  Tensor gk = go;
  if (!keep) { std::vector<i64> d = go.shape; d.insert(d.begin() + dim, 1); gk = op_reshape(go, d); }
  return raw_add(make(in_shape), gk);
}

// backward_impl, vearo-autograd/src/lib.rs:429-792.  Autograd is off while it runs, so the
// recorded-op helpers used inside the arms record nothing.
static void backward(const Tensor& output) {
  if (output.numel() != 1) fail("backward can only be called on scalar tensors");
  g_autograd = false;
  struct Restore { ~Restore() { g_autograd = true; } } restore;
  if (output.node < 0 || (uint32_t)(output.node >> 32) != g_tape.generation) return;
  int out_idx = (int)(output.node & 0xffffffff);
  std::vector<Node> nodes = g_tape.nodes;
  std::unordered_map<int, Tensor> gm;
  { float one = 1.0f; gm[out_idx] = from_data(&one, output.shape); }
  for (int ni = (int)nodes.size() - 1; ni >= 0; --ni) {
    Node& node = nodes[ni];
    auto it = gm.find(node.id);
    if (it == gm.end()) continue;
    if (node.saved.empty()) continue;
    Tensor go = it->second;
    std::vector<Tensor> gin;
    const std::vector<Tensor>& sv = node.saved;
    switch (node.op) {
      case ADD: gin = {reduce_to(go, sv[0].shape), reduce_to(go, sv[1].shape)}; break;
      case SUB: { Tensor gr = raw_mul(go, scalar1(-1.0f)); gin = {reduce_to(go, sv[0].shape), reduce_to(gr, sv[1].shape)}; break; }
      case MUL: { Tensor gl = raw_mul(go, sv[1]), gr = raw_mul(go, sv[0]); gin = {reduce_to(gl, sv[0].shape), reduce_to(gr, sv[1].shape)}; break; }
      case DIV: {
        Tensor gl = raw_div(go, sv[1]);
        Tensor gr = raw_div(raw_mul(raw_mul(go, scalar1(-1.0f)), sv[0]), raw_mul(sv[1], sv[1]));
        gin = {reduce_to(gl, sv[0].shape), reduce_to(gr, sv[1].shape)}; break;
      }
      case MATMUL: {
        Tensor lt = op_transpose(sv[0], sv[0].rank() - 2, sv[0].rank() - 1);
        Tensor rt = op_transpose(sv[1], sv[1].rank() - 2, sv[1].rank() - 1);
        Tensor gl = raw_matmul(go, rt), gr = raw_matmul(lt, go);
        gin = {reduce_to(gl, sv[0].shape), reduce_to(gr, sv[1].shape)}; break;
      }
      case RESHAPE: gin = {op_reshape(go, sv[0].shape)}; break;
      case TRANSPOSE: gin = {op_transpose(go, (int)node.a0, (int)node.a1)}; break;
      case PERMUTE: { std::vector<i64> inv(node.axes.size()); for (size_t i = 0; i < node.axes.size(); ++i) inv[node.axes[i]] = (i64)i; gin = {op_permute(go, inv)}; break; }
      case RELU: gin = {raw_mul(go, relu_grad_mask(sv[0]))}; break;
      case GELU: gin = {raw_mul(go, gelu_grad_mask(sv[0]))}; break;
      case SOFTMAX: {
        Tensor y = raw_softmax(sv[0], (int)node.a0);
        Tensor sgy = raw_sum(raw_mul(go, y), (int)node.a0, true, false);
        gin = {raw_mul(y, raw_sub(go, sgy))}; break;
      }
      case LAYERNORM: { Tensor gx, gw, gb; raw_layernorm_backward(sv[0], sv[1], sv[2], go, node.f0, gx, gw, gb); gin = {gx, gw, gb}; break; }
      case BATCHNORM: {
        Tensor gx, gw, gb; raw_batchnorm_backward(sv[0], sv[1], sv[3], sv[4], go, node.a0 != 0, node.f0, gx, gw, gb);
        gin = {gx, gw, gb, make(sv[3].shape), make(sv[4].shape)}; break;
      }
      case EMBEDDING: gin = {make(sv[0].shape), raw_embedding_backward(sv[0], sv[1], go)}; break;
      case CROSS_ENTROPY: gin = {raw_cross_entropy_backward(sv[0], sv[1], go), make(sv[1].shape)}; break;
      case FUSED_ATTENTION: {
        Tensor dq, dk, dv; const Tensor* mask = sv.size() > 3 ? &sv[3] : nullptr;
        raw_fused_attention_backward(sv[0], sv[1], sv[2], mask, go, dq, dk, dv);
        gin = {dq, dk, dv}; if (mask) gin.push_back(make(mask->shape)); break;
      }
      case CONV2D: { Tensor gi, gw, gb; raw_conv2d_backward(sv[0], sv[1], go, node.a0, node.a1, gi, gw, gb); gin = {gi, gw, gb}; break; }
      case MAXPOOL2D: gin = {raw_maxpool2d_backward(sv[0], go, node.a0, node.a1, node.a2)}; break;
      case AVGPOOL2D: gin = {raw_avgpool2d_backward(sv[0], go, node.a0, node.a1, node.a2)}; break;
      case SUM: gin = {expand_reduce_grad(go, sv[0].shape, (int)node.a0, node.a1 != 0)}; break;
      case MEAN: {
        Tensor e = expand_reduce_grad(go, sv[0].shape, (int)node.a0, node.a1 != 0);
        float count = (float)sv[0].shape[node.a0];
        gin = {raw_mul(e, scalar1(1.0f / count))}; break;
      }
      case LEAF: break;
    }
    for (size_t i = 0; i < node.inputs.size(); ++i) {
      int id = node.inputs[i];
      if (id < 0) continue;
      auto e = gm.find(id);
      if (e != gm.end()) e->second = raw_add(e->second, gin[i]);   // existing + new (736-737)
      else gm[id] = gin[i];
    }
  }
  // Publish gradients of leaves only (745-772).
  g_grads.clear();
  for (Node& node : nodes)
    for (size_t i = 0; i < node.saved.size(); ++i) {
      const Tensor& in = node.saved[i];
      if (in.node < 0 || (uint32_t)(in.node >> 32) != g_tape.generation) continue;
      int idx = (int)(in.node & 0xffffffff);
      if (!nodes[idx].inputs.empty() || nodes[idx].op != LEAF) continue;
      int id = node.inputs[i];
      if (id < 0) continue;
      auto e = gm.find(id);
      if (e != gm.end()) g_grads[in.buf.get()] = e->second;
    }
  g_tape.nodes.clear();
  g_tape.generation++;
}

// ---------------------------------------------------------------------------------
// Optimizers: vearo-optim/src/lib.rs, vearo-core/src/tensor.rs:931-1096.
// ---------------------------------------------------------------------------------
static float powi(float a, int n) {  // f32::powi -> repeated squaring (compiler-rt __powisf2)
  bool recip = n < 0; float r = 1.0f;
  while (true) { if (n & 1) r *= a; n /= 2; if (n == 0) break; a *= a; }
  return recip ? 1.0f / r : r;
}
// QuantizedState, vearo-optim/src/lib.rs:137-209: int8 values with one f32 scale (block maximum / 127) per 256 elements.
struct Quantized {
  std::vector<int8_t> data; std::vector<float> scales; size_t block = 256;
  explicit Quantized(size_t n = 0) : data(n, 0), scales((n + 255) / 256, 0.0f) {}
  void quantize(const std::vector<float>& src) {           // lib.rs:157-194
    const size_t n = src.size();
    for (size_t b = 0; b < scales.size(); ++b) {
      size_t start = b * block, end = std::min(start + block, n);
      if (start >= end) continue;
      float mx = 0.0f;
      for (size_t i = start; i < end; ++i) { float a = std::fabs(src[i]); if (a > mx) mx = a; }
      scales[b] = mx / 127.0f;
      if (mx > 0.0f) {
        float inv = 127.0f / mx;
        for (size_t i = start; i < end; ++i) {
          float q = std::round(src[i] * inv);                // f32::round: half away from zero
          q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
          data[i] = (int8_t)q;
        }
      } else {
        for (size_t i = start; i < end; ++i) data[i] = 0;
      }
    }
  }
  void dequantize(std::vector<float>& dst) const {           // lib.rs:197-208
    const size_t n = dst.size();
    for (size_t b = 0; b < scales.size(); ++b) {
      size_t start = b * block, end = std::min(start + block, n);
      for (size_t i = start; i < end; ++i) dst[i] = (float)data[i] * scales[b];
    }
  }
};
struct Optimizer {
  bool adam; std::vector<Tensor> params; float lr, b1, b2, eps, wd, momentum;
  std::vector<std::vector<float>> m, v; uint32_t t = 0;
  bool eight_bit = false; std::vector<Quantized> qm, qv;    // AdamW8bit, lib.rs:211-303
};
static void opt_step(Optimizer& o) {
  if (o.adam) o.t += 1;   // AdamW::step, vearo-optim/src/lib.rs:105-123
  for (size_t pi = 0; pi < o.params.size(); ++pi) {
    Tensor& p = o.params[pi];
    auto gi = g_grads.find(p.buf.get());
    if (gi == g_grads.end()) continue;
    Tensor g = contiguous(gi->second);
    if (g.shape != p.shape) fail("optimizer step shapes must match");
    if (!p.is_contiguous()) fail("optimizer step self must be contiguous");
    const float* gd = cdata(g); float* w = p.buf->data();
    i64 n = p.numel();
    if (o.adam) {   // adamw_step, tensor.rs:972-985
      float bc1 = 1.0f - powi(o.b1, (int)o.t), bc2 = 1.0f - powi(o.b2, (int)o.t);
      if (o.eight_bit) { o.qm[pi].dequantize(o.m[pi]); o.qv[pi].dequantize(o.v[pi]); }    // AdamW8bit::step, lib.rs:268-275
      float* m = o.m[pi].data(); float* v = o.v[pi].data();
      for (i64 i = 0; i < n; ++i) {
        float gv = gd[i];
        m[i] = o.b1 * m[i] + (1.0f - o.b1) * gv;
        v[i] = o.b2 * v[i] + (1.0f - o.b2) * gv * gv;
        float mh = m[i] / bc1, vh = v[i] / bc2;
        w[i] -= o.lr * o.wd * w[i];
        w[i] -= o.lr * mh / (std::sqrt(vh) + o.eps);
      }
      if (o.eight_bit) { o.qm[pi].quantize(o.m[pi]); o.qv[pi].quantize(o.v[pi]); }        // lib.rs:290-292
    } else {        // sgd_step, tensor.rs:1062-1069
      float* vel = o.m[pi].data();
      for (i64 i = 0; i < n; ++i) {
        float gv = gd[i];
        if (o.wd != 0.0f) gv += o.wd * w[i];
        vel[i] = o.momentum * vel[i] + gv;
        w[i] -= o.lr * vel[i];
      }
    }
  }
}
// clip_grad_norm, vearo-optim/src/lib.rs:360-383.  The reference asserts that every gradient is
// contiguous (365) and would therefore panic on the transposed-view gradient every Linear weight
// gets (vearo-autograd/src/lib.rs:525-528); here such a gradient is first made contiguous, as the
// optimizers do before their step (vearo-optim/src/lib.rs:36,109), and the sum runs over its
// logical row-major order.
static float clip_grad_norm(const std::vector<Tensor>& params, float max_norm) {
  std::vector<Tensor*> grads;
  for (const Tensor& p : params) {
    auto it = g_grads.find(p.buf.get());
    if (it == g_grads.end()) continue;
    if (!it->second.is_contiguous()) it->second = contiguous(it->second);
    grads.push_back(&it->second);
  }
  float total = 0.0f;
  for (Tensor* g : grads) {
    const float* d = cdata(*g);
    for (i64 i = 0, n = g->numel(); i < n; ++i) total = std::fmaf(d[i], d[i], total);
  }
  float norm = std::sqrt(total);
  if (norm > max_norm) {
    float scale = max_norm / (norm + 1e-6f);
    for (Tensor* g : grads) { float* d = g->buf->data(); for (i64 i = 0, n = g->numel(); i < n; ++i) d[i] = d[i] * scale; }
  }
  return norm;
}
// CosineSchedule::lr_at, vearo-optim/src/lib.rs:336-348
static float cosine_lr(float base, float min_lr, uint32_t warmup, uint32_t total, uint32_t step) {
  if (step < warmup) return base * ((float)step + 1.0f) / ((float)warmup + 1.0f);
  if (step > total) return min_lr;
  uint32_t denom = total > warmup ? total - warmup : 0; if (denom < 1) denom = 1;
  float progress = (float)(step - warmup) / (float)denom;
  float coeff = 0.5f * (1.0f + std::cos(3.14159265358979323846f * progress));
  return min_lr + coeff * (base - min_lr);
}

// Handle tables for the C interface.
static std::vector<std::unique_ptr<Tensor>> g_tensors;
static std::vector<std::unique_ptr<Optimizer>> g_opts;
static int put(const Tensor& t) { g_tensors.emplace_back(new Tensor(t)); return (int)g_tensors.size() - 1; }
static Tensor& at(int h) {
  if (h < 0 || h >= (int)g_tensors.size() || !g_tensors[h]) fail("bad tensor handle");
  return *g_tensors[h];
}
}  // namespace orc

// ---------------------------------------------------------------------------------
// C interface (ctypes).  Functions returning a handle return -1 on error; the message is
// available from orc_last_error(), mirroring the panic text of the reference.
// ---------------------------------------------------------------------------------
using namespace orc;
#define ORC_TRY(...) try { __VA_ARGS__; } catch (const std::exception& e) { g_err = e.what(); return -1; }

extern "C" {
const char* orc_last_error() { return g_err.c_str(); }
void orc_set_threads(int n) { g_threads = n; }
int orc_get_threads() { return n_threads(); }
void orc_set_training(int t) { g_training = t != 0; }
// Dropout::forward (vearo-nn/src/lib.rs:333-357) with SimpleRng (lib.rs:14-50) and the per-call counter (vearo-core/src/tensor.rs:1240-1285)
static uint64_t g_rng_counter = 0;
uint64_t orc_rng_counter() { return g_rng_counter; }
void orc_set_rng_counter(uint64_t v) { g_rng_counter = v; }
int orc_dropout(int x, float p, uint64_t seed) {
  ORC_TRY(Tensor& in = at(x);          // by reference: the tape token lives in the tensor
          if (p <= 0.0f || !g_training) return put(in);
          float scale = 1.0f / (1.0f - p);
          uint64_t call = g_rng_counter++;
          uint64_t st = seed ^ (call * 0x9E3779B97F4A7C15ull);
          if (st == 0) st = 0x123456789ABCDEF0ull;
          std::vector<float> mask((size_t)in.numel());
          for (float& m : mask) {
            st ^= st << 13; st ^= st >> 7; st ^= st << 17;
            float u = (float)st / (float)UINT64_MAX;
            m = u >= p ? scale : 0.0f;
          }
          Tensor mt = from_data(mask.data(), in.shape);
          return put(op_binary((Op)2, in, mt)));   // input.mul(&mask_t), recorded on the tape like any product
}
void orc_set_autograd(int e) { g_autograd = e != 0; }
void orc_reset_all() { g_tensors.clear(); g_opts.clear(); g_grads.clear(); g_tape.nodes.clear(); g_tape.generation++; g_autograd = true; g_training = true; g_rng_counter = 0; }
void orc_reset_tape() { g_tape.nodes.clear(); g_tape.generation++; }   // reset_active_tape, autograd lib.rs:831
void orc_zero_gradients() { g_grads.clear(); }                          // zero_gradients, autograd lib.rs:836
void orc_free(int h) { if (h >= 0 && h < (int)g_tensors.size()) g_tensors[h].reset(); }

int orc_tensor(const float* data, const int64_t* shape, int rank, int requires_grad) {
  ORC_TRY(Tensor t = from_data(data, std::vector<i64>(shape, shape + rank)); t.requires_grad = requires_grad != 0; return put(t));
}
int orc_rank(int h) { ORC_TRY(return at(h).rank()); }
int orc_shape(int h, int64_t* out) { ORC_TRY(Tensor& t = at(h); for (int i = 0; i < t.rank(); ++i) out[i] = t.shape[i]; return t.rank()); }
int64_t orc_numel(int h) { ORC_TRY(return at(h).numel()); }
int orc_is_contiguous(int h) { ORC_TRY(return at(h).is_contiguous() ? 1 : 0); }
int orc_read(int h, float* out) { ORC_TRY(Tensor c = contiguous(at(h)); if (c.numel()) std::memcpy(out, cdata(c), sizeof(float) * (size_t)c.numel()); return 0); }
int orc_write(int h, const float* in) { ORC_TRY(Tensor& t = at(h); if (!t.is_contiguous()) fail("write needs a contiguous tensor"); std::memcpy(t.buf->data(), in, sizeof(float) * (size_t)t.numel()); return 0); }
int orc_set_requires_grad(int h, int f) { ORC_TRY(at(h).requires_grad = f != 0; return 0); }

int orc_binary(int op, int a, int b) { ORC_TRY(return put(op_binary((Op)op, at(a), at(b)))); }   // 0 add 1 sub 2 mul 3 div
int orc_matmul(int a, int b) { ORC_TRY(return put(op_matmul(at(a), at(b)))); }
int orc_relu(int a) { ORC_TRY(return put(op_relu(at(a)))); }
int orc_gelu(int a) { ORC_TRY(return put(op_gelu(at(a)))); }
int orc_softmax(int a, int dim) { ORC_TRY(return put(op_softmax(at(a), dim))); }
int orc_sum(int a, int dim, int keep) { ORC_TRY(return put(op_sum(at(a), dim, keep != 0, false))); }
int orc_mean(int a, int dim, int keep) { ORC_TRY(return put(op_sum(at(a), dim, keep != 0, true))); }
int orc_layernorm(int x, int w, int b, float eps) { ORC_TRY(return put(op_layernorm(at(x), at(w), at(b), eps))); }
int orc_embedding(int idx, int w) { ORC_TRY(return put(op_embedding(at(idx), at(w)))); }
int orc_cross_entropy(int l, int t) { ORC_TRY(return put(op_cross_entropy(at(l), at(t)))); }
int orc_conv2d(int x, int w, int b, int stride, int pad) { ORC_TRY(return put(op_conv2d(at(x), at(w), at(b), stride, pad))); }
int orc_maxpool2d(int x, int k, int s, int p) { ORC_TRY(return put(op_maxpool2d(at(x), k, s, p))); }
int orc_avgpool2d(int x, int k, int s, int p) { ORC_TRY(return put(op_avgpool2d(at(x), k, s, p))); }
int orc_batchnorm(int x, int g, int b, int rm, int rv, int training, float mom, float eps) {
  ORC_TRY(return put(op_batchnorm(at(x), at(g), at(b), at(rm), at(rv), training != 0, mom, eps)));
}
int orc_fused_attention(int q, int k, int v, int mask) { ORC_TRY(return put(op_fused_attention(at(q), at(k), at(v), mask >= 0 ? &at(mask) : nullptr))); }
int orc_reshape(int a, const int64_t* shape, int rank) { ORC_TRY(return put(op_reshape(at(a), std::vector<i64>(shape, shape + rank)))); }
int orc_transpose(int a, int d0, int d1) { ORC_TRY(return put(op_transpose(at(a), d0, d1))); }
int orc_permute(int a, const int64_t* axes, int rank) { ORC_TRY(return put(op_permute(at(a), std::vector<i64>(axes, axes + rank)))); }
int orc_contiguous(int a) { ORC_TRY(return put(contiguous(at(a)))); }

// The explicit *_backward fields of BackendOps (vearo-core/src/tensor.rs:1135-1174); out = handles.
int orc_layernorm_backward(int x, int w, int b, int go, float eps, int* out) {
  ORC_TRY(Tensor gx, gw, gb; raw_layernorm_backward(at(x), at(w), at(b), at(go), eps, gx, gw, gb); out[0] = put(gx); out[1] = put(gw); out[2] = put(gb); return 0);
}
int orc_embedding_backward(int idx, int w, int go) { ORC_TRY(return put(raw_embedding_backward(at(idx), at(w), at(go)))); }
int orc_cross_entropy_backward(int l, int t, int go) { ORC_TRY(return put(raw_cross_entropy_backward(at(l), at(t), at(go)))); }
int orc_conv2d_backward(int x, int w, int go, int stride, int pad, int* out) {
  ORC_TRY(Tensor gi, gw, gb; raw_conv2d_backward(at(x), at(w), at(go), stride, pad, gi, gw, gb); out[0] = put(gi); out[1] = put(gw); out[2] = put(gb); return 0);
}
int orc_maxpool2d_backward(int x, int go, int k, int s, int p) { ORC_TRY(return put(raw_maxpool2d_backward(at(x), at(go), k, s, p))); }
int orc_avgpool2d_backward(int x, int go, int k, int s, int p) { ORC_TRY(return put(raw_avgpool2d_backward(at(x), at(go), k, s, p))); }
int orc_batchnorm_backward(int x, int g, int rm, int rv, int go, int training, float eps, int* out) {
  ORC_TRY(Tensor gx, gw, gb; raw_batchnorm_backward(at(x), at(g), at(rm), at(rv), at(go), training != 0, eps, gx, gw, gb); out[0] = put(gx); out[1] = put(gw); out[2] = put(gb); return 0);
}
int orc_fused_attention_backward(int q, int k, int v, int mask, int go, int* out) {
  ORC_TRY(Tensor dq, dk, dv; raw_fused_attention_backward(at(q), at(k), at(v), mask >= 0 ? &at(mask) : nullptr, at(go), dq, dk, dv); out[0] = put(dq); out[1] = put(dk); out[2] = put(dv); return 0);
}
int orc_reduce_to(int g, const int64_t* shape, int rank) { ORC_TRY(return put(reduce_to(at(g), std::vector<i64>(shape, shape + rank)))); }

int orc_backward(int h) { ORC_TRY(backward(at(h)); return 0); }
int orc_grad(int h) { ORC_TRY(auto it = g_grads.find(at(h).buf.get()); if (it == g_grads.end()) return -2; return put(it->second)); }

int orc_adamw_create(const int* params, int n, float lr, float b1, float b2, float eps, float wd) {
  ORC_TRY(auto o = std::make_unique<Optimizer>(); o->adam = true; o->lr = lr; o->b1 = b1; o->b2 = b2; o->eps = eps; o->wd = wd; o->momentum = 0;
          for (int i = 0; i < n; ++i) { o->params.push_back(at(params[i])); o->m.emplace_back((size_t)at(params[i]).numel(), 0.0f); o->v.emplace_back((size_t)at(params[i]).numel(), 0.0f); }
          g_opts.push_back(std::move(o)); return (int)g_opts.size() - 1);
}
int orc_adamw8bit_create(const int* params, int n, float lr, float b1, float b2, float eps, float wd) {
  ORC_TRY(auto o = std::make_unique<Optimizer>(); o->adam = true; o->eight_bit = true; o->lr = lr; o->b1 = b1; o->b2 = b2; o->eps = eps; o->wd = wd; o->momentum = 0;
          for (int i = 0; i < n; ++i) {
            size_t cnt = (size_t)at(params[i]).numel();
            o->params.push_back(at(params[i])); o->m.emplace_back(cnt, 0.0f); o->v.emplace_back(cnt, 0.0f);
            o->qm.emplace_back(cnt); o->qv.emplace_back(cnt);
          }
          g_opts.push_back(std::move(o)); return (int)g_opts.size() - 1);
}
// Quantized state of parameter `param` of an 8-bit optimizer: int8 values (numel) and block scales ((numel + 255) / 256), m then v.
int orc_opt_state8(int o, int param, int8_t* m8, float* ms, int8_t* v8, float* vs) {
  ORC_TRY(if (o < 0 || o >= (int)g_opts.size() || !g_opts[o]->eight_bit) fail("not an 8-bit optimizer");
          Optimizer& op = *g_opts[o];
          if (param < 0 || param >= (int)op.qm.size()) fail("bad parameter index");
          std::copy(op.qm[param].data.begin(), op.qm[param].data.end(), m8); std::copy(op.qm[param].scales.begin(), op.qm[param].scales.end(), ms);
          std::copy(op.qv[param].data.begin(), op.qv[param].data.end(), v8); std::copy(op.qv[param].scales.begin(), op.qv[param].scales.end(), vs);
          return 0);
}
int orc_sgd_create(const int* params, int n, float lr, float momentum, float wd) {
  ORC_TRY(auto o = std::make_unique<Optimizer>(); o->adam = false; o->lr = lr; o->momentum = momentum; o->wd = wd; o->b1 = o->b2 = o->eps = 0;
          for (int i = 0; i < n; ++i) { o->params.push_back(at(params[i])); o->m.emplace_back((size_t)at(params[i]).numel(), 0.0f); }
          g_opts.push_back(std::move(o)); return (int)g_opts.size() - 1);
}
int orc_opt_step(int o) { ORC_TRY(if (o < 0 || o >= (int)g_opts.size()) fail("bad optimizer handle"); opt_step(*g_opts[o]); return 0); }
int orc_opt_set_lr(int o, float lr) { ORC_TRY(if (o < 0 || o >= (int)g_opts.size()) fail("bad optimizer handle"); g_opts[o]->lr = lr; return 0); }
float orc_clip_grad_norm(const int* params, int n, float max_norm) {
  try { std::vector<Tensor> ps; for (int i = 0; i < n; ++i) ps.push_back(at(params[i])); return clip_grad_norm(ps, max_norm); }
  catch (const std::exception& e) { g_err = e.what(); return -1.0f; }
}
float orc_cosine_lr(float base, float min_lr, uint32_t warmup, uint32_t total, uint32_t step) { return cosine_lr(base, min_lr, warmup, total, step); }

// The bare 4x8 block, exported so a test can compare it bit-for-bit with the reference's
// assembly kernel (src/asm/x86_64/matmul.s) built into oracle/_ref.
void orc_block_4x8(float* out, const float* lhs, const float* rhs, size_t k_l, size_t n) { block_4x8(out, lhs, rhs, k_l, n); }
}
