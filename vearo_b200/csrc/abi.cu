// The extern "C" op entry points: shape checks, output allocation, view handling, kernel choice.
// Each function is the device-side counterpart of one `BackendOps` field of the reference
// (crates/vearo-core/src/tensor.rs:1111-1175) or of a host-side helper of its autograd
// (crates/vearo-autograd/src/lib.rs:316-403); include/vearo_b200.h carries the per-function citations.
#include "common.h"
#include <cmath>
#include <cstdlib>
#include <unordered_map>
#include <cstring>

using namespace vb;

namespace {

int broadcast_dims(const vb_tensor& a, const vb_tensor& b, int* rank, i64* dims) {
  int r = a.rank > b.rank ? a.rank : b.rank;
  for (int i = 0; i < r; ++i) {
    i64 da = i < r - a.rank ? 1 : a.dims[i - (r - a.rank)];
    i64 db = i < r - b.rank ? 1 : b.dims[i - (r - b.rank)];
    if (da == db || da == 1 || db == 1) dims[i] = da == 1 ? db : da;
    else return set_error(VB_ERR_INVALID, "Shapes are not broadcastable");
  }
  *rank = r;
  return VB_OK;
}

int binary(int op, const vb_tensor* a, const vb_tensor* b, vb_tensor* out) {
  float *pa, *pb;
  VB_TRY(tensor_ptr(a, &pa)); VB_TRY(tensor_ptr(b, &pb));
  int r; i64 dims[VB_MAX_RANK];
  VB_TRY(broadcast_dims(*a, *b, &r, dims));
  VB_TRY(new_output(out, r, dims));
  i64 n = numel(*out);
  if (n == 0) return VB_OK;
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  bool ca = is_contiguous(*a), cb = is_contiguous(*b);
  i64 na = numel(*a), nb = numel(*b);
  if (ca && cb && na == n && nb == n) return launch_binary(op, pa, pb, po, n);
  if (ca && na == n && nb == 1) return launch_binary_scalar(op, pa, pb, po, n, true);
  if (cb && nb == n && na == 1) return launch_binary_scalar(op, pa, pb, po, n, false);
  i64 last = dims[r - 1];
  if (ca && cb && na == n && nb == last && b->dims[b->rank - 1] == last) return launch_binary_rowvec(op, pa, pb, po, n, last, true);
  if (ca && cb && nb == n && na == last && a->dims[a->rank - 1] == last) return launch_binary_rowvec(op, pa, pb, po, n, last, false);
  Strided s{}; s.rank = r;
  for (int i = 0; i < r; ++i) {
    s.dims[i] = dims[i];
    int ia = i - (r - a->rank), ib = i - (r - b->rank);
    s.sa[i] = (ia >= 0 && a->dims[ia] != 1) ? a->strides[ia] : 0;
    s.sb[i] = (ib >= 0 && b->dims[ib] != 1) ? b->strides[ib] : 0;
  }
  return launch_binary_strided(op, pa, pb, po, n, s);
}

int unary(int op, const vb_tensor* x, vb_tensor* out) {
  Temp hx; const float* px;
  VB_TRY(contiguous_ptr(x, &px, hx));
  VB_TRY(new_output(out, x->rank, x->dims));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_unary(op, px, po, numel(*x));
}
int unary_backward(int op, const vb_tensor* x, const vb_tensor* g, vb_tensor* gx) {
  VB_CHECK(same_shape(*x, *g), "x and grad_out shapes differ");
  Temp hx, hg; const float *px, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(g, &pg, hg));
  VB_TRY(new_output(gx, x->rank, x->dims));
  float* po; VB_TRY(slot_ptr(gx->slot, &po));
  return launch_unary_backward(op, px, pg, po, numel(*x));
}

int reduce_axis(const vb_tensor* x, int dim, int keep, bool mean, vb_tensor* out) {
  VB_CHECK(dim >= 0 && dim < x->rank, "Reduction dim out of range");
  Temp hx; const float* px;
  VB_TRY(contiguous_ptr(x, &px, hx));
  i64 od[VB_MAX_RANK]; int orank = 0;
  i64 outer = 1, inner = 1, d = x->dims[dim];
  for (int i = 0; i < x->rank; ++i) {
    if (i < dim) outer *= x->dims[i]; else if (i > dim) inner *= x->dims[i];
    if (i == dim) { if (keep) od[orank++] = 1; } else od[orank++] = x->dims[i];
  }
  VB_TRY(new_output(out, orank, od, true));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  if (numel(*x) == 0) return VB_OK;
  return launch_sum_axis(px, po, outer, d, inner, mean);
}

// Collapse the broadcast batch dims of a matmul into at most two levels.
struct BatchPlan { int levels; i64 n[VB_MAX_RANK], sa[VB_MAX_RANK], sb[VB_MAX_RANK], sc[VB_MAX_RANK]; };
void plan_batches(int r, const i64* dims, const i64* sa, const i64* sb, const i64* sc, BatchPlan& p) {
  p.levels = 0;
  for (int i = 0; i < r; ++i) {
    if (dims[i] == 1) continue;
    if (p.levels > 0) {
      int l = p.levels - 1;   // try to merge with the previous level
      if (p.sa[l] == sa[i] * dims[i] && p.sb[l] == sb[i] * dims[i] && p.sc[l] == sc[i] * dims[i]) {
        p.n[l] *= dims[i]; p.sa[l] = sa[i]; p.sb[l] = sb[i]; p.sc[l] = sc[i];
        continue;
      }
    }
    p.n[p.levels] = dims[i]; p.sa[p.levels] = sa[i]; p.sb[p.levels] = sb[i]; p.sc[p.levels] = sc[i];
    ++p.levels;
  }
}
int run_gemm_levels(GemmArgs g, const BatchPlan& p, int level, i64 offa, i64 offb, i64 offc) {
  int remaining = p.levels - level;
  if (remaining <= 2) {
    g.A += offa; g.B += offb; g.C += offc;
    g.nb1 = g.nb2 = 1; g.a_b1 = g.a_b2 = g.b_b1 = g.b_b2 = g.c_b1 = g.c_b2 = 0;
    if (remaining == 2) { g.nb1 = p.n[level]; g.a_b1 = p.sa[level]; g.b_b1 = p.sb[level]; g.c_b1 = p.sc[level];
                          g.nb2 = p.n[level + 1]; g.a_b2 = p.sa[level + 1]; g.b_b2 = p.sb[level + 1]; g.c_b2 = p.sc[level + 1]; }
    else if (remaining == 1) { g.nb2 = p.n[level]; g.a_b2 = p.sa[level]; g.b_b2 = p.sb[level]; g.c_b2 = p.sc[level]; }
    return launch_gemm(g);
  }
  for (i64 i = 0; i < p.n[level]; ++i)
    VB_TRY(run_gemm_levels(g, p, level + 1, offa + i * p.sa[level], offb + i * p.sb[level], offc + i * p.sc[level]));
  return VB_OK;
}

// a [.., M, K] (any strides) x b [.., K, N] -> contiguous out; alpha scaling and optional bias.
int matmul_impl(const vb_tensor* a, const vb_tensor* b, vb_tensor* out, float alpha, const float* bias) {
  float *pa, *pb;
  VB_TRY(tensor_ptr(a, &pa)); VB_TRY(tensor_ptr(b, &pb));
  VB_CHECK(a->rank >= 2 && b->rank >= 2, "Matmul requires rank >= 2");
  i64 M = a->dims[a->rank - 2], K = a->dims[a->rank - 1], K2 = b->dims[b->rank - 2], N = b->dims[b->rank - 1];
  VB_CHECK(K == K2, "Incompatible dimensions for matmul");
  vb_tensor ba = *a, bb = *b; ba.rank -= 2; bb.rank -= 2;
  int br; i64 bd[VB_MAX_RANK];
  VB_TRY(broadcast_dims(ba, bb, &br, bd));
  VB_CHECK(br + 2 <= VB_MAX_RANK, "rank too large");
  i64 od[VB_MAX_RANK];
  for (int i = 0; i < br; ++i) od[i] = bd[i];
  od[br] = M; od[br + 1] = N;
  VB_TRY(new_output(out, br + 2, od));
  if (numel(*out) == 0) return VB_OK;
  float* pc; VB_TRY(slot_ptr(out->slot, &pc));
  i64 sa[VB_MAX_RANK], sb[VB_MAX_RANK], sc[VB_MAX_RANK];
  for (int i = 0; i < br; ++i) {
    int ia = i - (br - ba.rank), ib = i - (br - bb.rank);
    sa[i] = (ia >= 0 && a->dims[ia] != 1) ? a->strides[ia] : 0;
    sb[i] = (ib >= 0 && b->dims[ib] != 1) ? b->strides[ib] : 0;
    sc[i] = out->strides[i];
  }
  BatchPlan p; plan_batches(br, bd, sa, sb, sc, p);
  GemmArgs g = gemm_args();
  g.A = pa; g.B = pb; g.C = pc; g.bias = bias; g.M = M; g.N = N; g.K = K; g.alpha = alpha;
  g.a_rs = a->strides[a->rank - 2]; g.a_cs = a->strides[a->rank - 1];
  g.b_rs = b->strides[b->rank - 2]; g.b_cs = b->strides[b->rank - 1];
  g.c_rs = N; g.c_cs = 1;
  if (K == 0) return launch_fill(pc, 0.0f, numel(*out));
  return run_gemm_levels(g, p, 0, 0, 0, 0);
}

// Flatten all leading dims of a contiguous-or-viewable tensor into rows: returns rows and a
// contiguous pointer (copying only when the view cannot be read as [rows, last] with a row stride).
int rows_of(const vb_tensor* t, i64* rows, i64* last) {
  VB_CHECK(t->rank >= 1, "rank must be >= 1");
  *last = t->dims[t->rank - 1];
  *rows = *last ? numel(*t) / *last : 0;
  return VB_OK;
}

int pool_dims(const vb_tensor* x, int k, int s, int p, i64* oh, i64* ow) {
  VB_CHECK(x->rank == 4, "pooling input must be rank 4 (N, C, H, W)");
  VB_CHECK(k > 0 && s > 0 && p >= 0, "bad pooling parameters");
  VB_CHECK(x->dims[2] + 2 * p >= k && x->dims[3] + 2 * p >= k, "window larger than padded input");
  *oh = (x->dims[2] + 2 * p - k) / s + 1; *ow = (x->dims[3] + 2 * p - k) / s + 1;
  return VB_OK;
}

}  // namespace

extern "C" {

int vb_add(const vb_tensor* a, const vb_tensor* b, vb_tensor* out) { return binary(0, a, b, out); }
int vb_sub(const vb_tensor* a, const vb_tensor* b, vb_tensor* out) { return binary(1, a, b, out); }
int vb_mul(const vb_tensor* a, const vb_tensor* b, vb_tensor* out) { return binary(2, a, b, out); }
int vb_div(const vb_tensor* a, const vb_tensor* b, vb_tensor* out) { return binary(3, a, b, out); }
int vb_matmul(const vb_tensor* a, const vb_tensor* b, vb_tensor* out) { return matmul_impl(a, b, out, 1.0f, nullptr); }
int vb_relu(const vb_tensor* x, vb_tensor* out) { return unary(0, x, out); }
int vb_gelu(const vb_tensor* x, vb_tensor* out) { return unary(1, x, out); }
namespace { bool col_sums_enabled(); void col_sums_adopt(const vb_tensor* t, i64 rows, i64 cols, vb_slot sums); }     // defined with the table below
// A large activation gradient is about to be the output gradient of a Linear layer: the kernel leaves its column sums (that
// layer's bias gradient) beside it.
static int unary_backward_summed(int op, const vb_tensor* x, const vb_tensor* g, vb_tensor* gx) {
  i64 rows = 0, cols = 0;
  if (x->rank >= 2) { cols = x->dims[x->rank - 1]; rows = cols ? numel(*x) / cols : 0; }
  // (rows of fewer than 1024 floats do not fill the band kernel's 256 threads: the flat kernel plus a later column sum is faster there)
  if (!col_sums_enabled() || rows < 1024 || cols < 1024 || cols > 4096 || (cols & 3) || !is_contiguous(*x) || !is_contiguous(*g)) return unary_backward(op, x, g, gx);
  VB_CHECK(same_shape(*x, *g), "x and grad_out shapes differ");
  float *px, *pg; VB_TRY(tensor_ptr(x, &px)); VB_TRY(tensor_ptr(g, &pg));
  if (((reinterpret_cast<uintptr_t>(px) | reinterpret_cast<uintptr_t>(pg)) & 15) != 0) return unary_backward(op, x, g, gx);
  vb_slot sums = 0;
  if (slot_alloc(cols, false, &sums) != VB_OK) return unary_backward(op, x, g, gx);
  float* ps = nullptr; slot_ptr(sums, &ps);
  int rc = new_output(gx, x->rank, x->dims);
  float* po = nullptr;
  if (rc == VB_OK) rc = slot_ptr(gx->slot, &po);
  if (rc == VB_OK) rc = launch_unary_backward_colsum(op, px, pg, po, rows, cols, ps);
  if (rc == VB_OK) col_sums_adopt(gx, rows, cols, sums); else slot_release(sums, nullptr);
  return rc;
}
int vb_relu_backward(const vb_tensor* x, const vb_tensor* g, vb_tensor* gx) { return unary_backward_summed(0, x, g, gx); }
int vb_gelu_backward(const vb_tensor* x, const vb_tensor* g, vb_tensor* gx) { return unary_backward_summed(1, x, g, gx); }
int vb_sum(const vb_tensor* x, int dim, int keep, vb_tensor* out) { return reduce_axis(x, dim, keep, false, out); }
int vb_mean(const vb_tensor* x, int dim, int keep, vb_tensor* out) { return reduce_axis(x, dim, keep, true, out); }

int vb_softmax(const vb_tensor* x, int dim, vb_tensor* out) {
  VB_CHECK(dim >= 0 && dim < x->rank, "Softmax dim out of range");
  Temp hx; const float* px;
  VB_TRY(contiguous_ptr(x, &px, hx));
  VB_TRY(new_output(out, x->rank, x->dims));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  if (numel(*x) == 0) return VB_OK;
  i64 outer = 1, inner = 1, d = x->dims[dim];
  for (int i = 0; i < dim; ++i) outer *= x->dims[i];
  for (int i = dim + 1; i < x->rank; ++i) inner *= x->dims[i];
  return inner == 1 ? launch_softmax_rows(px, po, outer, d) : launch_softmax_strided(px, po, outer, d, inner);
}
int vb_softmax_backward(const vb_tensor* x, const vb_tensor* g, int dim, vb_tensor* gx) {
  VB_CHECK(dim >= 0 && dim < x->rank, "Softmax dim out of range");
  VB_CHECK(same_shape(*x, *g), "x and grad_out shapes differ");
  Temp hx, hg; const float *px, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(g, &pg, hg));
  VB_TRY(new_output(gx, x->rank, x->dims));
  float* po; VB_TRY(slot_ptr(gx->slot, &po));
  if (numel(*x) == 0) return VB_OK;
  i64 outer = 1, inner = 1, d = x->dims[dim];
  for (int i = 0; i < dim; ++i) outer *= x->dims[i];
  for (int i = dim + 1; i < x->rank; ++i) inner *= x->dims[i];
  return inner == 1 ? launch_softmax_backward_rows(px, pg, po, outer, d) : launch_softmax_backward_strided(px, pg, po, outer, d, inner);
}

namespace { bool activation_lo_enabled(); void lo_plane_adopt(vb_slot slot, vb_slot lo, i64 n); }     // defined with the lo-plane table below
int vb_layernorm(const vb_tensor* x, const vb_tensor* w, const vb_tensor* b, float eps, vb_tensor* out) {
  VB_CHECK(x->rank >= 1, "LayerNorm input must be at least rank 1");
  i64 rows, c; VB_TRY(rows_of(x, &rows, &c));
  VB_CHECK(w->rank == 1 && b->rank == 1, "LayerNorm weight and bias must be rank 1");
  VB_CHECK(w->dims[0] == c && b->dims[0] == c, "Weight/Bias dimension must match norm_dim");
  Temp hx, hw, hb; const float *px, *pw, *pb;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(w, &pw, hw)); VB_TRY(contiguous_ptr(b, &pb, hb));
  VB_TRY(new_output(out, x->rank, x->dims));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  // A large normalised activation is about to be the B operand of a weight-gradient product: its TF32 remainders are written
  // along with it (4 more bytes per element) and kept as the lo plane of the output's slot until that slot is released.
  vb_slot lo_slot = 0; float* plo = nullptr;
  if (activation_lo_enabled() && rows >= 1024 && rows * c >= ((i64)1 << 18) && slot_alloc(rows * c, false, &lo_slot) == VB_OK) slot_ptr(lo_slot, &plo);
  bool lo_done = false;
  int rc = launch_layernorm(px, pw, pb, po, rows, c, eps, plo, &lo_done);
  if (lo_slot) { if (rc == VB_OK && lo_done) lo_plane_adopt(out->slot, lo_slot, rows * c); else slot_release(lo_slot, nullptr); }
  return rc;
}
int vb_layernorm_backward(const vb_tensor* x, const vb_tensor* w, const vb_tensor* b, const vb_tensor* g, float eps,
                          vb_tensor* gx, vb_tensor* gw, vb_tensor* gb) {
  VB_CHECK(x->rank >= 1, "LayerNorm input must be at least rank 1");
  i64 rows, c; VB_TRY(rows_of(x, &rows, &c));
  VB_CHECK(w->rank == 1 && b->rank == 1 && w->dims[0] == c && b->dims[0] == c, "Weight/Bias dimension must match norm_dim");
  VB_CHECK(same_shape(*x, *g), "x and grad_out shapes differ");
  Temp hx, hw, hg; const float *px, *pw, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(w, &pw, hw)); VB_TRY(contiguous_ptr(g, &pg, hg));
  VB_TRY(new_output(gx, x->rank, x->dims));
  VB_TRY(new_output(gw, 1, &c)); VB_TRY(new_output(gb, 1, &c));
  float *pgx, *pgw, *pgb;
  VB_TRY(slot_ptr(gx->slot, &pgx)); VB_TRY(slot_ptr(gw->slot, &pgw)); VB_TRY(slot_ptr(gb->slot, &pgb));
  // the input gradient of a residual stream is usually the output gradient of the Linear layer before it: keep its column sums
  vb_slot sums = 0; float* ps = nullptr;
  if (col_sums_enabled() && rows >= 1024 && x->rank >= 2 && slot_alloc(c, false, &sums) == VB_OK) slot_ptr(sums, &ps);
  bool summed = false;
  int rc = launch_layernorm_backward(px, pw, pg, pgx, pgw, pgb, rows, c, eps, nullptr, ps, &summed);
  if (sums) { if (rc == VB_OK && summed) col_sums_adopt(gx, rows, c, sums); else slot_release(sums, nullptr); }
  return rc;
}
// The same, added to an existing gradient of x in place: grad_in += dx (one pass instead of a fresh dx and an accumulate).
int vb_layernorm_backward_accum(const vb_tensor* x, const vb_tensor* w, const vb_tensor* b, const vb_tensor* g, float eps,
                                const vb_tensor* grad_in, vb_tensor* gw, vb_tensor* gb) {
  VB_CHECK(x->rank >= 1, "LayerNorm input must be at least rank 1");
  i64 rows, c; VB_TRY(rows_of(x, &rows, &c));
  VB_CHECK(w->rank == 1 && b->rank == 1 && w->dims[0] == c && b->dims[0] == c, "Weight/Bias dimension must match norm_dim");
  VB_CHECK(same_shape(*x, *g), "x and grad_out shapes differ");
  VB_CHECK(grad_in && same_shape(*x, *grad_in) && is_contiguous(*grad_in), "grad_in must be a contiguous tensor of x's shape");
  Temp hx, hw, hg; const float *px, *pw, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(w, &pw, hw)); VB_TRY(contiguous_ptr(g, &pg, hg));
  float* pacc; VB_TRY(tensor_ptr(grad_in, &pacc));
  VB_TRY(new_output(gw, 1, &c)); VB_TRY(new_output(gb, 1, &c));
  float *pgw, *pgb;
  VB_TRY(slot_ptr(gw->slot, &pgw)); VB_TRY(slot_ptr(gb->slot, &pgb));
  slot_touch(grad_in->slot);
  if (rows == 0) return launch_layernorm_backward(px, pw, pg, pacc, pgw, pgb, rows, c, eps);
  vb_slot sums = 0; float* ps = nullptr;
  if (col_sums_enabled() && rows >= 1024 && x->rank >= 2 && slot_alloc(c, false, &sums) == VB_OK) slot_ptr(sums, &ps);
  bool summed = false;
  int rc = launch_layernorm_backward(px, pw, pg, pacc, pgw, pgb, rows, c, eps, pacc, ps, &summed);
  if (sums) { if (rc == VB_OK && summed) col_sums_adopt(grad_in, rows, c, sums); else slot_release(sums, nullptr); }
  return rc;
}

int vb_embedding(const vb_tensor* ids, const vb_tensor* weight, vb_tensor* out) {
  VB_CHECK(weight->rank == 2, "Weight must be rank 2 (vocab_size, embedding_dim)");
  VB_CHECK(ids->rank + 1 <= VB_MAX_RANK, "rank too large");
  Temp hi, hw; const float *pi, *pw;
  VB_TRY(contiguous_ptr(ids, &pi, hi)); VB_TRY(contiguous_ptr(weight, &pw, hw));
  i64 od[VB_MAX_RANK];
  for (int i = 0; i < ids->rank; ++i) od[i] = ids->dims[i];
  od[ids->rank] = weight->dims[1];
  VB_TRY(new_output(out, ids->rank + 1, od));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_embedding(pi, pw, po, numel(*ids), weight->dims[0], weight->dims[1]);
}
int vb_embedding_backward(const vb_tensor* ids, const vb_tensor* weight, const vb_tensor* g, vb_tensor* gw) {
  VB_CHECK(weight->rank == 2, "Weight must be rank 2 (vocab_size, embedding_dim)");
  VB_CHECK(g->rank == ids->rank + 1 && g->dims[g->rank - 1] == weight->dims[1], "grad_out shape must be x.shape() + [embedding_dim]");
  for (int i = 0; i < ids->rank; ++i) VB_CHECK(g->dims[i] == ids->dims[i], "grad_out shape must be x.shape() + [embedding_dim]");
  Temp hi, hg; const float *pi, *pg;
  VB_TRY(contiguous_ptr(ids, &pi, hi)); VB_TRY(contiguous_ptr(g, &pg, hg));
  VB_TRY(new_output(gw, 2, weight->dims, true));
  float* po; VB_TRY(slot_ptr(gw->slot, &po));
  return launch_embedding_backward(pi, pg, po, numel(*ids), weight->dims[0], weight->dims[1]);
}

int vb_cross_entropy(const vb_tensor* logits, const vb_tensor* targets, vb_tensor* loss, vb_tensor* row_stats) {
  VB_CHECK(logits->rank == 2, "Logits must be rank 2 (batch_size, vocab_size)");
  VB_CHECK(targets->rank == 1, "Targets must be rank 1 (batch_size)");
  i64 B = logits->dims[0], V = logits->dims[1];
  VB_CHECK(B > 0, "Batch size must be greater than 0");
  VB_CHECK(V > 0, "Vocabulary size must be greater than 0");
  VB_CHECK(targets->dims[0] == B, "Targets shape must match batch size");
  Temp hl, ht; const float *pl, *pt;
  VB_TRY(contiguous_ptr(logits, &pl, hl)); VB_TRY(contiguous_ptr(targets, &pt, ht));
  i64 one = 1;
  VB_TRY(new_output(loss, 1, &one));
  float* plo; VB_TRY(slot_ptr(loss->slot, &plo));
  float* pst = nullptr;
  if (row_stats) { i64 sd[2] = {B, 2}; VB_TRY(new_output(row_stats, 2, sd)); VB_TRY(slot_ptr(row_stats->slot, &pst)); }
  return launch_cross_entropy(pl, pt, plo, pst, B, V);
}
int vb_cross_entropy_fused(const vb_tensor* logits_inout, const vb_tensor* targets, vb_tensor* loss) {
  VB_CHECK(logits_inout->rank == 2, "Logits must be rank 2 (batch_size, vocab_size)");
  VB_CHECK(targets->rank == 1, "Targets must be rank 1 (batch_size)");
  i64 B = logits_inout->dims[0], V = logits_inout->dims[1];
  VB_CHECK(B > 0, "Batch size must be greater than 0");
  VB_CHECK(V > 0, "Vocabulary size must be greater than 0");
  VB_CHECK(targets->dims[0] == B, "Targets shape must match batch size");
  VB_CHECK(is_contiguous(*logits_inout), "cross_entropy_fused overwrites the logits: they must be contiguous");
  float* pl; VB_TRY(tensor_ptr(logits_inout, &pl));
  slot_touch(logits_inout->slot);        // overwritten with the gradient
  Temp ht; const float* pt;
  VB_TRY(contiguous_ptr(targets, &pt, ht));
  i64 one = 1;
  VB_TRY(new_output(loss, 1, &one));
  float* plo; VB_TRY(slot_ptr(loss->slot, &plo));
  return launch_cross_entropy_fused(pl, pt, plo, B, V);
}
int vb_cross_entropy_backward(const vb_tensor* logits, const vb_tensor* targets, const vb_tensor* g,
                              const vb_tensor* row_stats, vb_tensor* gl) {
  VB_CHECK(logits->rank == 2, "Logits must be rank 2 (batch_size, vocab_size)");
  VB_CHECK(targets->rank == 1, "Targets must be rank 1 (batch_size)");
  i64 B = logits->dims[0], V = logits->dims[1];
  VB_CHECK(B > 0, "Batch size must be greater than 0");
  VB_CHECK(targets->dims[0] == B, "Targets shape must match batch size");
  VB_CHECK(numel(*g) == 1, "grad_out must be a scalar");
  Temp hl, ht, hs; const float *pl, *pt, *ps = nullptr;
  VB_TRY(contiguous_ptr(logits, &pl, hl)); VB_TRY(contiguous_ptr(targets, &pt, ht));
  if (row_stats) { VB_CHECK(numel(*row_stats) == 2 * B, "row_stats must be [B,2]"); VB_TRY(contiguous_ptr(row_stats, &ps, hs)); }
  float* pg; VB_TRY(tensor_ptr(g, &pg));
  VB_TRY(new_output(gl, 2, logits->dims));
  float* po; VB_TRY(slot_ptr(gl->slot, &po));
  return launch_cross_entropy_backward(pl, pt, pg, ps, po, B, V);
}

int vb_conv2d(const vb_tensor* x, const vb_tensor* w, const vb_tensor* bias, int stride, int padding, vb_tensor* out) {
  VB_CHECK(x->rank == 4 && w->rank == 4, "conv2d expects NCHW input and OIHW weight");
  VB_CHECK(w->dims[1] == x->dims[1], "conv2d channel mismatch");
  VB_CHECK(bias->rank == 1 && bias->dims[0] == w->dims[0], "conv2d bias must be [Cout]");
  VB_CHECK(stride > 0 && padding >= 0, "bad stride / padding");
  i64 n = x->dims[0], cin = x->dims[1], h = x->dims[2], wd = x->dims[3], cout = w->dims[0], kh = w->dims[2], kw = w->dims[3];
  VB_CHECK(h + 2 * padding >= kh && wd + 2 * padding >= kw, "kernel larger than padded input");
  i64 oh = (h + 2 * padding - kh) / stride + 1, ow = (wd + 2 * padding - kw) / stride + 1;
  Temp hx, hw, hb; const float *px, *pw, *pb;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(w, &pw, hw)); VB_TRY(contiguous_ptr(bias, &pb, hb));
  i64 od[4] = {n, cout, oh, ow};
  VB_TRY(new_output(out, 4, od));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_conv2d(px, pw, pb, po, n, cin, h, wd, cout, kh, kw, oh, ow, stride, padding);
}
int vb_conv2d_backward(const vb_tensor* x, const vb_tensor* w, const vb_tensor* g, int stride, int padding,
                       vb_tensor* gx, vb_tensor* gw, vb_tensor* gb) {
  VB_CHECK(x->rank == 4 && w->rank == 4 && g->rank == 4, "conv2d_backward expects rank-4 tensors");
  i64 n = x->dims[0], cin = x->dims[1], h = x->dims[2], wd = x->dims[3], cout = w->dims[0], kh = w->dims[2], kw = w->dims[3];
  i64 oh = g->dims[2], ow = g->dims[3];
  VB_CHECK(g->dims[0] == n && g->dims[1] == cout, "grad_out shape mismatch");
  Temp hx, hw, hg; const float *px, *pw, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(w, &pw, hw)); VB_TRY(contiguous_ptr(g, &pg, hg));
  if (gx) VB_TRY(new_output(gx, 4, x->dims));
  VB_TRY(new_output(gw, 4, w->dims)); VB_TRY(new_output(gb, 1, &cout));
  float *pgx = nullptr, *pgw, *pgb;
  if (gx) VB_TRY(slot_ptr(gx->slot, &pgx));
  VB_TRY(slot_ptr(gw->slot, &pgw)); VB_TRY(slot_ptr(gb->slot, &pgb));
  return launch_conv2d_backward(px, pw, pg, pgx, pgw, pgb, n, cin, h, wd, cout, kh, kw, oh, ow, stride, padding);
}

int vb_maxpool2d(const vb_tensor* x, int k, int s, int p, vb_tensor* out) {
  i64 oh, ow; VB_TRY(pool_dims(x, k, s, p, &oh, &ow));
  Temp hx; const float* px; VB_TRY(contiguous_ptr(x, &px, hx));
  i64 od[4] = {x->dims[0], x->dims[1], oh, ow};
  VB_TRY(new_output(out, 4, od));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_maxpool2d(px, po, x->dims[0] * x->dims[1], x->dims[2], x->dims[3], oh, ow, k, s, p);
}
int vb_maxpool2d_backward(const vb_tensor* x, const vb_tensor* g, int k, int s, int p, vb_tensor* gx) {
  VB_CHECK(x->rank == 4 && g->rank == 4, "pooling tensors must be rank 4");
  Temp hx, hg; const float *px, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(g, &pg, hg));
  VB_TRY(new_output(gx, 4, x->dims));
  float* po; VB_TRY(slot_ptr(gx->slot, &po));
  return launch_maxpool2d_backward(px, pg, po, x->dims[0] * x->dims[1], x->dims[2], x->dims[3], g->dims[2], g->dims[3], k, s, p);
}
int vb_avgpool2d(const vb_tensor* x, int k, int s, int p, vb_tensor* out) {
  i64 oh, ow; VB_TRY(pool_dims(x, k, s, p, &oh, &ow));
  Temp hx; const float* px; VB_TRY(contiguous_ptr(x, &px, hx));
  i64 od[4] = {x->dims[0], x->dims[1], oh, ow};
  VB_TRY(new_output(out, 4, od));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_avgpool2d(px, po, x->dims[0] * x->dims[1], x->dims[2], x->dims[3], oh, ow, k, s, p);
}
int vb_avgpool2d_backward(const vb_tensor* x, const vb_tensor* g, int k, int s, int p, vb_tensor* gx) {
  VB_CHECK(x->rank == 4 && g->rank == 4, "pooling tensors must be rank 4");
  Temp hg; const float* pg; VB_TRY(contiguous_ptr(g, &pg, hg));
  VB_TRY(new_output(gx, 4, x->dims));
  float* po; VB_TRY(slot_ptr(gx->slot, &po));
  return launch_avgpool2d_backward(pg, po, x->dims[0] * x->dims[1], x->dims[2], x->dims[3], g->dims[2], g->dims[3], k, s, p);
}

int vb_batchnorm(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* rm, const vb_tensor* rv,
                 int training, float momentum, float eps, vb_tensor* out) {
  VB_CHECK(x->rank == 4, "BatchNorm2d input must be rank 4 (N, C, H, W)");
  i64 c = x->dims[1];
  VB_CHECK(gamma->rank == 1 && beta->rank == 1 && gamma->dims[0] == c && beta->dims[0] == c, "Gamma/Beta dim must match channels C");
  VB_CHECK(numel(*rm) == c && numel(*rv) == c && is_contiguous(*rm) && is_contiguous(*rv), "running stats must be contiguous [C]");
  Temp hx, hg, hb; const float *px, *pg, *pb;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(gamma, &pg, hg)); VB_TRY(contiguous_ptr(beta, &pb, hb));
  float *prm, *prv; VB_TRY(tensor_ptr(rm, &prm)); VB_TRY(tensor_ptr(rv, &prv));
  VB_TRY(new_output(out, 4, x->dims));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_batchnorm(px, pg, pb, prm, prv, po, x->dims[0], c, x->dims[2] * x->dims[3], training != 0, momentum, eps);
}
int vb_batchnorm_backward(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* rm, const vb_tensor* rv,
                          const vb_tensor* g, int training, float eps, vb_tensor* gx, vb_tensor* gw, vb_tensor* gb) {
  (void)beta;
  VB_CHECK(x->rank == 4 && same_shape(*x, *g), "BatchNorm2d tensors must be rank 4 and of equal shape");
  i64 c = x->dims[1];
  Temp hx, hg, hgo, hrm, hrv; const float *px, *pg, *pgo, *prm, *prv;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(gamma, &pg, hg)); VB_TRY(contiguous_ptr(g, &pgo, hgo));
  VB_TRY(contiguous_ptr(rm, &prm, hrm)); VB_TRY(contiguous_ptr(rv, &prv, hrv));
  VB_TRY(new_output(gx, 4, x->dims)); VB_TRY(new_output(gw, 1, &c)); VB_TRY(new_output(gb, 1, &c));
  float *pgx, *pgw, *pgb;
  VB_TRY(slot_ptr(gx->slot, &pgx)); VB_TRY(slot_ptr(gw->slot, &pgw)); VB_TRY(slot_ptr(gb->slot, &pgb));
  return launch_batchnorm_backward(px, pg, prm, prv, pgo, pgx, pgw, pgb, x->dims[0], c, x->dims[2] * x->dims[3], training != 0, eps);
}

int vb_bn_relu_maxpool(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* rm, const vb_tensor* rv,
                       int training, float momentum, float eps, vb_tensor* out, vb_tensor* stats) {
  VB_CHECK(x->rank == 4, "BatchNorm2d input must be rank 4 (N, C, H, W)");
  VB_CHECK(stats != nullptr, "vb_bn_relu_maxpool needs the stats output");
  i64 c = x->dims[1];
  VB_CHECK(gamma->rank == 1 && beta->rank == 1 && gamma->dims[0] == c && beta->dims[0] == c, "Gamma/Beta dim must match channels C");
  VB_CHECK(numel(*rm) == c && numel(*rv) == c && is_contiguous(*rm) && is_contiguous(*rv), "running stats must be contiguous [C]");
  VB_CHECK(x->dims[2] >= 2 && x->dims[3] >= 2, "pooling window larger than the input");
  Temp hx, hg, hb; const float *px, *pg, *pb;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(gamma, &pg, hg)); VB_TRY(contiguous_ptr(beta, &pb, hb));
  float *prm, *prv; VB_TRY(tensor_ptr(rm, &prm)); VB_TRY(tensor_ptr(rv, &prv));
  i64 od[4] = {x->dims[0], c, x->dims[2] / 2, x->dims[3] / 2}, sd[2] = {2, c};
  VB_TRY(new_output(out, 4, od)); VB_TRY(new_output(stats, 2, sd));
  float *po, *ps; VB_TRY(slot_ptr(out->slot, &po)); VB_TRY(slot_ptr(stats->slot, &ps));
  return launch_bn_relu_maxpool(px, pg, pb, prm, prv, ps, po, x->dims[0], c, x->dims[2], x->dims[3], training != 0, momentum, eps);
}
int vb_bn_relu_maxpool_backward(const vb_tensor* x, const vb_tensor* gamma, const vb_tensor* beta, const vb_tensor* stats,
                                const vb_tensor* g, int training, vb_tensor* gx, vb_tensor* gw, vb_tensor* gb) {
  VB_CHECK(x->rank == 4 && g->rank == 4, "BatchNorm2d tensors must be rank 4");
  i64 c = x->dims[1];
  VB_CHECK(g->dims[0] == x->dims[0] && g->dims[1] == c && g->dims[2] == x->dims[2] / 2 && g->dims[3] == x->dims[3] / 2, "grad_out shape mismatch");
  VB_CHECK(numel(*stats) == 2 * c, "stats must be [2, C]");
  Temp hx, hg, hb, hs, hgo; const float *px, *pg, *pb, *ps, *pgo;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(gamma, &pg, hg)); VB_TRY(contiguous_ptr(beta, &pb, hb));
  VB_TRY(contiguous_ptr(stats, &ps, hs)); VB_TRY(contiguous_ptr(g, &pgo, hgo));
  VB_TRY(new_output(gx, 4, x->dims)); VB_TRY(new_output(gw, 1, &c)); VB_TRY(new_output(gb, 1, &c));
  float *pgx, *pgw, *pgb;
  VB_TRY(slot_ptr(gx->slot, &pgx)); VB_TRY(slot_ptr(gw->slot, &pgw)); VB_TRY(slot_ptr(gb->slot, &pgb));
  return launch_bn_relu_maxpool_backward(px, pg, pb, ps, pgo, pgx, pgw, pgb, x->dims[0], c, x->dims[2], x->dims[3], training != 0);
}

// ---- attention -------------------------------------------------------------------------------
static int mask_strides(const vb_tensor* mask, i64 B, i64 H, i64 Sq, i64 Sk, const float** pm, i64 ms[4]) {
  *pm = nullptr; ms[0] = ms[1] = ms[2] = ms[3] = 0;
  if (!mask) return VB_OK;
  VB_CHECK(mask->rank <= 4, "mask rank must be <= 4");
  float* p; VB_TRY(tensor_ptr(mask, &p));
  i64 want[4] = {B, H, Sq, Sk};
  for (int i = 0; i < mask->rank; ++i) {
    int o = 4 - mask->rank + i;
    VB_CHECK(mask->dims[i] == 1 || mask->dims[i] == want[o], "mask is not broadcastable to [B,H,S,S]");
    ms[o] = mask->dims[i] == 1 ? 0 : mask->strides[i];
  }
  *pm = p;
  return VB_OK;
}
// Causal fast path.  A [S,S] additive mask that is 0 on/below the diagonal and <= -1e9 above it makes every
// probability above the diagonal exactly 0, so score tiles there need not be computed and the products with P / dS
// are triangular.  The pattern is checked on the device once per mask (slot contents are versioned) and the answer
// cached; shapes outside the tensor-core kernel's rules keep the general path.
static bool attention_is_causal(const vb_tensor* mask, const vb_tensor* q, i64 S, i64 dk) {
  static int disabled = -1;
  if (disabled < 0) { const char* e = getenv("VB200_NO_CAUSAL"); disabled = (e && e[0] == '1') ? 1 : 0; }
  if (disabled || !mask || S % 128 != 0 || S > 1024 || dk % 4 != 0 || dk < 32) return false;
  for (int i = 0; i < mask->rank - 2; ++i) if (mask->dims[i] != 1) return false;
  if (mask->rank < 2 || mask->dims[mask->rank - 1] != S || mask->dims[mask->rank - 2] != S || mask->strides[mask->rank - 1] != 1) return false;
  for (int i = 0; i < 4; ++i) if (q->strides[i] % 4 != 0 && i != 3) return false;
  struct Cache { vb_slot slot = 0; uint64_t serial = 0; i64 offset = -1, S = 0, rs = 0; bool causal = false; };
  static Cache c;
  i64 rs = mask->strides[mask->rank - 2];
  if (c.slot == mask->slot && c.serial == slot_serial(mask->slot) && c.offset == mask->offset && c.S == S && c.rs == rs) return c.causal;
  float* pm;
  if (tensor_ptr(mask, &pm) != VB_OK) return false;
  int* d_flag = reinterpret_cast<int*>(ctx().d_scalars + 8);
  int one = 1, h = 0;
  if (cudaMemcpyAsync(d_flag, &one, sizeof(int), cudaMemcpyHostToDevice, ctx().stream) != cudaSuccess) return false;
  if (launch_mask_is_causal(pm, S, rs, d_flag) != VB_OK) return false;
  if (cudaMemcpyAsync(&h, d_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx().stream) != cudaSuccess) return false;
  if (cudaStreamSynchronize(ctx().stream) != cudaSuccess) return false;
  c.slot = mask->slot; c.serial = slot_serial(mask->slot); c.offset = mask->offset; c.S = S; c.rs = rs; c.causal = h == 1;
  return c.causal;
}
// VB200_ATTN_FUSED=0 keeps attention on the GEMM + row-kernel route (the route every additive mask other than the causal one takes)
static bool attn_fused_enabled() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("VB200_ATTN_FUSED"); on = (e && e[0] == '0') ? 0 : 1; }
  return on != 0;
}
static void qk_gemm_operand(const vb_tensor* t, i64* rs, i64* cs, i64* b1, i64* b2) {
  *b1 = t->strides[0]; *b2 = t->strides[1]; *rs = t->strides[2]; *cs = t->strides[3];
}

// Attention results are laid out in memory as [B,S,H,dk] and returned as the [B,H,S,dk] view of that buffer: the
// `transpose(1,2).reshape([B,S,D])` that follows in MultiHeadAttention::forward (and its mirror image in the
// backward walk) is then a pure view, with no copy.
static int new_output_bshd(vb_tensor* out, i64 B, i64 H, i64 S, i64 dk) {
  i64 mem[4] = {B, S, H, dk};
  VB_TRY(new_output(out, 4, mem));
  out->dims[0] = B; out->dims[1] = H; out->dims[2] = S; out->dims[3] = dk;
  out->strides[0] = S * H * dk; out->strides[1] = dk; out->strides[2] = H * dk; out->strides[3] = 1;
  return VB_OK;
}

int vb_fused_attention(const vb_tensor* q, const vb_tensor* k, const vb_tensor* v, const vb_tensor* mask,
                       vb_tensor* out, vb_tensor* probs) {
  VB_CHECK(q->rank == 4 && same_shape(*q, *k) && same_shape(*q, *v), "fused_attention expects q, k, v of equal shape [B,H,S,dk]");
  i64 B = q->dims[0], H = q->dims[1], S = q->dims[2], dk = q->dims[3];
  float *pq, *pk, *pv; VB_TRY(tensor_ptr(q, &pq)); VB_TRY(tensor_ptr(k, &pk)); VB_TRY(tensor_ptr(v, &pv));
  const float* pm; i64 ms[4]; VB_TRY(mask_strides(mask, B, H, S, S, &pm, ms));
  VB_TRY(new_output_bshd(out, B, H, S, dk));
  if (numel(*q) == 0) { if (probs) { i64 pd[4] = {B, H, S, S}; VB_TRY(new_output(probs, 4, pd)); } return VB_OK; }
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  i64 pd[4] = {B, H, S, S};
  float scale = 1.0f / sqrtf((float)dk);
  const bool causal = attention_is_causal(mask, q, S, dk);
  if (causal || !mask) {
    // one kernel for scores, softmax and the product with V (attn_fused.cu); the probabilities leave the SM only when asked for,
    // and then the slot that takes them also takes a copy of the output behind them: the backward kernel wants both
    const AttnOperand oq{pq, q->strides[0], q->strides[1], q->strides[2], q->strides[3]};
    const AttnOperand ok{pk, k->strides[0], k->strides[1], k->strides[2], k->strides[3]};
    const AttnOperand ov{pv, v->strides[0], v->strides[1], v->strides[2], v->strides[3]};
    if (attn_fused_enabled() && attn_fused_supported(oq, ok, ov, B, H, S, dk)) {
      vb_tensor saved; saved.slot = 0;
      float* ps = nullptr;
      if (probs) {
        vb_slot sl; VB_TRY(slot_alloc(B * H * S * (S + dk), false, &sl));
        set_contiguous(saved, 4, pd); saved.slot = sl;
        VB_TRY(slot_ptr(sl, &ps));
      }
      int rc = launch_attn_fwd_fused(oq, ok, ov, po, H * dk, S * H * dk, ps, B, H, S, causal, scale);
      if (rc == VB_OK && probs) *probs = saved; else if (saved.slot) slot_release(saved.slot, nullptr);
      return rc;
    }
  }
  // scores / probabilities
  vb_tensor ptmp;
  VB_TRY(new_output(&ptmp, 4, pd));
  float* pp; VB_TRY(slot_ptr(ptmp.slot, &pp));
  GemmArgs g = gemm_args();
  g.M = S; g.N = S; g.K = dk; g.alpha = scale; g.nb1 = B; g.nb2 = H; g.causal = causal ? 1 : 0;
  g.A = pq; qk_gemm_operand(q, &g.a_rs, &g.a_cs, &g.a_b1, &g.a_b2);
  g.B = pk; { i64 rs, cs; qk_gemm_operand(k, &rs, &cs, &g.b_b1, &g.b_b2); g.b_rs = cs; g.b_cs = rs; }   // K^T
  g.C = pp; g.c_rs = S; g.c_cs = 1; g.c_b1 = H * S * S; g.c_b2 = S * S;
  int rc = launch_gemm(g);
  if (rc == VB_OK) rc = launch_attn_softmax(pp, pm, ms, causal, B, H, S, S, scale);
  if (rc == VB_OK) {
    GemmArgs o = gemm_args();
    o.M = S; o.N = dk; o.K = S; o.nb1 = B; o.nb2 = H; o.causal = causal ? 2 : 0;
    o.A = pp; o.a_rs = S; o.a_cs = 1; o.a_b1 = H * S * S; o.a_b2 = S * S;
    o.B = pv; qk_gemm_operand(v, &o.b_rs, &o.b_cs, &o.b_b1, &o.b_b2);
    o.C = po; o.c_rs = H * dk; o.c_cs = 1; o.c_b1 = S * H * dk; o.c_b2 = dk;
    rc = launch_gemm(o);
  }
  if (rc == VB_OK && probs) *probs = ptmp; else slot_release(ptmp.slot, nullptr);
  return rc;
}

// The backward products; gradients are written as [B,S,H,dk]-ordered rows of length `ld` floats (ld = H*dk for separate
// buffers, 3*H*dk when dq, dk and dv are the three column blocks of one packed [B,S,3*H*dk] buffer).
static int attention_backward_core(const vb_tensor* q, const vb_tensor* k, const vb_tensor* v, const vb_tensor* mask,
                                   const vb_tensor* gout, const vb_tensor* probs, float* pdq, float* pdk, float* pdv, i64 ld) {
  i64 B = q->dims[0], H = q->dims[1], S = q->dims[2], dk = q->dims[3];
  float *pq, *pk, *pv, *pg;
  VB_TRY(tensor_ptr(q, &pq)); VB_TRY(tensor_ptr(k, &pk)); VB_TRY(tensor_ptr(v, &pv)); VB_TRY(tensor_ptr(gout, &pg));
  float scale = 1.0f / sqrtf((float)dk);
  const bool causal = attention_is_causal(mask, q, S, dk);
  i64 SS = S * S;
  // probabilities: reuse the saved ones or recompute them
  vb_tensor ptmp; ptmp.slot = 0;
  const float* pp;
  if (probs) {
    VB_CHECK(numel(*probs) == B * H * SS && is_contiguous(*probs), "probs must be a contiguous [B,H,S,S] tensor");
    float* t; VB_TRY(tensor_ptr(probs, &t)); pp = t;
  } else {
    const float* pm; i64 ms[4]; VB_TRY(mask_strides(mask, B, H, S, S, &pm, ms));
    i64 pd[4] = {B, H, S, S};
    VB_TRY(new_output(&ptmp, 4, pd));
    float* t; VB_TRY(slot_ptr(ptmp.slot, &t));
    GemmArgs g = gemm_args();
    g.M = S; g.N = S; g.K = dk; g.alpha = scale; g.nb1 = B; g.nb2 = H; g.causal = causal ? 1 : 0;
    g.A = pq; qk_gemm_operand(q, &g.a_rs, &g.a_cs, &g.a_b1, &g.a_b2);
    g.B = pk; { i64 rs, cs; qk_gemm_operand(k, &rs, &cs, &g.b_b1, &g.b_b2); g.b_rs = cs; g.b_cs = rs; }
    g.C = t; g.c_rs = S; g.c_cs = 1; g.c_b1 = H * SS; g.c_b2 = SS;
    VB_TRY(launch_gemm(g));
    VB_TRY(launch_attn_softmax(t, pm, ms, causal, B, H, S, S, scale));
    pp = t;
  }
  void* dpv = nullptr;
  int rc = scratch_alloc((size_t)(B * H * SS) * sizeof(float), &dpv);
  float* pdp = (float*)dpv;
  // The probabilities of the fused forward kernel come with the output behind them: then dP, the softmax backward and dQ are one
  // kernel, which also leaves dS (scaled) in `pdp` for the dK product below.
  bool fused_dq = false;
  if (rc == VB_OK && probs && (causal || !mask) && attn_fused_enabled() && (ld & 3) == 0 && ((uintptr_t)pdq & 15) == 0) {
    const AttnOperand oq{pq, q->strides[0], q->strides[1], q->strides[2], q->strides[3]};
    const AttnOperand ok{pk, k->strides[0], k->strides[1], k->strides[2], k->strides[3]};
    const AttnOperand ov{pv, v->strides[0], v->strides[1], v->strides[2], v->strides[3]};
    const AttnOperand og{pg, gout->strides[0], gout->strides[1], gout->strides[2], gout->strides[3]};
    float* base; i64 cap = 0;
    if (attn_fused_supported(oq, ok, ov, B, H, S, dk) && attn_fused_operand_ok(og, B, H) && probs->offset == 0 &&
        slot_ptr(probs->slot, &base, &cap) == VB_OK && cap >= B * H * S * (S + dk)) {
      rc = launch_attn_bwd_dq_fused(ok, ov, og, pp, pdp, pdq, ld, S * ld, B, H, S, causal, scale);
      fused_dq = true;
    }
  }
  if (rc == VB_OK) {   // dV = P^T . dO
    GemmArgs g = gemm_args();
    g.M = S; g.N = dk; g.K = S; g.nb1 = B; g.nb2 = H; g.causal = causal ? 3 : 0;
    g.A = pp; g.a_rs = 1; g.a_cs = S; g.a_b1 = H * SS; g.a_b2 = SS;
    g.B = pg; qk_gemm_operand(gout, &g.b_rs, &g.b_cs, &g.b_b1, &g.b_b2);
    g.C = pdv; g.c_rs = ld; g.c_cs = 1; g.c_b1 = S * ld; g.c_b2 = dk;
    rc = launch_gemm(g);
  }
  if (rc == VB_OK && !fused_dq) {   // dP = dO . V^T
    GemmArgs g = gemm_args();
    g.M = S; g.N = S; g.K = dk; g.nb1 = B; g.nb2 = H; g.causal = causal ? 1 : 0;
    g.A = pg; qk_gemm_operand(gout, &g.a_rs, &g.a_cs, &g.a_b1, &g.a_b2);
    g.B = pv; { i64 rs, cs; qk_gemm_operand(v, &rs, &cs, &g.b_b1, &g.b_b2); g.b_rs = cs; g.b_cs = rs; }
    g.C = pdp; g.c_rs = S; g.c_cs = 1; g.c_b1 = H * SS; g.c_b2 = SS;
    rc = launch_gemm(g);
  }
  if (rc == VB_OK && !fused_dq) rc = launch_attn_softmax_backward(pp, pdp, B * H * S, S, scale, causal, S);   // dS * scale, in place
  if (rc == VB_OK && !fused_dq) {   // dQ = dS . K
    GemmArgs g = gemm_args();
    g.M = S; g.N = dk; g.K = S; g.nb1 = B; g.nb2 = H; g.causal = causal ? 2 : 0;
    g.A = pdp; g.a_rs = S; g.a_cs = 1; g.a_b1 = H * SS; g.a_b2 = SS;
    g.B = pk; qk_gemm_operand(k, &g.b_rs, &g.b_cs, &g.b_b1, &g.b_b2);
    g.C = pdq; g.c_rs = ld; g.c_cs = 1; g.c_b1 = S * ld; g.c_b2 = dk;
    rc = launch_gemm(g);
  }
  if (rc == VB_OK) {   // dK = dS^T . Q
    GemmArgs g = gemm_args();
    g.M = S; g.N = dk; g.K = S; g.nb1 = B; g.nb2 = H; g.causal = causal ? 3 : 0;
    g.A = pdp; g.a_rs = 1; g.a_cs = S; g.a_b1 = H * SS; g.a_b2 = SS;
    g.B = pq; qk_gemm_operand(q, &g.b_rs, &g.b_cs, &g.b_b1, &g.b_b2);
    g.C = pdk; g.c_rs = ld; g.c_cs = 1; g.c_b1 = S * ld; g.c_b2 = dk;
    rc = launch_gemm(g);
  }
  if (dpv) scratch_free(dpv);
  if (ptmp.slot) slot_release(ptmp.slot, nullptr);
  return rc;
}
int vb_fused_attention_backward(const vb_tensor* q, const vb_tensor* k, const vb_tensor* v, const vb_tensor* mask,
                                const vb_tensor* gout, const vb_tensor* probs, vb_tensor* dq, vb_tensor* dk_, vb_tensor* dv) {
  VB_CHECK(q->rank == 4 && same_shape(*q, *k) && same_shape(*q, *v) && same_shape(*q, *gout), "fused_attention_backward expects [B,H,S,dk] tensors");
  i64 B = q->dims[0], H = q->dims[1], S = q->dims[2], dk = q->dims[3];
  VB_TRY(new_output_bshd(dq, B, H, S, dk)); VB_TRY(new_output_bshd(dk_, B, H, S, dk)); VB_TRY(new_output_bshd(dv, B, H, S, dk));
  if (numel(*q) == 0) return VB_OK;
  float *pdq, *pdk, *pdv;
  VB_TRY(slot_ptr(dq->slot, &pdq)); VB_TRY(slot_ptr(dk_->slot, &pdk)); VB_TRY(slot_ptr(dv->slot, &pdv));
  return attention_backward_core(q, k, v, mask, gout, probs, pdq, pdk, pdv, H * dk);
}

// Attention over a packed projection: qkv is a contiguous [B, S, 3*D] tensor whose column blocks [0,D), [D,2D), [2D,3D) are
// q, k and v with heads side by side (what one Linear with the three weight matrices stacked produces).  The result is
// the [B, S, D] context; the backward returns one [B, S, 3*D] gradient with the same column blocks, written by the
// products themselves.
static int packed_views(const vb_tensor* qkv, int n_head, vb_tensor* q, vb_tensor* k, vb_tensor* v) {
  VB_CHECK(qkv->rank == 3 && is_contiguous(*qkv) && qkv->dims[2] % 3 == 0, "packed qkv must be a contiguous [B, S, 3*D] tensor");
  i64 B = qkv->dims[0], S = qkv->dims[1], D = qkv->dims[2] / 3;
  VB_CHECK(n_head > 0 && D % n_head == 0, "D must be divisible by the number of heads");
  i64 dk = D / n_head;
  vb_tensor t = *qkv;
  t.rank = 4; t.dims[0] = B; t.dims[1] = n_head; t.dims[2] = S; t.dims[3] = dk;
  t.strides[0] = S * 3 * D; t.strides[1] = dk; t.strides[2] = 3 * D; t.strides[3] = 1;
  *q = t; *k = t; *v = t;
  k->offset += D; v->offset += 2 * D;
  return VB_OK;
}
int vb_fused_attention_packed(const vb_tensor* qkv, int n_head, const vb_tensor* mask, vb_tensor* out, vb_tensor* probs) {
  vb_tensor q, k, v;
  VB_TRY(packed_views(qkv, n_head, &q, &k, &v));
  VB_TRY(vb_fused_attention(&q, &k, &v, mask, out, probs));
  // the [B,H,S,dk] view of the [B,S,H,dk] buffer, seen as [B,S,D]
  i64 B = qkv->dims[0], S = qkv->dims[1], D = qkv->dims[2] / 3;
  out->rank = 3; out->dims[0] = B; out->dims[1] = S; out->dims[2] = D;
  out->strides[0] = S * D; out->strides[1] = D; out->strides[2] = 1;
  return VB_OK;
}
int vb_fused_attention_packed_backward(const vb_tensor* qkv, int n_head, const vb_tensor* mask, const vb_tensor* gout,
                                       const vb_tensor* probs, vb_tensor* dqkv) {
  vb_tensor q, k, v;
  VB_TRY(packed_views(qkv, n_head, &q, &k, &v));
  i64 B = qkv->dims[0], S = qkv->dims[1], D = qkv->dims[2] / 3, dk = D / n_head;
  VB_CHECK(gout->rank == 3 && gout->dims[0] == B && gout->dims[1] == S && gout->dims[2] == D, "grad_out must be [B, S, D]");
  Temp hg; const float* pg;
  VB_TRY(contiguous_ptr(gout, &pg, hg));
  vb_tensor g4 = *gout;                      // [B,S,D] rows seen as [B,H,S,dk]
  vb_tensor gc; gc.slot = 0;
  if (!is_contiguous(*gout)) { VB_TRY(vb_contiguous(gout, &gc)); g4 = gc; }
  g4.rank = 4; g4.dims[0] = B; g4.dims[1] = n_head; g4.dims[2] = S; g4.dims[3] = dk;
  g4.strides[0] = S * D; g4.strides[1] = dk; g4.strides[2] = D; g4.strides[3] = 1;
  int rc = new_output(dqkv, 3, qkv->dims);
  float* pd = nullptr;
  if (rc == VB_OK && numel(*qkv) > 0) rc = slot_ptr(dqkv->slot, &pd);
  if (rc == VB_OK && numel(*qkv) > 0) rc = attention_backward_core(&q, &k, &v, mask, &g4, probs, pd, pd + D, pd + 2 * D, 3 * D);
  if (gc.slot) slot_release(gc.slot, nullptr);
  return rc;
}

// ---- host-side autograd helpers moved to the device --------------------------------------------
int vb_reduce_to(const vb_tensor* grad, const int64_t* tdims, int trank, vb_tensor* out) {
  VB_CHECK(grad->rank >= trank, "Grad rank must be >= target rank");
  bool same = grad->rank == trank;
  for (int i = 0; same && i < trank; ++i) same = grad->dims[i] == tdims[i];
  Temp hg; const float* pg;
  VB_TRY(contiguous_ptr(grad, &pg, hg));
  VB_TRY(new_output(out, trank, tdims, true));
  i64 on = numel(*out), gn = numel(*grad);
  if (on == 0 || gn == 0) return VB_OK;
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  if (same) { VB_CUDA(cudaMemcpyAsync(po, pg, (size_t)gn * sizeof(float), cudaMemcpyDeviceToDevice, ctx().stream)); return VB_OK; }
  int lead = grad->rank - trank;
  // leading dims reduced entirely, trailing dims kept as they are -> column sum of [rows, cols]
  int split = trank;          // first target dim (from the left) that equals the gradient's
  for (int d = trank - 1; d >= 0; --d) { if (tdims[d] == grad->dims[lead + d] ) split = d; else break; }
  bool prefix_reduced = true;
  for (int d = 0; d < split; ++d) if (tdims[d] != 1) prefix_reduced = false;
  if (prefix_reduced) {
    i64 cols = 1; for (int d = split; d < trank; ++d) cols *= tdims[d];
    return launch_colsum(pg, po, gn / cols, cols, false);
  }
  Strided kept{}, red{};
  i64 gs[VB_MAX_RANK]; { i64 s = 1; for (int i = grad->rank - 1; i >= 0; --i) { gs[i] = s; s *= grad->dims[i]; } }
  i64 red_count = 1;
  for (int i = 0; i < grad->rank; ++i) {
    int td = i - lead;
    bool is_kept = td >= 0 && tdims[td] != 1;
    if (is_kept) { VB_CHECK(tdims[td] == grad->dims[i], "target shape does not broadcast to the gradient"); kept.dims[kept.rank] = grad->dims[i]; kept.sa[kept.rank++] = gs[i]; }
    else { red.dims[red.rank] = grad->dims[i]; red.sa[red.rank++] = gs[i]; red_count *= grad->dims[i]; }
  }
  return launch_reduce_general(pg, po, on, kept, red, red_count);
}

int vb_accumulate(const vb_tensor* dst, const vb_tensor* src) {
  slot_touch(dst->slot);
  VB_CHECK(is_contiguous(*dst), "accumulate destination must be contiguous");
  VB_CHECK(numel(*dst) == numel(*src), "accumulate sizes differ");
  float* pd; VB_TRY(tensor_ptr(dst, &pd));
  Temp hs; const float* ps; VB_TRY(contiguous_ptr(src, &ps, hs));
  return launch_axpy(pd, ps, numel(*dst));
}
int vb_copy(const vb_tensor* dst, const vb_tensor* src) {
  slot_touch(dst->slot);
  VB_CHECK(is_contiguous(*dst), "copy destination must be contiguous");
  VB_CHECK(numel(*dst) == numel(*src), "copy sizes differ");
  float *pd, *ps; VB_TRY(tensor_ptr(dst, &pd)); VB_TRY(tensor_ptr(src, &ps));
  i64 n = numel(*dst);
  if (n == 0) return VB_OK;
  if (is_contiguous(*src)) { VB_CUDA(cudaMemcpyAsync(pd, ps, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, ctx().stream)); return VB_OK; }
  Strided s{}; s.rank = src->rank;
  for (int i = 0; i < src->rank; ++i) { s.dims[i] = src->dims[i]; s.sa[i] = src->strides[i]; }
  return launch_strided_copy(ps, pd, n, s);
}
int vb_scale(const vb_tensor* x, float alpha, vb_tensor* out) {
  Temp hx; const float* px; VB_TRY(contiguous_ptr(x, &px, hx));
  VB_TRY(new_output(out, x->rank, x->dims));
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  return launch_scale(px, alpha, po, numel(*x));
}
int vb_contiguous(const vb_tensor* x, vb_tensor* out) {
  VB_TRY(new_output(out, x->rank, x->dims));
  return vb_copy(out, x);
}
int vb_fill(const vb_tensor* dst, float value) {
  slot_touch(dst->slot);
  VB_CHECK(is_contiguous(*dst), "fill destination must be contiguous");
  float* pd; VB_TRY(tensor_ptr(dst, &pd));
  return launch_fill(pd, value, numel(*dst));
}

// ---- fused linear layer ------------------------------------------------------------------------
// TF32 remainders ("lo plane") of a Linear weight, kept beside the weight while its contents stand: the tensor-core GEMM then
// loads them instead of recomputing them in every tile of the forward product and of the input-gradient product.  Keyed by the
// weight's slot; valid while the slot's serial is unchanged (every call of this library that writes into an existing slot --
// vb_write, vb_copy, vb_fill, vb_accumulate, the optimizer steps, vb_clip_grad_norm, vb_dp_allreduce, vb_cross_entropy_fused,
// vb_linear_backward_into -- advances it).  One plane covers the whole slot, so
// parameters that are views of one block share it.  Returns null where the plane does not pay or cannot be had.
namespace {
// Column sums of a [rows, cols] gradient, left by the kernel that produced it (an activation's backward, LayerNorm backward):
// the bias gradient of the Linear layer whose output gradient that tensor is.  Keyed by the tensor's slot, valid for exactly
// the view that was summed and while the slot's serial is unchanged -- the same rule as for the lo planes below.
struct ColSums { vb_slot sums = 0; uint64_t serial = 0; i64 offset = 0, rows = 0, cols = 0; };
std::unordered_map<vb_slot, ColSums>& col_sums() { static auto* m = new std::unordered_map<vb_slot, ColSums>(); return *m; }
bool col_sums_enabled() {
  static const bool on = [] { const char* e = getenv("VB200_COLSUM_REUSE"); return !(e && e[0] == '0'); }();
  return on;
}
// `sums` (a slot of its own holding cols floats) now describes the contiguous view t = [rows, cols] as it stands
void col_sums_adopt(const vb_tensor* t, i64 rows, i64 cols, vb_slot sums) {
  auto& tab = col_sums();
  if (tab.size() > 64) {        // forget sums of slots that have been handed out again or rewritten since
    for (auto it = tab.begin(); it != tab.end();) {
      if (slot_serial(it->first) != it->second.serial) { slot_release(it->second.sums, nullptr); it = tab.erase(it); } else ++it;
    }
  }
  ColSums& e = tab[t->slot];
  if (e.sums) slot_release(e.sums, nullptr);
  e.sums = sums; e.serial = slot_serial(t->slot); e.offset = t->offset; e.rows = rows; e.cols = cols;
}
const float* col_sums_of(const vb_tensor* t, i64 rows, i64 cols) {
  if (!col_sums_enabled()) return nullptr;
  auto& tab = col_sums();
  auto it = tab.find(t->slot);
  if (it == tab.end()) return nullptr;
  const ColSums& e = it->second;
  if (e.sums == 0 || e.serial != slot_serial(t->slot) || e.offset != t->offset || e.rows != rows || e.cols != cols || !is_contiguous(*t)) return nullptr;
  float* p;
  return slot_ptr(e.sums, &p) == VB_OK ? p : nullptr;
}
struct LoPlane { vb_slot lo = 0; uint64_t serial = 0; i64 numel = 0; };
std::unordered_map<vb_slot, LoPlane>& lo_planes() { static auto* m = new std::unordered_map<vb_slot, LoPlane>(); return *m; }
bool activation_lo_enabled() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("VB200_ACT_LO"); const char* w = getenv("VB200_WEIGHT_LO"); on = ((e && e[0] == '0') || (w && w[0] == '0')) ? 0 : 1; }
  return on != 0;
}
// the plane `lo` (a slot of its own) now belongs to `slot`, whose present contents it matches
void lo_plane_adopt(vb_slot slot, vb_slot lo, i64 n) {
  LoPlane& e = lo_planes()[slot];
  if (e.lo) slot_release(e.lo, nullptr);
  e.lo = lo; e.numel = n; e.serial = slot_serial(slot);
}
// the plane of an activation, if its producer left one and the contents have not changed since (never made here)
const float* existing_lo_plane(const vb_tensor* t, const float* pt) {
  auto& tab = lo_planes();
  auto it = tab.find(t->slot);
  if (it == tab.end() || it->second.lo == 0 || it->second.serial != slot_serial(t->slot)) return nullptr;
  float *base, *lo; i64 n;
  if (slot_ptr(t->slot, &base, &n) != VB_OK || n != it->second.numel || slot_ptr(it->second.lo, &lo) != VB_OK) return nullptr;
  return lo + (pt - base);
}
const float* weight_lo_plane(const vb_tensor* w, const float* pw) {
  static int on = -1;
  if (on < 0) { const char* e = getenv("VB200_WEIGHT_LO"); on = (e && e[0] == '0') ? 0 : 1; }
  if (!on) return nullptr;
  float* base; i64 n;
  if (slot_ptr(w->slot, &base, &n) != VB_OK || n < (i64)1 << 18) return nullptr;       // small weights: their products are not tensor-core bound
  auto& tab = lo_planes();
  if (tab.size() > 512) {        // forget planes of slots that have been handed out again since
    for (auto it = tab.begin(); it != tab.end();) {
      if (slot_serial(it->first) != it->second.serial) { slot_release(it->second.lo, nullptr); it = tab.erase(it); } else ++it;
    }
  }
  LoPlane& e = tab[w->slot];
  const uint64_t serial = slot_serial(w->slot);
  if (e.lo == 0 || e.numel != n) {
    if (e.lo) { slot_release(e.lo, nullptr); e.lo = 0; }
    if (slot_alloc(n, false, &e.lo) != VB_OK) { tab.erase(w->slot); return nullptr; }
    e.numel = n; e.serial = 0;
  }
  float* lo;
  if (slot_ptr(e.lo, &lo) != VB_OK) return nullptr;
  if (e.serial != serial) {
    if (launch_tf32_lo(base, lo, n) != VB_OK) return nullptr;
    e.serial = serial;
  }
  return lo + (pw - base);
}
}  // namespace
extern "C++" {
namespace vb {
void lo_planes_forget_all() { lo_planes().clear(); col_sums().clear(); }
void lo_plane_on_release(vb_slot slot) {
  auto& cs = col_sums();
  if (!cs.empty()) {
    auto ic = cs.find(slot);
    if (ic != cs.end()) { vb_slot sums = ic->second.sums; cs.erase(ic); if (sums) slot_release(sums, nullptr); }
  }
  auto& tab = lo_planes();
  if (tab.empty()) return;
  auto it = tab.find(slot);
  if (it == tab.end()) return;
  vb_slot lo = it->second.lo;
  tab.erase(it);
  if (lo) slot_release(lo, nullptr);
}
float* lo_plane_base_for(vb_slot weight_slot, float** weight_base) {
  auto& tab = lo_planes();
  auto it = tab.find(weight_slot);
  if (it == tab.end() || it->second.lo == 0) return nullptr;
  float *base, *lo; i64 n;
  if (slot_ptr(weight_slot, &base, &n) != VB_OK || n != it->second.numel || slot_ptr(it->second.lo, &lo) != VB_OK) return nullptr;
  if (weight_base) *weight_base = base;
  return lo;
}
bool lo_plane_is_current(vb_slot weight_slot) {
  auto it = lo_planes().find(weight_slot);
  return it != lo_planes().end() && it->second.lo != 0 && it->second.serial == slot_serial(weight_slot);
}
void lo_plane_mark_current(vb_slot weight_slot) {
  auto it = lo_planes().find(weight_slot);
  if (it != lo_planes().end()) it->second.serial = slot_serial(weight_slot);
}
}  // namespace vb
}  // extern "C++"

static int linear_forward_impl(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* bias, vb_tensor* out, vb_tensor* act);
int vb_linear(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* bias, vb_tensor* out) {
  return linear_forward_impl(x, weight, bias, out, nullptr);
}
int vb_linear_gelu(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* bias, vb_tensor* pre, vb_tensor* act) {
  VB_CHECK(pre && act, "linear_gelu needs both outputs");
  return linear_forward_impl(x, weight, bias, pre, act);
}
// act (optional): GELU(out), formed in the GEMM's epilogue from the values it is storing anyway where the tensor-core kernel
// takes the product as whole tiles, else by the activation kernel
static int linear_forward_impl(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* bias, vb_tensor* out, vb_tensor* act) {
  VB_CHECK(weight->rank == 2 && x->rank >= 1, "linear expects weight [out, in]");
  VB_CHECK(x->dims[x->rank - 1] == weight->dims[1], "Incompatible dimensions for matmul");
  Temp hx, hb; const float* px; VB_TRY(contiguous_ptr(x, &px, hx));
  float* pw; VB_TRY(tensor_ptr(weight, &pw));
  const float* pb = nullptr;
  if (bias) { VB_CHECK(numel(*bias) == weight->dims[0], "bias must be [out]"); VB_TRY(contiguous_ptr(bias, &pb, hb)); }
  i64 od[VB_MAX_RANK];
  for (int i = 0; i < x->rank - 1; ++i) od[i] = x->dims[i];
  od[x->rank - 1] = weight->dims[0];
  VB_TRY(new_output(out, x->rank, od));
  if (act) VB_TRY(new_output(act, x->rank, od));
  if (numel(*out) == 0) return VB_OK;
  float* po; VB_TRY(slot_ptr(out->slot, &po));
  float* pa = nullptr; if (act) VB_TRY(slot_ptr(act->slot, &pa));
  i64 rows, in; VB_TRY(rows_of(x, &rows, &in));
  GemmArgs g = gemm_args();
  g.M = rows; g.N = weight->dims[0]; g.K = in;
  g.A = px; g.a_rs = in; g.a_cs = 1;
  g.B = pw; g.b_rs = weight->strides[1]; g.b_cs = weight->strides[0];   // W^T
  g.C = po; g.c_rs = g.N; g.c_cs = 1; g.bias = pb;
  if (rows >= 1024) g.B_lo = weight_lo_plane(weight, pw);
  if (g.B_lo && !hx.p) g.A_lo = existing_lo_plane(x, px);        // a normalised input brings its own remainders
  int fused = 0;
  g.act_out = pa; g.act_fused = &fused;
  VB_TRY(launch_gemm(g));
  if (act && !fused) VB_TRY(launch_unary(1, po, pa, numel(*out)));
  return VB_OK;
}
// gw_into / gb_into: existing contiguous tensors the weight and bias gradients are written into (a parameter's slice of
// the flat gradient arena) instead of fresh outputs.
static int linear_backward_impl(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* gout, vb_tensor* gx, vb_tensor* gw, vb_tensor* gb,
                                const vb_tensor* gw_into, const vb_tensor* gb_into) {
  VB_CHECK(weight->rank == 2 && x->rank >= 1 && gout->rank == x->rank, "linear_backward shape mismatch");
  i64 rows, in; VB_TRY(rows_of(x, &rows, &in));
  i64 outf = weight->dims[0];
  VB_CHECK(in == weight->dims[1] && gout->dims[gout->rank - 1] == outf && numel(*gout) == rows * outf, "linear_backward shape mismatch");
  if (gw_into) VB_CHECK(is_contiguous(*gw_into) && numel(*gw_into) == outf * in, "weight-gradient destination must be a contiguous [out, in] tensor");
  if (gb_into) VB_CHECK(is_contiguous(*gb_into) && numel(*gb_into) == outf, "bias-gradient destination must be a contiguous [out] tensor");
  Temp hx, hg; const float *px, *pg;
  VB_TRY(contiguous_ptr(x, &px, hx)); VB_TRY(contiguous_ptr(gout, &pg, hg));
  float* pw; VB_TRY(tensor_ptr(weight, &pw));
  if (gx) {   // gx = gy . W
    VB_TRY(new_output(gx, x->rank, x->dims));
    if (numel(*gx)) {
      float* p; VB_TRY(slot_ptr(gx->slot, &p));
      GemmArgs g = gemm_args();
      g.M = rows; g.N = in; g.K = outf;
      g.A = pg; g.a_rs = outf; g.a_cs = 1;
      g.B = pw; g.b_rs = weight->strides[0]; g.b_cs = weight->strides[1];
      g.C = p; g.c_rs = in; g.c_cs = 1;
      if (rows >= 1024) g.B_lo = weight_lo_plane(weight, pw);
      VB_TRY(launch_gemm(g));
    }
  }
  if (gw || gw_into) {   // gw[out, in] = gy^T . x
    float* p;
    if (gw_into) { VB_TRY(tensor_ptr(gw_into, &p)); slot_touch(gw_into->slot); }
    else { i64 wd[2] = {outf, in}; VB_TRY(new_output(gw, 2, wd)); VB_TRY(slot_ptr(gw->slot, &p)); }
    if (rows == 0) VB_TRY(launch_fill(p, 0.0f, outf * in));
    else {
      GemmArgs g = gemm_args();
      g.M = outf; g.N = in; g.K = rows;
      g.A = pg; g.a_rs = 1; g.a_cs = outf;
      g.B = px; g.b_rs = in; g.b_cs = 1;
      g.C = p; g.c_rs = in; g.c_cs = 1;
      if (!hx.p) g.B_lo = existing_lo_plane(x, px);        // x consumed in place and its producer left a lo plane
      VB_TRY(launch_gemm(g));
    }
  }
  if (gb || gb_into) {
    float* p;
    if (gb_into) { VB_TRY(tensor_ptr(gb_into, &p)); slot_touch(gb_into->slot); }
    else { VB_TRY(new_output(gb, 1, &outf, true)); VB_TRY(slot_ptr(gb->slot, &p)); }
    const float* known = (rows > 0 && !hg.p) ? col_sums_of(gout, rows, outf) : nullptr;      // its producer summed the columns already
    if (known) VB_CUDA(cudaMemcpyAsync(p, known, (size_t)outf * sizeof(float), cudaMemcpyDeviceToDevice, ctx().stream));
    else if (rows > 0) VB_TRY(launch_colsum(pg, p, rows, outf, false));
    else if (gb_into) VB_TRY(launch_fill(p, 0.0f, outf));
  }
  return VB_OK;
}
int vb_linear_backward(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* gout, vb_tensor* gx, vb_tensor* gw, vb_tensor* gb) {
  return linear_backward_impl(x, weight, gout, gx, gw, gb, nullptr, nullptr);
}
int vb_linear_backward_into(const vb_tensor* x, const vb_tensor* weight, const vb_tensor* gout, vb_tensor* gx,
                            const vb_tensor* gw_into, const vb_tensor* gb_into) {
  return linear_backward_impl(x, weight, gout, gx, nullptr, nullptr, gw_into, gb_into);
}

}  // extern "C"
