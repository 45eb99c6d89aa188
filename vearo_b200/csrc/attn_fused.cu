// Scaled-dot-product attention with the score matrix kept on the SM: Q.K^T, the softmax and P.V in one kernel (forward), and
// dP = dO.V^T, the softmax backward and dQ = dS.K in one kernel (backward).  FP32-accurate: every product is a 3xTF32 split
// product on the tcgen05 tensor cores, accumulators in tensor memory, operand tiles staged in shared memory by TMA (no
// multicast).  The probability / score-gradient operand of the second product of each kernel never touches shared memory: the
// row warps write it (split into its TF32 hi and lo parts) to tensor memory and the MMA reads its A operand from there.
//
// Semantics: crates/vearo-backend-cpu/src/lib.rs:2412-2471 (forward row: score = q.k * scale + mask, p = exp(score - max) *
// (1 / (sum + 1e-9)), out = sum p v) and :2480-2630 (backward: ds = p * (dp - sum_j dp_j p_j), dq = ds.k * scale, ...).
// Mask forms handled here: none, or the causal pattern (0 on and below the diagonal, <= -1e9 above it, for which every
// probability above the diagonal is exactly 0 in f32); any other additive mask takes the GEMM + row-kernel route of abi.cu.
// Head size 64.
//
// Forward, one CTA per 128 query rows of one (batch, head), 448 threads:
//   warp 0       TMA producer: Q once, then the K and V blocks (128 keys each)
//   warp 1       allocates tensor memory and issues every MMA from one thread
//   warps 2-5    converters: the TF32 remainders ("lo") of Q, K and V tiles, written beside the raw tiles (the raw f32 tile is
//                the hi operand: the tensor core reads it cut to TF32)
//   warps 6-13   row warps: thread = one query row x 64 of the block's 128 keys
//   pass 1: S = Q.K^T block by block, running row maximum and sum of exp (K double-buffered through the idle V region);
//   pass 2: S again, p = exp(s - max) / (sum + 1e-9) exactly as the reference forms it, P -> tensor memory (hi, lo) and -- when
//           the caller keeps the probabilities for the backward pass -- to global memory through staged TMA block stores, then
//           O += P.V.  No running rescale of O is ever needed, and the stored P is final.
// Backward (dQ part), one CTA per 128 query rows, same warp roles; dP is formed 128 keys at a time (one V tile), dS and dQ in
// 64-key halves (K double-buffered):
//   the dO rows go to tensor memory once (hi, lo: the A operand of dP = dO.V^T); per block the row warps take their P block
//   (asynchronous copies two blocks ahead), ds = p * (dp - delta) * scale with delta = dO.O (= sum_j dp_j p_j, the reference's
//   row term), dS -> tensor memory (hi, lo) and global memory (for the dK product), dQ += dS.K.
// dV = P^T.dO and dK = dS^T.Q are left to the batched GEMM kernel (triangular k ranges under the causal mask).
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises the device error word, lets its copies land,
// frees its tensor memory and returns.
#include "common.h"
#include "tc_util.cuh"
#include <cuda.h>
#include <cstring>

namespace vb {
namespace {
using namespace tc;

constexpr int kTile = 128 * 64 * 4;            // one 128 x 64 f32 operand tile: two 32-column chunks of 16 KB
constexpr int kChunk = 128 * 32 * 4;
constexpr int kFwdThreads = 32 * 14;
constexpr int kRowWarpsFwd = 8;

struct AttnFwdParams {
  int S, n_qtiles, causal, store_p;
  int H;
  float scale_l2e;          // 1/sqrt(dk) * log2(e): scores are kept in the base-2 domain, exp(x) = 2^(x log2 e)
  int* err;
};

// 2^x on the special-function unit (relative error about 2^-22; -inf gives 0).  With the argument formed by one FMA from the raw
// score, a probability comes out within about 1e-6 of exp(score - max) for |score - max| up to a few tens, two orders inside
// the parity bar, for two instructions instead of expf's twenty.
__device__ __forceinline__ float fast_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// barrier indices of the forward kernel
enum { B_QFULL = 0, B_QCONV, B_KFULL0, B_KFULL1, B_KCONV0, B_KCONV1, B_KFREE0, B_KFREE1, B_VFULL, B_VCONV, B_SFULL, B_SFREE, B_PREADY, B_PVDONE, B_COUNT };

__device__ __forceinline__ void stage_put(float4* stg, int lane, int j4, float4 x) { stg[lane * 8 + (j4 ^ (lane & 7))] = x; }

__device__ __forceinline__ void convert_tile(const uint8_t* raw, uint8_t* lo, int tid, int nthreads) {
  const float4* s = (const float4*)raw; float4* d = (float4*)lo;
  // 16 independent loads per thread in flight before the first store (the loop is latency-bound otherwise)
  float4 x[8];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = s[tid + (h * 8 + i) * nthreads];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 l;
      l.x = tf32_lo_of_raw(x[i].x); l.y = tf32_lo_of_raw(x[i].y); l.z = tf32_lo_of_raw(x[i].z); l.w = tf32_lo_of_raw(x[i].w);
      d[tid + (h * 8 + i) * nthreads] = l;
    }
  }
}
// MN-major descriptor of a [128 k rows x 32 floats] block sequence (SWIZZLE_128B with 32-byte base), `rows` k rows per 32-wide block
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr, int rows) { return make_desc_mn_sw128(addr, rows); }

__global__ void __launch_bounds__(kFwdThreads, 1)
k_attn_fwd(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
           const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_o, const __grid_constant__ CUtensorMap map_o2,
           AttnFwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* q_hi = smem; uint8_t* q_lo = smem + kTile;
  uint8_t* kbuf[2] = {smem + 2 * kTile, smem + 4 * kTile};     // [hi | lo] each; buffer 1 is the V region (pass 1 only)
  uint8_t* v_hi = smem + 4 * kTile; uint8_t* v_lo = smem + 5 * kTile;
  uint8_t* staging = smem + 6 * kTile;                          // 8 x 4 KB, one block per row warp
  uint64_t* bars = (uint64_t*)(staging + kRowWarpsFwd * 4096);
  uint32_t* tmem_slot = (uint32_t*)(bars + B_COUNT);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int qt = p.n_qtiles - 1 - (int)blockIdx.y;              // longest tiles first
  const int n_kv_all = (p.S + 127) / 128;
  const int n_kv = p.causal ? (qt + 1 < n_kv_all ? qt + 1 : n_kv_all) : n_kv_all;

  if (threadIdx.x == 0) {
    mbar_init(&bars[B_QFULL], 1); mbar_init(&bars[B_QCONV], 4);
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[B_KFULL0 + i], 1); mbar_init(&bars[B_KCONV0 + i], 4); mbar_init(&bars[B_KFREE0 + i], 1); }
    mbar_init(&bars[B_VFULL], 1); mbar_init(&bars[B_VCONV], 4);
    mbar_init(&bars[B_SFULL], 1); mbar_init(&bars[B_SFREE], kRowWarpsFwd);
    mbar_init(&bars[B_PREADY], kRowWarpsFwd); mbar_init(&bars[B_PVDONE], 2);      // (two lanes issue P.V, each commits its own MMAs)
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // (two accumulators for O, taking alternate k steps: consecutive MMAs then do not wait on each other's result; summed in the epilogue)
  const uint32_t t_s = tmem, t_phi = tmem + 128, t_plo = tmem + 256, t_o = tmem + 384, t_o2 = tmem + 448;

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      int kuse[2] = {0, 0};
      mbar_arrive_expect_tx(&bars[B_QFULL], kTile);
      tma_load_4d(q_hi, &map_q, &bars[B_QFULL], 0, qt * 128, h, b);
      tma_load_4d(q_hi + kChunk, &map_q, &bars[B_QFULL], 32, qt * 128, h, b);
      auto load_k = [&](int kb, int j) -> bool {
        if (kuse[kb] > 0 && !mbar_wait(&bars[B_KFREE0 + kb], (uint32_t)(kuse[kb] - 1) & 1, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars[B_KFULL0 + kb], kTile);
        tma_load_4d(kbuf[kb], &map_k, &bars[B_KFULL0 + kb], 0, j * 128, h, b);
        tma_load_4d(kbuf[kb] + kChunk, &map_k, &bars[B_KFULL0 + kb], 32, j * 128, h, b);
        ++kuse[kb];
        return true;
      };
      for (int j = 0; j < n_kv && ok; ++j) ok = load_k(j & 1, j);         // pass 1: K alternates between its own region and V's
      if (ok) ok = load_k(0, 0);                                           // pass 2: K(j + 1) goes out ahead of V(j), in the order the MMAs free them
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) { ok = load_k(0, j + 1); if (!ok) break; }
        // the V region was pass 1's second K buffer: its last reader must be done; later blocks wait for the previous P.V
        if (j == 0) { if (kuse[1] > 0) ok = mbar_wait(&bars[B_KFREE1], (uint32_t)(kuse[1] - 1) & 1, abort_flag); }
        else ok = mbar_wait(&bars[B_PVDONE], (uint32_t)(j - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[B_VFULL], kTile);
        tma_load_4d(v_hi, &map_v, &bars[B_VFULL], 0, j * 128, h, b);
        tma_load_4d(v_hi + kChunk, &map_v, &bars[B_VFULL], 32, j * 128, h, b);
      }
      if (*abort_flag) {      // give copies already issued a bounded time to land before the CTA exits
        for (int i = 0; i < B_COUNT; ++i) {
          if (i != B_QFULL && i != B_KFULL0 && i != B_KFULL1 && i != B_VFULL) continue;
          uint32_t addr = smem_u32(&bars[i]), done = 0;
          for (uint32_t n = 0; n < (1u << 14) && !done; ++n)
            asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}" : "=r"(done) : "r"(addr), "r"(0u) : "memory");
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ------------------------------------------------------------------------------------------------------
    // Issuing one MMA costs the issuing thread about as long as a 128 x 128 x 8 product takes to execute, so the narrower P.V
    // products (N = 64) would leave the tensor pipe half idle behind one thread: two lanes issue them, each the k steps of
    // one parity into its own accumulator.  Lane 0 alone issues Q.K^T.
    if (lane < 2) {
      const uint32_t idesc_qk = make_idesc(128, 128, 0, 0), idesc_pv = make_idesc(128, 64, 0, 1);
      const uint64_t dq_hi = make_desc_k(smem_u32(q_hi), 32), dq_lo = make_desc_k(smem_u32(q_lo), 32);
      const uint64_t dk_hi[2] = {make_desc_k(smem_u32(kbuf[0]), 32), make_desc_k(smem_u32(kbuf[1]), 32)};
      const uint64_t dk_lo[2] = {make_desc_k(smem_u32(kbuf[0] + kTile), 32), make_desc_k(smem_u32(kbuf[1] + kTile), 32)};
      const uint64_t dv_hi = desc_mn(smem_u32(v_hi), 128), dv_lo = desc_mn(smem_u32(v_lo), 128);
      bool ok = mbar_wait(&bars[B_QCONV], 0, abort_flag);
      int muse[2] = {0, 0}, g = 0;                  // uses of each K buffer; S tiles produced so far
      auto issue_qk = [&](int kb) -> bool {
        if (!mbar_wait(&bars[B_KCONV0 + kb], (uint32_t)muse[kb] & 1, abort_flag)) return false;
        if (g > 0 && !mbar_wait(&bars[B_SFREE], (uint32_t)(g - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        uint32_t acc = 0;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const uint64_t off = (uint64_t)((c * kChunk + s * 32) >> 4);
            mma_tf32(t_s, dq_lo + off, dk_hi[kb] + off, idesc_qk, acc);
            mma_tf32(t_s, dq_hi + off, dk_lo[kb] + off, idesc_qk, 1u);
            mma_tf32(t_s, dq_hi + off, dk_hi[kb] + off, idesc_qk, 1u);
            acc = 1u;
          }
        mma_commit(&bars[B_KFREE0 + kb]);
        mma_commit(&bars[B_SFULL]);
        ++muse[kb]; ++g;
        return true;
      };
      if (lane == 0) {
        for (int j = 0; j < n_kv && ok; ++j) ok = issue_qk(j & 1);        // pass 1: scores only
        if (ok) ok = issue_qk(0);                                          // pass 2, block 0
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (lane == 0 && j + 1 < n_kv) { ok = issue_qk(0); if (!ok) break; }   // the next block's scores run under this block's softmax
        ok = mbar_wait(&bars[B_PREADY], (uint32_t)j & 1, abort_flag);
        ok = ok && mbar_wait(&bars[B_VCONV], (uint32_t)j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = lane ? t_o2 : t_o;
#pragma unroll
        for (int t2 = 0; t2 < 8; ++t2) {
          const int t = 2 * t2 + lane;
          const uint64_t off = (uint64_t)((t * 1024) >> 4);
          mma_tf32_ta(acc, t_plo + 8 * t, dv_hi + off, idesc_pv, (j > 0 || t2 > 0) ? 1u : 0u);
          mma_tf32_ta(acc, t_phi + 8 * t, dv_lo + off, idesc_pv, 1u);
          mma_tf32_ta(acc, t_phi + 8 * t, dv_hi + off, idesc_pv, 1u);
        }
        mma_commit(&bars[B_PVDONE]);
      }
    }
  } else if (warp < 6) {
    // ---- converters ------------------------------------------------------------------------------------------------------
    const int tid = threadIdx.x - 64;
    bool ok = mbar_wait(&bars[B_QFULL], 0, abort_flag);
    if (ok) {
      convert_tile(q_hi, q_lo, tid, 128);
      fence_async_smem(); __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_QCONV]);
    }
    int cuse[2] = {0, 0};
    auto conv_k = [&](int kb) -> bool {
      if (!mbar_wait(&bars[B_KFULL0 + kb], (uint32_t)cuse[kb] & 1, abort_flag)) return false;
      convert_tile(kbuf[kb], kbuf[kb] + kTile, tid, 128);
      fence_async_smem(); __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_KCONV0 + kb]);
      ++cuse[kb];
      return true;
    };
    for (int j = 0; j < n_kv && ok; ++j) ok = conv_k(j & 1);
    if (ok) ok = conv_k(0);
    for (int j = 0; j < n_kv && ok; ++j) {            // the producer's order: K(j + 1), then V(j)
      if (j + 1 < n_kv) { ok = conv_k(0); if (!ok) break; }
      ok = mbar_wait(&bars[B_VFULL], (uint32_t)j & 1, abort_flag);
      if (!ok) break;
      convert_tile(v_hi, v_lo, tid, 128);
      fence_async_smem(); __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_VCONV]);
    }
  } else {
    // ---- row warps -------------------------------------------------------------------------------------------------------
    const int w = warp - 6, quarter = warp & 3, half = w >> 2;
    const int row = quarter * 32 + lane;                       // row of the tile held by this thread
    const int grow = qt * 128 + row;                           // query index
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    float4* stg = (float4*)(staging + w * 4096);
    float* xm = (float*)staging; float* xl = xm + 256;         // pass-1 statistics of the two column halves (staging is idle then)
    bool ok = true;
    int g = 0;
    float m = -INFINITY, l = 0.0f;
    uint32_t v[64];
    // scores of this thread for block j: scaled (base-2 domain), with masked columns at -inf
    auto load_scores = [&](int j) -> bool {
      if (!mbar_wait(&bars[B_SFULL], (uint32_t)g & 1, abort_flag)) return false;
      tc_fence_after();
      tmem_ld32(t_s + lane_off + (uint32_t)(half * 64), v);
      tmem_ld32(t_s + lane_off + (uint32_t)(half * 64 + 32), v + 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_SFREE]);
      ++g;
      const int col0 = j * 128 + half * 64;
      const int lim = p.causal ? (grow < p.S - 1 ? grow : p.S - 1) : p.S - 1;      // last live column
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float x = __uint_as_float(v[c]) * p.scale_l2e;
        v[c] = __float_as_uint(col0 + c <= lim ? x : -INFINITY);
      }
      return true;
    };
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = load_scores(j);
      if (!ok) break;
      float bm = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) bm = fmaxf(bm, __uint_as_float(v[c]));
      const float mn = fmaxf(m, bm);
      if (mn > -INFINITY) {
        float s = 0.0f;
#pragma unroll
        for (int c = 0; c < 64; ++c) s += fast_exp2(__uint_as_float(v[c]) - mn);
        l = l * fast_exp2(m - mn) + s;
        m = mn;
      }
    }
    // the two halves of a row agree on its maximum and sum
    xm[half * 128 + row] = m; xl[half * 128 + row] = l;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    {
      const float mo = xm[(1 - half) * 128 + row], lo_ = xl[(1 - half) * 128 + row];
      const float M = fmaxf(m, mo);
      float L = 0.0f;
      if (m > -INFINITY) L += l * fast_exp2(m - M);
      if (mo > -INFINITY) L += lo_ * fast_exp2(mo - M);
      m = M; l = 1.0f / (L + 1e-9f);
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");            // (the staging area is about to carry stores)
    const float rmax = m, inv = l;
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = load_scores(j);
      if (!ok) break;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        v[c] = __float_as_uint(fast_exp2(__uint_as_float(v[c]) - rmax) * inv);      // (masked columns: 2^-inf = 0)
      }
      if (j > 0) { ok = mbar_wait(&bars[B_PVDONE], (uint32_t)(j - 1) & 1, abort_flag); if (!ok) break; tc_fence_after(); }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) t[e] = v[c * 32 + e] & 0xffffe000u;
        tmem_st32(t_phi + lane_off + (uint32_t)(half * 64 + c * 32), t);
#pragma unroll
        for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(tf32_lo_of_raw(__uint_as_float(v[c * 32 + e])));
        tmem_st32(t_plo + lane_off + (uint32_t)(half * 64 + c * 32), t);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_PREADY]);
      if (p.store_p) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4)
            stage_put(stg, lane, j4, make_float4(__uint_as_float(v[c * 32 + 4 * j4]), __uint_as_float(v[c * 32 + 4 * j4 + 1]),
                                                 __uint_as_float(v[c * 32 + 4 * j4 + 2]), __uint_as_float(v[c * 32 + 4 * j4 + 3])));
          fence_async_smem();
          __syncwarp();
          if (lane == 0) tma_store_3d(&map_p, stg, j * 128 + half * 64 + c * 32, qt * 128 + quarter * 32, bh);
        }
      }
    }
    // ---- epilogue: O (already normalised, P was) -> staged block -> global ----
    if (ok) ok = mbar_wait(&bars[B_PVDONE], (uint32_t)(n_kv - 1) & 1, abort_flag);
    if (ok) {
      tc_fence_after();
      tmem_ld32(t_o + lane_off + (uint32_t)(half * 32), v);
      tmem_ld32(t_o2 + lane_off + (uint32_t)(half * 32), v + 32);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(v[32 + c]));
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4)
        stage_put(stg, lane, j4, make_float4(__uint_as_float(v[4 * j4]), __uint_as_float(v[4 * j4 + 1]), __uint_as_float(v[4 * j4 + 2]), __uint_as_float(v[4 * j4 + 3])));
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_block(&map_o, stg, half * 32, qt * 128 + quarter * 32, h, b);
        if (p.store_p) tma_store_block(&map_o2, stg, half * 32, qt * 128 + quarter * 32, h, b);     // the backward's copy, behind the probabilities
      }
    }
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.err, ERRBIT_WAIT_TIMEOUT);
}


// ---- backward: dP = dO.V^T, dS = P (dP - delta) scale, dQ += dS.K ------------------------------------------------------------
struct AttnBwdParams {
  int S, n_qtiles, causal, H;
  float scale;
  const float* P;            // [BH, S, S] probabilities
  const float* O;            // [BH, S, 64] attention output (contiguous)
  const float* dO; i64 do_sb, do_sh, do_ss;     // [B,H,S,64] view of the output gradient
  int* err;
};
enum { D_VFULL = 0, D_VCONV, D_VFREE, D_KFULL0, D_KFULL1, D_KCONV0, D_KCONV1, D_KFREE0, D_KFREE1,
       D_DPFULL, D_DPFREE, D_DSREADY, D_DQDONE, D_DOREADY, D_COUNT };
constexpr int kHalfTile = 64 * 64 * 4;          // a 64-key operand block: 16 KB (two 32-column chunks of 8 KB)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;          // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

__global__ void __launch_bounds__(kFwdThreads, 1)
k_attn_bwd_dq(const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_ds,
              const __grid_constant__ CUtensorMap map_dq, AttnBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // V: one 128-key K-major tile [hi | lo] (the B operand of dP = dO.V^T, N = 128: an MMA instruction costs its issuer about the
  // same whether it is 64 or 128 wide, so dP is formed 128 keys at a time); K: 64-key MN-major blocks, two stages [hi | lo] (the B
  // operand of dQ += dS.K, whose width is the head size)
  uint8_t* v_hi = smem; uint8_t* v_lo = smem + kTile;
  uint8_t* kbuf[2] = {smem + 4 * kHalfTile, smem + 6 * kHalfTile};
  uint8_t* staging = smem + 8 * kHalfTile;                                  // 8 row warps x 3 blocks of 4 KB
  uint64_t* bars = (uint64_t*)(staging + kRowWarpsFwd * 3 * 4096);
  float* xd = (float*)(bars + D_COUNT);                                     // delta halves [2][128]
  uint32_t* tmem_slot = (uint32_t*)(xd + 256);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int qt = p.n_qtiles - 1 - (int)blockIdx.y;
  const int n_all = (p.S + 127) / 128;
  const int n_big = p.causal ? (qt + 1 < n_all ? qt + 1 : n_all) : n_all;      // 128-key blocks
  const int n_kv = 2 * n_big;                                                   // 64-key sub-blocks (one past the end of S reads zeros)

  if (threadIdx.x == 0) {
    mbar_init(&bars[D_VFULL], 1); mbar_init(&bars[D_VCONV], 4); mbar_init(&bars[D_VFREE], 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[D_KFULL0 + i], 1); mbar_init(&bars[D_KCONV0 + i], 4); mbar_init(&bars[D_KFREE0 + i], 2); }
    mbar_init(&bars[D_DPFULL], 1); mbar_init(&bars[D_DPFREE], kRowWarpsFwd); mbar_init(&bars[D_DSREADY], kRowWarpsFwd);
    mbar_init(&bars[D_DQDONE], 2); mbar_init(&bars[D_DOREADY], kRowWarpsFwd);          // (two lanes issue the MMAs, each commits its own)
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // (dQ has two accumulators taking alternate k steps, one per issuing lane)
  const uint32_t t_dohi = tmem, t_dolo = tmem + 64, t_dp = tmem + 128, t_dshi = tmem + 256, t_dslo = tmem + 320, t_dq = tmem + 384, t_dq2 = tmem + 448;

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1, u = j >> 1;
        if ((j & 1) == 0) {          // the 128-key V tile of block J = j / 2
          if (u > 0) ok = mbar_wait(&bars[D_VFREE], (uint32_t)(u - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars[D_VFULL], kTile);
          tma_load_4d(v_hi, &map_v, &bars[D_VFULL], 0, u * 128, h, b);
          tma_load_4d(v_hi + kChunk, &map_v, &bars[D_VFULL], 32, u * 128, h, b);
        }
        if (u > 0) ok = mbar_wait(&bars[D_KFREE0 + st], (uint32_t)(u - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[D_KFULL0 + st], kHalfTile);
        tma_load_4d(kbuf[st], &map_k, &bars[D_KFULL0 + st], 0, j * 64, h, b);
        tma_load_4d(kbuf[st] + kHalfTile / 2, &map_k, &bars[D_KFULL0 + st], 32, j * 64, h, b);
      }
      if (*abort_flag)        // give copies already issued a bounded time to land before the CTA exits
        for (int i = 0; i < 3; ++i) {
          uint32_t addr = smem_u32(&bars[i == 2 ? D_VFULL : D_KFULL0 + i]), done = 0;
          for (uint32_t n = 0; n < (1u << 14) && !done; ++n)
            asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}" : "=r"(done) : "r"(addr), "r"(0u) : "memory");
        }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ------------------------------------------------------------------------------------------------------
    // (two lanes issue, each the k steps of one parity into its own accumulator: see the forward kernel)
    if (lane < 2) {
      const uint32_t idesc_dq = make_idesc(128, 64, 0, 1);
      const uint32_t idesc_dp128 = make_idesc(128, 128, 0, 0);
      const uint64_t dv_hi = make_desc_k(smem_u32(v_hi), 32), dv_lo = make_desc_k(smem_u32(v_lo), 32);
      uint64_t dk_hi[2], dk_lo[2];
      for (int i = 0; i < 2; ++i) { dk_hi[i] = desc_mn(smem_u32(kbuf[i]), 64); dk_lo[i] = desc_mn(smem_u32(kbuf[i] + kHalfTile), 64); }
      bool ok = mbar_wait(&bars[D_DOREADY], 0, abort_flag);
      // dP of the 128-key block J (lane 0 alone: 128-wide instructions keep the tensor pipe busy by themselves)
      auto issue_dp = [&](int J) -> bool {
        if (!mbar_wait(&bars[D_VCONV], (uint32_t)J & 1, abort_flag)) return false;
        if (J > 0 && !mbar_wait(&bars[D_DPFREE], (uint32_t)(J - 1) & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const uint64_t off = (uint64_t)(((t >> 2) * kChunk + (t & 3) * 32) >> 4);
          mma_tf32_ta(t_dp, t_dolo + 8 * t, dv_hi + off, idesc_dp128, t > 0 ? 1u : 0u);
          mma_tf32_ta(t_dp, t_dohi + 8 * t, dv_lo + off, idesc_dp128, 1u);
          mma_tf32_ta(t_dp, t_dohi + 8 * t, dv_hi + off, idesc_dp128, 1u);
        }
        mma_commit(&bars[D_VFREE]);
        mma_commit(&bars[D_DPFULL]);
        return true;
      };
      if (ok && lane == 0) ok = issue_dp(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1, u = j >> 1;
        // order on the pipe: dQ(J, first half), dP(J + 1), dQ(J, second half) -- the next block's V has landed by then and its
        // dP runs while the row warps work on the second half
        if (lane == 0 && (j & 1) == 1 && u + 1 < n_big) { ok = issue_dp(u + 1); if (!ok) break; }
        ok = mbar_wait(&bars[D_DSREADY], (uint32_t)j & 1, abort_flag) && mbar_wait(&bars[D_KCONV0 + st], (uint32_t)u & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = lane ? t_dq2 : t_dq;
#pragma unroll
        for (int t2 = 0; t2 < 4; ++t2) {
          const int t = 2 * t2 + lane;
          const uint64_t off = (uint64_t)((t * 1024) >> 4);
          mma_tf32_ta(acc, t_dslo + 8 * t, dk_hi[st] + off, idesc_dq, (j > 0 || t2 > 0) ? 1u : 0u);
          mma_tf32_ta(acc, t_dshi + 8 * t, dk_lo[st] + off, idesc_dq, 1u);
          mma_tf32_ta(acc, t_dshi + 8 * t, dk_hi[st] + off, idesc_dq, 1u);
        }
        mma_commit(&bars[D_KFREE0 + st]);
        mma_commit(&bars[D_DQDONE]);
      }
    }
  } else if (warp < 6) {
    // ---- converters ------------------------------------------------------------------------------------------------------
    const int tid = threadIdx.x - 64;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int st = j & 1, u = j >> 1;
      if ((j & 1) == 0) {
        ok = mbar_wait(&bars[D_VFULL], (uint32_t)u & 1, abort_flag);
        if (!ok) break;
        convert_tile(v_hi, v_lo, tid, 128);
        fence_async_smem(); __syncwarp();
        if (lane == 0) mbar_arrive(&bars[D_VCONV]);
      }
      ok = mbar_wait(&bars[D_KFULL0 + st], (uint32_t)u & 1, abort_flag);
      if (!ok) break;
      const float4* s4 = (const float4*)kbuf[st]; float4* d4 = (float4*)(kbuf[st] + kHalfTile);
      float4 x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = s4[tid + i * 128];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 l;
        l.x = tf32_lo_of_raw(x[i].x); l.y = tf32_lo_of_raw(x[i].y); l.z = tf32_lo_of_raw(x[i].z); l.w = tf32_lo_of_raw(x[i].w);
        d4[tid + i * 128] = l;
      }
      fence_async_smem(); __syncwarp();
      if (lane == 0) mbar_arrive(&bars[D_KCONV0 + st]);
    }
  } else {
    // ---- row warps -------------------------------------------------------------------------------------------------------
    const int w = warp - 6, quarter = warp & 3, half = w >> 2;
    const int row = quarter * 32 + lane, grow = qt * 128 + row;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    uint8_t* bufs = staging + w * 3 * 4096;
    bool ok = true;
    uint32_t v[32];
    // P block of (this warp, key block j): rows qt*128 + quarter*32 .. +32, columns j*64 + half*32 .. +32, into buffer j % 3
    auto prefetch_p = [&](int j) {
      if (j < n_kv) {
        uint8_t* dst = bufs + (j % 3) * 4096;
        const int col0 = j * 64 + half * 32, row0 = qt * 128 + quarter * 32;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int u = e * 32 + lane, r = u >> 3, c4 = u & 7;
          const bool valid = row0 + r < p.S && col0 + 4 * c4 < p.S && VB_BC(r * 128 + ((c4 ^ (r & 7)) << 4), 4096);
          const float* src = valid ? p.P + ((i64)bh * p.S + row0 + r) * p.S + col0 + 4 * c4 : p.P;
          cp_async16(dst + r * 128 + ((c4 ^ (r & 7)) << 4), src, valid);
        }
      }
      cp_async_commit();                 // (an empty group past the last block keeps the group count uniform)
    };
    // dO row -> tensor memory (hi, lo); delta = dO . O.  These loads go out first: every CTA of a wave starts at once and the
    // first product waits for them, while the P blocks (requested right behind) are not needed before its result.
    float delta = 0.0f;
    {
      uint32_t t[32];
      float4 g[8], o[8];
      if (grow < p.S) {
        const float4* g4 = (const float4*)(p.dO + (i64)b * p.do_sb + (i64)h * p.do_sh + (i64)grow * p.do_ss + half * 32);
        const float4* o4 = (const float4*)(p.O + ((i64)bh * p.S + grow) * 64 + half * 32);
#pragma unroll
        for (int e = 0; e < 8; ++e) { g[e] = __ldg(g4 + e); o[e] = __ldg(o4 + e); }      // all sixteen in flight before the first use
      }
      prefetch_p(0);
      prefetch_p(1);
      if (grow < p.S) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[4 * e] = __float_as_uint(g[e].x); v[4 * e + 1] = __float_as_uint(g[e].y); v[4 * e + 2] = __float_as_uint(g[e].z); v[4 * e + 3] = __float_as_uint(g[e].w);
          delta = fmaf(g[e].x, o[e].x, delta); delta = fmaf(g[e].y, o[e].y, delta); delta = fmaf(g[e].z, o[e].z, delta); delta = fmaf(g[e].w, o[e].w, delta);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = 0u;
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) t[e] = v[e] & 0xffffe000u;
      tmem_st32(t_dohi + lane_off + (uint32_t)(half * 32), t);
#pragma unroll
      for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(tf32_lo_of_raw(__uint_as_float(v[e])));
      tmem_st32(t_dolo + lane_off + (uint32_t)(half * 32), t);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[D_DOREADY]);
    }
    xd[half * 128 + row] = delta;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    delta = xd[row] + xd[128 + row];
    for (int j = 0; j < n_kv && ok; ++j) {
      float4* buf = (float4*)(bufs + (j % 3) * 4096);
      cp_async_wait1();
      __syncwarp();
      float pv[32];
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) { const float4 x = buf[lane * 8 + (j4 ^ (lane & 7))]; pv[4 * j4] = x.x; pv[4 * j4 + 1] = x.y; pv[4 * j4 + 2] = x.z; pv[4 * j4 + 3] = x.w; }
      // dP holds 128 keys: this warp's 32 columns of sub-block j & 1; the accumulator is released after the second sub-block's read
      if ((j & 1) == 0) { ok = mbar_wait(&bars[D_DPFULL], (uint32_t)(j >> 1) & 1, abort_flag); if (!ok) break; }
      tc_fence_after();
      tmem_ld32(t_dp + lane_off + (uint32_t)((j & 1) * 64 + half * 32), v);
      tmem_wait_ld();
      if (j & 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[D_DPFREE]);
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) pv[c] = (pv[c] * (__uint_as_float(v[c]) - delta)) * p.scale;
      if (j > 0) { ok = mbar_wait(&bars[D_DQDONE], (uint32_t)(j - 1) & 1, abort_flag); if (!ok) break; tc_fence_after(); }
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(pv[c]) & 0xffffe000u;
      tmem_st32(t_dshi + lane_off + (uint32_t)(half * 32), v);
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(tf32_lo_of_raw(pv[c]));
      tmem_st32(t_dslo + lane_off + (uint32_t)(half * 32), v);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[D_DSREADY]);
      // dS block -> the buffer its P came from -> global (the dK product reads it)
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) buf[lane * 8 + (j4 ^ (lane & 7))] = make_float4(pv[4 * j4], pv[4 * j4 + 1], pv[4 * j4 + 2], pv[4 * j4 + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (j * 64 + half * 32 < p.S) {
          tma_store_3d(&map_ds, buf, j * 64 + half * 32, qt * 128 + quarter * 32, bh);
          tma_store_wait_read1();        // the store before this one has left its buffer: that buffer takes the P block two ahead
        } else tma_store_wait_read();    // (a sub-block past the last key: nothing to store)
      }
      __syncwarp();
      prefetch_p(j + 2);
    }
    // ---- epilogue: dQ -> staged block -> global ----
    if (ok) ok = mbar_wait(&bars[D_DQDONE], (uint32_t)(n_kv - 1) & 1, abort_flag);
    if (ok) {
      tc_fence_after();
      uint32_t v2[32];
      tmem_ld32(t_dq + lane_off + (uint32_t)(half * 32), v);
      tmem_ld32(t_dq2 + lane_off + (uint32_t)(half * 32), v2);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(v2[c]));
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
      float4* stg = (float4*)bufs;
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4)
        stage_put(stg, lane, j4, make_float4(__uint_as_float(v[4 * j4]), __uint_as_float(v[4 * j4 + 1]), __uint_as_float(v[4 * j4 + 2]), __uint_as_float(v[4 * j4 + 3])));
      fence_async_smem();
      __syncwarp();
      if (lane == 0) tma_store_block(&map_dq, stg, half * 32, qt * 128 + quarter * 32, h, b);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.err, ERRBIT_WAIT_TIMEOUT);
}

// ---- host side --------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
    else cudaGetLastError();
  }
  return fn;
}
// [B,H,S,64] view with element strides {sb, sh, ss, 1}: dims {64, S, H, B}; boxes of 32 columns x `rows` rows
int head_map(CUtensorMap* map, const float* base, i64 S, i64 H, i64 B, i64 ss, i64 sh, i64 sb, int rows, CUtensorMapSwizzle sw) {
  cuuint64_t dims[4] = {64, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 4, (cuuint64_t)(H > 1 ? sh : ss * S) * 4, (cuuint64_t)(B > 1 ? sb : (H > 1 ? sh * H : ss * S)) * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)rows, 1, 1}, estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(VB_ERR_CUDA, "cuTensorMapEncodeTiled (attention operand) failed with code " + std::to_string((int)r));
  return VB_OK;
}
// [BH, S, S] probabilities / score gradients: dims {S, S, BH}; boxes of 32 columns x `rows` rows
int square_map(CUtensorMap* map, const float* base, i64 S, i64 BH, int rows) {
  cuuint64_t dims[3] = {(cuuint64_t)S, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)S * 4, (cuuint64_t)S * (cuuint64_t)S * 4};
  cuuint32_t box[3] = {32, (cuuint32_t)rows, 1}, estr[3] = {1, 1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(VB_ERR_CUDA, "cuTensorMapEncodeTiled (attention scores) failed with code " + std::to_string((int)r));
  return VB_OK;
}
bool strides_ok(const float* p, i64 ss, i64 sh, i64 sb, i64 H, i64 B) {
  if ((uintptr_t)p & 15) return false;
  if (ss <= 0 || (ss & 3)) return false;
  if (H > 1 && (sh <= 0 || (sh & 3))) return false;
  if (B > 1 && (sb <= 0 || (sb & 3))) return false;
  return true;
}

}  // namespace

bool attn_fused_supported(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, i64 B, i64 H, i64 S, i64 dk) {
  if (!encode_fn() || dk != 64 || S < 128 || (S & 3) || S > 65535 * 128 || B * H < 1 || B * H > 0x7fffffff) return false;
  for (const AttnOperand* o : {&q, &k, &v}) if (o->sd != 1 || !strides_ok(o->p, o->ss, o->sh, o->sb, H, B)) return false;
  return true;
}

bool attn_fused_operand_ok(const AttnOperand& o, i64 B, i64 H) { return o.sd == 1 && strides_ok(o.p, o.ss, o.sh, o.sb, H, B); }

// out: [B,S,H,64]-ordered buffer (row stride o_ss, head stride 64); probs: null, or room for the [B,H,S,S] probabilities followed by a
// [B,H,S,64] copy of the output (what the backward kernel reads)
int launch_attn_fwd_fused(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, float* out, i64 o_ss, i64 o_sb, float* probs,
                          i64 B, i64 H, i64 S, bool causal, float scale) {
  CUtensorMap mq, mk, mv, mp, mo, mo2;
  VB_TRY(head_map(&mq, q.p, S, H, B, q.ss, q.sh, q.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B));
  VB_TRY(head_map(&mk, k.p, S, H, B, k.ss, k.sh, k.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B));
  VB_TRY(head_map(&mv, v.p, S, H, B, v.ss, v.sh, v.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B));
  VB_TRY(head_map(&mo, out, S, H, B, o_ss, 64, o_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B));
  memset(&mp, 0, sizeof mp); memset(&mo2, 0, sizeof mo2);
  if (probs) {
    VB_TRY(square_map(&mp, probs, S, B * H, 32));
    VB_TRY(head_map(&mo2, probs + B * H * S * S, S, H, B, 64, S * 64, H * S * 64, 32, CU_TENSOR_MAP_SWIZZLE_128B));     // [B,H,S,64] behind the probabilities
  }
  AttnFwdParams p{};
  p.S = (int)S; p.n_qtiles = (int)((S + 127) / 128); p.causal = causal ? 1 : 0; p.store_p = probs ? 1 : 0; p.H = (int)H; p.scale_l2e = scale * 1.4426950408889634f;
  p.err = ctx().d_err;
  const size_t smem = 6 * (size_t)kTile + kRowWarpsFwd * 4096 + B_COUNT * sizeof(uint64_t) + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) { VB_CUDA(cudaFuncSetAttribute(k_attn_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_set = true; }
  // useful flops: Q.K^T and P.V over the blocks that are computed (the second Q.K^T pass is the kernel's own business)
  const double nq = (double)p.n_qtiles, blocks = causal ? nq * (nq + 1) / 2 : nq * nq;
  const double dense = 2.0 * 2.0 * (double)S * (double)S * 64.0 * (double)(B * H);
  const double live = 2.0 * 2.0 * 128.0 * 128.0 * 64.0 * blocks * (double)(B * H);
  ProfScope prof("attn_fused_fwd", live < dense ? live : dense, dense);
  dim3 grid((unsigned)(B * H), (unsigned)p.n_qtiles, 1);
  k_attn_fwd<<<grid, kFwdThreads, smem, ctx().stream>>>(mq, mk, mv, mp, mo, mo2, p);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

// saved: what the fused forward left for the backward, [B,H,S,S] probabilities followed by the [B,H,S,64] output; ds: [B,H,S,S]
// scratch that receives scale * P (dP - delta) (up to the end of each row's diagonal tile under the causal mask); dq: rows of 64
// floats per head at dq + b*dq_sb + s*dq_ss + h*64
int launch_attn_bwd_dq_fused(const AttnOperand& k, const AttnOperand& v, const AttnOperand& gout, const float* saved, float* ds,
                             float* dq, i64 dq_ss, i64 dq_sb, i64 B, i64 H, i64 S, bool causal, float scale) {
  CUtensorMap mv, mk, mds, mdq;
  VB_TRY(head_map(&mv, v.p, S, H, B, v.ss, v.sh, v.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B));              // 128-key tiles (dP)
  VB_TRY(head_map(&mk, k.p, S, H, B, k.ss, k.sh, k.sb, 64, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B));      // 64-key blocks (dQ)
  VB_TRY(square_map(&mds, ds, S, B * H, 32));
  VB_TRY(head_map(&mdq, dq, S, H, B, dq_ss, 64, dq_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B));
  AttnBwdParams p{};
  p.S = (int)S; p.n_qtiles = (int)((S + 127) / 128); p.causal = causal ? 1 : 0; p.H = (int)H; p.scale = scale;
  p.P = saved; p.O = saved + B * H * S * S;
  p.dO = gout.p; p.do_sb = gout.sb; p.do_sh = gout.sh; p.do_ss = gout.ss;
  p.err = ctx().d_err;
  const size_t smem = 8 * (size_t)kHalfTile + kRowWarpsFwd * 3 * 4096 + D_COUNT * sizeof(uint64_t) + 256 * sizeof(float) + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) { VB_CUDA(cudaFuncSetAttribute(k_attn_bwd_dq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_set = true; }
  const double nq = (double)p.n_qtiles, blocks = causal ? nq * (nq + 1) / 2 : nq * nq;
  const double dense = 2.0 * 2.0 * (double)S * (double)S * 64.0 * (double)(B * H);
  const double live = 2.0 * 2.0 * 128.0 * 128.0 * 64.0 * blocks * (double)(B * H);
  ProfScope prof("attn_fused_bwd_dq", live < dense ? live : dense, dense);
  dim3 grid((unsigned)(B * H), (unsigned)p.n_qtiles, 1);
  k_attn_bwd_dq<<<grid, kFwdThreads, smem, ctx().stream>>>(mv, mk, mds, mdq, p);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
