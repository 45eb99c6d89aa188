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
// Backward (dQ part), one CTA per 128 query rows, 64-key blocks, 256 threads:
//   dP = dO.V^T -> row warps read P (TMA-loaded tile), ds = p * (dp - delta) * scale with delta = dO.O (= sum_j dp_j p_j),
//   dS -> tensor memory (hi, lo) and global memory (for the dK product), dQ += dS.K.
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
  float scale;
  int* err;
};

// barrier indices of the forward kernel
enum { B_QFULL = 0, B_QCONV, B_KFULL0, B_KFULL1, B_KCONV0, B_KCONV1, B_KFREE0, B_KFREE1, B_VFULL, B_VCONV, B_SFULL, B_SFREE, B_PREADY, B_PVDONE, B_COUNT };

__device__ __forceinline__ void stage_put(float4* stg, int lane, int j4, float4 x) { stg[lane * 8 + (j4 ^ (lane & 7))] = x; }

__device__ __forceinline__ void convert_tile(const uint8_t* raw, uint8_t* lo, int tid, int nthreads) {
  const float4* s = (const float4*)raw; float4* d = (float4*)lo;
#pragma unroll 4
  for (int i = tid; i < kTile / 16; i += nthreads) {
    float4 x = s[i], l;
    l.x = tf32_lo_of_raw(x.x); l.y = tf32_lo_of_raw(x.y); l.z = tf32_lo_of_raw(x.z); l.w = tf32_lo_of_raw(x.w);
    d[i] = l;
  }
}
// MN-major descriptor of a [128 k rows x 32 floats] block sequence (SWIZZLE_128B with 32-byte base), `rows` k rows per 32-wide block
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr, int rows) { return make_desc_mn_sw128(addr, rows); }

__global__ void __launch_bounds__(kFwdThreads, 1)
k_attn_fwd(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
           const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_o, AttnFwdParams p) {
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
    mbar_init(&bars[B_PREADY], kRowWarpsFwd); mbar_init(&bars[B_PVDONE], 1);
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
  const uint32_t t_s = tmem, t_phi = tmem + 128, t_plo = tmem + 256, t_o = tmem + 384;

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
    if (lane == 0) {
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
      for (int j = 0; j < n_kv && ok; ++j) ok = issue_qk(j & 1);          // pass 1: scores only
      if (ok) ok = issue_qk(0);                                            // pass 2, block 0
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) { ok = issue_qk(0); if (!ok) break; }            // the next block's scores run under this block's softmax
        ok = mbar_wait(&bars[B_PREADY], (uint32_t)j & 1, abort_flag) && mbar_wait(&bars[B_VCONV], (uint32_t)j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const uint64_t off = (uint64_t)((t * 1024) >> 4);
          mma_tf32_ta(t_o, t_plo + 8 * t, dv_hi + off, idesc_pv, (j > 0 || t > 0) ? 1u : 0u);
          mma_tf32_ta(t_o, t_phi + 8 * t, dv_lo + off, idesc_pv, 1u);
          mma_tf32_ta(t_o, t_phi + 8 * t, dv_hi + off, idesc_pv, 1u);
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
    // scores of this thread for block j: scaled, with masked columns at -inf
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
        float x = __uint_as_float(v[c]) * p.scale;
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
        for (int c = 0; c < 64; ++c) s += expf(__uint_as_float(v[c]) - mn);
        l = l * expf(m - mn) + s;
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
      if (m > -INFINITY) L += l * expf(m - M);
      if (mo > -INFINITY) L += lo_ * expf(mo - M);
      m = M; l = 1.0f / (L + 1e-9f);
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");            // (the staging area is about to carry stores)
    const float rmax = m, inv = l;
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = load_scores(j);
      if (!ok) break;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float x = __uint_as_float(v[c]);
        v[c] = __float_as_uint(x > -INFINITY ? expf(x - rmax) * inv : 0.0f);
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
      tmem_wait_ld();
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4)
        stage_put(stg, lane, j4, make_float4(__uint_as_float(v[4 * j4]), __uint_as_float(v[4 * j4 + 1]), __uint_as_float(v[4 * j4 + 2]), __uint_as_float(v[4 * j4 + 3])));
      fence_async_smem();
      __syncwarp();
      if (lane == 0) tma_store_block(&map_o, stg, half * 32, qt * 128 + quarter * 32, h, b);
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

// out: [B,S,H,64]-ordered buffer (row stride o_ss, head stride 64); probs: contiguous [B,H,S,S] or null
int launch_attn_fwd_fused(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, float* out, i64 o_ss, i64 o_sb, float* probs,
                          i64 B, i64 H, i64 S, bool causal, float scale) {
  CUtensorMap mq, mk, mv, mp, mo;
  VB_TRY(head_map(&mq, q.p, S, H, B, q.ss, q.sh, q.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B));
  VB_TRY(head_map(&mk, k.p, S, H, B, k.ss, k.sh, k.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B));
  VB_TRY(head_map(&mv, v.p, S, H, B, v.ss, v.sh, v.sb, 128, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B));
  VB_TRY(head_map(&mo, out, S, H, B, o_ss, 64, o_sb, 32, CU_TENSOR_MAP_SWIZZLE_128B));
  memset(&mp, 0, sizeof mp);
  if (probs) VB_TRY(square_map(&mp, probs, S, B * H, 32));
  AttnFwdParams p{};
  p.S = (int)S; p.n_qtiles = (int)((S + 127) / 128); p.causal = causal ? 1 : 0; p.store_p = probs ? 1 : 0; p.H = (int)H; p.scale = scale;
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
  k_attn_fwd<<<grid, kFwdThreads, smem, ctx().stream>>>(mq, mk, mv, mp, mo, p);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

}  // namespace vb
