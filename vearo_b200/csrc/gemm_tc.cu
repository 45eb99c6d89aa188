// FP32-accurate GEMM on the 5th-generation tensor cores: 3xTF32 split precision, tcgen05.mma with
// the accumulator in tensor memory, operands staged in shared memory by TMA (no multicast).
//
//   C[b] = alpha * A[b] . B[b] (+ beta * C[b]) (+ bias),  A [M,K] and B^T [N,K] both K-contiguous.
//
// Every f32 operand value x is split as x = hi + lo with hi = tf32(x) (round to nearest) and
// lo = tf32(x - hi); the product is accumulated as lo_a*hi_b + hi_a*lo_b + hi_a*hi_b (small terms
// first) in one FP32 accumulator, which leaves a relative error of about 2^-22 per product instead
// of TF32's 2^-11.  The tensor pipe therefore issues three TF32 MMAs per useful multiply-add: the
// useful-flop ceiling of this kernel is one third of the TF32 peak.
//
// CTA = 192 threads, one 128 x BN output tile (BN = 64, 128 or 256 chosen per call):
//   warp 0      TMA producer: raw f32 tiles of A and B (BK = 16 columns, 64-byte swizzle) into a
//               4..6-stage ring, completion signalled on `full[s]` by transaction bytes.
//   warps 2-5   converters: wait `full[s]`, rewrite the stage in place as `hi` and write `lo` to a
//               twin buffer at the same offsets (the split is elementwise, so the swizzle pattern is
//               irrelevant), fence the generic-proxy writes towards the async proxy, arrive `conv[s]`.
//               After the main loop the same warps run the epilogue (tcgen05.ld -> registers -> global).
//   warp 1      allocates tensor memory, waits `conv[s]`, issues the 3 x (BK/8) MMAs of the stage from
//               one thread, and releases the stage with tcgen05.commit -> `empty[s]`.
// Split-K (grid.z) spreads long-K, few-tile problems (weight gradients) over all 148 SMs; partial
// tiles go to scratch and a second kernel adds them in a fixed order.
//
// Operands that are not K-contiguous (transposed views) are first repacked by a tiled transpose
// kernel into K-contiguous scratch; shapes that break TMA's alignment rules (row stride not a
// multiple of 16 bytes, unaligned base) fall back to the CUDA-core kernel in gemm_simt.cu.
//
// Every wait on an mbarrier is bounded: when a wait runs out the CTA raises a flag in the device
// error word, drains what it has in flight, frees its tensor memory and returns.
#include "common.h"
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

namespace vb {

namespace {

constexpr int BM = 128;
constexpr int BK = 16;                    // f32 columns per stage: 64-byte rows, SWIZZLE_64B
constexpr int kConvWarps = 8;                 // converter / epilogue warps
constexpr int kThreads = 64 + 32 * kConvWarps;
constexpr uint32_t kSpinLimit = 1u << 20; // polls of try_wait (each waits a bounded time) before giving up

struct TcParams {
  float* C; const float* bias; float* partial;   // partial: [splits][nbatch][M][N] when splits > 1
  i64 M, N, K;
  i64 c_rs, c_b1, c_b2;
  i64 nb1, nb2;
  int a_bcast1, a_bcast2, b_bcast1, b_bcast2;     // 1: batch level is broadcast for that operand (coordinate 0)
  int bn, stages, lstages, splits, kblocks_per_split;   // stages: raw-tile ring (TMA in flight); lstages: lo-tile ring
  int a_mn, b_mn;                                 // 1: operand tile is MN-contiguous (transposed view), staged as 32-wide boxes, 128-byte swizzle with 32-byte base
  int causal;                                     // see GemmArgs::causal
  int debug;                                      // timing experiments only (results are wrong): 1 skip the split, 2 issue one MMA of three
  int raw_hi;                                     // 1: the raw f32 tile is used as the hi operand (the MMA ignores the low 13 mantissa bits)
  float alpha, beta;
  int* err;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait; false when the limit ran out (or another role already aborted).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 1023) == 1023 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// Shared-memory matrix descriptor, K-major, SWIZZLE_64B: rows of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t make_desc_k_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(512 >> 4) << 32;                     // stride byte offset: 8 rows * 64 B
  d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
  d |= (uint64_t)4 << 61;                              // layout type: SWIZZLE_64B
  return d;
}
// Shared-memory matrix descriptor, MN-major.  For 32-bit operands the only MN-major layout the tensor core accepts
// is the 128-byte swizzle with a 32-byte base: the tile is a row of 32-float (128-byte) MN blocks, each block BK rows
// (k) of 128 bytes; blocks are 2048 bytes apart (leading offset), groups of 4 k rows 512 bytes apart (stride offset).
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((BK * 128) >> 4) << 16;              // leading byte offset: next 32-wide MN block
  d |= (uint64_t)(512 >> 4) << 32;                     // stride byte offset: next group of 4 k rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;                              // layout type: SWIZZLE_128B_BASE32B
  return d;
}
__device__ __forceinline__ uint64_t make_desc(uint32_t base, int ks, int mn_major) {
  return mn_major ? make_desc_mn_sw128(base + ks * 1024) : make_desc_k_sw64(base + ks * 32);
}
// Instruction descriptor: D = F32, A = B = TF32, M = 128, N = bn, operand majors as given.
__device__ __forceinline__ uint32_t make_idesc(int bn, int a_mn, int b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(kThreads, 2)
k_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: raw ring [stages][ A | B ] (TMA destination, read by the MMA as the hi operand), lo ring [lstages][ A_lo | B_lo ], barriers.
  // The raw ring is deep (it has to cover the latency of TMA loads from HBM); the lo ring only spans convert -> MMA.
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzle atoms need 1024-byte alignment in the shared window
  const int bn = p.bn, stages = p.stages, lstages = p.lstages;
  const uint32_t a_bytes = BM * BK * 4, b_bytes = (uint32_t)bn * BK * 4, raw_bytes = a_bytes + b_bytes;
  uint8_t* lo_ring = smem + (size_t)stages * raw_bytes;
  uint64_t* bars = (uint64_t*)(lo_ring + (size_t)lstages * raw_bytes);
  uint64_t* full = bars; uint64_t* empty = bars + stages; uint64_t* conv = bars + 2 * stages; uint64_t* lo_empty = conv + lstages;
  uint64_t* tmem_full = lo_empty + lstages;
  uint32_t* tmem_slot = (uint32_t*)(tmem_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const i64 tile_n = blockIdx.x, tile_m = blockIdx.y;
  const i64 nbatch = p.nb1 * p.nb2;
  const i64 bz = blockIdx.z % nbatch; const int split = (int)(blockIdx.z / nbatch);
  const int b1 = (int)(bz / p.nb2), b2 = (int)(bz % p.nb2);
  const i64 kblocks_total = (p.K + BK - 1) / BK;
  i64 kb0 = (i64)split * p.kblocks_per_split;
  i64 kb1 = kb0 + p.kblocks_per_split; if (kb1 > kblocks_total) kb1 = kblocks_total;
  if (p.causal == 1 && tile_n * p.bn >= (tile_m + 1) * BM) return;                       // whole tile above the diagonal (uniform exit, nothing allocated yet)
  if (p.causal == 2) { i64 lim = ((tile_m + 1) * BM + BK - 1) / BK; if (kb1 > lim) kb1 = lim; }
  if (p.causal == 3) { i64 lo = (tile_m * BM) / BK; if (kb0 < lo) kb0 = lo; }
  const int nkb = (int)(kb1 > kb0 ? kb1 - kb0 : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < lstages; ++s) { mbar_init(&conv[s], kConvWarps); mbar_init(&lo_empty[s], 1); }
    mbar_init(tmem_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // tensor memory: bn columns hold the 128 x bn f32 accumulator (so that several CTAs can share an SM's 512 columns)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)bn) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------------
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        int s = kb % stages; uint32_t ph = (uint32_t)(kb / stages) & 1;
        if (kb >= stages && !mbar_wait(&empty[s], ph ^ 1, abort_flag)) break;
        uint8_t* st = smem + (size_t)s * raw_bytes;
        mbar_arrive_expect_tx(&full[s], raw_bytes);
        int k = (int)((kb0 + kb) * BK);
        const int ab2 = p.a_bcast2 ? 0 : b2, ab1 = p.a_bcast1 ? 0 : b1, bb2 = p.b_bcast2 ? 0 : b2, bb1 = p.b_bcast1 ? 0 : b1;
        if (!p.a_mn) tma_load_4d(st, &map_a, &full[s], k, (int)(tile_m * BM), ab2, ab1);
        else for (int j = 0; j < BM / 32; ++j) tma_load_4d(st + j * (BK * 128), &map_a, &full[s], (int)(tile_m * BM) + 32 * j, k, ab2, ab1);
        if (!p.b_mn) tma_load_4d(st + a_bytes, &map_b, &full[s], k, (int)(tile_n * bn), bb2, bb1);
        else for (int j = 0; j < bn / 32; ++j) tma_load_4d(st + a_bytes + j * (BK * 128), &map_b, &full[s], (int)(tile_n * bn) + 32 * j, k, bb2, bb1);
        issued = kb + 1;
      }
      // after an abort: give the copies already issued a bounded time to land before the CTA exits
      if (*abort_flag)
        for (int kb = (issued > stages ? issued - stages : 0); kb < issued; ++kb) {
          uint32_t addr = smem_u32(&full[kb % stages]), ph = (uint32_t)(kb / stages) & 1, done = 0;
          for (uint32_t it = 0; it < (1u << 16) && !done; ++it)
            asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}" : "=r"(done) : "r"(addr), "r"(ph) : "memory");
        }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(bn, p.a_mn, p.b_mn);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        int s = kb % stages, l = kb % lstages; uint32_t lph = (uint32_t)(kb / lstages) & 1;
        ok = mbar_wait(&conv[l], lph, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t st = smem_u32(smem + (size_t)s * raw_bytes), lt = smem_u32(lo_ring + (size_t)l * raw_bytes);
        uint32_t a_hi = st, b_hi = st + a_bytes, a_lo = lt, b_lo = lt + a_bytes;
#pragma unroll
        for (int ks = 0; ks < BK / 8; ++ks) {
          // one MMA covers 8 k: 32 bytes along a K-major row, or one 1024-byte k group of an MN-major tile
          uint64_t da_hi = make_desc(a_hi, ks, p.a_mn), db_hi = make_desc(b_hi, ks, p.b_mn);
          uint64_t da_lo = make_desc(a_lo, ks, p.a_mn), db_lo = make_desc(b_lo, ks, p.b_mn);
          if (p.debug & 2) { mma_tf32(tmem_base, da_hi, db_hi, idesc, (kb | ks) ? 1u : 0u); continue; }
          mma_tf32(tmem_base, da_lo, db_hi, idesc, (kb | ks) ? 1u : 0u);
          mma_tf32(tmem_base, da_hi, db_lo, idesc, 1u);
          mma_tf32(tmem_base, da_hi, db_hi, idesc, 1u);
        }
        mma_commit(&empty[s]);          // frees the raw stage once these MMAs have read it
        mma_commit(&lo_empty[l]);       // ... and the lo stage
      }
      if (ok) mma_commit(tmem_full);    // accumulator complete
    }
  } else {
    // ---- converters, then epilogue ------------------------------------------------------------
    const int cw = warp - 2, ct = cw * 32 + lane;            // 0 .. 32*kConvWarps-1
    constexpr int kConvThreads = 32 * kConvWarps;
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      int s = kb % stages, l = kb % lstages; uint32_t ph = (uint32_t)(kb / stages) & 1, lph = (uint32_t)(kb / lstages) & 1;
      if (kb >= lstages) ok = mbar_wait(&lo_empty[l], lph ^ 1, abort_flag);
      if (ok) ok = mbar_wait(&full[s], ph, abort_flag);
      if (!ok) break;
      float4* hi = (float4*)(smem + (size_t)s * raw_bytes);
      float4* lo = (float4*)(lo_ring + (size_t)l * raw_bytes);
      const int n4 = (int)(raw_bytes / 16);      // 768, 1024 or 1536: a multiple of kConvThreads
      if (p.debug & 1) {
      } else if (p.raw_hi) {
#pragma unroll 3
        for (int i = ct; i < n4; i += kConvThreads) {
          float4 x = hi[i], l;
          l.x = tf32_rna(x.x - __uint_as_float(__float_as_uint(x.x) & 0xffffe000u));
          l.y = tf32_rna(x.y - __uint_as_float(__float_as_uint(x.y) & 0xffffe000u));
          l.z = tf32_rna(x.z - __uint_as_float(__float_as_uint(x.z) & 0xffffe000u));
          l.w = tf32_rna(x.w - __uint_as_float(__float_as_uint(x.w) & 0xffffe000u));
          lo[i] = l;
        }
      } else {
#pragma unroll 3
        for (int i = ct; i < n4; i += kConvThreads) {
          float4 x = hi[i], h, l;
          h.x = tf32_rna(x.x); h.y = tf32_rna(x.y); h.z = tf32_rna(x.z); h.w = tf32_rna(x.w);
          l.x = tf32_rna(x.x - h.x); l.y = tf32_rna(x.y - h.y); l.z = tf32_rna(x.z - h.z); l.w = tf32_rna(x.w - h.w);
          hi[i] = h; lo[i] = l;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&conv[l]);
    }
    // epilogue: TMEM lane quarter of this warp is (warp % 4)
    if (nkb == 0) ok = true;
    if (ok && nkb > 0) ok = mbar_wait(tmem_full, 0, abort_flag);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int q = warp & 3;
      const i64 row = tile_m * BM + q * 32 + lane;
      const bool direct = p.splits == 1;
      float* out = direct ? p.C + (i64)b1 * p.c_b1 + (i64)b2 * p.c_b2 + row * p.c_rs
                          : p.partial + (((i64)split * nbatch + bz) * p.M + row) * p.N;
      const bool vec_ok = direct ? ((p.c_rs & 3) == 0 && (((uintptr_t)p.C | (uintptr_t)(p.c_b1 * 4) | (uintptr_t)(p.c_b2 * 4)) & 15) == 0) : ((p.N & 3) == 0);
      const int half = (warp - 2) >> 2, ncol_half = bn / 2;      // two warps share a lane quarter; each takes half the columns
      for (int c0 = half * ncol_half; c0 < (half + 1) * ncol_half; c0 += 32) {
        i64 col0 = tile_n * bn + c0;
        if (col0 >= p.N) break;
        uint32_t r[32];
        if (nkb > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            i64 col = col0 + j;
            if (col >= p.N) break;
            float v[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) v[t] = __uint_as_float(r[j + t]);
            if (direct) {
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                v[t] *= p.alpha;
                if (col + t < p.N) {
                  if (p.beta != 0.0f) v[t] += p.beta * out[col + t];
                  if (p.bias) v[t] += p.bias[col + t];
                }
              }
            }
            if (vec_ok && col + 3 < p.N) *reinterpret_cast<float4*>(out + col) = make_float4(v[0], v[1], v[2], v[3]);
            else for (int t = 0; t < 4 && col + t < p.N; ++t) out[col + t] = v[t];
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)bn) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.err, ERRBIT_WAIT_TIMEOUT);
}

// Sum the split-K partial tiles in split order, then apply alpha / beta / bias.
__global__ void k_splitk_reduce(const float* __restrict__ partial, float* __restrict__ C, const float* __restrict__ bias,
                                i64 M, i64 N, i64 nb2, i64 nbatch, int splits, i64 c_rs, i64 c_b1, i64 c_b2, float alpha, float beta) {
  i64 total = nbatch * M * N;
  for (i64 idx = blockIdx.x * (i64)blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    i64 n = idx % N, m = (idx / N) % M, bz = idx / (N * M);
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += partial[(i64)k * total + idx];
    float* c = C + (bz / nb2) * c_b1 + (bz % nb2) * c_b2 + m * c_rs + n;
    float v = alpha * s;
    if (beta != 0.0f) v += beta * *c;
    if (bias) v += bias[n];
    *c = v;
  }
}

// Repack a [R, K] operand whose K axis is not contiguous into K-contiguous rows of length Kp
// (tiled 32x32 transpose through shared memory; batch levels are flattened into the output).
__global__ void k_repack_kmajor(const float* __restrict__ src, float* __restrict__ dst, i64 R, i64 K, i64 Kp, i64 rs, i64 cs,
                                i64 nb2, i64 sb1, i64 sb2) {
  __shared__ float tile[32][33];
  i64 bz = blockIdx.z;
  const float* s = src + (bz / nb2) * sb1 + (bz % nb2) * sb2;
  float* d = dst + bz * R * Kp;
  i64 r0 = (i64)blockIdx.y * 32, k0 = (i64)blockIdx.x * 32;
  // read with the row index fastest (the contiguous axis of a transposed view)
  for (int i = threadIdx.y; i < 32; i += 8) {
    i64 r = r0 + threadIdx.x, k = k0 + i;
    tile[i][threadIdx.x] = (r < R && k < K) ? s[r * rs + k * cs] : 0.0f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    i64 r = r0 + i, k = k0 + threadIdx.x;
    if (r < R && k < Kp) d[r * Kp + k] = tile[threadIdx.x][i];
  }
}

// ---- host side --------------------------------------------------------------------------------
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

struct Operand { const float* p; i64 rows, rs, b1, b2; bool bc1, bc2; bool mn; };   // [rows, K]; rs = row stride (K-major) or k stride (MN-major)

bool tma_ok(const Operand& o, i64 nb1, i64 nb2) {
  if ((uintptr_t)o.p & 15) return false;
  if (o.rs & 3) return false;
  if (!o.bc1 && nb1 > 1 && (o.b1 & 3)) return false;
  if (!o.bc2 && nb2 > 1 && (o.b2 & 3)) return false;
  if (o.rs <= 0 || (!o.bc1 && nb1 > 1 && o.b1 <= 0) || (!o.bc2 && nb2 > 1 && o.b2 <= 0)) return false;
  return true;
}
int make_map(CUtensorMap* map, const Operand& o, i64 K, i64 nb1, i64 nb2, int box_rows) {
  i64 d2 = o.bc2 ? 1 : nb2, d3 = o.bc1 ? 1 : nb1;
  // K-major: dims {K, rows}, one box of BK x box_rows, 64-byte swizzle.  MN-major: dims {rows, K}, boxes of 32 x BK, 128-byte swizzle on 32-byte units.
  i64 inner = o.mn ? o.rows : K, outer = o.mn ? K : o.rows;
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)d2, (cuuint64_t)d3};
  // a batch level of extent 1 never advances: any 16-byte-multiple stride is acceptable there
  i64 s2 = d2 > 1 ? o.b2 : o.rs * (outer > 0 ? outer : 1), s3 = d3 > 1 ? o.b1 : s2 * d2;
  cuuint64_t strides[3] = {(cuuint64_t)o.rs * 4, (cuuint64_t)s2 * 4, (cuuint64_t)s3 * 4};
  cuuint32_t box[4] = {(cuuint32_t)(o.mn ? 32 : BK), (cuuint32_t)(o.mn ? BK : box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)o.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           o.mn ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(VB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return VB_OK;
}

}  // namespace

int launch_gemm_tc(const GemmArgs& g, bool* handled) {
  *handled = false;
  if (!encode_fn()) return VB_OK;
  if (g.c_cs != 1) return VB_OK;
  const i64 nb = g.nb1 * g.nb2;
  // worth a tensor-core launch?  (tiny products stay on the CUDA cores: exact and launch-bound anyway)
  if (g.M < 32 || g.N < 32 || g.K < 8) return VB_OK;
  if (!g.causal && (double)g.M * (double)g.N * (double)g.K * (double)nb < 4.0e6) return VB_OK;
  if (g.M > 0x7fffffffLL || g.N > 0x7fffffffLL || g.K > 0x7fffffffLL || nb > 60000) return VB_OK;
  if (g.nb1 > 1 && g.c_b1 <= 0) return VB_OK;
  if (g.nb2 > 1 && g.c_b2 <= 0) return VB_OK;

  Temp hold_a, hold_b;
  auto prepare = [&](const float* p, i64 rows, i64 rs, i64 cs, i64 sb1, i64 sb2, Temp& hold, Operand* o) -> int {
    bool bc1 = g.nb1 > 1 && sb1 == 0, bc2 = g.nb2 > 1 && sb2 == 0;
    *o = Operand{p, rows, rs, sb1, sb2, bc1, bc2, false};
    if (cs == 1 && tma_ok(*o, g.nb1, g.nb2)) return VB_OK;
    // MN-contiguous (a transposed view): consumed in place through MN-major descriptors
    static int no_mn = -1;
    if (no_mn < 0) { const char* e = getenv("VB200_TC_NO_MN"); no_mn = (e && e[0] == '1') ? 1 : 0; }
    Operand mn{p, rows, cs, sb1, sb2, bc1, bc2, true};
    if (!no_mn && rs == 1 && rows >= 32 && tma_ok(mn, g.nb1, g.nb2)) { *o = mn; return VB_OK; }
    // repack into K-contiguous scratch, one plane per (non-broadcast) batch
    i64 e1 = bc1 ? 1 : g.nb1, e2 = bc2 ? 1 : g.nb2;
    i64 Kp = (g.K + 3) & ~i64(3);
    VB_TRY(scratch_alloc((size_t)(e1 * e2 * rows * Kp) * sizeof(float), &hold.p));
    ProfScope prof("gemm_repack", 2.0 * (double)(e1 * e2 * rows * g.K) * 4.0);
    dim3 grid((unsigned)((Kp + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)(e1 * e2)), block(32, 8);
    if (grid.y > 65535 || grid.z > 65535) return set_error(VB_ERR_UNSUPPORTED, "operand too tall to repack");
    k_repack_kmajor<<<grid, block, 0, ctx().stream>>>(p, (float*)hold.p, rows, g.K, Kp, rs, cs, e2, bc1 ? 0 : sb1, bc2 ? 0 : sb2);
    VB_LAUNCH_CHECK();
    *o = Operand{(const float*)hold.p, rows, Kp, e2 * rows * Kp, rows * Kp, bc1, bc2, false};
    return VB_OK;
  };
  Operand oa, ob;
  VB_TRY(prepare(g.A, g.M, g.a_rs, g.a_cs, g.a_b1, g.a_b2, hold_a, &oa));
  VB_TRY(prepare(g.B, g.N, g.b_cs, g.b_rs, g.b_b1, g.b_b2, hold_b, &ob));   // B^T rows are the columns of B

  TcParams p{};
  // Tile width and split-K factor: minimise an estimate of the run time in units of one 256-wide k-block.
  // A k-block of a 128-wide tile costs ~0.62 of a 256-wide one (same A traffic for half the flops); the epilogue of a
  // tile costs about 10 (256) / 6 (128) k-blocks; split-K adds a pass over the partial tiles.
  const i64 kblocks = (g.K + BK - 1) / BK;
  const i64 slots = (i64)ctx().sm_count * 2;          // two resident CTAs per SM
  p.bn = g.N <= 64 ? 64 : (g.N <= 128 ? 128 : 256);
  int splits = 1;
  if (p.bn == 256) {
    double best = 1e300;
    for (int bn : {256, 128}) {
      i64 tiles = ((g.M + BM - 1) / BM) * ((g.N + bn - 1) / bn) * nb;
      for (int sk : {1, 2, 3, 4, 6, 8, 12, 16}) {
        if (sk > 1 && kblocks / sk < 24) break;
        i64 units = tiles * sk, waves = (units + slots - 1) / slots;
        double kb_cost = bn == 256 ? 1.0 : 0.62, epi = bn == 256 ? 10.0 : 6.0;
        double t = (double)waves * ((double)((kblocks + sk - 1) / sk) * kb_cost + epi);
        if (sk > 1) t += (double)tiles * (double)sk * epi * 0.5 / (double)slots + epi;      // partial tiles written, then summed
        if (t < best * 0.97) { best = t; p.bn = bn; splits = sk; }
      }
    }
  } else {
    i64 tiles = ((g.M + BM - 1) / BM) * nb;
    if (tiles < slots && kblocks >= 48) { splits = (int)((slots + tiles - 1) / tiles); if (splits > kblocks / 24) splits = (int)(kblocks / 24); if (splits < 1) splits = 1; }
  }
  const i64 tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + p.bn - 1) / p.bn;
  const size_t raw_bytes = (size_t)(BM + p.bn) * BK * 4;
  // Small rings on purpose: two CTAs then share an SM, and one CTA's epilogue and pipeline bubbles are covered by
  // the other's main loop; measured faster than one CTA per SM with a deep ring.
  p.lstages = 2;
  p.stages = p.bn == 256 ? 2 : 3;
  p.kblocks_per_split = (int)((kblocks + splits - 1) / splits);
  splits = (int)((kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split);
  p.splits = splits;
  if (tiles_m > 65535 || nb * splits > 65535) return VB_OK;

  CUtensorMap map_a, map_b;
  VB_TRY(make_map(&map_a, oa, g.K, g.nb1, g.nb2, BM));
  VB_TRY(make_map(&map_b, ob, g.K, g.nb1, g.nb2, p.bn));
  Temp part;
  if (splits > 1) VB_TRY(scratch_alloc((size_t)((i64)splits * nb * g.M * g.N) * sizeof(float), &part.p));
  p.C = g.C; p.bias = g.bias; p.partial = (float*)part.p;
  p.M = g.M; p.N = g.N; p.K = g.K; p.c_rs = g.c_rs; p.c_b1 = g.c_b1; p.c_b2 = g.c_b2; p.nb1 = g.nb1; p.nb2 = g.nb2;
  p.a_bcast1 = oa.bc1; p.a_bcast2 = oa.bc2; p.b_bcast1 = ob.bc1; p.b_bcast2 = ob.bc2;
  p.a_mn = oa.mn; p.b_mn = ob.mn;
  p.alpha = g.alpha; p.beta = g.beta; p.err = ctx().d_err;
  p.causal = (splits == 1 && g.M == (g.causal == 1 ? g.N : g.K)) ? g.causal : 0;

  static int raw_hi_env = -1;
  if (raw_hi_env < 0) { const char* e = getenv("VB200_TC_RAW_HI"); raw_hi_env = (e && e[0] == '0') ? 0 : 1; }
  p.raw_hi = raw_hi_env;
  { static int dbg = -1; if (dbg < 0) { const char* e = getenv("VB200_TC_DEBUG"); dbg = e ? atoi(e) : 0; } p.debug = dbg; }
  { const char* e = getenv("VB200_TC_STAGES"); if (e) { int r = 0, l = 0; if (sscanf(e, "%d,%d", &r, &l) == 2 && r >= 1 && l >= 1 && (size_t)(r + l) * raw_bytes <= 204 * 1024) { p.stages = r; p.lstages = l; } } }
  size_t smem = (size_t)(p.stages + p.lstages) * raw_bytes + (2 * p.stages + 2 * p.lstages + 1) * sizeof(uint64_t) + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) { VB_CUDA(cudaFuncSetAttribute(k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); attr_set = true; }
  {
    static int shapes = -1;
    if (shapes < 0) { const char* e = getenv("VB200_PROF_SHAPES"); shapes = (e && e[0] == '1') ? 1 : 0; }
    char fam[96];
    if (shapes) snprintf(fam, sizeof fam, "gemm_tc M%lld N%lld K%lld nb%lld a%d b%d bn%d sk%d", (long long)g.M, (long long)g.N, (long long)g.K, (long long)nb, (int)oa.mn, (int)ob.mn, p.bn, splits);
    else snprintf(fam, sizeof fam, "%s", nb > 1 ? "gemm_tc_batched" : "gemm_tc");
    ProfScope prof(fam, 2.0 * (double)g.M * (double)g.N * (double)g.K * (double)nb);
    dim3 grid((unsigned)tiles_n, (unsigned)tiles_m, (unsigned)(nb * splits));
    k_gemm_tc<<<grid, kThreads, smem, ctx().stream>>>(map_a, map_b, p);
    VB_LAUNCH_CHECK();
    if (splits > 1) {
      i64 total = nb * g.M * g.N;
      i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 16; if (blocks > cap) blocks = cap;
      k_splitk_reduce<<<(unsigned)blocks, 256, 0, ctx().stream>>>((const float*)part.p, g.C, g.bias, g.M, g.N, g.nb2, nb, splits,
                                                                   g.c_rs, g.c_b1, g.c_b2, g.alpha, g.beta);
      VB_LAUNCH_CHECK();
    }
  }
  *handled = true;
  return VB_OK;
}

}  // namespace vb
