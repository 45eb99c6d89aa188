// FP32-accurate GEMM on the 5th-generation tensor cores: 3xTF32 split precision, tcgen05.mma with
// the accumulator in tensor memory, operands staged in shared memory by TMA (no multicast).
//
//   C[b] = alpha * A[b] . B[b] (+ beta * C[b]) (+ bias),  A [M,K] and B^T [N,K] both K-contiguous.
//
// Every f32 operand value x is split as x = hi + lo with hi = x cut to TF32's 10 mantissa bits (what the
// tensor core reads of a raw f32 operand) and lo = tf32(x - hi), exact remainder rounded to nearest; the
// product is accumulated as lo_a*hi_b + hi_a*lo_b + hi_a*hi_b (small terms first) in one FP32
// accumulator, which leaves a relative error of about 2^-20 per product instead of TF32's 2^-10.  The tensor pipe therefore issues three TF32 MMAs per useful multiply-add: the
// useful-flop ceiling of this kernel is one third of the TF32 peak.
//
// CTA = 320 threads, one 128 x BN output tile (BN = 64, 128, 192 or 256 chosen per call), two CTAs per SM:
//   warp 0      TMA producer: raw f32 tiles of A and B (16 k per stage; 32 for the 64-wide tiles, whose cost is the per-stage
//               hand-offs) into a ring of 2-4 stages; one TMA box per operand tile; completion signalled on `full[s]` by
//               transaction bytes.
//   warps 2-9   converters: wait `full[s]`, write the `lo` parts of the stage into a second (2-3 stage) ring at the same
//               offsets (the split is elementwise, so the swizzle pattern is irrelevant); the raw tile itself serves as
//               `hi`, because the tensor core ignores the low 13 mantissa bits of a TF32 operand.  Then fence the
//               generic-proxy writes towards the async proxy and arrive `conv[l]`.  After the main loop the same warps
//               run the epilogue: tcgen05.ld -> registers (alpha, biases) -> staged in the idle lo ring in the 128-byte-swizzled
//               layout -> one TMA store per 32 x 32 block, which overlaps the next block's read from tensor memory
//               (ordinary coalesced stores when the output breaks TMA's alignment rules or beta != 0).
//   warp 1      allocates tensor memory, waits `conv[l]`, issues the 3 x (BK/8) MMAs of the stage from one thread, and
//               releases the stages with tcgen05.commit -> `empty[s]`, `lo_empty[l]`.
// Shared memory bandwidth is what bounds the main loop (operand reads of three MMAs + the converters' read and write
// + the TMA writes); everything per k-block in the two single-thread roles is kept to a handful of instructions.
//
// Few-tile, long-K products (weight gradients) are split along K: either tiled split-K (grid.z; partial tiles go to
// scratch and a second kernel adds them in a fixed order) or, where a tile would have three or four parts at most,
// stream-K: the k-blocks of all tiles are dealt evenly to one CTA per slot and the CTA that completes a shared tile last
// adds the parts in k order inside the kernel.  Short-K products with many tiles (attention scores, the vocabulary
// projection) deal whole tiles round-robin to resident CTAs; triangular products (attention under a causal mask) clamp
// each tile row's k range and dispatch the longest rows first.
//
// Operands: K-contiguous rows go through 64-byte-swizzle boxes; transposed views (MN-contiguous) are consumed in place
// through 32-float boxes in the 128-byte swizzle with a 32-byte base, the only MN-major layout the tensor core takes
// for 32-bit data.  Anything else (neither axis contiguous, strides that break TMA's 16-byte rules) is first repacked
// into K-contiguous scratch; shapes the tensor-core path declines fall back to the CUDA-core kernel in gemm_simt.cu.
//
// Every wait on an mbarrier is bounded: when a wait runs out the CTA raises a flag in the device error word, drains
// what it has in flight, frees its tensor memory and returns.
#include "common.h"
#include "tc_util.cuh"
#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace vb {

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 16;                    // f32 columns per stage: 64-byte rows, SWIZZLE_64B
constexpr int kConvWarps = 8;             // converter warps; the same warps run the epilogue
constexpr int kThreads = 64 + 32 * kConvWarps;

struct TcParams {
  float* C; const float* bias; const float* bias_m; float* partial;   // partial: [splits][nbatch][M][N] when splits > 1
  i64 M, N, K;
  i64 c_rs, c_b1, c_b2;
  i64 nb1, nb2;
  int a_bcast1, a_bcast2, b_bcast1, b_bcast2;     // 1: batch level is broadcast for that operand (coordinate 0)
  int tmem_cols;                                  // tensor-memory columns allocated: bn rounded up to a power of two
  int b_lo;                                       // the lo part of B comes pre-split from memory (map_blo) instead of from the converters
  int a_lo;                                       // ... and the lo part of A (map_alo); a_lo implies b_lo (the converters then have nothing to split)
  int tma_out;                                    // results leave through TMA stores of the staged 32 x 32 blocks (map_c)
  int act;                                        // 1: the epilogue also stores GELU(result) through map_act (whole tiles, tma_out only)
  // B is the unfolded ("im2col") matrix of a zero-padded NHWC image batch, never materialised: a 5-D tensor map {(j,c), x, y, tap row i, n}
  // whose boxes are the tiles (see GemmArgs::conv).  1: K-major, rows = the pixels of image b2 (forward / input gradient);
  // 2: MN-major, K = all pixels of all images, N = the taps (weight gradient)
  int b_conv;
  int cv_run, cv_w, cv_h;                         // floats per tap row (3 * C), image width and height
  int bk;                                         // k per stage: 16, or 32 for the narrow (64-wide) tiles whose per-stage hand-offs dominate
  int bn, stages, lstages, splits, kblocks_per_split;   // stages: raw-tile ring (TMA in flight); lstages: lo-tile ring
  int a_fold, b_fold;                             // 1: MN-contiguous operand whose tensor map is folded into 32-wide blocks (one TMA box per tile)
  int a_mn, b_mn;                                 // 1: operand tile is MN-contiguous (transposed view), staged as 32-wide boxes, 128-byte swizzle with 32-byte base
  int long_first;                                 // triangular products (causal 2, 3), tiled mode: gridDim = (tiles_n, batch, tiles_m) and the tile rows with the longest k range are dispatched first
  int causal;                                     // see GemmArgs::causal
  float alpha, beta;
  int* err;
  int persistent;                                 // 1: stream-K launch, 2: whole tiles dealt round-robin to resident CTAs (see WorkIter)
  i64 total_kb, tiles_m, tiles_n;                 // stream-K: k-blocks of all tiles; tile grid
  i64 live_tiles, live_per_batch;                 // round-robin: tiles that are computed (all, or those on and below the diagonal)
  float* ws;                                      // stream-K: partial sums, two 128 x bn slots per CTA
  int* counters;                                  // stream-K: arrivals per tile (all zero between launches)
};

// One operand tile of `rows` rows starting at row r0, k-block starting at k.  Three layouts of the tensor map (see make_map):
//   K-major            dims {K, rows, 1, b2, b1}        one box BK x rows
//   MN-major, folded   dims {32, K, rows/32, b2, b1}    one box 32 x BK x rows/32 (the 32-wide blocks of the tile land one after another)
//   MN-major, plain    dims {rows, K, 1, b2, b1}        one box 32 x BK per 32-wide block (row counts that are not multiples of 32)
__device__ __forceinline__ void tma_load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int mode, int rows, int r0, int k, int b2, int b1, int bk) {
  if (mode == 0) tma_load_5d(dst, map, bar, k, r0, 0, b2, b1);
  else if (mode == 2) tma_load_5d(dst, map, bar, 0, k, r0 >> 5, b2, b1);
  else for (int j = 0; j < rows / 32; ++j) tma_load_5d(dst + j * (bk * 128), map, bar, r0 + 32 * j, k, 0, b2, b1);
}

// One unit of work of a CTA: a k-block range of one output tile.
struct Work {
  int tile;            // linear tile index (stream-K mode)
  int tile_m, tile_n, bz;
  int b1, b2, split;
  int kb0, nkb;        // first k-block (absolute) and count
  int whole;           // the range is the tile's whole K extent
  int which;           // stream-K: 0 when the range starts at the group's first k-block, else 1 (selects the partial slot)
};

// Work of this CTA (one 128 x bn tile at a time).
// One launch is either "tiled" (gridDim = tiles x batch*splits, one unit per CTA, what a CTA does follows from blockIdx),
// "stream-K" (gridDim.x CTAs share tiles*kblocks k-blocks evenly; CTA c owns the contiguous range [c*W/G, (c+1)*W/G) of the
// tile-major k-block sequence, so a tile may be covered by several CTAs) or "round-robin" (whole tiles dealt to resident CTAs).
struct WorkIter {
  i64 w, w0, w1;
  int done;
  __device__ __forceinline__ void init(const TcParams& p) {
    done = 0;
    if (p.persistent == 2) { w = blockIdx.x; return; }
    if (p.persistent) {
      const i64 G = gridDim.x, c = blockIdx.x;
      w0 = (c * p.total_kb) / G; w1 = ((c + 1) * p.total_kb) / G; w = w0;
    }
  }
  __device__ __forceinline__ bool next(const TcParams& p, Work& o) {
    const i64 kblocks_total = (p.K + p.bk - 1) / p.bk;
    if (p.persistent == 2) {
      // whole tiles, the u-th computed tile to group u mod G: no launch / allocation / barrier set-up per tile, and the producer
      // runs ahead into the next tile while this one is stored.  With tiles skipped above the diagonal (causal 1) only the
      // computed ones are counted, so that every group gets the same number of them.
      if (w >= p.live_tiles) return false;
      const i64 u = w; w += gridDim.x;
      o.bz = (int)(u / p.live_per_batch);
      int j = (int)(u - (i64)o.bz * p.live_per_batch), m = 0;
      if (p.causal == 1) {
        for (;; ++m) {
          i64 c = (((i64)m + 1) * BM + p.bn - 1) / p.bn; if (c > p.tiles_n) c = p.tiles_n;      // computed tiles of tile row m
          if (j < c) break;
          j -= (int)c;
        }
      } else { m = j / (int)p.tiles_n; j -= m * (int)p.tiles_n; }
      o.tile_m = m; o.tile_n = j; o.tile = 0; o.which = 0; o.split = 0;
      o.b1 = o.bz / (int)p.nb2; o.b2 = o.bz % (int)p.nb2;
      o.kb0 = 0; o.nkb = (int)kblocks_total; o.whole = 1;
      return true;
    }
    if (p.persistent) {
      if (w >= w1) return false;
      o.tile = (int)(w / kblocks_total);
      i64 kb = w - (i64)o.tile * kblocks_total, n = kblocks_total - kb;
      if (n > w1 - w) n = w1 - w;
      o.kb0 = (int)kb; o.nkb = (int)n; o.whole = n == kblocks_total; o.which = w == w0 ? 0 : 1; o.split = 0;
      const int tiles_mn = (int)(p.tiles_m * p.tiles_n);
      o.bz = o.tile / tiles_mn; const int t = o.tile - o.bz * tiles_mn;
      o.tile_m = t / (int)p.tiles_n; o.tile_n = t - o.tile_m * (int)p.tiles_n;
      o.b1 = o.bz / (int)p.nb2; o.b2 = o.bz % (int)p.nb2;
      w += n;
      return true;
    }
    if (done) return false;
    done = 1;
    // blocks are dispatched x first, z last: with long_first the slowest index walks the tile rows from the longest k range to the
    // shortest, over all batches, so that the launch does not end on a few long tiles
    const unsigned gy = p.long_first ? (p.causal == 2 ? gridDim.z - 1 - blockIdx.z : blockIdx.z) : blockIdx.y;
    const unsigned gz = p.long_first ? blockIdx.y : blockIdx.z;
    o.tile_n = blockIdx.x; o.tile_m = (int)gy; o.tile = 0; o.which = 0;
    const i64 nbatch = p.nb1 * p.nb2;
    o.bz = (int)(gz % nbatch); o.split = (int)(gz / nbatch);
    o.b1 = o.bz / (int)p.nb2; o.b2 = o.bz % (int)p.nb2;
    i64 kb0 = (i64)o.split * p.kblocks_per_split, kb1 = kb0 + p.kblocks_per_split;
    if (kb1 > kblocks_total) kb1 = kblocks_total;
    if (p.causal == 2) { i64 lim = (((i64)o.tile_m + 1) * BM + p.bk - 1) / p.bk; if (kb1 > lim) kb1 = lim; }
    if (p.causal == 3) { i64 lo = ((i64)o.tile_m * BM) / p.bk; if (kb0 < lo) kb0 = lo; }
    o.kb0 = (int)kb0; o.nkb = (int)(kb1 > kb0 ? kb1 - kb0 : 0); o.whole = p.splits == 1;
    return true;
  }
};

// Store one 32-row x 32-column block of results held one row per lane (v[j] = column j of row `lane`).  The block is
// transposed through a 4 KB per-warp staging area (XOR-swizzled 16-byte units, conflict-free both ways) so that every store
// instruction writes four full 128-byte row segments instead of 32 scattered ones.
//   fin: apply alpha, beta * C and bias (final result); otherwise the raw sums are stored.
__device__ __forceinline__ void stage_put(float4* stg, int lane, int j4, float4 x) { stg[lane * 8 + (j4 ^ (lane & 7))] = x; }
__device__ __forceinline__ void stage_write_out(const TcParams& p, float4* stg, int lane, float* base, i64 rs, i64 row0, i64 col0, bool fin, bool vec_ok);
__device__ __forceinline__ void store_block(const TcParams& p, const uint32_t* v, float4* stg, int lane, float* base, i64 rs, i64 row0, i64 col0,
                                            bool fin, bool vec_ok) {
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4)
    stage_put(stg, lane, j4, make_float4(__uint_as_float(v[4 * j4]), __uint_as_float(v[4 * j4 + 1]), __uint_as_float(v[4 * j4 + 2]), __uint_as_float(v[4 * j4 + 3])));
  stage_write_out(p, stg, lane, base, rs, row0, col0, fin, vec_ok);
}
// Second half: read the staged block back one row segment per 8 lanes and store it (apply alpha / beta / biases when `fin`).
__device__ __forceinline__ void stage_write_out(const TcParams& p, float4* stg, int lane, float* base, i64 rs, i64 row0, i64 col0, bool fin, bool vec_ok) {
  __syncwarp();
  const int c4 = lane & 7;
  const i64 col = col0 + 4 * c4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    float4 x = stg[rr * 8 + (c4 ^ (rr & 7))];
    const i64 row = row0 + rr;
    if (row >= p.M || col >= p.N) continue;
    float* out = base + row * rs + col;
    float e[4] = {x.x, x.y, x.z, x.w};
    if (fin) {
      const float bm = p.bias_m ? p.bias_m[row] : 0.0f;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        e[t] *= p.alpha;
        if (col + t < p.N) {
          if (p.beta != 0.0f) e[t] += p.beta * out[t];
          if (p.bias) e[t] += p.bias[col + t];
          e[t] += bm;
        }
      }
    }
    if (vec_ok && col + 3 < p.N) *reinterpret_cast<float4*>(out) = make_float4(e[0], e[1], e[2], e[3]);
    else for (int t = 0; t < 4 && col + t < p.N; ++t) out[t] = e[t];
  }
  __syncwarp();
}

// The CTA owns a 128 x bn output tile at a time (see the file header for the roles of its warps).
// ACT: the instance whose epilogue also stores GELU(result) (kept apart: the activation's registers would spill the plain kernel).
template <bool ACT>
__global__ void __launch_bounds__(kThreads, 2)
k_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
          const __grid_constant__ CUtensorMap map_blo, const __grid_constant__ CUtensorMap map_alo, const __grid_constant__ CUtensorMap map_act,
          TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: raw ring [stages][ A | B ] (TMA destination, read by the MMA as the hi operand), lo ring [lstages][ A_lo | B_lo ]
  // (doubles as the epilogue's staging area: nothing converts while a tile is being stored), barriers.
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzle atoms need 1024-byte alignment in the shared window
  const int bn = p.bn, stages = p.stages, lstages = p.lstages;
  const int bk = p.bk;
  const uint32_t a_bytes = BM * bk * 4, b_bytes = (uint32_t)bn * bk * 4, raw_bytes = a_bytes + b_bytes;
  uint8_t* lo_ring = smem + (size_t)stages * raw_bytes;
  uint64_t* bars = (uint64_t*)(lo_ring + (size_t)lstages * raw_bytes);
  uint64_t* full = bars; uint64_t* empty = bars + stages; uint64_t* conv = bars + 2 * stages; uint64_t* lo_empty = conv + lstages;
  uint64_t* tmem_full = lo_empty + lstages;
  uint64_t* tmem_empty = tmem_full + 1;
  uint64_t* stg_free = tmem_empty + 1;          // pre-split B in the persistent modes: the epilogue has left the staging area (= the lo ring)
  uint32_t* tmem_slot = (uint32_t*)(stg_free + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.causal == 1 && !p.persistent && (i64)blockIdx.x * p.bn >= ((i64)blockIdx.y + 1) * BM) return;   // whole tile above the diagonal (nothing allocated yet)

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < lstages; ++s) { mbar_init(&conv[s], kConvWarps + (p.b_lo ? 1 : 0)); mbar_init(&lo_empty[s], 1); }    // (+1: the producer's expect_tx arrival for the pre-split lo part of B)
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, kConvWarps);
    mbar_init(stg_free, kConvWarps);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // tensor memory: bn columns hold the 128 x bn f32 accumulator rows of this CTA (so that two CTAs can share an SM's 512 columns)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  WorkIter wi; wi.init(p);
  Work wk;
  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------------------
    // One thread: everything it does per k-block is on the critical path, so ring position and phase are carried in
    // registers instead of being derived from the k-block count.
    if (lane == 0) {
      int it = 0;                       // k-blocks issued by this CTA so far
      int s = 0; uint32_t ph = 1;       // ring slot and the parity of `empty` that says the slot was released
      bool ok = true;
      const int amode = p.a_mn + p.a_fold, bmode = p.b_mn + p.b_fold;
      int unit = 0;
      while (ok && wi.next(p, wk)) {
        // pre-split B, persistent modes: the lo ring doubles as the epilogue's staging area, so the lo parts of this unit may not
        // land before the converter warps have finished the previous unit's epilogue
        if (p.b_lo && p.persistent && unit > 0 && !mbar_wait(stg_free, (uint32_t)(unit - 1) & 1, abort_flag)) { ok = false; break; }
        ++unit;
        const int ab2 = p.a_bcast2 ? 0 : wk.b2, ab1 = p.a_bcast1 ? 0 : wk.b1, bb2 = p.b_bcast2 ? 0 : wk.b2, bb1 = p.b_bcast1 ? 0 : wk.b1;
        const int m0 = wk.tile_m * BM, n0 = wk.tile_n * bn;
        int k = wk.kb0 * bk;
        for (int kb = 0; kb < wk.nkb; ++kb, ++it, k += bk) {
          if (it >= stages && !mbar_wait(&empty[s], ph, abort_flag)) { ok = false; break; }
          uint8_t* st = smem + (size_t)s * raw_bytes;
          mbar_arrive_expect_tx(&full[s], raw_bytes);
          tma_load_tile(st, &map_a, &full[s], amode, BM, m0, k, ab2, ab1, bk);
          if (p.b_conv == 1) {
            // tile rows n0 .. n0 + bn are the pixels (y0 .., all x) of image bb2; k = (tap row, position inside its run of 3 * C floats)
            tma_load_5d(st + a_bytes, &map_b, &full[s], k % p.cv_run, 0, n0 / p.cv_w, k / p.cv_run, bb2);
          } else if (p.b_conv == 2) {
            // k = (image, y, x) of the first of bk pixels; every 32-wide block of taps is one box (blocks past the last tap read zeros)
            const int kx = k % p.cv_w, ky = (k / p.cv_w) % p.cv_h, kn = k / (p.cv_w * p.cv_h);
            for (int j = 0; j < bn / 32; ++j) {
              const int nn = n0 + 32 * j;
              tma_load_5d(st + a_bytes + j * (bk * 128), &map_b, &full[s], nn % p.cv_run, kx, ky, nn / p.cv_run, kn);
            }
          } else
          tma_load_tile(st + a_bytes, &map_b, &full[s], bmode, bn, n0, k, bb2, bb1, bk);
          if (p.b_lo) {
            // the lo part of B lands straight in the lo stage (the converters fill only the A part); it completes on the stage's
            // `conv` barrier together with their arrivals
            const int l = it % lstages;                                   // (derived, not carried: this role has no register to spare)
            const uint32_t lph = (((uint32_t)(it / lstages)) & 1u) ^ 1u;    // parity of `lo_empty` that says the slot was released
            if (it >= lstages && !mbar_wait(&lo_empty[l], lph, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&conv[l], p.a_lo ? raw_bytes : b_bytes);
            tma_load_tile(lo_ring + (size_t)l * raw_bytes + a_bytes, &map_blo, &conv[l], bmode, bn, n0, k, bb2, bb1, bk);
            if (p.a_lo) tma_load_tile(lo_ring + (size_t)l * raw_bytes, &map_alo, &conv[l], amode, BM, m0, k, ab2, ab1, bk);
          }
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
      // after an abort: give the copies already issued a bounded time to land before the CTA exits
      if (*abort_flag)
        for (int kb = (it > stages ? it - stages : 0); kb < it; ++kb) {
          uint32_t addr = smem_u32(&full[kb % stages]), php = (uint32_t)(kb / stages) & 1, done = 0;
          for (uint32_t n = 0; n < (1u << 16) && !done; ++n)
            asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}" : "=r"(done) : "r"(addr), "r"(php) : "memory");
        }
      // (the pre-split lo copies complete on `conv`, which also needs the converters: polled for the same bounded time, as a delay)
      if (*abort_flag && p.b_lo)
        for (int kb = (it > lstages ? it - lstages : 0); kb < it; ++kb) {
          uint32_t addr = smem_u32(&conv[kb % lstages]), php = (uint32_t)(kb / lstages) & 1, done = 0;
          for (uint32_t n = 0; n < (1u << 16) && !done; ++n)
            asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}" : "=r"(done) : "r"(addr), "r"(php) : "memory");
        }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------------
    // One thread again: descriptors of every ring slot differ only in the start-address field, so they are advanced by
    // additions; nothing else is computed per k-block.
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, bn, p.a_mn, p.b_mn);
      const uint64_t a_hi0 = make_desc(smem_u32(smem), 0, p.a_mn, bk), b_hi0 = make_desc(smem_u32(smem) + a_bytes, 0, p.b_mn, bk);
      const uint64_t a_lo0 = make_desc(smem_u32(lo_ring), 0, p.a_mn, bk), b_lo0 = make_desc(smem_u32(lo_ring) + a_bytes, 0, p.b_mn, bk);
      const uint64_t a_ks = p.a_mn ? (1024 >> 4) : (32 >> 4), b_ks = p.b_mn ? (1024 >> 4) : (32 >> 4);   // second 8-wide k step of a k-block
      const uint64_t stage16 = raw_bytes >> 4;
      uint64_t a_hi = a_hi0, b_hi = b_hi0, a_lo = a_lo0, b_lo = b_lo0;
      int s = 0, l = 0; uint32_t lph = 0;
      bool ok = true;
      int unit = 0;
      while (ok && wi.next(p, wk)) {
        if (wk.nkb == 0) continue;
        if (unit > 0) {                 // the previous unit's accumulator must have left tensor memory
          ok = mbar_wait(tmem_empty, (uint32_t)(unit - 1) & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        uint32_t acc = 0;
        for (int kb = 0; kb < wk.nkb; ++kb) {
          ok = mbar_wait(&conv[l], lph, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          // one MMA covers 8 k: 32 bytes along a K-major row, or one 1024-byte k group of an MN-major tile
          mma_tf32(tmem_base, a_lo, b_hi, idesc, acc);
          mma_tf32(tmem_base, a_hi, b_lo, idesc, 1u);
          mma_tf32(tmem_base, a_hi, b_hi, idesc, 1u);
          mma_tf32(tmem_base, a_lo + a_ks, b_hi + b_ks, idesc, 1u);
          mma_tf32(tmem_base, a_hi + a_ks, b_lo + b_ks, idesc, 1u);
          mma_tf32(tmem_base, a_hi + a_ks, b_hi + b_ks, idesc, 1u);
          if (bk == 32) {         // two more 8-wide k steps
            mma_tf32(tmem_base, a_lo + 2 * a_ks, b_hi + 2 * b_ks, idesc, 1u);
            mma_tf32(tmem_base, a_hi + 2 * a_ks, b_lo + 2 * b_ks, idesc, 1u);
            mma_tf32(tmem_base, a_hi + 2 * a_ks, b_hi + 2 * b_ks, idesc, 1u);
            mma_tf32(tmem_base, a_lo + 3 * a_ks, b_hi + 3 * b_ks, idesc, 1u);
            mma_tf32(tmem_base, a_hi + 3 * a_ks, b_lo + 3 * b_ks, idesc, 1u);
            mma_tf32(tmem_base, a_hi + 3 * a_ks, b_hi + 3 * b_ks, idesc, 1u);
          }
          acc = 1u;
          // frees the raw stage and the lo stage once these MMAs have read them
          mma_commit(&empty[s]); mma_commit(&lo_empty[l]);
          if (++s == stages) { s = 0; a_hi = a_hi0; b_hi = b_hi0; } else { a_hi += stage16; b_hi += stage16; }
          if (++l == lstages) { l = 0; lph ^= 1; a_lo = a_lo0; b_lo = b_lo0; } else { a_lo += stage16; b_lo += stage16; }
        }
        if (ok) mma_commit(tmem_full);    // accumulator complete
        ++unit;
      }
    }
  } else {
    // ---- converters, then epilogue ------------------------------------------------------------
    const int cw = warp - 2, ct = cw * 32 + lane;            // 0 .. 255
    constexpr int kConvThreads = 32 * kConvWarps;
    const int q = warp & 3;                                  // TMEM lane quarter this warp may read
    const int half = cw >> 2, ncol_half = bn / 2;            // two warps share a lane quarter; each takes half the columns
    float4* stg = (float4*)(lo_ring + (size_t)cw * 4096);    // staging block of this warp (the lo ring is at least 32 KB)
    bool ok = true;
    int it = 0, unit = 0;
    int s = 0, l = 0; uint32_t ph = 0, lph = 1;   // ring slots; parities of `full` (tile landed) and `lo_empty` (lo slot released)
    while (wi.next(p, wk)) {            // every warp walks the whole list (the named barriers below need all of them), aborted or not
      for (int kb = 0; kb < wk.nkb && ok; ++kb, ++it) {
        if (it >= lstages) ok = mbar_wait(&lo_empty[l], lph, abort_flag);
        if (ok) ok = mbar_wait(&full[s], ph, abort_flag);
        if (!ok) break;
        float4* hi = (float4*)(smem + (size_t)s * raw_bytes);
        float4* lo = (float4*)(lo_ring + (size_t)l * raw_bytes);
        const int n4 = p.a_lo ? 0 : (p.b_lo ? (int)(a_bytes / 16) : (int)(raw_bytes / 16));     // what is left to split: nothing, the A part, or both parts
#pragma unroll 3
        for (int i = ct; i < n4; i += kConvThreads) {
          float4 x = hi[i], l;
          l.x = tf32_lo_of_raw(x.x); l.y = tf32_lo_of_raw(x.y); l.z = tf32_lo_of_raw(x.z); l.w = tf32_lo_of_raw(x.w);
          lo[i] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv[l]);
        if (++s == stages) { s = 0; ph ^= 1; }
        if (++l == lstages) { l = 0; lph ^= 1; }
      }
      // ---- epilogue of this unit ----
      bool have = ok;
      if (have && wk.nkb > 0) have = ok = mbar_wait(tmem_full, (uint32_t)unit & 1, abort_flag);
      if (have) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const i64 row0 = (i64)wk.tile_m * BM + q * 32;
      const bool streamk_part = p.persistent && !wk.whole;
      float* cbase = p.C + (i64)wk.b1 * p.c_b1 + (i64)wk.b2 * p.c_b2;
      const bool c_vec = (p.c_rs & 3) == 0 && (((uintptr_t)p.C | (uintptr_t)(p.c_b1 * 4) | (uintptr_t)(p.c_b2 * 4)) & 15) == 0;
      float* pbase = p.partial + ((i64)wk.split * (p.nb1 * p.nb2) + wk.bz) * p.M * p.N;       // split-K scratch of the tiled mode
      const i64 slot_floats = (i64)BM * bn;
      float4* slot = (float4*)p.ws + ((i64)(2 * blockIdx.x + wk.which) * slot_floats) / 4;     // stream-K partial of this CTA
      if (have) {
        for (int c0 = half * ncol_half; c0 < (half + 1) * ncol_half; c0 += 32) {
          i64 col0 = (i64)wk.tile_n * bn + c0;
          if (col0 >= p.N) break;
          uint32_t r[32];
          if (wk.nkb > 0) {
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (streamk_part) {
            // partial sums of a tile shared with other groups: [32-column block][lane quarter][4-column group][lane], 512 contiguous bytes per store
            float4* dst = slot + ((c0 >> 5) * 4 + q) * 256 + lane;
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4)
              dst[j4 * 32] = make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]), __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3]));
          } else if (p.tma_out) {
            // final values (or raw split-K sums) are formed in registers, staged, and stored by the copy engine: the store of
            // one block overlaps the read of the next from tensor memory
            if (wk.whole) {
              const float bm = (p.bias_m && row0 + lane < p.M) ? p.bias_m[row0 + lane] : 0.0f;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float e = __uint_as_float(r[j]) * p.alpha;
                if (p.bias && col0 + j < p.N) e += __ldg(p.bias + col0 + j);
                r[j] = __float_as_uint(e + bm);
              }
            }
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4)
              stage_put(stg, lane, j4, make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]), __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3])));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && row0 < p.M) {
              if (wk.whole) tma_store_block(&map_c, stg, (int)col0, (int)row0, wk.b2, wk.b1);
              else tma_store_block(&map_c, stg, (int)col0, (int)row0, (int)((i64)wk.split * (p.nb1 * p.nb2) + wk.bz), 0);
            }
            if (ACT && p.act && wk.whole) {
              // the activation of the block just stored, from the same registers: GELU as the standalone kernel computes it
              // (crates/vearo-backend-cpu/src/lib.rs:458-497)
              // (staged in a block of its own, in the raw ring: this launch mode has one unit per CTA, whose loads are all consumed)
              float4* stg2 = (float4*)(smem + (size_t)cw * 4096);
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(gelu_value(__uint_as_float(r[j])));
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4)
                stage_put(stg2, lane, j4, make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]), __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3])));
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0 && row0 < p.M) tma_store_block(&map_act, stg2, (int)col0, (int)row0, wk.b2, wk.b1);
            }
          } else if (wk.whole) {
            store_block(p, r, stg, lane, cbase, p.c_rs, row0, col0, true, c_vec);
          } else {
            store_block(p, r, stg, lane, pbase, p.N, row0, col0, false, (p.N & 3) == 0);
          }
        }
      }
      if (p.tma_out) { if (lane == 0) tma_store_wait_read(); __syncwarp(); }     // the staging area is the lo ring of the next unit
      if (wk.nkb > 0) {                 // the accumulator has been read: the next unit's first MMA may overwrite it
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0 && have) mbar_arrive(tmem_empty);
        ++unit;
      }
      if (streamk_part) {
        // Who finishes the tile?  Every CTA holding a part of it publishes its partial sums, then counts itself in; the CTA that
        // counts last adds all parts in k order (its own included, read back from memory: the order of the additions is then
        // the same whichever CTA happens to be last) and writes the result.  Nobody waits for anybody.
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kConvWarps) : "memory");
        const i64 kblocks_total = (p.K + p.bk - 1) / p.bk;
        const i64 x0 = (i64)wk.tile * kblocks_total, G = gridDim.x, W = p.total_kb;
        // first and last group whose range meets [x0, x0 + kblocks_total): group c starts at floor(c*W/G)
        i64 cf = ((x0 + 1) * G + W - 1) / W - 1;
        while (cf + 1 < G && ((cf + 1) * W) / G <= x0) ++cf;
        while (cf > 0 && (cf * W) / G > x0) --cf;
        i64 cl = ((x0 + kblocks_total) * G + W - 1) / W - 1;
        while (cl + 1 < G && ((cl + 1) * W) / G <= x0 + kblocks_total - 1) ++cl;
        while (cl > 0 && (cl * W) / G > x0 + kblocks_total - 1) --cl;
        const int np = (int)(cl - cf + 1);
        int* counter = p.counters + wk.tile;
        if (ct == 0) {
          int last = 0;
          if (!*abort_flag) {
            int old = atomicAdd(counter, 1);
            if (old == np - 1) { last = 1; *counter = 0; }     // reset for the next launch (nobody else touches it any more)
          }
          *last_flag = last;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kConvWarps) : "memory");
        const int last = *last_flag;
        if (last && !*abort_flag) {
          __threadfence();
          for (int c0 = half * ncol_half; c0 < (half + 1) * ncol_half; c0 += 32) {
            i64 col0 = (i64)wk.tile_n * bn + c0;
            if (col0 >= p.N) break;
            // part by part, accumulating in the staging block itself (every thread re-reads only what it wrote): eight loads in
            // flight per thread, and no accumulator registers beyond the eight values just loaded
            const i64 unit = ((c0 >> 5) * 4 + q) * 256 + lane;
            if (p.tma_out) { if (lane == 0) tma_store_wait_read(); __syncwarp(); }
            for (int i = 0; i < np; ++i) {
              const i64 c = cf + i;
              const int which = ((c * W) / G >= x0) ? 0 : 1;
              const float4* src = (const float4*)p.ws + ((2 * c + which) * slot_floats) / 4 + unit;
              float4 x[8];
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) x[j4] = __ldcg(src + j4 * 32);
              if (i == 0) {
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) stage_put(stg, lane, j4, x[j4]);
              } else {
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                  float4 a = stg[lane * 8 + (j4 ^ (lane & 7))];
                  a.x += x[j4].x; a.y += x[j4].y; a.z += x[j4].z; a.w += x[j4].w;
                  stage_put(stg, lane, j4, a);
                }
              }
            }
            if (p.tma_out) {          // finish row `lane` of the staged block in place, then hand the block to the copy engine
              const float bm = (p.bias_m && row0 + lane < p.M) ? p.bias_m[row0 + lane] : 0.0f;
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) {
                float4 a = stg[lane * 8 + (j4 ^ (lane & 7))];
                float e[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  e[t] *= p.alpha;
                  if (p.bias && col0 + 4 * j4 + t < p.N) e[t] += __ldg(p.bias + col0 + 4 * j4 + t);
                  e[t] += bm;
                }
                stage_put(stg, lane, j4, make_float4(e[0], e[1], e[2], e[3]));
              }
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0 && row0 < p.M) tma_store_block(&map_c, stg, (int)col0, (int)row0, wk.b2, wk.b1);
            } else {
              stage_write_out(p, stg, lane, cbase, p.c_rs, row0, col0, true, c_vec);
            }
          }
          if (p.tma_out) { if (lane == 0) tma_store_wait_read(); __syncwarp(); }
        }
      }
      // the staging area is the lo ring, and last_flag is per unit: nobody starts converting the next unit before all have finished this one
      if (p.persistent) asm volatile("bar.sync 1, %0;" ::"n"(32 * kConvWarps) : "memory");
      if (p.b_lo && p.persistent && lane == 0) mbar_arrive(stg_free);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.err, ERRBIT_WAIT_TIMEOUT);
}

// Sum the split-K partial tiles in split order, then apply alpha / beta / bias.
__global__ void k_splitk_reduce(const float* __restrict__ partial, float* __restrict__ C, const float* __restrict__ bias, const float* __restrict__ bias_m,
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
    if (bias_m) v += bias_m[m];
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

// lo[i] = the TF32 remainder of x[i], exactly what the converters compute
__global__ void __launch_bounds__(256) k_tf32_lo(const float* __restrict__ x, float* __restrict__ lo, i64 n) {
  const i64 stride = (i64)gridDim.x * blockDim.x;
  const i64 n4 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(lo)) & 15) == 0 ? n / 4 : 0;
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<float4*>(lo)[i] = make_float4(tf32_lo_of_raw(v.x), tf32_lo_of_raw(v.y), tf32_lo_of_raw(v.z), tf32_lo_of_raw(v.w));
  }
  for (i64 i = n4 * 4 + blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += stride) lo[i] = tf32_lo_of_raw(x[i]);
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
int make_map(CUtensorMap* map, const Operand& o, i64 K, i64 nb1, i64 nb2, int box_rows, int bk, bool* folded) {
  i64 d2 = o.bc2 ? 1 : nb2, d3 = o.bc1 ? 1 : nb1;
  *folded = o.mn && (o.rows % 32) == 0;
  // a batch level of extent 1 never advances: any 16-byte-multiple stride is acceptable there
  i64 plane = o.mn ? o.rs * (K > 0 ? K : 1) : o.rs * (o.rows > 0 ? o.rows : 1);
  i64 s2 = d2 > 1 ? o.b2 : plane, s3 = d3 > 1 ? o.b1 : s2 * d2;
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
  if (!o.mn) {            // K-major: one box of BK x box_rows, 64-byte swizzle
    dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)o.rows; dims[2] = 1;
    strides[0] = (cuuint64_t)o.rs * 4; strides[1] = (cuuint64_t)plane * 4;
    box[0] = (cuuint32_t)bk; box[1] = (cuuint32_t)box_rows; box[2] = 1;
  } else if (*folded) {   // MN-major, rows a multiple of 32: {32, K, rows/32}, one box of 32 x BK x box_rows/32, 128-byte swizzle on 32-byte units
    dims[0] = 32; dims[1] = (cuuint64_t)K; dims[2] = (cuuint64_t)(o.rows / 32);
    strides[0] = (cuuint64_t)o.rs * 4; strides[1] = 128;
    box[0] = 32; box[1] = (cuuint32_t)bk; box[2] = (cuuint32_t)(box_rows / 32);
  } else {                // MN-major, any row count: boxes of 32 x BK
    dims[0] = (cuuint64_t)o.rows; dims[1] = (cuuint64_t)K; dims[2] = 1;
    strides[0] = (cuuint64_t)o.rs * 4; strides[1] = (cuuint64_t)plane * 4;
    box[0] = 32; box[1] = (cuuint32_t)bk; box[2] = 1;
  }
  dims[3] = (cuuint64_t)d2; dims[4] = (cuuint64_t)d3;
  strides[2] = (cuuint64_t)s2 * 4; strides[3] = (cuuint64_t)s3 * 4;
  box[3] = 1; box[4] = 1;
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, (void*)o.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           o.mn ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(VB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return VB_OK;
}

// Map of the output (or of the split-K scratch) for the epilogue's block stores: {columns, rows, inner batch, outer batch}, boxes of
// 32 x 32 with the 128-byte swizzle.  False when the layout cannot be described (unaligned base or strides): the kernel then
// stores with ordinary instructions.
bool make_out_map(CUtensorMap* map, float* base, i64 N, i64 M, i64 d2, i64 d3, i64 rs, i64 s2, i64 s3) {
  if (((uintptr_t)base & 15) || (rs & 3) || rs <= 0 || N <= 0 || M <= 0) return false;
  if (d2 <= 1) { d2 = 1; s2 = rs * M; }
  if (d3 <= 1) { d3 = 1; s3 = s2 * d2; }
  if ((s2 & 3) || (s3 & 3) || s2 <= 0 || s3 <= 0) return false;
  const i64 lim = (i64)1 << 38;     // strides in bytes must stay below 2^40
  if (rs >= lim || s2 >= lim || s3 >= lim || N > 0x7fffffff || M > 0x7fffffff || d2 > 0x7fffffff || d3 > 0x7fffffff) return false;
  cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)d2, (cuuint64_t)d3};
  cuuint64_t strides[3] = {(cuuint64_t)rs * 4, (cuuint64_t)s2 * 4, (cuuint64_t)s3 * 4};
  cuuint32_t box[4] = {32, 32, 1, 1}, estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The unfolded matrix of a zero-padded NHWC batch xp [n, H + 2, W + 2, C] (3 x 3 window, stride 1) as a tensor map:
// dims {3C (tap column j and channel, contiguous), W (x), H (y), 3 (tap row i), n}; element (jc, x, y, i, n) = xp[n, y + i, x, jc].
// mode 1: boxes {bk, W, rows / W, 1, 1} (K-major tile of `rows` pixels); mode 2: boxes {32, bx, bk / bx, 1, 1} (MN-major, bk pixels).
bool make_conv_map(CUtensorMap* map, const ConvOperand& cv, int mode, int rows, int bk) {
  const i64 C = cv.c, W = cv.w, H = cv.h;
  if (((uintptr_t)cv.xp & 15) || (C & 3) || W <= 0 || H <= 0) return false;
  cuuint64_t dims[5] = {(cuuint64_t)(3 * C), (cuuint64_t)W, (cuuint64_t)H, 3, (cuuint64_t)cv.n};
  cuuint64_t strides[4] = {(cuuint64_t)C * 4, (cuuint64_t)(W + 2) * C * 4, (cuuint64_t)(W + 2) * C * 4, (cuuint64_t)(H + 2) * (W + 2) * C * 4};
  cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
  if (mode == 1) {
    if (rows % W || rows / W > 256 || W > 256) return false;
    box[0] = (cuuint32_t)bk; box[1] = (cuuint32_t)W; box[2] = (cuuint32_t)(rows / W); box[3] = 1; box[4] = 1;
  } else {
    const i64 bx = W < bk ? W : bk;
    if (bk % bx || W % bx) return false;
    box[0] = 32; box[1] = (cuuint32_t)bx; box[2] = (cuuint32_t)(bk / bx); box[3] = 1; box[4] = 1;
  }
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, (void*)cv.xp, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           mode == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int* g_tile_counters = nullptr;     // stream-K arrival counters (zero between launches)

}  // namespace

int64_t g_tc_launches = 0;          // launches of k_gemm_tc so far (vb_tc_launch_count)

// After a device-side wait ran out a tile may have been left half counted: start from zero again.
int gemm_tc_reset_state() {
  if (g_tile_counters) VB_CUDA(cudaMemsetAsync(g_tile_counters, 0, 4096 * sizeof(int), ctx().stream));
  return VB_OK;
}

int launch_tf32_lo(const float* x, float* lo, i64 n) {
  if (n <= 0) return VB_OK;
  ProfScope prof("tf32_lo", 8.0 * (double)n);
  i64 blocks = (n / 4 + 255) / 256, cap = (i64)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap; if (blocks < 1) blocks = 1;
  k_tf32_lo<<<(unsigned)blocks, 256, 0, ctx().stream>>>(x, lo, n);
  VB_LAUNCH_CHECK();
  return VB_OK;
}

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
    Operand mn{p, rows, cs, sb1, sb2, bc1, bc2, true};
    if (rs == 1 && rows >= 32 && tma_ok(mn, g.nb1, g.nb2)) { *o = mn; return VB_OK; }
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
  const int b_conv = g.conv ? g.conv->mode : 0;
  if (b_conv) {
    // B is described by the padded image batch itself; the geometry has to fit whole boxes
    const ConvOperand& cv = *g.conv;
    if (hold_a.p || (3 * cv.c) % 32 || (b_conv == 1 && (g.nb1 != 1 || g.nb2 != cv.n || g.N != cv.h * cv.w || g.K != 9 * cv.c)) ||
        (b_conv == 2 && (nb != 1 || g.N != 9 * cv.c || g.K != cv.n * cv.h * cv.w || (cv.h * cv.w) % 32))) return VB_OK;
    ob = Operand{cv.xp, g.N, 0, 0, 0, false, false, b_conv == 2};
  } else
  VB_TRY(prepare(g.B, g.N, g.b_cs, g.b_rs, g.b_b1, g.b_b2, hold_b, &ob));   // B^T rows are the columns of B

  TcParams p{};
  // 64-wide tiles do a quarter of the work of 256-wide ones per k-block but pay the same hand-offs: twice the k per stage
  const int bk = (g.N <= 64 && g.K >= 64) ? 32 : BK;
  const i64 kblocks = (g.K + bk - 1) / bk;
  const i64 slots = (i64)ctx().sm_count * 2;     // resident CTAs: two per SM
  p.bn = g.N <= 64 ? 64 : (g.N <= 128 ? 128 : 256);
  int splits = 1;
  if (p.bn == 256) {
    // Tile width and split-K factor: minimise an estimate of the run time in units of one 256-wide k-block.
    // A k-block of a 128-wide tile costs ~0.62 of a 256-wide one (same A traffic for half the flops); the epilogue of a
    // tile costs about 10 (256) / 6 (128) k-blocks; split-K adds a pass over the partial tiles.
    double best = 1e300;
    // 192-wide tiles only where they make a single wave fuller (8192 x 768 . 768 x 768: 256 tiles instead of 192 for 296 slots,
    // 62.7 us against 74.7 us); on multi-wave products they measured no better than 256
    for (int bn : {256, 192, 128}) {
      i64 tiles = ((g.M + BM - 1) / BM) * ((g.N + bn - 1) / bn) * nb;
      for (int sk : {1, 2, 3, 4, 5, 6, 8, 10, 12, 16}) {
        if (sk > 1 && kblocks / sk < 24) break;
        if (bn == 192 && (sk > 1 || tiles > slots)) break;
        i64 units = tiles * sk, waves = (units + slots - 1) / slots;
        double kb_cost = bn == 256 ? 1.0 : (bn == 192 ? 0.81 : 0.62), epi = bn == 256 ? 10.0 : (bn == 192 ? 8.0 : 6.0);
        double t = (double)waves * ((double)((kblocks + sk - 1) / sk) * kb_cost + epi);
        if (sk > 1) t += (double)tiles * (double)sk * epi * 0.5 / (double)slots + epi;      // partial tiles written, then summed
        if (t < best * 0.97) { best = t; p.bn = bn; splits = sk; }
      }
    }
  } else {
    i64 tiles = ((g.M + BM - 1) / BM) * nb;
    if (tiles < slots && kblocks >= 48) { splits = (int)((slots + tiles - 1) / tiles); if (splits > kblocks / 24) splits = (int)(kblocks / 24); if (splits < 1) splits = 1; }
  }
  // Stream-K instead of split-K where a tile would be shared by three or four CTAs at most: the k-blocks of all tiles are
  // dealt evenly to one CTA per slot and shared tiles are finished inside the kernel (no pass over partial tiles).
  // Measured slower than plain tiles when nothing needs splitting (CTAs at different k positions stop sharing
  // operand lines in L2) and when a tile has many parts (the CTA finishing a tile adds them alone).
  bool persistent = false;
  i64 streamk_groups = 0;
  // ... and where whole 256-wide tiles would fill one wave and less than half of a second one (measured on 4096 x 1024 . 1024 x 3072:
  // 384 tiles for 296 slots, 157 us against 187 us with 128-wide tiles)
  const i64 tiles256 = ((g.M + BM - 1) / BM) * ((g.N + 255) / 256) * nb;
  const bool ragged_wave = splits == 1 && g.N > 128 && tiles256 > slots && 2 * tiles256 <= 3 * slots && kblocks >= 32;
  if (!g.causal && p.bn >= 128 && (splits > 1 || ragged_wave)) {
    int bn = 256;
    if (g.N <= 128 || ((g.N + 127) / 128) * 128 * 5 <= ((g.N + 255) / 256) * 256 * 4) bn = 128;     // a 256-wide last tile would be mostly padding
    i64 tiles = ((g.M + BM - 1) / BM) * ((g.N + bn - 1) / bn) * nb;
    i64 W = tiles * kblocks, G = slots;
    if (G > W / 8) G = W / 8;                          // at least 8 k-blocks per CTA
    if (G < 1) G = 1;
    // (very long K: plain split-K measured faster, 2.74 ms against 2.90 ms for 8192 x 50304 . 50304 x 768)
    if (tiles <= 4096 && W / G >= kblocks / 3 && kblocks <= 1024) { persistent = true; streamk_groups = G; p.bn = bn; splits = 1; }
  }
  p.tmem_cols = p.bn <= 64 ? 64 : (p.bn <= 128 ? 128 : 256);
  const i64 tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + p.bn - 1) / p.bn;
  // Short-K products with many tiles per slot (attention scores, the vocabulary projection): resident CTAs take whole tiles
  // round-robin instead of one launch slot per tile.
  const int causal_eff = (splits == 1 && !persistent && g.M == (g.causal == 1 ? g.N : g.K)) ? g.causal : 0;
  i64 live_per_batch = tiles_m * tiles_n;
  if (causal_eff == 1) {
    live_per_batch = 0;
    for (i64 m = 0; m < tiles_m; ++m) { i64 c = ((m + 1) * BM + p.bn - 1) / p.bn; live_per_batch += c < tiles_n ? c : tiles_n; }
  }
  const bool round_robin = !persistent && splits == 1 && kblocks <= 64 && causal_eff <= 1 && live_per_batch * nb >= 4 * slots;
  const size_t raw_bytes = (size_t)(BM + p.bn) * bk * 4;
  p.bk = bk;
  // Small rings on purpose: two CTAs then share an SM, and one CTA's epilogue and pipeline bubbles are covered by
  // the other's main loop; measured faster than one CTA per SM with a deep ring.  The lo ring is at least 32 KB
  // because the epilogue stages its stores there.
  p.lstages = (int)((32 * 1024 + raw_bytes - 1) / raw_bytes); if (p.lstages < 2) p.lstages = 2;
  p.stages = (int)((100 * 1024 - (size_t)p.lstages * raw_bytes) / raw_bytes); if (p.stages > 4) p.stages = 4; if (p.stages < 2) p.stages = 2;
  p.kblocks_per_split = (int)((kblocks + splits - 1) / splits);
  splits = (int)((kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split);
  p.splits = splits;
  if (!persistent && !round_robin && (tiles_m > 65535 || nb * splits > 65535)) return VB_OK;

  CUtensorMap map_a, map_b;
  bool fold_a = false, fold_b = false;
  VB_TRY(make_map(&map_a, oa, g.K, g.nb1, g.nb2, BM, bk, &fold_a));
  if (b_conv) {
    const ConvOperand& cv = *g.conv;
    // tiles must be whole image rows (mode 1) / the k-blocks whole runs of pixels inside an image (mode 2); split-K ranges and the
    // stream-K deal keep k-block granularity, so they need nothing more
    if ((b_conv == 1 && p.bn % cv.w) || (3 * cv.c) % bk ||
        !make_conv_map(&map_b, cv, b_conv, p.bn, bk)) return VB_OK;
    p.b_conv = b_conv; p.cv_run = (int)(3 * cv.c); p.cv_w = (int)cv.w; p.cv_h = (int)cv.h;
    if (g.conv_used) *g.conv_used = 1;
  } else
  VB_TRY(make_map(&map_b, ob, g.K, g.nb1, g.nb2, p.bn, bk, &fold_b));
  p.a_fold = fold_a; p.b_fold = fold_b;
  Temp part, ws;
  if (splits > 1) VB_TRY(scratch_alloc((size_t)((i64)splits * nb * g.M * g.N) * sizeof(float), &part.p));
  if (persistent) {
    if (!g_tile_counters) {
      VB_CUDA(cudaMalloc(&g_tile_counters, 4096 * sizeof(int)));
      VB_CUDA(cudaMemsetAsync(g_tile_counters, 0, 4096 * sizeof(int), ctx().stream));
    }
    VB_TRY(scratch_alloc((size_t)streamk_groups * 2 * BM * p.bn * sizeof(float), &ws.p));
    p.persistent = 1; p.total_kb = tiles_m * tiles_n * nb * kblocks; p.tiles_m = tiles_m; p.tiles_n = tiles_n;
    p.ws = (float*)ws.p; p.counters = g_tile_counters;
  }
  p.C = g.C; p.bias = g.bias; p.bias_m = g.bias_m; p.partial = (float*)part.p;
  p.M = g.M; p.N = g.N; p.K = g.K; p.c_rs = g.c_rs; p.c_b1 = g.c_b1; p.c_b2 = g.c_b2; p.nb1 = g.nb1; p.nb2 = g.nb2;
  p.a_bcast1 = oa.bc1; p.a_bcast2 = oa.bc2; p.b_bcast1 = ob.bc1; p.b_bcast2 = ob.bc2;
  p.a_mn = oa.mn; p.b_mn = ob.mn;
  p.alpha = g.alpha; p.beta = g.beta; p.err = ctx().d_err;
  p.causal = causal_eff;
  p.long_first = (!persistent && !round_robin && causal_eff >= 2 && tiles_m <= 65535 && nb * splits <= 65535) ? 1 : 0;
  if (round_robin) { p.persistent = 2; p.tiles_m = tiles_m; p.tiles_n = tiles_n; p.live_per_batch = live_per_batch; p.live_tiles = live_per_batch * nb; }

  // Results leave through the copy engine when the layout allows and nothing has to be read back (beta = 0).
  CUtensorMap map_c, map_act;
  memset(&map_c, 0, sizeof map_c); memset(&map_act, 0, sizeof map_act);
  if (g.beta == 0.0f) {
    if (splits == 1) p.tma_out = make_out_map(&map_c, g.C, g.N, g.M, g.nb2, g.nb1, g.c_rs, g.c_b2, g.c_b1) ? 1 : 0;
    else p.tma_out = make_out_map(&map_c, (float*)part.p, g.N, g.M, (i64)splits * nb, 1, g.N, g.M * g.N, 0) ? 1 : 0;
  }
  // GELU of the result as a second output of the epilogue (same layout as C): whole tiles stored by the copy engine only; in
  // every other mode the caller runs the activation as a kernel of its own
  if (g.act_out && p.tma_out && splits == 1 && !persistent && !round_robin && g.alpha == 1.0f && (size_t)p.stages * raw_bytes >= 32 * 1024 &&
      make_out_map(&map_act, g.act_out, g.N, g.M, g.nb2, g.nb1, g.c_rs, g.c_b2, g.c_b1)) {
    p.act = 1;
    if (g.act_fused) *g.act_fused = 1;
  }

  // Pre-split lo part of B: B consumed in place (the lo plane has B's layout).  (In the persistent modes the
  // producer holds the lo parts of the next tile back until the epilogue has left the lo ring, its staging area.)
  CUtensorMap map_blo;
  memset(&map_blo, 0, sizeof map_blo);
  if (g.B_lo && !hold_b.p) {
    Operand obl = ob; obl.p = g.B_lo;
    bool f2 = false;
    if (tma_ok(obl, g.nb1, g.nb2) && make_map(&map_blo, obl, g.K, g.nb1, g.nb2, p.bn, bk, &f2) == VB_OK && f2 == fold_b) p.b_lo = 1;
  }
  CUtensorMap map_alo;
  memset(&map_alo, 0, sizeof map_alo);
  if (p.b_lo && g.A_lo && !hold_a.p) {
    Operand oal = oa; oal.p = g.A_lo;
    bool f2 = false;
    if (tma_ok(oal, g.nb1, g.nb2) && make_map(&map_alo, oal, g.K, g.nb1, g.nb2, BM, bk, &f2) == VB_OK && f2 == fold_a) p.a_lo = 1;
  }

  size_t smem = (size_t)(p.stages + p.lstages) * raw_bytes + (2 * p.stages + 2 * p.lstages + 3) * sizeof(uint64_t) + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA(cudaFuncSetAttribute(k_gemm_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    VB_CUDA(cudaFuncSetAttribute(k_gemm_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
  {
    static int shapes = -1;
    if (shapes < 0) { const char* e = getenv("VB200_PROF_SHAPES"); shapes = (e && e[0] == '1') ? 1 : 0; }
    char fam[96];
    if (shapes) snprintf(fam, sizeof fam, "gemm_tc M%lld N%lld K%lld nb%lld a%d b%d bn%d sk%d%s", (long long)g.M, (long long)g.N, (long long)g.K, (long long)nb, (int)oa.mn, (int)ob.mn, p.bn, splits, persistent ? " streamk" : (round_robin ? " roundrobin" : ""));
    else snprintf(fam, sizeof fam, "%s", nb > 1 ? "gemm_tc_batched" : "gemm_tc");
    // flops of the tiles and k ranges that are actually issued (a causal product skips or clamps some), next to the dense count
    const double dense = 2.0 * (double)g.M * (double)g.N * (double)g.K * (double)nb;
    double issued = dense;
    if (causal_eff == 1) issued = 2.0 * (double)live_per_batch * BM * p.bn * (double)g.K * (double)nb;
    else if (causal_eff >= 2) {
      issued = 0.0;
      for (i64 m = 0; m < tiles_m; ++m) {
        i64 kr = causal_eff == 2 ? ((m + 1) * BM < g.K ? (m + 1) * BM : g.K) : (g.K - m * BM > 0 ? g.K - m * BM : 0);
        issued += 2.0 * BM * (double)g.N * (double)kr * (double)nb;
      }
    }
    ProfScope prof(fam, issued < dense ? issued : dense, dense);
    dim3 grid((unsigned)tiles_n, (unsigned)tiles_m, (unsigned)(nb * splits));
    if (p.long_first) grid = dim3((unsigned)tiles_n, (unsigned)(nb * splits), (unsigned)tiles_m);
    if (persistent) grid = dim3((unsigned)streamk_groups, 1, 1);
    if (round_robin) grid = dim3((unsigned)slots, 1, 1);
    if (p.act) k_gemm_tc<true><<<grid, kThreads, smem, ctx().stream>>>(map_a, map_b, map_c, map_blo, map_alo, map_act, p);
    else k_gemm_tc<false><<<grid, kThreads, smem, ctx().stream>>>(map_a, map_b, map_c, map_blo, map_alo, map_act, p);
    VB_LAUNCH_CHECK();
    ++g_tc_launches;
    if (splits > 1) {
      i64 total = nb * g.M * g.N;
      i64 blocks = (total + 255) / 256, cap = (i64)ctx().sm_count * 16; if (blocks > cap) blocks = cap;
      k_splitk_reduce<<<(unsigned)blocks, 256, 0, ctx().stream>>>((const float*)part.p, g.C, g.bias, g.bias_m, g.M, g.N, g.nb2, nb, splits,
                                                                   g.c_rs, g.c_b1, g.c_b2, g.alpha, g.beta);
      VB_LAUNCH_CHECK();
    }
  }
  *handled = true;
  return VB_OK;
}

}  // namespace vb
