// Tensor-core TPA forward for sm_100a: bf16 factors, head_dim 64 or 128, lengths that are
// multiples of 128.  Replaces _fwd_kernel (tpa/tpa.py:245-443) for those shapes.
//
// One CTA owns 256 query rows (two 128-row units) of one head of one batch element and
// walks the key/value rows 128 at a time.  Two variants share the softmax and MMA roles and
// differ in where the per-head Q, K, V tiles are rebuilt from the rank factors
// (Q, K, V = sums over rank of a[row, r, head] * b[row, r, :], tpa/tpa.py:317,364,417):
//
//   FUSED   the attention kernel rebuilds them itself: 8 warps turn factor rows into
//           shared-memory tiles while the tensor pipe works.  No scratch memory.  Every CTA
//           of a head rebuilds the K/V tiles it visits, so this is the choice when there is
//           one CTA per head (lq <= 256) and the rebuild is not repeated.
//   STAGED  a staging kernel rebuilds every 128-row tile of Q, K and V once, already in the
//           swizzled shared-memory image, into caller scratch; the attention kernel then
//           only moves 16/32 KB tiles with cp.async.bulk.  For long sequences this removes
//           the lq/256-fold repetition of the rebuild (64x on average at T = 32768).
//
// Roles, by warp:
//   FUSED   warps 0-3 / 4-7: online softmax of unit 0 / unit 1, one thread per query row
//           (= TMEM lane); warps 8-11 / 12-15: rebuild the K / V tile (all eight rebuild Q once
//           at the start); warp 16: issues tcgen05.mma: S_u = Q_u K^T (fp32 in TMEM), O_u += P_u V
//   STAGED  warps 0-7 / 8-15: online softmax of unit 0 / unit 1, two threads per query row
//           (each takes 64 of the 128 keys of a tile and half of the accumulator columns);
//           warp 16: one thread issues the bulk copies of the staged tiles; warp 17: one thread
//           issues the logits S_u = Q_u K^T; warp 18: one thread issues O_u += P_u V
//
// The 1/R_q, 1/R_k means and sm_scale * log2(e) are folded into Q once; the 1/R_k of V is
// applied with the final 1/l.  K and V tiles are double buffered, in the 128-byte-swizzled
// layout the tcgen05 shared-memory descriptors describe.
//
// FUSED: P (bf16) overwrites S in TMEM and feeds the second MMA from there, so per unit
// softmax(j) -> P V(j) -> S(j+1) -> softmax(j+1) is one serial chain; the two units alternate on
// the tensor pipe and the softmax of one overlaps the MMAs of the other.
//
// STAGED breaks that chain.  A softmax thread takes its 64 logits into registers the moment
// they are complete and releases the columns; P gets columns of its own.  The next logits of a
// unit are therefore computed while its softmax still works on the current ones, and only
// P V waits for the softmax.  (With D = 128, TMEM has room for one set of logit columns beside
// P0, P1, O0, O1: the two units use it in turn, which also keeps their exponentials apart on
// the MUFU pipe.)  Issuing a tile's eight MMAs holds the issuing thread for about as long as
// the tensor pipe needs for what is queued ahead of them, so logits and P V have a thread each:
// neither sits in an issue while an event the other could act on arrives.  Measured (cycle
// counters, longest CTA, T = 16384): 3590 cycles per 256 x 128 tile pair with P over S and one
// issuing thread, 4100 with the logits drained but one issuing thread, 2900 with two.
//
// The running maximum is only raised when a tile exceeds it by more than 2^8 (the accumulator
// and row sum are then rescaled); the final 1/l division makes the result independent of which
// maximum was subtracted.  STAGED: each thread finds the maximum of its 64 logits, one one-bit
// vote of the two warps that share the rows says whether any row needs a raise, and only then
// do the halves exchange their maxima through shared memory.
//
// Every mbarrier wait is bounded: after ~2^28 cycles the waiter records where it gave up in
// the status block, raises a CTA-wide abort flag that makes all later waits fall through,
// and the CTA runs to its normal end (TMEM is freed).
#include <math_constants.h>

#include <climits>

#include <type_traits>

#include "sm100_ptx.cuh"
#include "tpa_common.cuh"

namespace tpa {
namespace {

using namespace ptx;

constexpr int kRebuildWarps = 8;
template <bool STAGED>
struct Roles {
  // STAGED: two softmax threads per query row (16 warps); FUSED: one (8 warps)
  static constexpr int kSoftmaxWarps = STAGED ? 16 : 8;
  static constexpr int kProducerWarps = STAGED ? 1 : kRebuildWarps;
  static constexpr int kMmaWarp = kSoftmaxWarps + kProducerWarps;
  // STAGED has two issuing warps: kMmaWarp issues the logits S = Q K^T, kMmaWarp + 1 the P V
  static constexpr int kMmaWarps = STAGED ? 2 : 1;
  static constexpr int kThreads = (kMmaWarp + kMmaWarps) * 32;  // STAGED 19 warps, FUSED 17
};
constexpr int kUnitRows = 128;
constexpr int kTileKv = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr float kOptimisticSumLimit = 32768.f;  // 2^15, see the softmax role
constexpr long long kWaitCycles = 1ll << 28;
struct Barriers {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2], p_ready[2], o_done[2];
  uint64_t s_free[2];  // STAGED: the unit's softmax warps have taken their logits out of TMEM
  uint32_t tmem_base;
  volatile uint32_t abort;
  // key segment ids of the tile in each V stage (filled and released together with it)
  alignas(16) int32_t kseg[2][kTileKv];
  // exchange between the two threads of a row (STAGED): [slot][unit][column half][row]
  float xch[2][2][2][kUnitRows];
};

#ifdef TPA_DEBUG_CYCLES
// tuning builds only: thread-private slots of the status block (words 8..63) get clock values
#define TPA_TICK(slot) do { if (dbg_on && (slot) < 56) p.status[8 + (slot)] = (uint32_t)clock64(); } while (0)
// five ticks per tile for tiles 4..13
#define TPA_TICK5(k) do { if (j >= 4 && j < 14) TPA_TICK(1 + (j - 4) * 5 + (k)); } while (0)
#else
#define TPA_TICK(slot) do { } while (0)
#define TPA_TICK5(k) do { } while (0)
#endif

struct Waiter {
  Barriers* bars;
  uint32_t* status;
  long long budget = kWaitCycles;
  // Returns when the phase with this parity has completed, or after the cycle budget.
  __device__ __forceinline__ void operator()(uint64_t* bar, uint32_t parity, uint32_t where) const {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
      if (bars->abort) return;
      if ((++spins & 63u) == 0 && clock64() - t0 > budget) {
        bars->abort = 1;
        if (status != nullptr && atomicCAS(status, 0u, 1u) == 0u) {
          status[1] = where;
          status[2] = blockIdx.x;
          status[3] = spins;
        }
        return;
      }
    }
  }
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// two fp32 values in one 64-bit register, for the packed add below
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Key tiles are walked, and staged, in an order of their own.  With the causal comparison on
// part-local indices (TPA_FLAG_CAUSAL_PER_PART) the tiles with the same index inside their parts
// are adjacent: walk index = local tile * parts + part.  Every row block then sees a prefix of the
// walk, as it does for one part, and nothing else in the tile loops changes.  Otherwise the walk
// is the key array's own order.
__device__ __forceinline__ int walk_group(const Params& p) { return p.per_part ? p.kv_parts : 1; }
// walk index -> tile index in the key array
__device__ __forceinline__ int walk_to_key_tile(const Params& p, int kt) {
  if (!p.per_part) return kt;
  return (kt % p.kv_parts) * (p.part_len / kTileKv) + kt / p.kv_parts;
}
// tile index in the key array -> walk index
__device__ __forceinline__ int key_tile_to_walk(const Params& p, int tile) {
  if (!p.per_part) return tile;
  const int tps = p.part_len / kTileKv;
  return (tile % tps) * p.kv_parts + tile / tps;
}

// dst tile rows [0,128): dst[row][:] = scale * sum_r a[row0+row, r] * b[row0+row, r, :], bf16,
// in 64-column sub-tiles of 16 KB with the 128-byte swizzle.  `nthreads` threads cooperate.
template <int D>
__device__ __forceinline__ void rebuild_tile(uint8_t* dst, const __nv_bfloat16* a,
                                             int64_t a_row, int64_t a_rank,
                                             const __nv_bfloat16* b, int64_t b_row, int64_t b_rank,
                                             int rank, int64_t row0, int64_t row_end, float scale,
                                             int tid, int nthreads) {
  constexpr int CH = D / 8;  // 16-byte chunks per row
  const int chunk = tid % CH;
  const int rows_per_pass = nthreads / CH;
  const int r_in = tid / CH;
  const __nv_bfloat16* bcol = b + chunk * 8;
  uint8_t* dsub = dst + (chunk >> 3) * (kUnitRows * 128);
#pragma unroll 2
  for (int row = r_in; row < kUnitRows; row += rows_per_pass) {
    const int64_t g = row0 + row;
    const __nv_bfloat16* ap = a + g * a_row;
    const __nv_bfloat16* bp = bcol + g * b_row;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    const int nr = g < row_end ? rank : 0;  // rows past the end of a ragged last tile stay zero
#pragma unroll 4
    for (int r = 0; r < nr; ++r) {
      const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bp + r * b_rank));
      const float av = __bfloat162float(ap[r * a_rank]);
      const uint32_t w[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] = fmaf(av, __uint_as_float(w[e] << 16), acc[2 * e]);
        acc[2 * e + 1] = fmaf(av, __uint_as_float(w[e] & 0xffff0000u), acc[2 * e + 1]);
      }
    }
    uint4 out;
    out.x = pack_bf16(acc[0] * scale, acc[1] * scale);
    out.y = pack_bf16(acc[2] * scale, acc[3] * scale);
    out.z = pack_bf16(acc[4] * scale, acc[5] * scale);
    out.w = pack_bf16(acc[6] * scale, acc[7] * scale);
    *reinterpret_cast<uint4*>(dsub + sw128_offset(row, chunk & 7)) = out;
  }
}

// ---------------------------------------------------------------------------------------------
// Staging kernel: one CTA rebuilds one 128-row tile of Q, K or V for 8 heads and writes each
// head's tile as the exact shared-memory image (64-column sub-tiles of 16 KB, 128-byte swizzle)
// at ws[((batch * heads + head) * tiles + tile) * tile_bytes].
// grid = (heads/8, lq/128 + 2 * lk/128, batch), 256 threads: the head groups of one tile are
// adjacent in launch order, so the factor rows they share are read from HBM once.
template <int D>
__global__ void __launch_bounds__(256, 2) tpa_stage_tiles_kernel(const Params p, uint8_t* ws_q,
                                                              uint8_t* ws_k, uint8_t* ws_v,
                                                              float qscale, int first_tile) {
  constexpr int CH = D / 8;
  constexpr int kTileBytes = kUnitRows * D * 2;
  const int nq = (p.lq + kUnitRows - 1) / kUnitRows, nk = (p.lk + kTileKv - 1) / kTileKv;
  int tile = blockIdx.y + first_tile;  // first_tile = lq/128 skips the Q tiles (already staged)
  const TpaFactor *fa, *fb;
  uint8_t* ws;
  int rank, ntiles, length;
  float scale;
  bool is_q = false, is_v = false;
  if (tile < nq) {
    fa = &p.qa; fb = &p.qb; ws = ws_q; rank = p.rank_q; ntiles = nq; scale = qscale; length = p.lq; is_q = true;
  } else if (tile < nq + nk) {
    tile -= nq;
    fa = &p.ka; fb = &p.kb; ws = ws_k; rank = p.rank_k; ntiles = nk; scale = 1.f; length = p.lk;
  } else {
    tile -= nq + nk;
    fa = &p.va; fb = &p.vb; ws = ws_v; rank = p.rank_k; ntiles = nk; scale = 1.f; length = p.lk; is_v = true;
  }
  const int hg = blockIdx.x, batch = blockIdx.z;
  // keys in parts: rows of this tile start part * part_stride into the factor (the tile lies in
  // one part), and its image goes to its place in the walk order
  int slot = tile;
  int64_t part_off = 0;
  if (!is_q && p.kv_parts > 1) {
    const int part = tile / (p.part_len / kTileKv);
    part_off = (int64_t)part * (is_v ? p.v_part_stride : p.k_part_stride) - (int64_t)part * p.part_len * fa->stride[1];
    slot = key_tile_to_walk(p, tile);
  }
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(fa->ptr) + batch * fa->stride[0] + part_off + hg * 8;
  const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(fb->ptr) + batch * fb->stride[0] + part_off;
  const int chunk = threadIdx.x % CH, r_in = threadIdx.x / CH;
  uint8_t* out0 = ws + (((int64_t)batch * p.heads + hg * 8) * ntiles + slot) * kTileBytes +
                  (chunk >> 3) * (kUnitRows * 128);
  // rotary embedding of Q and K rows: table row = row index + offset
  const bool rope = p.rope_cos != nullptr && !is_v;
  const int64_t rope_off = is_q ? p.rope_q_offset : p.rope_k_offset;
  // Two fp32 columns ride in one 64-bit register and every multiply-add is a packed fma.f32x2:
  // the kernel is bound by instruction issue, and this halves its FMA count.  The scale is folded
  // into the head factor (8 multiplies per rank instead of 64 per row).
  const uint64_t scale2 = pack2(scale, scale);
  for (int row = r_in; row < kUnitRows; row += 256 / CH) {
    const int64_t g = (int64_t)tile * kUnitRows + row;
    const __nv_bfloat16* ap = a + g * fa->stride[1];
    const __nv_bfloat16* bp = b + g * fb->stride[1] + chunk * 8;
    uint64_t acc[8][4];
#pragma unroll
    for (int h = 0; h < 8; ++h)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[h][e] = 0ull;
    // four ranks at a time: their eight 16-byte loads are issued before any of the FMAs
    // rows past the end of a ragged last tile stay zero (the attention kernel masks them)
    for (int r0 = 0; r0 < (g < length ? rank : 0); r0 += 4) {
      uint4 bv[4], av[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = min(r0 + i, rank - 1);  // clamped loads; ranks past the end are skipped below
        bv[i] = __ldg(reinterpret_cast<const uint4*>(bp + r * fb->stride[2]));
        av[i] = __ldg(reinterpret_cast<const uint4*>(ap + r * fa->stride[2]));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (r0 + i < rank) {
          const uint32_t bw[4] = {bv[i].x, bv[i].y, bv[i].z, bv[i].w};
          const uint32_t aw[4] = {av[i].x, av[i].y, av[i].z, av[i].w};
          uint64_t b2[4];  // columns (2e, 2e + 1) of this thread's eight
#pragma unroll
          for (int e = 0; e < 4; ++e)
            b2[e] = pack2(__uint_as_float(bw[e] << 16), __uint_as_float(bw[e] & 0xffff0000u));
#pragma unroll
          for (int h = 0; h < 8; ++h) {
            const float ah = __uint_as_float((h & 1) ? (aw[h >> 1] & 0xffff0000u) : (aw[h >> 1] << 16));
            const uint64_t a2 = mul2(pack2(ah, ah), scale2);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[h][e] = fma2(a2, b2[e], acc[h][e]);
          }
        }
      }
    }
    if (rope && g < length) {
      // this thread's 8 columns are 4 whole pairs; the rotation is the same for every head
      const float4 cs = __ldg(reinterpret_cast<const float4*>(p.rope_cos + (g + rope_off) * (D / 2) + chunk * 4));
      const float4 sn = __ldg(reinterpret_cast<const float4*>(p.rope_sin + (g + rope_off) * (D / 2) + chunk * 4));
      const float c4[4] = {cs.x, cs.y, cs.z, cs.w}, s4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
      for (int h = 0; h < 8; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x, y;
          unpack2(acc[h][e], x, y);
          acc[h][e] = pack2(x * c4[e] - y * s4[e], x * s4[e] + y * c4[e]);
        }
    }
    const uint32_t off = sw128_offset(row, chunk & 7);
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x, y;
        unpack2(acc[h][e], x, y);
        w[e] = pack_bf16(x, y);
      }
      *reinterpret_cast<uint4*>(out0 + (int64_t)h * ntiles * kTileBytes + off) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Segment ids: which key tiles can each 256-row block see at all?  One CTA per (row block,
// batch element) finds the id range of its two 128-row units and of every 128-key tile and
// writes {first tile, end tile of unit 0, end tile of unit 1, 0}: the attention kernel then
// walks only [first, end).  With packed sequences (ids non-decreasing) that is exactly the
// tiles of the block's own segments; for arbitrary ids it is a superset, and the element-wise
// test inside the tiles still decides.  grid = (pairs, batch), 128 threads.
__global__ void __launch_bounds__(128) tpa_seg_ranges_kernel(const Params p, int4* ranges) {
  __shared__ int red[4][4];   // per warp: min/max of unit 0, min/max of unit 1
  __shared__ int first, last[2];
  // one bit per key tile (walk order): set when the tile's keys do not all carry the block's one id
  constexpr int kBitmapTiles = 8192;
  __shared__ uint32_t odd_tile[kBitmapTiles / 32];
  __shared__ int mixed;
  const int pair = blockIdx.x, batch = blockIdx.y, t = threadIdx.x;
  const int32_t* qs = p.q_seg + (int64_t)batch * p.q_seg_bstride;
  const int32_t* ks = p.kv_seg + (int64_t)batch * p.kv_seg_bstride;
  const int n_kv = (p.lk + kTileKv - 1) / kTileKv;
  int lo[2], hi[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int row = pair * 2 * kUnitRows + u * kUnitRows + t;
    const int id = row < p.lq ? qs[row] : 0;
    lo[u] = __reduce_min_sync(0xffffffffu, row < p.lq ? id : INT_MAX);
    hi[u] = __reduce_max_sync(0xffffffffu, row < p.lq ? id : INT_MIN);
  }
  if ((t & 31) == 0) {
    red[t >> 5][0] = lo[0]; red[t >> 5][1] = hi[0]; red[t >> 5][2] = lo[1]; red[t >> 5][3] = hi[1];
  }
  if (t == 0) { first = n_kv; last[0] = -1; last[1] = -1; mixed = 0; }
  for (int i = t; i < kBitmapTiles / 32; i += 128) odd_tile[i] = 0u;
  __syncthreads();
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    lo[u] = min(min(red[0][2 * u], red[1][2 * u]), min(red[2][2 * u], red[3][2 * u]));
    hi[u] = max(max(red[0][2 * u + 1], red[1][2 * u + 1]), max(red[2][2 * u + 1], red[3][2 * u + 1]));
  }
  // do all rows of the block carry one id?  (an absent second unit has lo > hi)
  const bool one_id = lo[0] == hi[0] && (lo[1] > hi[1] || (lo[1] == hi[1] && lo[1] == lo[0]));
  for (int tile = t; tile < n_kv; tile += 128) {  // `tile` counts in walk order
    const int key_tile = walk_to_key_tile(p, tile);
    const int4* src = reinterpret_cast<const int4*>(ks + kseg_offset(p, key_tile * kTileKv));
    int kmin = INT_MAX, kmax = INT_MIN;
    const int n4 = min(kTileKv, p.lk - key_tile * kTileKv) / 4;  // lk % 4 == 0
    for (int i = 0; i < n4; ++i) {
      const int4 v = __ldg(src + i);
      kmin = min(kmin, min(min(v.x, v.y), min(v.z, v.w)));
      kmax = max(kmax, max(max(v.x, v.y), max(v.z, v.w)));
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (kmin <= hi[u] && kmax >= lo[u]) {  // id ranges intersect (never true for an absent unit)
        atomicMin(&first, tile);
        atomicMax(&last[u], tile);
      }
    }
    if (!(kmin == kmax && kmin == lo[0])) {
      if (tile < kBitmapTiles) atomicOr(&odd_tile[tile >> 5], 1u << (tile & 31));
      else mixed = 1;  // beyond the bitmap: no claim
    }
  }
  __syncthreads();
  // Uniform: one id on every row of the block and on every key of every tile it walks.  The
  // attention kernel then drops the id handling for this block altogether (no key ids copied, no
  // per-tile test): the all-zero ids a ring call must pass cost nothing.
  const int f = first < n_kv ? first : 0;
  const int e = max(f, max(last[0], last[1]) + 1);
  for (int w = (f >> 5) + t; w <= ((e - 1) >> 5) && e > f && w < kBitmapTiles / 32; w += 128) {
    uint32_t bits = odd_tile[w];
    if (w == (f >> 5)) bits &= 0xffffffffu << (f & 31);
    if (w == ((e - 1) >> 5) && ((e & 31) != 0)) bits &= 0xffffffffu >> (32 - (e & 31));
    if (bits != 0u) mixed = 1;
  }
  __syncthreads();
  if (t == 0) {
    const int uniform = (one_id && mixed == 0) ? 1 : 0;
    ranges[(int64_t)batch * gridDim.x + pair] = make_int4(f, max(f, last[0] + 1), max(f, last[1] + 1), uniform);
  }
}

// MODE 0: the reference's call.  1: key parts (a ring in one call).  2: windows / dilation as well.
// The plain instantiation keeps none of the others' arithmetic (one position per key, the walk is
// the key array's order), and parts alone cost one counter per tile.
template <int D, bool STAGED, int MODE>
__global__ void __launch_bounds__(Roles<STAGED>::kThreads, 1)
tpa_fwd_sm100_kernel(const Params p, const uint8_t* ws_q, const uint8_t* ws_k, const uint8_t* ws_v,
                     const int pairs, const int group, const int4* seg_ranges) {
  constexpr int kMmaWarp = Roles<STAGED>::kMmaWarp;
  constexpr int kSoftmaxWarps = Roles<STAGED>::kSoftmaxWarps;
  constexpr int kTileBytes = kUnitRows * D * 2;  // one Q unit, one K stage or one V stage
  constexpr uint32_t kIdescS = make_idesc(128, kTileKv, false, false);
  constexpr uint32_t kIdescPV = make_idesc(128, D, false, true);
  // TMEM columns (512).  FUSED: S0 [0,128) S1 [128,256), P_u over S_u, O_u at 256 + u D.
  // STAGED keeps P out of the logits' columns, so that the next logits of a unit can be computed
  // while its softmax still works on the current ones (they are taken into registers at once):
  //   D = 128: S [0,128) shared by the two units in turn, P0 [128,192) P1 [192,256), O0 [256,384) O1 [384,512)
  //   D = 64:  S0 [0,128) S1 [128,256), P0 [256,320) P1 [320,384), O0 [384,448) O1 [448,512)
  constexpr bool kSharedS = STAGED;  // at D = 64 there is room for two, but taking turns keeps the units' exponentials apart
  auto s_col = [](int u) -> uint32_t { return kSharedS ? 0u : (uint32_t)u * 128u; };
  auto p_col = [](int u) -> uint32_t {
    return !STAGED ? (uint32_t)u * 128u : (D == 128 ? 128u + 64u * u : 256u + 64u * u);
  };
  auto o_col = [](int u) -> uint32_t {
    return !STAGED ? 256u + (uint32_t)u * D : (D == 128 ? 256u + 128u * u : 384u + 64u * u);
  };

#ifdef TPA_DEBUG_CYCLES
  const long long dbg_t_entry = clock64();
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + 2 * kTileBytes;
  uint8_t* sV = smem + 4 * kTileBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + 6 * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Launch order decides what shares L2 and how the kernel ends (see launch_sm100): the
  // (batch, head) slices are taken `group` at a time; within a group the longest causal rows
  // of every slice go first and the slices of one row block are adjacent.
  const int per_group = group * pairs;
  const int slice = (blockIdx.x / per_group) * group + (blockIdx.x % per_group) % group;
  const int pair = pairs - 1 - (blockIdx.x % per_group) / group;
  const int head = slice % p.heads;
  const int batch = slice / p.heads;
  const int q0 = pair * 2 * kUnitRows;
  const bool causal = (p.flags & TPA_FLAG_CAUSAL) != 0;
  bool has_seg = p.q_seg != nullptr;  // cleared below for a block whose rows and walked keys all carry one id
  const bool load_state = (p.flags & TPA_FLAG_STATE_LOAD) != 0;
  const bool store_state = (p.flags & TPA_FLAG_STATE_STORE) != 0;

  // number of key tiles each unit can see (tpa/tpa.py:427-431, with global offsets)
  // Tiles are counted in walk order (see walk_group): G tiles share one position range.
  const int n_kv = (p.lk + kTileKv - 1) / kTileKv;
  constexpr bool kParts = MODE >= 1;
  const int G = kParts ? walk_group(p) : 1;
  const int n_loc = n_kv / G;
  const bool windowed = MODE == 2 && p.window > 0;
  const bool dilated = MODE == 2 && p.dilation > 1;
  const int span = windowed ? p.window * p.dilation : 0;
  int n_vis[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int q0u = q0 + u * kUnitRows;
    int hi = q0u >= p.lq ? 0 : n_loc;
    const int64_t last = (int64_t)q0u + kUnitRows - 1 + p.q_offset - p.k_offset;  // position of the last row, key-relative
    if (hi > 0 && causal) hi = last < 0 ? 0 : (int)min((int64_t)n_loc, last / kTileKv + 1);
    if (hi > 0 && windowed && !causal)  // keys at most span - 1 ahead of the last row
      hi = last + span - 1 < 0 ? 0 : (int)min((int64_t)hi, (last + span - 1) / kTileKv + 1);
    n_vis[u] = hi * G;
  }
  // A window starts the walk at the tile of the first key the block's first row can see.
  // With segment ids the walk starts at the first tile any row of the block can match and ends
  // where the unit's last match is (tpa_seg_ranges_kernel).  From here on tiles are counted
  // from j0: tile j of the loops below is walk tile j0 + j.
  int j0 = 0;
  if (windowed) {
    const int64_t first = (int64_t)q0 + p.q_offset - p.k_offset - (span - 1);
    if (first > 0) j0 = (int)min((int64_t)n_loc, first / kTileKv) * G;
  }
  if (seg_ranges != nullptr) {
    const int4 r = seg_ranges[(int64_t)batch * pairs + pair];
    if (r.w != 0) has_seg = false;
    j0 = max(j0, r.x);
    n_vis[0] = min(n_vis[0], r.y);
    n_vis[1] = min(n_vis[1], r.z);
  }
  n_vis[0] = max(0, n_vis[0] - j0);
  n_vis[1] = max(0, n_vis[1] - j0);
  // Key splits (gridDim.y > 1, few query rows against many keys): this CTA walks only its share
  // of the tiles and leaves a partial (o, lse) in its own slice of the scratch that
  // tpa_combine_splits_kernel merges; the host has set STATE_STORE and pointed state_o/lse there.
  const int split = blockIdx.y;
  if (gridDim.y > 1) {
    const int chunk = (max(n_vis[0], n_vis[1]) + gridDim.y - 1) / gridDim.y;
    const int begin = split * chunk;
    j0 += begin;
    n_vis[0] = min(max(0, n_vis[0] - begin), chunk);
    n_vis[1] = min(max(0, n_vis[1] - begin), chunk);
  }
  const int n_tiles = max(n_vis[0], n_vis[1]);
  const int64_t split_rows = (int64_t)split * p.batch * p.lq * p.heads;
  float* const st_o = p.state_o + split_rows * D;
  float* const st_lse = p.state_lse + split_rows;

  if (threadIdx.x == 0) {
    // producers: one expect_tx arrival (STAGED) or one arrival per rebuild warp (FUSED)
    mbar_init(&bars->q_full, STAGED ? 1 : kRebuildWarps);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->k_full[s], STAGED ? 1 : kRebuildWarps / 2);
      mbar_init(&bars->v_full[s], STAGED ? 1 : kRebuildWarps / 2);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_ready[s], kSoftmaxWarps / 2);  // one arrival per softmax warp of the unit
      mbar_init(&bars->o_done[s], 1);
      mbar_init(&bars->s_free[s], kSoftmaxWarps / 2);
    }
    bars->abort = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const Waiter wait{bars, p.status, kWaitCycles};
  const __nv_bfloat16* qa = static_cast<const __nv_bfloat16*>(p.qa.ptr) + batch * p.qa.stride[0] + head;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(p.qb.ptr) + batch * p.qb.stride[0];
  const __nv_bfloat16* ka = static_cast<const __nv_bfloat16*>(p.ka.ptr) + batch * p.ka.stride[0] + head;
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(p.kb.ptr) + batch * p.kb.stride[0];
  const __nv_bfloat16* va = static_cast<const __nv_bfloat16*>(p.va.ptr) + batch * p.va.stride[0] + head;
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(p.vb.ptr) + batch * p.vb.stride[0];

  if (warp < kSoftmaxWarps) {
   if constexpr (STAGED) {
    // ------------------------------------------------------------------ softmax + epilogue (STAGED)
    // Two threads per query row: 16 warps, warp w serves unit w >> 3, column half (w >> 2) & 1
    // and TMEM lanes 32 (w & 3)...  Thread (unit, half, row) exponentiates 64 of the 128 keys of
    // each tile and owns D/2 columns of the accumulator row.  The two warps that share 32 rows
    // meet on their own named barrier: a one-bit vote per tile on the fast path, the row
    // maximum (through shared memory) on the exact path, the row sum at the end.
    const int u = warp >> 3;
    const int half = (warp >> 2) & 1;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int pair_bar = 1 + u * 4 + quarter;  // named barrier of the two partner warps
    const int n_u = n_vis[u];
    const int q0u = q0 + u * kUnitRows;
    const int grow = q0u + row;
    const bool live = q0u < p.lq;      // the unit exists
    const bool row_ok = grow < p.lq;   // this thread's row exists (the last unit may be ragged)
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tSh = tmem + lane_base + s_col(u) + half * 64;      // this thread's 64 logits
    const uint32_t tPh = tmem + lane_base + p_col(u) + half * 32;      // ... and where their bf16 P goes
    const uint32_t tOh = tmem + lane_base + o_col(u) + half * (D / 2);  // its D/2 accumulators
    const int64_t rh = row_ok ? ((int64_t)batch * p.lq + grow) * p.heads + head : 0;
    const int64_t qpos = (int64_t)grow + p.q_offset;
    const int qseg = (has_seg && row_ok) ? p.q_seg[(int64_t)batch * p.q_seg_bstride + grow] : 0;
    const float rk = (float)p.rank_k;
    constexpr int kOChunks = D / 64;  // 32-column chunks of the accumulator this thread owns

    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
    auto pair_any = [&](bool pred) -> bool {
      uint32_t out;
      asm volatile(
          "{\n\t.reg .pred pin, pout;\n\t"
          "setp.ne.u32 pin, %1, 0;\n\t"
          "bar.red.or.pred pout, %2, 64, pin;\n\t"
          "selp.u32 %0, 1, 0, pout;\n\t}"
          : "=r"(out)
          : "r"((uint32_t)pred), "r"(pair_bar)
          : "memory");
      return out != 0;
    };

    float m = -CUDART_INF_F, l = 0.f;  // m is the same in both halves of a row; l is this half's share
    bool loaded = false;
    if (load_state && live && n_u > 0) {
      // carried partial (tpa/ring_tpa.py:69-71): accumulator = o_prev (times R_k, see header),
      // row sum 1 (counted once, in half 0), maximum = previous LSE
      const float prev = row_ok ? st_lse[rh] : -CUDART_INF_F;
      const bool has = prev != -CUDART_INF_F;
      if (has) {
        m = prev * kLog2e;
        l = half == 0 ? 1.f : 0.f;
      }
      const float* so = st_o + rh * D + half * (D / 2);
#pragma unroll
      for (int c = 0; c < kOChunks; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float4 v = has ? *reinterpret_cast<const float4*>(so + c * 32 + e) : make_float4(0.f, 0.f, 0.f, 0.f);
          r[e] = __float_as_uint(v.x * rk);
          r[e + 1] = __float_as_uint(v.y * rk);
          r[e + 2] = __float_as_uint(v.z * rk);
          r[e + 3] = __float_as_uint(v.w * rk);
        }
        tmem_st32(tOh + c * 32, r);
      }
      tmem_st_wait();
      loaded = true;
    }

#ifdef TPA_DEBUG_CYCLES
    const bool dbg_on = blockIdx.x == TPA_DEBUG_CYCLES && warp == 8 && lane == 0 && p.status != nullptr;  // unit 1, half 0
    if (dbg_on) p.status[8 + 52] = (uint32_t)dbg_t_entry;
    TPA_TICK(0);
#endif
    // position of walk tile j0 + j: tile (j0 + j) / G of its part, kept by counting
    int pos_tile = kParts ? j0 / G : j0, pos_cnt = kParts ? j0 % G : 0;
    for (int j = 0; j < n_u; ++j) {
      wait(&bars->s_full[u], j & 1, 0x100 + u);
      tc_fence_after();
      // The thread's 64 logits leave TMEM at once; the MMA warp may then overwrite them with the
      // next tile's (of this unit, or of the other one where the two share the columns) while
      // this tile's softmax runs.
      uint32_t r0[32], r1[32];
      tmem_ld32(tSh, r0);
      tmem_ld32(tSh + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_free[u]);
      TPA_TICK5(0);
      // this thread's 64 columns: index of the first in the walk (= in the key array unless the
      // walk is interleaved, and then no tile is ragged) and its position in the comparisons
      const int k0 = (j0 + j) * kTileKv + half * 64;
      const int64_t kp0 = (int64_t)pos_tile * kTileKv + half * 64 + p.k_offset;
      if (kParts) {
        if (++pos_cnt == G) { pos_cnt = 0; ++pos_tile; }
      } else {
        ++pos_tile;
      }
      const int64_t q_lo = (int64_t)q0u + p.q_offset;
      // does any (row of the unit, column of this half) pair fall to the causal or window rule?
      const bool edge = (causal && kp0 + 63 > q_lo) ||
                        (windowed && (q_lo + kUnitRows - 1 - kp0 >= span || (!causal && kp0 + 63 - q_lo >= span)));
      const bool tail = G == 1 && k0 + 63 >= p.lk;  // columns past the last key (zero rows in the staged tile)
      // Segment ids: when every key of these 64 columns and every row of this warp carry the
      // same id, nothing is masked and the element-wise test is skipped (warp-uniform).
      const int32_t* ks = bars->kseg[j & 1] + half * 64;
      bool seg_mask = false;
      if (has_seg) {
        wait(&bars->v_full[j & 1], (j >> 1) & 1, 0x700 + u);
        const int2 k2 = *reinterpret_cast<const int2*>(ks + lane * 2);
        const int kmin = __reduce_min_sync(0xffffffffu, min(k2.x, k2.y));
        const int kmax = __reduce_max_sync(0xffffffffu, max(k2.x, k2.y));
        seg_mask = !__all_sync(0xffffffffu, kmin == kmax && qseg == kmin);
      }
      const bool masked = edge || seg_mask || tail || dilated;
      if (masked) {
        // The causal rule, the window and the end of the keys leave this thread a range [lo, hi) of
        // its 64 columns.  rel = its row's position minus its first column's, clamped to 32 bits
        // (see MaskRule); column c is kept by the causal rule iff c <= rel, by the window iff
        // |rel - c| < span.
        int lo = 0, hi = 64, phase = 0;
        const int rel = clamp_diff(qpos - kp0);
        if (tail) hi = min(hi, p.lk - k0);
        if (edge) {
          if (causal) hi = min(hi, rel + 1);
          else if (windowed) hi = min(hi, rel + span);
          if (windowed) lo = max(lo, rel - span + 1);
        }
        if (dilated) phase = diff_phase(qpos - kp0, p.dilation);
        const unsigned width = hi > lo ? (unsigned)(hi - lo) : 0u;
        auto mask_chunk = [&](uint32_t(&r)[32], int c) {
          if (edge || tail) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if ((unsigned)(c * 32 + e - lo) >= width) r[e] = 0xff800000u;  // -inf
          }
          if (seg_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (qseg != ks[c * 32 + e]) r[e] = 0xff800000u;
          }
          if (dilated) {  // a loop of its own: the remainders are only computed when asked for
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if ((phase - (c * 32 + e)) % p.dilation != 0) r[e] = 0xff800000u;
          }
        };
        mask_chunk(r0, 0);
        mask_chunk(r1, 1);
      }
      // Maximum of the thread's 64 logits.  The reference maximum m carried from earlier tiles
      // stays as long as no logit of the row exceeds it by more than 2^8 (the final 1 / l makes
      // the result independent of which maximum was subtracted): one one-bit vote of the two
      // warps that share the rows.  Only when some row needs a new maximum do the halves
      // exchange theirs through shared memory.  m is identical in both halves of a row, so both
      // warps of a pair always take the same branches.
      float cm4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int e = 0; e < 32; e += 4) {  // four independent chains
        cm4[0] = max3(cm4[0], __uint_as_float(r0[e]), __uint_as_float(r0[e + 1]));
        cm4[1] = max3(cm4[1], __uint_as_float(r0[e + 2]), __uint_as_float(r0[e + 3]));
        cm4[2] = max3(cm4[2], __uint_as_float(r1[e]), __uint_as_float(r1[e + 1]));
        cm4[3] = max3(cm4[3], __uint_as_float(r1[e + 2]), __uint_as_float(r1[e + 3]));
      }
      const float cm = fmaxf(fmaxf(cm4[0], cm4[1]), fmaxf(cm4[2], cm4[3]));
      const bool need = (m == -CUDART_INF_F) ? (cm != -CUDART_INF_F) : (cm - m > kRescaleThreshold);
      if (pair_any(__any_sync(0xffffffffu, need))) {
        // row maximum over both halves, through shared memory (slot alternates with the tile)
        float* xch = bars->xch[j & 1][u][0];
        xch[half * kUnitRows + row] = cm;
        pair_sync();
        const float m_new = fmaxf(m, fmaxf(xch[row], xch[kUnitRows + row]));
        float factor = 1.f;
        if (m == -CUDART_INF_F) {
          m = m_new;  // nothing accumulated for this row yet (l = 0, accumulator row is 0)
        } else if (m_new - m > kRescaleThreshold) {
          factor = fast_exp2(m - m_new);
          m = m_new;
        }
        if (__any_sync(0xffffffffu, factor != 1.f) && (j > 0 || loaded)) {
          if (j > 0) {
            wait(&bars->o_done[u], (j - 1) & 1, 0x200 + u);
            tc_fence_after();
          }
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t a[16];
            tmem_ld16(tOh + c * 16, a);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) a[e] = __float_as_uint(__uint_as_float(a[e]) * factor);
            tmem_st16(tOh + c * 16, a);
          }
        }
        l *= factor;
      }
      TPA_TICK5(1);
      // p = 2^(s - m), packed to bf16, and the row sum in four packed partial sums
      const float neg_m = (m == -CUDART_INF_F) ? 0.f : -m;
      const uint64_t neg_m2 = pack2(neg_m, neg_m);
      uint64_t lsum[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t pk[32];
      auto exp_chunk = [&](const uint32_t(&r)[32], uint32_t* out) {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float x0, x1;
          unpack2(add2(pack2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), neg_m2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          lsum[(e >> 1) & 3] = add2(lsum[(e >> 1) & 3], pack2(p0, p1));
          out[e / 2] = pack_bf16(p0, p1);
        }
      };
      exp_chunk(r0, pk);
      TPA_TICK5(2);
      exp_chunk(r1, pk + 16);
      {
        float a0, a1, a2, a3;
        unpack2(add2(lsum[0], lsum[1]), a0, a1);
        unpack2(add2(lsum[2], lsum[3]), a2, a3);
        l += (a0 + a1) + (a2 + a3);
      }
      TPA_TICK5(3);
      // P has columns of its own: key k of the tile is at column k / 2.  They are free once the
      // previous tile's P V has been read out (the same barrier the accumulator rescale waits on).
      if (j > 0) {
        wait(&bars->o_done[u], (j - 1) & 1, 0x210 + u);
        tc_fence_after();
      }
      tmem_st32(tPh, pk);
      tmem_st_wait();  // warp-wide: every lane's P (and any rescaled accumulator) has landed
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready[u]);
      TPA_TICK5(4);
    }

    TPA_TICK(53);
    // ---- epilogue: o = acc / (l * R_k), lse = ln2 * (m + log2 l); NaN / -inf for empty rows
    if (live) {
      if (n_u > 0) {
        wait(&bars->o_done[u], (n_u - 1) & 1, 0x300 + u);
        tc_fence_after();
      }
      TPA_TICK(54);
      // row sum = this half's share + the partner's
      float* xch = bars->xch[n_u & 1][u][0];
      xch[half * kUnitRows + row] = l;
      pair_sync();
      l = xch[row] + xch[kUnitRows + row];
      const bool empty = !(l > 0.f);
      float inv = empty ? 0.f : 1.f / (l * rk);
      float lse = empty ? -CUDART_INF_F : (m + log2f(l)) * kLn2;
      const bool passthrough = (n_u == 0) && load_state;  // nothing visible: carry the state over
      if (passthrough) {
        lse = row_ok ? st_lse[rh] : -CUDART_INF_F;
        inv = 1.f;
      }
      const bool none = passthrough ? (lse == -CUDART_INF_F) : empty;
      __nv_bfloat16* orow = store_state ? nullptr
                                        : static_cast<__nv_bfloat16*>(p.o) + rh * D + half * (D / 2);
      float* srow = (store_state || passthrough) ? st_o + rh * D + half * (D / 2) : nullptr;
#pragma unroll
      for (int c = 0; c < kOChunks; ++c) {
        uint32_t r[32];
        if (n_u > 0) {
          tmem_ld32(tOh + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            r[e] = (passthrough && !none) ? __float_as_uint(srow[c * 32 + e]) : 0u;
        }
        if (store_state) {
          if (!passthrough) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              float4 v = make_float4(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv,
                                     __uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
              if (row_ok) *reinterpret_cast<float4*>(srow + c * 32 + e) = v;
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float x0 = none ? CUDART_NAN_F : __uint_as_float(r[e + 2 * k]) * inv;
              const float x1 = none ? CUDART_NAN_F : __uint_as_float(r[e + 2 * k + 1]) * inv;
              w[k] = pack_bf16(x0, x1);
            }
            if (row_ok) *reinterpret_cast<uint4*>(orow + c * 32 + e) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (half == 0 && row_ok) {
        if (store_state) {
          if (!passthrough) st_lse[rh] = lse;
        } else if (p.lse != nullptr) {
          p.lse[rh] = lse;
        }
      }
    }
    TPA_TICK(55);
   } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int u = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int n_u = n_vis[u];
    const int q0u = q0 + u * kUnitRows;
    const int grow = q0u + row;
    const bool live = q0u < p.lq;      // the unit exists
    const bool row_ok = grow < p.lq;   // this thread's row exists (the last unit may be ragged)
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_base + u * 128;
    const uint32_t tO = tmem + lane_base + o_col(u);
    const int64_t rh = row_ok ? ((int64_t)batch * p.lq + grow) * p.heads + head : 0;
    const int64_t qpos = (int64_t)grow + p.q_offset;
    const int qseg = (has_seg && row_ok) ? p.q_seg[(int64_t)batch * p.q_seg_bstride + grow] : 0;
    const float rk = (float)p.rank_k;

    float m = -CUDART_INF_F, l = 0.f;
    bool loaded = false;
    if (load_state && live && n_u > 0) {
      // carried partial (tpa/ring_tpa.py:69-71): accumulator = o_prev (times R_k, see header),
      // row sum 1, maximum = previous LSE
      const float prev = row_ok ? st_lse[rh] : -CUDART_INF_F;
      const bool has = prev != -CUDART_INF_F;
      if (has) {
        m = prev * kLog2e;
        l = 1.f;
      }
      const float* so = st_o + rh * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float4 v = has ? *reinterpret_cast<const float4*>(so + c * 32 + e) : make_float4(0.f, 0.f, 0.f, 0.f);
          r[e] = __float_as_uint(v.x * rk);
          r[e + 1] = __float_as_uint(v.y * rk);
          r[e + 2] = __float_as_uint(v.z * rk);
          r[e + 3] = __float_as_uint(v.w * rk);
        }
        tmem_st32(tO + c * 32, r);
      }
      tmem_st_wait();
      loaded = true;
    }

    for (int j = 0; j < n_u; ++j) {
      wait(&bars->s_full[u], j & 1, 0x100 + u);
      tc_fence_after();
      const int k0 = (j0 + j) * kTileKv;
      const bool diag = causal && ((int64_t)k0 + kTileKv - 1 + p.k_offset > (int64_t)q0u + p.q_offset);
      const bool tail = k0 + kTileKv - 1 >= p.lk;  // columns past the last key
      // Segment ids: when every key of the tile and every row of this warp carry the same
      // id, nothing is masked and the element-wise test is skipped (warp-uniform decision).
      const int32_t* ks = bars->kseg[j & 1];
      bool seg_mask = false;
      if (has_seg) {
        wait(&bars->v_full[j & 1], (j >> 1) & 1, 0x700 + u);
        const int4 k4 = *reinterpret_cast<const int4*>(ks + lane * 4);
        const int kmin = __reduce_min_sync(0xffffffffu, min(min(k4.x, k4.y), min(k4.z, k4.w)));
        const int kmax = __reduce_max_sync(0xffffffffu, max(max(k4.x, k4.y), max(k4.z, k4.w)));
        seg_mask = !__all_sync(0xffffffffu, kmin == kmax && qseg == kmin);
      }
      const bool masked = diag || seg_mask || tail;

      // pass 1: row maximum of the (masked) logits; they are already in log2 units
      float tmax = -CUDART_INF_F;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + c * 32, r);
        tmem_ld_wait();
        if (masked) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kc = k0 + c * 32 + e;
            bool keep = kc < p.lk;
            if (diag) keep = keep && qpos >= (int64_t)kc + p.k_offset;
            if (seg_mask) keep = keep && (qseg == ks[c * 32 + e]);
            if (keep) tmax = fmaxf(tmax, __uint_as_float(r[e]));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) tmax = fmaxf(tmax, __uint_as_float(r[e]));
        }
      }
      const float m_new = fmaxf(m, tmax);
      float factor = 1.f;
      if (m == -CUDART_INF_F) {
        m = m_new;  // nothing accumulated for this row yet (l = 0, accumulator row is 0)
      } else if (m_new - m > kRescaleThreshold) {
        factor = fast_exp2(m - m_new);
        m = m_new;
      }
      if (__any_sync(0xffffffffu, factor != 1.f) && (j > 0 || loaded)) {
        if (j > 0) {
          wait(&bars->o_done[u], (j - 1) & 1, 0x200 + u);
          tc_fence_after();
        }
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * factor);
          tmem_st32(tO + c * 32, r);
        }
        tmem_st_wait();
      }
      l *= factor;
      const float m_sub = (m == -CUDART_INF_F) ? 0.f : m;

      // pass 2: p = 2^(s - m), row sum, bf16 P over the first 64 columns of S
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t pk[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = half * 2 + cc;
          uint32_t r[32];
          tmem_ld32(tS + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float s0 = __uint_as_float(r[e]), s1 = __uint_as_float(r[e + 1]);
            if (masked) {
              const int kc = k0 + c * 32 + e;
              bool keep0 = kc < p.lk, keep1 = kc + 1 < p.lk;
              if (diag) {
                keep0 = keep0 && qpos >= (int64_t)kc + p.k_offset;
                keep1 = keep1 && qpos >= (int64_t)kc + 1 + p.k_offset;
              }
              if (seg_mask) {
                keep0 = keep0 && (qseg == ks[c * 32 + e]);
                keep1 = keep1 && (qseg == ks[c * 32 + e + 1]);
              }
              if (!keep0) s0 = -CUDART_INF_F;
              if (!keep1) s1 = -CUDART_INF_F;
            }
            const float p0 = fast_exp2(s0 - m_sub), p1 = fast_exp2(s1 - m_sub);
            l += p0 + p1;
            pk[cc * 16 + e / 2] = pack_bf16(p0, p1);
          }
        }
        tmem_st32(tS + half * 32, pk);
      }
      tmem_st_wait();  // warp-wide: every lane's P has landed in TMEM
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready[u]);
    }

    // ---- epilogue: o = acc / (l * R_k), lse = ln2 * (m + log2 l); NaN / -inf for empty rows
    if (live) {
      if (n_u > 0) {
        wait(&bars->o_done[u], (n_u - 1) & 1, 0x300 + u);
        tc_fence_after();
      }
      const bool empty = !(l > 0.f);
      float inv = empty ? 0.f : 1.f / (l * rk);
      float lse = empty ? -CUDART_INF_F : (m + log2f(l)) * kLn2;
      const bool passthrough = (n_u == 0) && load_state;  // nothing visible: carry the state over
      if (passthrough) {
        lse = row_ok ? st_lse[rh] : -CUDART_INF_F;
        inv = 1.f;
      }
      const bool none = passthrough ? (lse == -CUDART_INF_F) : empty;
      __nv_bfloat16* orow = store_state ? nullptr : static_cast<__nv_bfloat16*>(p.o) + rh * D;
      float* srow = (store_state || passthrough) ? st_o + rh * D : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (n_u > 0) {
          tmem_ld32(tO + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            r[e] = (passthrough && !none) ? __float_as_uint(srow[c * 32 + e]) : 0u;
        }
        if (store_state) {
          if (!passthrough) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              float4 v = make_float4(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv,
                                     __uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
              if (row_ok) *reinterpret_cast<float4*>(srow + c * 32 + e) = v;
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float x0 = none ? CUDART_NAN_F : __uint_as_float(r[e + 2 * k]) * inv;
              const float x1 = none ? CUDART_NAN_F : __uint_as_float(r[e + 2 * k + 1]) * inv;
              w[k] = pack_bf16(x0, x1);
            }
            if (row_ok) *reinterpret_cast<uint4*>(orow + c * 32 + e) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (!row_ok) {
      } else if (store_state) {
        if (!passthrough) st_lse[rh] = lse;
      } else if (p.lse != nullptr) {
        p.lse[rh] = lse;
      }
    }
   }
  } else if (warp < kMmaWarp) {
   if constexpr (STAGED) {
    // ------------------------------------------------------------------ bulk copies of staged tiles
    if (lane == 0) {
      const int64_t bh = (int64_t)batch * p.heads + head;
      const uint8_t* gq = ws_q + (bh * ((p.lq + kUnitRows - 1) / kUnitRows) + pair * 2) * kTileBytes;
      const uint8_t* gk = ws_k + bh * n_kv * kTileBytes;
      const uint8_t* gv = ws_v + bh * n_kv * kTileBytes;
      const int units = (q0 + kUnitRows < p.lq) ? 2 : 1;
      mbar_arrive_expect_tx(&bars->q_full, units * kTileBytes);
      bulk_g2s(sQ, gq, units * kTileBytes, &bars->q_full);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (j >= 2) wait(&bars->k_empty[s], ((j >> 1) - 1) & 1, 0x400);
        mbar_arrive_expect_tx(&bars->k_full[s], kTileBytes);
        bulk_g2s(sK + s * kTileBytes, gk + (int64_t)(j0 + j) * kTileBytes, kTileBytes, &bars->k_full[s]);
        if (j >= 2) wait(&bars->v_empty[s], ((j >> 1) - 1) & 1, 0x500);
        // ids of a ragged last tile: only the keys that exist (lk % 4 == 0, so 16-byte multiples)
        const int key_tile = walk_to_key_tile(p, j0 + j);
        const int n_ids = min(kTileKv, p.lk - key_tile * kTileKv);
        mbar_arrive_expect_tx(&bars->v_full[s], kTileBytes + (has_seg ? n_ids * 4 : 0));
        bulk_g2s(sV + s * kTileBytes, gv + (int64_t)(j0 + j) * kTileBytes, kTileBytes, &bars->v_full[s]);
        if (has_seg)
          bulk_g2s(bars->kseg[s], p.kv_seg + (int64_t)batch * p.kv_seg_bstride + kseg_offset(p, key_tile * kTileKv),
                   n_ids * 4, &bars->v_full[s]);
      }
    }
    __syncwarp();
   } else {
    // ------------------------------------------------------------------ rebuild Q, then K or V tiles
    const int rt = threadIdx.x - kSoftmaxWarps * 32;  // 0..255
    const float qscale = p.sm_scale * kLog2e / ((float)p.rank_q * (float)p.rank_k);
    for (int u = 0; u < 2; ++u) {
      if (q0 + u * kUnitRows < p.lq)
        rebuild_tile<D>(sQ + u * kTileBytes, qa, p.qa.stride[1], p.qa.stride[2], qb, p.qb.stride[1],
                        p.qb.stride[2], p.rank_q, q0 + u * kUnitRows, p.lq, qscale, rt, kRebuildWarps * 32);
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars->q_full);

    const bool is_k = rt < kRebuildWarps * 16;
    const int t = is_k ? rt : rt - kRebuildWarps * 16;
    const __nv_bfloat16* fa = is_k ? ka : va;
    const __nv_bfloat16* fb = is_k ? kb : vb;
    const TpaFactor& sa = is_k ? p.ka : p.va;
    const TpaFactor& sb = is_k ? p.kb : p.vb;
    uint8_t* stages = is_k ? sK : sV;
    uint64_t* full = is_k ? bars->k_full : bars->v_full;
    uint64_t* empty = is_k ? bars->k_empty : bars->v_empty;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      if (j >= 2) wait(&empty[s], ((j >> 1) - 1) & 1, is_k ? 0x400 : 0x500);
      rebuild_tile<D>(stages + s * kTileBytes, fa, sa.stride[1], sa.stride[2], fb, sb.stride[1],
                      sb.stride[2], p.rank_k, (int64_t)(j0 + j) * kTileKv, p.lk, 1.f, t, kRebuildWarps * 16);
      if (!is_k && has_seg)
        bars->kseg[s][t] = ((j0 + j) * kTileKv + t < p.lk)
                               ? p.kv_seg[(int64_t)batch * p.kv_seg_bstride + (int64_t)(j0 + j) * kTileKv + t]
                               : 0;
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
    }
   }
  } else {
    // ------------------------------------------------------------------ MMA issue (one thread)
    if (lane == 0 && n_tiles > 0) {
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      auto issue_s = [&](int u, int j) {
        const uint32_t qbase = aQ + u * kTileBytes, kbase = aK + (j & 1) * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * (kUnitRows * 128) + (ks & 3) * 32;
          mma_ss(tmem + s_col(u), make_desc(qbase + off, 16, 1024), make_desc(kbase + off, 16, 1024),
                 kIdescS, ks > 0);
        }
        tc_commit(&bars->s_full[u]);
      };
      auto issue_pv = [&](int u, int j, bool acc) {
        const uint32_t vbase = aV + (j & 1) * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kTileKv / 16; ++ks) {
          // P of key k is at column k / 2 of the unit's P columns
          mma_ts(tmem + o_col(u), tmem + p_col(u) + ks * 8,
                 make_desc(vbase + ks * 2048, kTileKv * 128, 1024), kIdescPV, (acc || ks > 0) ? 1u : 0u);
        }
        tc_commit(&bars->o_done[u]);
      };
      if constexpr (STAGED) {
        // Two issuing threads.  Issuing tcgen05.mma holds the thread for about as long as the
        // tensor pipe needs for what is queued before it (measured: ~670 cycles for the eight
        // MMAs of a tile), so one thread that issues everything cannot also be waiting for the
        // next softmax event while the pipe works: every hand-over then costs its full latency
        // in pipe idle time.  Here one thread issues the logits and another the P V; each waits
        // only for its own events, and the pipe takes from both.
        //
        // The softmax warps take a tile's logits into registers as soon as they are complete and
        // say so (s_free); from then on the columns may be overwritten, so S_u(j+1) is issued
        // while softmax_u(j) still runs and only P_u(j) V waits for it.  With D = 128 the two
        // units share one set of logit columns and use it in turn, S0(j) S1(j) S0(j+1) ..., each
        // after the previous user has drained.
        if (warp == kMmaWarp) {
          wait(&bars->q_full, 0, 0x600);
          tc_fence_after();
          int last_u = -1, last_j = 0;  // the last logits issued into the shared columns
          for (int j = 0; j < n_tiles; ++j) {
            wait(&bars->k_full[j & 1], (j >> 1) & 1, 0x601);
            tc_fence_after();
            for (int u = 0; u < 2; ++u) {
              if (j >= n_vis[u]) continue;
              if (kSharedS) {
                if (last_u >= 0) {
                  wait(&bars->s_free[last_u], last_j & 1, 0x620 + last_u);
                  tc_fence_after();
                }
              } else if (j > 0) {
                wait(&bars->s_free[u], (j - 1) & 1, 0x620 + u);
                tc_fence_after();
              }
              issue_s(u, j);
              last_u = u;
              last_j = j;
            }
            tc_commit(&bars->k_empty[j & 1]);  // both units' logits of tile j are issued
          }
        } else {
          for (int j = 0; j < n_tiles; ++j) {
            wait(&bars->v_full[j & 1], (j >> 1) & 1, 0x602);
            tc_fence_after();
            for (int u = 0; u < 2; ++u) {
              if (j >= n_vis[u]) continue;
              wait(&bars->p_ready[u], j & 1, 0x610 + u);
              tc_fence_after();
              issue_pv(u, j, load_state || j > 0);
            }
            tc_commit(&bars->v_empty[j & 1]);  // both units' P V of tile j are issued
          }
        }
      } else {
        // Per unit the order is fixed: S(j), O += P V of tile j, S(j+1) (which overwrites P).  The
        // units are interleaved in a fixed order too, PV0(j) S0(j+1) PV1(j) S1(j+1): it keeps them
        // half a tile apart, so that the softmax of one always has the other's MMAs to hide behind.
        wait(&bars->q_full, 0, 0x600);
        tc_fence_after();
        wait(&bars->k_full[0], 0, 0x601);
        tc_fence_after();
        for (int u = 0; u < 2; ++u)
          if (n_vis[u] > 0) issue_s(u, 0);
        tc_commit(&bars->k_empty[0]);
        for (int j = 0; j < n_tiles; ++j) {
          wait(&bars->v_full[j & 1], (j >> 1) & 1, 0x602);
          tc_fence_after();
          bool k_waited = false;
          for (int u = 0; u < 2; ++u) {
            if (j < n_vis[u]) {
              wait(&bars->p_ready[u], j & 1, 0x610 + u);
              tc_fence_after();
              issue_pv(u, j, load_state || j > 0);
            }
            if (j + 1 < n_vis[u]) {
              if (!k_waited) {
                wait(&bars->k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, 0x603);
                tc_fence_after();
                k_waited = true;
              }
              issue_s(u, j + 1);
            }
          }
          tc_commit(&bars->v_empty[j & 1]);
          if (j + 1 < n_tiles) tc_commit(&bars->k_empty[(j + 1) & 1]);
        }
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// Self-test of the bounded wait: one warp waits, with a short cycle budget, on an mbarrier that
// nothing ever arrives at.  The wait runs out, the status block records {1, where, block, spins},
// the abort flag makes the second wait fall through at once, and the kernel ends normally.
__global__ void __launch_bounds__(32) tpa_wait_selftest_kernel(uint32_t* status, long long budget) {
  __shared__ Barriers bars;
  if (threadIdx.x == 0) {
    mbar_init(&bars.q_full, 1);
    bars.abort = 0;
    fence_mbar_init();
  }
  __syncwarp();
  const Waiter wait{&bars, status, budget};
  if (threadIdx.x == 0) {
    wait(&bars.q_full, 0, 0x7e57);
    wait(&bars.q_full, 0, 0x7e58);  // falls through: the abort flag is up
  }
  __syncwarp();
}

template <int D>
constexpr size_t smem_bytes() {
  return 6 * (size_t)kUnitRows * D * 2 + sizeof(Barriers) + 1024;
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }
inline bool factor_vec_ok(const TpaFactor& f) {
  return aligned16(f.ptr) && f.stride[0] % 8 == 0 && f.stride[1] % 8 == 0 && f.stride[2] % 8 == 0;
}
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
inline size_t ceil128(size_t x) { return (x + 127) / 128 * 128; }  // whole tiles are staged
inline size_t staged_q_bytes(const Params& p) { return align256((size_t)p.batch * p.heads * ceil128(p.lq) * p.dk * 2); }
inline size_t staged_kv_bytes(const Params& p) { return align256((size_t)p.batch * p.heads * ceil128(p.lk) * p.dk * 2); }

template <int D, bool STAGED, int MODE>
cudaError_t launch_attn(const Params& p, const uint8_t* wq, const uint8_t* wk, const uint8_t* wv,
                        dim3 grid, int pairs, int group, const int4* seg_ranges, size_t smem,
                        cudaStream_t stream) {
  auto kern = tpa_fwd_sm100_kernel<D, STAGED, MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<grid, Roles<STAGED>::kThreads, smem, stream>>>(p, wq, wk, wv, pairs, group, seg_ranges);
  return cudaGetLastError();
}

}  // namespace

// Merges the partial (o, lse) of the key splits (and the caller's carried state, if loaded) the
// way the ring merges steps (tpa/ring_tpa.py:82-91): weights exp(lse_i - max), normalised.
//
// One CTA of 8 warps serves whole (row, head) items, never a part of one: with STATE_LOAD and
// STATE_STORE on the same buffers (every middle ring step) the old state_lse / state_o of an item
// are read by the same CTA that overwrites them, after a barrier, so no other block can see a
// half-updated item.  WPR = warps per item: 1 (eight items per CTA; a handful of splits) or 8 (one
// item per CTA; the hundreds of partials of a decode call, warps striding over the splits and
// meeting in shared memory).  Lanes own the columns (float4 each, two when dv > 128).
template <int WPR>
__global__ void __launch_bounds__(256) tpa_combine_splits_kernel(const Params p, const float* part_o,
                                                                 const float* part_lse, int splits) {
  constexpr int kItems = 8 / WPR;
  __shared__ float4 red_acc[WPR > 1 ? 8 : 1][64];
  __shared__ float red_w[8];
  const int d = p.dv, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = warp % WPR;
  const int64_t rows = (int64_t)p.batch * p.lq * p.heads;
  const int64_t rh_raw = (int64_t)blockIdx.x * kItems + warp / WPR;
  const bool item_ok = rh_raw < rows;
  const int64_t rh = item_ok ? rh_raw : rows - 1;  // idle warps shadow the last item and write nothing
  const bool load = (p.flags & TPA_FLAG_STATE_LOAD) != 0, store = (p.flags & TPA_FLAG_STATE_STORE) != 0;
  const int nchunk = d / 4;  // float4 chunks per row (dv is a multiple of 4 here)
  const float old_lse = load ? p.state_lse[rh] : -CUDART_INF_F;

  // every warp finds the maximum over all splits itself (splits / 32 loads per lane)
  float m = old_lse;
  for (int s = lane; s < splits; s += 32) m = fmaxf(m, part_lse[s * rows + rh]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));

  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  float wsum = 0.f;
  auto add = [&](const float* o, float lse) {
    if (lse == -CUDART_INF_F) return;  // warp-uniform
    const float w = expf(lse - m);
    wsum += w;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunk) {
        const float4 v = *reinterpret_cast<const float4*>(o + c * 4);
        acc[i].x += w * v.x; acc[i].y += w * v.y; acc[i].z += w * v.z; acc[i].w += w * v.w;
      }
    }
  };
  if (m != -CUDART_INF_F) {
    if (load && sub == 0) add(p.state_o + rh * d, old_lse);
#pragma unroll 4
    for (int s = sub; s < splits; s += WPR) add(part_o + (s * rows + rh) * d, part_lse[s * rows + rh]);
  }
  if constexpr (WPR > 1) {
    // the eight warps of the item meet in shared memory, warp 0 finishes
    if (lane == 0) red_w[warp] = wsum;
    if (warp > 0) {
      red_acc[warp][lane] = acc[0];
      red_acc[warp][lane + 32] = acc[1];
    }
    __syncthreads();
    if (warp > 0) return;
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      wsum += red_w[w];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float4 v = red_acc[w][lane + 32 * i];
        acc[i].x += v.x; acc[i].y += v.y; acc[i].z += v.z; acc[i].w += v.w;
      }
    }
  } else {
    __syncthreads();  // all items of the CTA have read their old state before anyone overwrites it
  }
  if (!item_ok) return;
  const bool none = !(wsum > 0.f);
  const float inv = none ? 0.f : 1.f / wsum;
  const float lse = none ? -CUDART_INF_F : m + logf(wsum);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int c = lane + 32 * i;
    if (c >= nchunk) continue;
    if (store) {
      *reinterpret_cast<float4*>(p.state_o + rh * d + c * 4) =
          make_float4(acc[i].x * inv, acc[i].y * inv, acc[i].z * inv, acc[i].w * inv);
    } else {
      const float q = none ? CUDART_NAN_F : 1.f;  // rows that saw no key are NaN (tpa/tpa.py:439)
      if (p.dtype == TPA_DTYPE_F32) {  // the generic kernel's partials
        *reinterpret_cast<float4*>(static_cast<float*>(p.o) + rh * d + c * 4) =
            make_float4(acc[i].x * inv * q, acc[i].y * inv * q, acc[i].z * inv * q, acc[i].w * inv * q);
      } else {
        uint2 o;
        o.x = pack_bf16(acc[i].x * inv * q, acc[i].y * inv * q);
        o.y = pack_bf16(acc[i].z * inv * q, acc[i].w * inv * q);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.o) + rh * d + c * 4) = o;
      }
    }
  }
  if (lane == 0) {
    if (store) p.state_lse[rh] = lse;
    else if (p.lse != nullptr) p.lse[rh] = lse;
  }
}

cudaError_t launch_combine_splits(const Params& p, const float* part_o, const float* part_lse, int splits,
                                  cudaStream_t stream) {
  const int64_t rows = (int64_t)p.batch * p.lq * p.heads;
  if (splits > 32)
    tpa_combine_splits_kernel<8><<<(unsigned)rows, 256, 0, stream>>>(p, part_o, part_lse, splits);
  else
    tpa_combine_splits_kernel<1><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(p, part_o, part_lse, splits);
  count_launch(1);
  return cudaGetLastError();
}

// Rebuilds every 128-row tile of Q (times qscale), K and V of all heads into the three arrays
// (the staging launch of the STAGED forward; the backward reads the same images).
cudaError_t launch_stage_tiles(const Params& p, uint8_t* wq, uint8_t* wk, uint8_t* wv, float qscale,
                               cudaStream_t stream) {
  const int nq = (p.lq + kUnitRows - 1) / kUnitRows, nk = (p.lk + kTileKv - 1) / kTileKv;
  dim3 sgrid(p.heads / 8, nq + 2 * nk, p.batch);
  if (p.dk == 128) tpa_stage_tiles_kernel<128><<<sgrid, 256, 0, stream>>>(p, wq, wk, wv, qscale, 0);
  else tpa_stage_tiles_kernel<64><<<sgrid, 256, 0, stream>>>(p, wq, wk, wv, qscale, 0);
  count_launch(1);
  return cudaGetLastError();
}

bool sm100_supported(const Params& p) {
  if (p.dtype != TPA_DTYPE_BF16) return false;
  if (p.dk != p.dv || (p.dk != 64 && p.dk != 128)) return false;
  // lengths need not be multiples of the 128-row tiles: ragged last tiles are zero-padded and
  // masked.  Key ids travel as 16-byte multiples.
  if (p.kv_seg != nullptr && p.lk % 4 != 0) return false;
  if (p.heads % 8 != 0) return false;
  if (p.kv_parts > 1 && p.part_len % kTileKv != 0) return false;  // a key tile lies in one part
  if (p.kv_parts > 1 && (p.k_part_stride % 8 != 0 || p.v_part_stride % 8 != 0)) return false;
  if (p.kv_parts > 1 && p.kv_seg != nullptr && p.kseg_part_stride % 4 != 0) return false;
  if (p.rope_cos != nullptr && (!aligned16(p.rope_cos) || !aligned16(p.rope_sin))) return false;
  // factors are read with 16-byte loads; output rows are written with them
  if (!factor_vec_ok(p.qa) || !factor_vec_ok(p.ka) || !factor_vec_ok(p.va)) return false;
  if (!factor_vec_ok(p.qb) || !factor_vec_ok(p.kb) || !factor_vec_ok(p.vb)) return false;
  if (!(p.flags & TPA_FLAG_STATE_STORE) && !aligned16(p.o)) return false;
  if ((p.flags & (TPA_FLAG_STATE_STORE | TPA_FLAG_STATE_LOAD)) && !aligned16(p.state_o)) return false;
  // key segment ids travel to shared memory as 512-byte bulk copies
  if (p.kv_seg != nullptr && (!aligned16(p.kv_seg) || p.kv_seg_bstride % 4 != 0)) return false;
  return true;
}

// STAGED is the default whenever the shape allows a tensor-core kernel: measured against FUSED it
// wins from 256 x 256 (45 vs 50 us) to 128 x 32768 (0.25 vs 0.61 ms) and T = 32768 (8.1 vs 36.8 ms).
// FUSED stays selectable for callers that want no scratch at all.
int sm100_pick_variant(const Params&) { return TPA_KERNEL_SM100_STAGED; }

// one int4 per (batch, 256-row block) when segment ids are given
inline size_t seg_range_bytes(const Params& p) {
  if (p.q_seg == nullptr) return 0;
  const size_t pairs = (p.lq + 2 * kUnitRows - 1) / (2 * kUnitRows);
  return align256((size_t)p.batch * pairs * sizeof(int4));
}

// Few 256-row blocks against many keys (decode-like, cross attention) would leave most SMs idle:
// the key tiles are then split over several CTAs per block and the partials merged afterwards.
constexpr int kNumSms = 148;
int sm100_pick_splits(const Params& p) {
  const int pairs = (p.lq + 2 * kUnitRows - 1) / (2 * kUnitRows);
  const int64_t items = (int64_t)pairs * p.heads * p.batch;
  const int n_kv = (p.lk + kTileKv - 1) / kTileKv;
  if (items * 2 > kNumSms || n_kv < 8) return 1;
  int splits = (int)(kNumSms / items);
  if (splits > n_kv / 4) splits = n_kv / 4;
  if (splits > 16) splits = 16;
  return splits < 2 ? 1 : splits;
}
inline size_t split_bytes(const Params& p) {
  const int splits = sm100_pick_splits(p);
  if (splits == 1) return 0;
  return align256((size_t)splits * p.batch * p.lq * p.heads * (p.dv + 1) * sizeof(float));
}

size_t sm100_workspace_bytes(const Params& p, int variant) {
  const size_t common = seg_range_bytes(p) + split_bytes(p);
  if (variant != TPA_KERNEL_SM100_STAGED) return common;
  return common + staged_q_bytes(p) + 2 * staged_kv_bytes(p);
}

cudaError_t launch_sm100(const Params& p, int variant, void* workspace, TpaKernelInfo* info,
                         bool dry_run, cudaStream_t stream) {
  const bool staged = variant == TPA_KERNEL_SM100_STAGED;
  const size_t smem = p.dk == 128 ? smem_bytes<128>() : smem_bytes<64>();
  const int pairs = (p.lq + 2 * kUnitRows - 1) / (2 * kUnitRows);
  // Taking all (batch, head) slices of the longest rows first balances best and leaves only
  // short CTAs for the end, but the concurrent CTAs then touch the staged K/V of every slice.
  // So slices are taken in groups whose K/V (lk * d * 4 bytes each) fit in about half of L2:
  // the CTAs of a group stream the same tiles together, and the kernel still ends on the
  // shortest rows of the last group instead of on a whole head's longest ones.
  const int slices = p.heads * p.batch;
  int group = slices;
  if (staged) {
    const size_t per_slice = (size_t)p.lk * p.dk * 4;
    while (group > 1 && ((size_t)group * per_slice > ((size_t)72 << 20) || slices % group != 0)) --group;
  }
  const int splits = sm100_pick_splits(p);
  dim3 grid((unsigned)(pairs * slices), (unsigned)splits, 1);
  if (info) {
    info->kernel = variant;
    info->block_q = 2 * kUnitRows;
    info->block_kv = kTileKv;
    info->threads = staged ? Roles<true>::kThreads : Roles<false>::kThreads;
    info->grid[0] = grid.x;
    info->grid[1] = grid.y;
    info->grid[2] = grid.z;
    info->smem_bytes = (int)smem;
    const bool stage_nothing = (p.flags & TPA_FLAG_REUSE_STAGED_Q) && (p.flags & TPA_FLAG_REUSE_STAGED_KV);
    info->launches = (staged && !stage_nothing ? 2 : 1) + (p.q_seg != nullptr ? 1 : 0) + (splits > 1 ? 1 : 0);
  }
  if (dry_run) return cudaSuccess;
  cudaError_t e;
  // Scratch layout: staged Q, K, V tiles first (STAGED only; the Q tiles are then at the same
  // place whatever the key length is, which is what lets consecutive calls with other keys keep
  // them), then the per-block key-tile ranges, then the key-split partials.
  uint8_t* const after_tiles = static_cast<uint8_t*>(workspace) + (staged ? staged_q_bytes(p) + 2 * staged_kv_bytes(p) : 0);
  int4* seg_ranges = nullptr;
  if (p.q_seg != nullptr) {
    seg_ranges = reinterpret_cast<int4*>(after_tiles);
    tpa_seg_ranges_kernel<<<dim3(pairs, p.batch), 128, 0, stream>>>(p, seg_ranges);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    count_launch(1);
  }
  // with key splits the attention kernel stores partials (as a ring step would) into scratch
  Params pk = p;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    part_o = reinterpret_cast<float*>(after_tiles + seg_range_bytes(p));
    part_lse = part_o + (size_t)splits * p.batch * p.lq * p.heads * p.dv;
    pk.flags = (p.flags & TPA_FLAG_CAUSAL) | TPA_FLAG_STATE_STORE;
    pk.state_o = part_o;
    pk.state_lse = part_lse;
  }
  uint8_t *wq = nullptr, *wk = nullptr, *wv = nullptr;
  if (staged) {
    wq = static_cast<uint8_t*>(workspace);
    wk = wq + staged_q_bytes(p);
    wv = wk + staged_kv_bytes(p);
    const float qscale = p.sm_scale * kLog2e / ((float)p.rank_q * (float)p.rank_k);
    // ring steps after the first keep the Q tiles the previous call staged in this workspace
    const int nq = (p.lq + kUnitRows - 1) / kUnitRows, nk = (p.lk + kTileKv - 1) / kTileKv;
    // ... and two query chunks against the same gathered keys keep the K and V tiles
    const int first_tile = (p.flags & TPA_FLAG_REUSE_STAGED_Q) ? nq : 0;
    const int end_tile = (p.flags & TPA_FLAG_REUSE_STAGED_KV) ? nq : nq + 2 * nk;
    if (end_tile > first_tile) {
      dim3 sgrid(p.heads / 8, end_tile - first_tile, p.batch);
      if (p.dk == 128)
        tpa_stage_tiles_kernel<128><<<sgrid, 256, 0, stream>>>(p, wq, wk, wv, qscale, first_tile);
      else
        tpa_stage_tiles_kernel<64><<<sgrid, 256, 0, stream>>>(p, wq, wk, wv, qscale, first_tile);
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      count_launch(1);
    }
    const int mode = p.has_window() ? 2 : (p.kv_parts > 1 ? 1 : 0);
    auto go = [&](auto kern_d) {
      constexpr int DD = decltype(kern_d)::value;
      switch (mode) {
        case 0: return launch_attn<DD, true, 0>(pk, wq, wk, wv, grid, pairs, group, seg_ranges, smem, stream);
        case 1: return launch_attn<DD, true, 1>(pk, wq, wk, wv, grid, pairs, group, seg_ranges, smem, stream);
        default: return launch_attn<DD, true, 2>(pk, wq, wk, wv, grid, pairs, group, seg_ranges, smem, stream);
      }
    };
    e = p.dk == 128 ? go(std::integral_constant<int, 128>{}) : go(std::integral_constant<int, 64>{});
  } else {
    e = p.dk == 128 ? launch_attn<128, false, 0>(pk, wq, wk, wv, grid, pairs, group, seg_ranges, smem, stream)
                    : launch_attn<64, false, 0>(pk, wq, wk, wv, grid, pairs, group, seg_ranges, smem, stream);
  }
  if (e != cudaSuccess) return e;
  count_launch(1);
  if (splits > 1) e = launch_combine_splits(p, part_o, part_lse, splits, stream);
  return e;
}

cudaError_t launch_wait_selftest(uint32_t* status, long long budget_cycles, cudaStream_t stream) {
  tpa_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, budget_cycles);
  count_launch(1);
  return cudaGetLastError();
}

}  // namespace tpa
