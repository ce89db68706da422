// Tensor-core TPA backward for sm_100a: bf16 factors, head_dim 64 or 128, any lengths.
// Replaces _bwd_kernel (tpa/tpa.py:546-820) for those shapes; the arithmetic is the
// materialising branch of the reference (tpa/tpa.py:777-799).
//
// Per 128 x 128 (query tile, key tile) pair and head, with S2 = log2(e) sm_scale q k^T:
//     p  = 2^(S2 - log2(e) lse)                 masked entries 0      tpa/tpa.py:662-677
//     ds = p (do v^T - delta)                                          tpa/tpa.py:783-786
//     dv += p^T do     dk += sm_scale ds^T q     dq += sm_scale ds k   tpa/tpa.py:778,789,796
//
// The reference gives a program one key block and adds its dq contribution with atomics
// (tpa/tpa.py:806-807).  Here ONE kernel template runs twice, without atomics:
//
//   KV_OWNER   a CTA owns a key tile (K, V resident in shared memory) and streams the query
//              tiles (Q, dO, row statistics) past it.  It computes the TRANSPOSED tiles
//              S^T = K Q^T and dP^T = V dO^T, so that p^T and ds^T sit in TMEM with keys on the
//              lanes and feed dV += p^T dO and dK += ds^T Q as the TMEM (A) operand.
//   !KV_OWNER  a CTA owns a query tile (Q, dO resident) and streams the key tiles (K, V):
//              S = Q K^T, dP = dO V^T, dQ += ds K with ds as the TMEM operand.
//
// Seven tile GEMMs instead of five, all tcgen05.mma with fp32 accumulators in TMEM, in
// exchange for bitwise reproducible gradients and no zero-fill or atomic traffic.  Both passes
// read the same staged operands: tpa_stage_tiles_kernel (shared with the forward) rebuilds the
// per-head Q, K, V tiles from the factors once, tpa_bwd_stage_do_kernel lays dO out the same
// way, and tpa_bwd_stats_kernel writes log2(e) lse and delta per (head, row).  One staged tile
// serves as a K-major operand of the first two GEMMs and as an MN-major operand of the
// accumulating ones; only the descriptor differs.
//
// Roles, by warp: 0-15 element-wise (four threads per TMEM lane, 32 columns each) and the epilogue;
// 16: one thread issues the bulk copies; 17: one thread issues tcgen05.mma.
//
// Pipeline.  A tile has two dependency chains, T1 -> p -> (dV) and T2 -> ds -> (dK | dQ).  A
// commit -> waiter -> arrive -> issuer round trip costs about 500 cycles on top of the MMAs, and
// TMEM is full, so there is no second tile to hide it behind; instead the chains are interleaved:
// the element-wise warps turn T1 into p while the tensor pipe computes T2, and T2 into ds while
// it runs the accumulating GEMM fed by p and the next tile's T1.
// TMEM columns: T1 [0,128) (S, then p as bf16), T2 [128,256) (dP, then ds as bf16),
// accumulators from 256 (dQ, or dK and dV).  Dense fp32 dQ / dK / dV go to scratch; the
// factor contraction (tpa_bwd_contract_kernel) is shared with the SIMT path.
//
// Every mbarrier wait is bounded (~2^28 cycles): the waiter then records where it gave up in
// the status block, raises a CTA-wide abort flag that makes later waits fall through, and the
// CTA runs to its normal end (TMEM is freed).
#include <math_constants.h>

#include "sm100_ptx.cuh"
#include "tpa_common.cuh"

namespace tpa {
namespace {

using namespace ptx;

constexpr int kRows = 128;  // rows of every tile (queries or keys)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr long long kWaitCycles = 1ll << 28;
constexpr int kEwWarps = 16;
constexpr int kProducerWarp = kEwWarps;
constexpr int kMmaWarp = kEwWarps + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;

struct BwdBarriers {
  uint64_t x_full;                   // the CTA's own two tiles have landed
  uint64_t y_full[3], y_empty[3];    // streamed tiles (+ row statistics), two or three stages
  uint64_t t_full[2], p_ready[2], acc_done;  // [0]: T1 written / read (p stored); [1]: T2 written / ds stored
  uint32_t tmem_base;
  volatile uint32_t abort;
  alignas(16) float stats[3][2][kRows];  // [stage][-log2e*lse | -delta][query row] (KV_OWNER)
};

struct BoundedWait {
  BwdBarriers* bars;
  uint32_t* status;
  __device__ __forceinline__ void operator()(uint64_t* bar, uint32_t parity, uint32_t where) const {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
      if (bars->abort) return;
      if ((++spins & 63u) == 0 && clock64() - t0 > kWaitCycles) {
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

// two fp32 values in one 64-bit register for the packed add / mul / fma (half the issue slots)
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
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------
// Row statistics, one warp per (batch, padded row, head):
//   stats[((batch*heads + head) * tiles + row/128) * 256 + row%128]       = -log2(e) * lse
//   stats[...                                       + 128 + row%128]      = -delta
// (negated: the pair kernel only ever adds them).  delta = nansum(o * do) (tpa/tpa.py:976-980).
// Rows that saw no key (lse = -inf) and the padding rows of a ragged last tile get -inf in the
// first slot, so that p = 2^(s - inf) = 0 for them.
__global__ void __launch_bounds__(256) tpa_bwd_stats_kernel(const Params p, const __nv_bfloat16* d_o,
                                                            float* stats, int tiles) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t total = (int64_t)p.batch * tiles * kRows * p.heads;
  if (w >= total) return;
  const int head = (int)(w % p.heads);
  const int64_t rest = w / p.heads;
  const int row = (int)(rest % ((int64_t)tiles * kRows));
  const int batch = (int)(rest / ((int64_t)tiles * kRows));
  float acc = 0.f, nl2 = -CUDART_INF_F;
  if (row < p.lq) {
    const int64_t rh = ((int64_t)batch * p.lq + row) * p.heads + head;
    const __nv_bfloat16* o = static_cast<const __nv_bfloat16*>(p.o) + rh * p.dv;
    const __nv_bfloat16* g = d_o + rh * p.dv;
    for (int t = lane; t < p.dv; t += 32) {
      const float x = __bfloat162float(o[t]) * __bfloat162float(g[t]);
      if (x == x) acc += x;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    const float lse = p.lse[rh];
    if (lse != -CUDART_INF_F) nl2 = -lse * kLog2e;
  }
  if (lane == 0) {
    float* dst = stats + (((int64_t)batch * p.heads + head) * tiles + row / kRows) * (2 * kRows) + row % kRows;
    dst[0] = nl2;
    dst[kRows] = -acc;
  }
}

// dO[batch, lq, heads, D] -> per (batch, head, tile) shared-memory images (64-column sub-tiles of
// 16 KB, 128-byte swizzle), rows past lq zero.  grid = (tiles, batch), 256 threads.
template <int D>
__global__ void __launch_bounds__(256) tpa_bwd_stage_do_kernel(const Params p, const __nv_bfloat16* d_o,
                                                               uint8_t* ws, int tiles) {
  constexpr int CH = D / 8;
  constexpr int kTileBytes = kRows * D * 2;
  const int tile = blockIdx.x, batch = blockIdx.y;
  const int per_row = p.heads * CH;
  for (int idx = threadIdx.x; idx < kRows * per_row; idx += 256) {
    const int row = idx / per_row, rem = idx - row * per_row;
    const int head = rem / CH, chunk = rem - head * CH;
    const int64_t g = (int64_t)tile * kRows + row;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (g < p.lq)
      v = __ldg(reinterpret_cast<const uint4*>(d_o + (((int64_t)batch * p.lq + g) * p.heads + head) * D + chunk * 8));
    uint8_t* dst = ws + (((int64_t)batch * p.heads + head) * tiles + tile) * kTileBytes +
                   (chunk >> 3) * (kRows * 128) + sw128_offset(row, chunk & 7);
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

// ---------------------------------------------------------------------------------------------
// The pair kernel.  "own" = the tile pair the CTA keeps (K,V or Q,dO), "moving" = the tiles it
// streams (Q,dO or K,V).  T1 = own0 moving0^T, T2 = own1 moving1^T; acc0 += ds moving0,
// acc1 += p moving1 (KV_OWNER only).  dense0 / dense1: fp32 [batch, len, heads, D].
template <int D, bool KV_OWNER>
__global__ void __launch_bounds__(kThreads, 1)
tpa_bwd_sm100_kernel(const Params p, const uint8_t* ws_q, const uint8_t* ws_k, const uint8_t* ws_v,
                     const uint8_t* ws_do, const float* stats, float* dense0, float* dense1,
                     const int own_tiles, const int group) {
  constexpr int kTileBytes = kRows * D * 2;
  constexpr uint32_t kIdescT = make_idesc(128, kRows, false, false);
  constexpr uint32_t kIdescAcc = make_idesc(128, D, false, true);
  constexpr int kT2 = 128, kAcc = 256;
  // Where TMEM has room (all but the key-owner pass at head_dim 128) the CTA's own two tiles live
  // there as the A operands of the first two GEMMs: an operand in TMEM is not re-read from shared
  // memory by every MMA (an M128 N128 K16 MMA with both operands in shared memory needs all of
  // its 128 B/clk, leaving nothing for the bulk copies), and the 2 tiles of shared memory it
  // frees hold a third stage of streamed tiles.
  constexpr bool kOwnTmem = !KV_OWNER || D == 64;
  constexpr int kStages = kOwnTmem ? 3 : 2;
  constexpr int kOwnCol = kAcc + (KV_OWNER ? 2 : 1) * D;  // own tile g: columns kOwnCol + g * D/2
  static_assert(kOwnCol + (kOwnTmem ? D : 0) <= 512, "TMEM budget");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sX = smem;                   // own tiles (unless in TMEM): [0] K or Q, [1] V or dO
  uint8_t* sY = smem + (kOwnTmem ? 0 : 2) * kTileBytes;  // moving tiles: stage s at s * 2 tiles: [0] Q or K, [1] dO or V
  BwdBarriers* bars = reinterpret_cast<BwdBarriers*>(sY + kStages * 2 * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.lq + kRows - 1) / kRows, nk = (p.lk + kRows - 1) / kRows;
  // (batch, head) slices are taken `group` at a time so that the CTAs running together stream
  // the same moving tiles through L2; within a group the tiles with the longest walk go first.
  const int per_group = group * own_tiles;
  const int slice = (blockIdx.x / per_group) * group + (blockIdx.x % per_group) % group;
  const int ord = (blockIdx.x % per_group) / group;
  const int own = KV_OWNER ? ord : own_tiles - 1 - ord;
  const int head = slice % p.heads, batch = slice / p.heads;
  const int own0 = own * kRows;
  const bool causal = (p.flags & TPA_FLAG_CAUSAL) != 0;
  const bool has_seg = p.q_seg != nullptr;

  // moving tiles that can hold a visible pair
  int t_lo = 0, t_hi = KV_OWNER ? nq : nk;
  if (causal) {
    if (KV_OWNER) {
      const int64_t first = (int64_t)own0 + p.k_offset - p.q_offset;  // first row that sees key own0
      if (first > 0) t_lo = (int)min((int64_t)t_hi, first / kRows);
    } else {
      const int64_t last = (int64_t)own0 + kRows - 1 + p.q_offset - p.k_offset;  // last visible key
      t_hi = last < 0 ? 0 : (int)min((int64_t)t_hi, last / kRows + 1);
    }
  }
  const int n_tiles = max(0, t_hi - t_lo);

  if (threadIdx.x == 0) {
    mbar_init(&bars->x_full, kOwnTmem ? kEwWarps : 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->y_full[s], 1);
      mbar_init(&bars->y_empty[s], 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(&bars->t_full[h], 1);
      mbar_init(&bars->p_ready[h], kEwWarps);
    }
    mbar_init(&bars->acc_done, 1);
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
  const BoundedWait wait{bars, p.status};
  const int64_t bh = (int64_t)batch * p.heads + head;

  if (warp < kEwWarps) {
    // ------------------------------------------------------------------ element-wise + epilogue
    // Four threads per TMEM lane: warp w serves lanes 32 (w & 3)... and the 32 columns (moving
    // rows) 32 (w >> 2)... of T1 and T2.  Per tile: phase 1 turns T1 into p, phase 2 turns T2
    // into ds; each has its own pair of barriers.
    const int quarter = warp & 3, cq = warp >> 2;
    const int row = quarter * 32 + lane;  // TMEM lane = row of the own tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int own_idx = own0 + row;
    const bool own_ok = own_idx < (KV_OWNER ? p.lk : p.lq);
    const int64_t own_pos = (int64_t)own_idx + (KV_OWNER ? p.k_offset : p.q_offset);
    const int mov_len = KV_OWNER ? p.lq : p.lk;
    const int64_t mov_off = KV_OWNER ? p.q_offset : p.k_offset;
    int own_seg = 0;
    const int32_t* mov_seg = nullptr;
    if (has_seg) {
      const int32_t* own_ids = KV_OWNER ? p.kv_seg + (int64_t)batch * p.kv_seg_bstride
                                        : p.q_seg + (int64_t)batch * p.q_seg_bstride;
      mov_seg = KV_OWNER ? p.q_seg + (int64_t)batch * p.q_seg_bstride
                         : p.kv_seg + (int64_t)batch * p.kv_seg_bstride;
      if (own_ok) own_seg = own_ids[own_idx];
    }
    float my_nl2 = -CUDART_INF_F, my_ndl = 0.f;  // !KV_OWNER: this lane's query row
    if (!KV_OWNER) {
      const float* st = stats + (bh * nq + own) * (2 * kRows);
      my_nl2 = st[row];
      my_ndl = st[kRows + row];
    }
    const float inv_rk = 1.f / (float)p.rank_k;
    const uint64_t my_nl2_2 = pack2(my_nl2, my_nl2), my_ndl_2 = pack2(my_ndl, my_ndl), inv_rk_2 = pack2(inv_rk, inv_rk);
    const int64_t lane0_pos = (int64_t)own0 + quarter * 32 + (KV_OWNER ? p.k_offset : p.q_offset);

    if (kOwnTmem && n_tiles > 0) {
      // own tiles -> TMEM in the layout of a tcgen05.mma A operand: lane = row, one 32-bit column
      // per two consecutive bf16 of the row.  Read straight from the staged (swizzled) images.
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint8_t* src = KV_OWNER ? (g == 0 ? ws_k : ws_v) + (bh * nk + own) * kTileBytes
                                      : (g == 0 ? ws_q : ws_do) + (bh * nq + own) * kTileBytes;
#pragma unroll
        for (int i = 0; i < D / 64; ++i) {  // this thread: D/4 elements = D/32 chunks of 16 bytes, 4 at a time
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int chunk = cq * (D / 32) + i * 2 + j;
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (chunk >> 3) * (kRows * 128) +
                                                                 sw128_offset(row, chunk & 7)));
            w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
          }
          tmem_st8(tmem + lane_base + kOwnCol + g * (D / 2) + cq * (D / 8) + i * 8, w);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->x_full);
    }

    const int c0 = cq * 32;  // this thread's 32 columns (moving rows) of every tile
    for (int n = 0; n < n_tiles; ++n) {
      const int s = n % kStages;
      const int m0 = (t_lo + n) * kRows + c0;  // first moving row of those columns
      // does any pair of these 32 lanes x 32 columns need the element-wise test?
      bool masked = has_seg;
      if (causal) {
        if (KV_OWNER) masked = masked || ((int64_t)m0 + mov_off < lane0_pos + 31);  // min q < max key
        else masked = masked || ((int64_t)m0 + 31 + mov_off > lane0_pos);            // max key > min q
      }
      if (!KV_OWNER) masked = masked || (m0 + 32 > p.lk);  // padded keys of a ragged last tile

      // ---- phase 1: p = 2^(T1 + (-log2e lse)), as soon as the first GEMM is done (the second runs meanwhile)
      wait(&bars->t_full[0], n & 1, 0x100);
      tc_fence_after();
      if (KV_OWNER) wait(&bars->y_full[s], (n / kStages) & 1, 0x102);  // the statistics have landed
      uint32_t ppk[16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t1[16];
        tmem_ld16(tmem + lane_base + c0 + c * 16, t1);
        float l2v[16];
        if (KV_OWNER) {
          const float4* a4 = reinterpret_cast<const float4*>(bars->stats[s][0] + c0 + c * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 a = a4[i];
            l2v[4 * i] = a.x; l2v[4 * i + 1] = a.y; l2v[4 * i + 2] = a.z; l2v[4 * i + 3] = a.w;
          }
        }
        tmem_ld_wait();
        if (masked) {  // rare (diagonal and ragged tiles, segment ids): -inf logits give p = 0 below
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int mi = m0 + c * 16 + e;
            const int64_t mpos = (int64_t)mi + mov_off;
            bool keep = mi < mov_len;
            if (causal) keep = keep && (KV_OWNER ? (mpos >= own_pos) : (own_pos >= mpos));
            if (has_seg && keep) keep = mov_seg[mi] == own_seg;
            if (!keep) t1[e] = 0xff800000u;
          }
        }
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          float x0, x1;
          unpack2(add2(pack2(__uint_as_float(t1[e]), __uint_as_float(t1[e + 1])),
                       KV_OWNER ? pack2(l2v[e], l2v[e + 1]) : my_nl2_2), x0, x1);
          ppk[c * 8 + e / 2] = pack_bf16(ex2(x0), ex2(x1));
        }
      }
      // bf16 p overwrites the first 16 of the thread's own 32 fp32 columns: moving row k of the
      // tile is at column (k / 32) * 32 + (k % 32) / 2.  The query-owner pass needs p only here.
      if (KV_OWNER) {
        tmem_st16(tmem + lane_base + c0, ppk);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready[0]);  // T1 has been read (and holds p)

      // ---- phase 2: ds = p (T2 / R_k + (-delta)), p as rounded to bf16 above
      wait(&bars->t_full[1], n & 1, 0x101);
      tc_fence_after();
      uint32_t dpk[16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t2[16];
        tmem_ld16(tmem + lane_base + kT2 + c0 + c * 16, t2);
        float dlv[16];
        if (KV_OWNER) {
          const float4* b4 = reinterpret_cast<const float4*>(bars->stats[s][1] + c0 + c * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 b = b4[i];
            dlv[4 * i] = b.x; dlv[4 * i + 1] = b.y; dlv[4 * i + 2] = b.z; dlv[4 * i + 3] = b.w;
          }
        }
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const uint32_t pw = ppk[c * 8 + e / 2];
          const uint64_t p2 = pack2(__uint_as_float(pw << 16), __uint_as_float(pw & 0xffff0000u));
          float d0, d1;
          unpack2(mul2(p2, fma2(pack2(__uint_as_float(t2[e]), __uint_as_float(t2[e + 1])), inv_rk_2,
                                KV_OWNER ? pack2(dlv[e], dlv[e + 1]) : my_ndl_2)), d0, d1);
          dpk[c * 8 + e / 2] = pack_bf16(d0, d1);
        }
      }
      tmem_st16(tmem + lane_base + kT2 + c0, dpk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready[1]);  // T2 holds ds
    }

    // epilogue: accumulators -> dense fp32 rows (zeros when nothing was visible)
    if (n_tiles > 0) {
      wait(&bars->acc_done, 0, 0x200);
      tc_fence_after();
    }
    const int own_len = KV_OWNER ? p.lk : p.lq;
    const float scale0 = KV_OWNER ? (float)p.rank_k * kLn2 : p.sm_scale * inv_rk;
#pragma unroll
    for (int a = 0; a < (KV_OWNER ? 2 : 1); ++a) {
      float* dst = (a == 0 ? dense0 : dense1) +
                   (((int64_t)batch * own_len + own_idx) * p.heads + head) * D + cq * (D / 4);
      const float scale = a == 0 ? scale0 : 1.f;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[16];
        if (n_tiles > 0) {
          tmem_ld16(tmem + lane_base + kAcc + a * D + cq * (D / 4) + c * 16, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) r[e] = 0u;
        }
        if (own_ok) {
#pragma unroll
          for (int e = 0; e < 16; e += 4)
            *reinterpret_cast<float4*>(dst + c * 16 + e) =
                make_float4(__uint_as_float(r[e]) * scale, __uint_as_float(r[e + 1]) * scale,
                            __uint_as_float(r[e + 2]) * scale, __uint_as_float(r[e + 3]) * scale);
        }
      }
    }
  } else if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ bulk copies of staged tiles
    if (lane == 0 && n_tiles > 0) {  // every copy issued here is waited for by the MMA thread
      const uint8_t* gx0 = (KV_OWNER ? ws_k + (bh * nk + own) * kTileBytes : ws_q + (bh * nq + own) * kTileBytes);
      const uint8_t* gx1 = (KV_OWNER ? ws_v + (bh * nk + own) * kTileBytes : ws_do + (bh * nq + own) * kTileBytes);
      if (!kOwnTmem) {
        mbar_arrive_expect_tx(&bars->x_full, 2 * kTileBytes);
        bulk_g2s(sX, gx0, kTileBytes, &bars->x_full);
        bulk_g2s(sX + kTileBytes, gx1, kTileBytes, &bars->x_full);
      }
      for (int n = 0; n < n_tiles; ++n) {
        const int s = n % kStages;
        const int64_t t = t_lo + n;
        if (n >= kStages) wait(&bars->y_empty[s], ((n / kStages) - 1) & 1, 0x400);
        const uint8_t* gy0 = KV_OWNER ? ws_q + (bh * nq + t) * kTileBytes : ws_k + (bh * nk + t) * kTileBytes;
        const uint8_t* gy1 = KV_OWNER ? ws_do + (bh * nq + t) * kTileBytes : ws_v + (bh * nk + t) * kTileBytes;
        mbar_arrive_expect_tx(&bars->y_full[s], 2 * kTileBytes + (KV_OWNER ? 2 * kRows * 4 : 0));
        bulk_g2s(sY + s * 2 * kTileBytes, gy0, kTileBytes, &bars->y_full[s]);
        bulk_g2s(sY + s * 2 * kTileBytes + kTileBytes, gy1, kTileBytes, &bars->y_full[s]);
        if (KV_OWNER)
          bulk_g2s(bars->stats[s], stats + (bh * nq + t) * (2 * kRows), 2 * kRows * 4, &bars->y_full[s]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ MMA issue (one thread)
    if (lane == 0 && n_tiles > 0) {
      const uint32_t aX = smem_u32(sX), aY = smem_u32(sY);
      // Descriptors are built once; an MMA then only adds its byte offset (>> 4) to the address field.
      const uint64_t dX0 = make_desc(aX, 16, 1024), dX1 = make_desc(aX + kTileBytes, 16, 1024);
      const uint64_t dYk0 = make_desc(aY, 16, 1024);            // moving tiles as K-major operands
      const uint64_t dYm0 = make_desc(aY, kRows * 128, 1024);   // ... and as MN-major operands
      auto stage_off = [&](int n) { return (uint32_t)(((n % kStages) * 2 * kTileBytes) >> 4); };
      // g = 0: T1 = own0 moving0^T;  g = 1: T2 = own1 moving1^T  (M128 N128, D/16 K steps)
      auto issue_t = [&](int n, int g) {
        const uint64_t dy = dYk0 + stage_off(n) + ((g * kTileBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * (kRows * 128) + (ks & 3) * 32) >> 4;
          if (kOwnTmem) mma_ts(tmem + g * kT2, tmem + kOwnCol + g * (D / 2) + ks * 8, dy + off, kIdescT, ks > 0);
          else mma_ss(tmem + g * kT2, (g == 0 ? dX0 : dX1) + off, dy + off, kIdescT, ks > 0);
        }
        tc_commit(&bars->t_full[g]);
      };
      // a = 0: acc0 += ds moving0 (ds in T2);  a = 1: acc1 += p moving1 (p in T1); eight K steps of 16 rows
      auto issue_acc = [&](int n, int a) {
        const uint64_t dy = dYm0 + stage_off(n) + ((a * kTileBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < kRows / 16; ++ks) {
          const uint32_t acol = (ks >> 1) * 32 + (ks & 1) * 8;  // where the element-wise role put rows 16 ks ...
          mma_ts(tmem + kAcc + a * D, tmem + (a == 0 ? kT2 : 0) + acol, dy + ((ks * 2048) >> 4), kIdescAcc,
                 (n > 0 || ks > 0) ? 1u : 0u);
        }
      };
      // The two chains of a tile (T1 -> p -> acc1, T2 -> ds -> acc0) interleave, so that every wait
      // for the element-wise warps is covered by an independent GEMM already in the queue:
      //   T1(0) T2(0) | [p(n)] acc1(n) T1(n+1) | [ds(n)] acc0(n) T2(n+1) | ...
      // T1(n+1) overwrites p(n) after acc1(n) has read it, T2(n+1) overwrites ds(n) after acc0(n):
      // the tensor pipe executes in issue order.  (The query-owner pass has no acc1; there [p(n)]
      // only says that T1(n) has been read.)
      wait(&bars->x_full, 0, 0x600);
      tc_fence_after();
      wait(&bars->y_full[0], 0, 0x601);
      tc_fence_after();
      issue_t(0, 0);
      issue_t(0, 1);
      for (int n = 0; n < n_tiles; ++n) {
        const bool more = n + 1 < n_tiles;
        wait(&bars->p_ready[0], n & 1, 0x610);
        tc_fence_after();
        if (KV_OWNER) issue_acc(n, 1);
        if (more) {
          wait(&bars->y_full[(n + 1) % kStages], ((n + 1) / kStages) & 1, 0x602);
          tc_fence_after();
          issue_t(n + 1, 0);
        }
        wait(&bars->p_ready[1], n & 1, 0x611);
        tc_fence_after();
        issue_acc(n, 0);
        tc_commit(&bars->y_empty[n % kStages]);
        if (more) issue_t(n + 1, 1);
      }
      tc_commit(&bars->acc_done);
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
inline size_t ceil128(size_t x) { return (x + 127) / 128 * 128; }
inline size_t staged_bytes(const Params& p, int len) { return align256((size_t)p.batch * p.heads * ceil128(len) * p.dk * 2); }
inline size_t stats_bytes(const Params& p) { return align256((size_t)p.batch * p.heads * ceil128(p.lq) * 2 * sizeof(float)); }

template <int D, bool KV_OWNER>
cudaError_t launch_pairs(const Params& p, const uint8_t* wq, const uint8_t* wk, const uint8_t* wv,
                         const uint8_t* wdo, const float* stats, float* dense0, float* dense1,
                         cudaStream_t stream) {
  const int nq = (p.lq + kRows - 1) / kRows, nk = (p.lk + kRows - 1) / kRows;
  const int own_tiles = KV_OWNER ? nk : nq;
  const int slices = p.heads * p.batch;
  // slices whose streamed tiles (two arrays of len * D bf16) fit in about half of L2 run together
  const size_t per_slice = (size_t)(KV_OWNER ? p.lq : p.lk) * D * 4;
  int group = slices;
  while (group > 1 && ((size_t)group * per_slice > ((size_t)72 << 20) || slices % group != 0)) --group;
  const size_t smem = 6 * (size_t)kRows * D * 2 + sizeof(BwdBarriers) + 1024;  // 2 own + 2 x 2 streamed tiles, or 3 x 2 streamed
  auto kern = tpa_bwd_sm100_kernel<D, KV_OWNER>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)(own_tiles * slices), kThreads, smem, stream>>>(p, wq, wk, wv, wdo, stats, dense0, dense1,
                                                                  own_tiles, group);
  count_launch(1);
  return cudaGetLastError();
}

}  // namespace

bool bwd_sm100_supported(const BwdParams& bp) {
  return sm100_supported(bp.f) && (reinterpret_cast<uintptr_t>(bp.d_o) & 15) == 0;
}

// statistics + staged Q, K, V, dO
size_t bwd_sm100_workspace_bytes(const Params& p) {
  return stats_bytes(p) + 2 * staged_bytes(p, p.lq) + 2 * staged_bytes(p, p.lk);
}

// dense dQ / dK / dV of the whole batch into bp.{dq,dk,dv}_dense: statistics, two staging
// launches, the key-owner pass and the query-owner pass (five launches)
cudaError_t launch_bwd_pairs_sm100(const BwdParams& bp, void* workspace, cudaStream_t stream) {
  const Params& p = bp.f;
  const int nq = (p.lq + kRows - 1) / kRows;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* stats = reinterpret_cast<float*>(ws);
  uint8_t* wq = ws + stats_bytes(p);
  uint8_t* wdo = wq + staged_bytes(p, p.lq);
  uint8_t* wk = wdo + staged_bytes(p, p.lq);
  uint8_t* wv = wk + staged_bytes(p, p.lk);
  const __nv_bfloat16* d_o = static_cast<const __nv_bfloat16*>(bp.d_o);

  const int64_t warps = (int64_t)p.batch * nq * kRows * p.heads;
  tpa_bwd_stats_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(p, d_o, stats, nq);
  count_launch(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const float qscale = p.sm_scale * kLog2e / ((float)p.rank_q * (float)p.rank_k);
  e = launch_stage_tiles(p, wq, wk, wv, qscale, stream);
  if (e != cudaSuccess) return e;
  if (p.dk == 128) tpa_bwd_stage_do_kernel<128><<<dim3(nq, p.batch), 256, 0, stream>>>(p, d_o, wdo, nq);
  else tpa_bwd_stage_do_kernel<64><<<dim3(nq, p.batch), 256, 0, stream>>>(p, d_o, wdo, nq);
  count_launch(1);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (p.dk == 128) {
    e = launch_pairs<128, true>(p, wq, wk, wv, wdo, stats, bp.dk_dense, bp.dv_dense, stream);
    if (e == cudaSuccess) e = launch_pairs<128, false>(p, wq, wk, wv, wdo, stats, bp.dq_dense, nullptr, stream);
  } else {
    e = launch_pairs<64, true>(p, wq, wk, wv, wdo, stats, bp.dk_dense, bp.dv_dense, stream);
    if (e == cudaSuccess) e = launch_pairs<64, false>(p, wq, wk, wv, wdo, stats, bp.dq_dense, nullptr, stream);
  }
  return e;
}

}  // namespace tpa
