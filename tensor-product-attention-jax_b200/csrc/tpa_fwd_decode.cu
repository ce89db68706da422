// TPA forward for a handful of query rows against a long key/value factor cache (decode and
// cross shapes, tpa/tpa_test.py:67-70; bf16 factors).  K and V are never materialised:
//
//   logits  s[h, j] = c * sum_{rq, rk} qa[rq, h] ka[j, rk, h] (qb[rq, :] . kb[j, rk, :])       (mma.sync)
//           the rank-space form of the reference's `nomat` branch (tpa/tpa.py:333-359):
//           R_q R_k (d + h) multiply-adds per key instead of R_k h d
//   output  o[h, :] = (1 / R_k) sum_{j, rk} (p[h, j] va[j, rk, h]) vb[j, rk, :]                 (mma.sync)
//
// so every factor byte is read from HBM exactly once per query row and nothing else is: the
// staged tensor-core path rebuilds and writes all heads' dense K/V tiles first (h d / (R_k (h+d))
// = 12.8x the factor bytes at h = 32, d = 128, R_k = 2), which is what a single decode row cannot
// amortise.  The two contractions (qb kb^T and w vb) run on the tensor cores, the rest in fp32 on CUDA
// cores: measured 1.4-1.6 TB/s of factor stream (8.4x the staged path for one row, 24 % of the
// HBM roof); what remains is the fp32 logits / softmax / p * va pass and five block-wide syncs per tile.
//
// grid = (key splits, query rows, batch); 256 threads.  A CTA walks its share of the keys in tiles
// of 64 (key, rank) rows, keeps a running (max, sum) per head and the h x dv accumulator in
// mma.sync fragments (warp w owns value columns 16 w ... 16 w + 15 of every head), and leaves
// a normalised partial (o, lse) per split that tpa_combine_splits_kernel merges (with the caller's
// carried state, if any) exactly as a ring step's partials are merged (tpa/ring_tpa.py:82-91).
#include <math_constants.h>

#include "tpa_common.cuh"

namespace tpa {
namespace {

constexpr int DEC_THREADS = 256;
constexpr int DEC_JR = 64;  // (key, rank) rows per tile

__device__ __forceinline__ void bf16x8_to_float4(const uint4 v, float4& lo, float4& hi) {
  lo = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                   __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
  hi = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                   __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
}

// D (16 x 8, fp32) += A (16 x 16, bf16, row-major fragments) * B (16 x 8, bf16, "col" fragments)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t smem_addr(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}
// two / four 8 x 8 b16 matrices; lane l supplies the address of row l % 8 of matrix l / 8
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_addr(row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(row)));
}

// One factor array of a tile: 16-byte chunks (8 bf16) of the rows jr -> (key0 + jr / rank, jr % rank),
// fetched into registers while the previous tile is being computed and written to shared
// memory (as fp32, row pitch ld) at the start of the next iteration.  Thread t owns chunk
// t % CPR of the rows t / CPR + i * (256 / CPR), i < N (CPR = 16 or 8 chunks per row at most),
// so that nothing has to be divided inside the key loop.
template <int N, int CPR>
struct TileLoad {
  uint4 v[N];
  int goff[N];    // element offset of the chunk relative to the tile's first key, -1: no such chunk
  int keyrel[N];  // its key relative to the tile's first key
  __device__ __forceinline__ void init(const int64_t* st, int rank, int cols, int tid) {
    const int c = tid % CPR;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int jr = tid / CPR + i * (DEC_THREADS / CPR);
      keyrel[i] = jr / rank;
      const bool exists = c * 8 < cols && jr < (DEC_JR / rank) * rank;
      goff[i] = exists ? (int)(keyrel[i] * st[1] + (jr % rank) * st[2] + c * 8) : -1;
    }
  }
  __device__ __forceinline__ void fetch(const __nv_bfloat16* f, const int64_t* st, int key0, int key_end) {
    const __nv_bfloat16* base = f + (int64_t)key0 * st[1];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      v[i] = make_uint4(0u, 0u, 0u, 0u);
      if (goff[i] >= 0 && key0 + keyrel[i] < key_end) v[i] = __ldg(reinterpret_cast<const uint4*>(base + goff[i]));
    }
  }
  // the 16-byte chunks as they are (bf16 tile, row pitch `pitch` elements, a multiple of 8)
  __device__ __forceinline__ void store_raw(__nv_bfloat16* dst, int pitch, int cols, int tid) const {
    const int c = tid % CPR;
    if (c * 8 >= cols) return;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int jr = tid / CPR + i * (DEC_THREADS / CPR);
      *reinterpret_cast<uint4*>(dst + jr * pitch + c * 8) = v[i];
    }
  }
  __device__ __forceinline__ void store(float* dst, int ld, int cols, int tid) const {
    const int c = tid % CPR;
    if (c * 8 >= cols) return;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int jr = tid / CPR + i * (DEC_THREADS / CPR);
      float4 lo, hi;
      bf16x8_to_float4(v[i], lo, hi);
      float2* d = reinterpret_cast<float2*>(dst + jr * ld + c * 8);  // ld is even, not always a multiple of 4
      d[0] = make_float2(lo.x, lo.y);
      d[1] = make_float2(lo.z, lo.w);
      d[2] = make_float2(hi.x, hi.y);
      d[3] = make_float2(hi.z, hi.w);
    }
  }
};

// Shared-memory layout, shared by the kernel and the host-side size computation.
struct DecodeSmem {
  int qb16, kb16, vb16, w16;           // bf16 tiles (byte offsets), rows padded by 16 bytes
  int qa, ka, va, dots, s, m, l, c, kseg, total;  // fp32 / int32 arrays (byte offsets)
  int pk, pv, pw;                      // row pitches of the bf16 tiles, elements
  __host__ __device__ DecodeSmem(int h, int dk, int dv, int rq, int mt) {
    pk = dk + 8; pv = dv + 8; pw = DEC_JR + 8;
    int off = 0;
    qb16 = off; off += 16 * pk * 2;
    kb16 = off; off += DEC_JR * pk * 2;
    vb16 = off; off += DEC_JR * pv * 2;
    w16 = off; off += mt * 16 * pw * 2;
    qa = off; off += rq * h * 4;
    ka = off; off += DEC_JR * h * 4;
    va = off; off += DEC_JR * h * 4;
    dots = off; off += DEC_JR * rq * 4;
    s = off; off += h * (DEC_JR + 1) * 4;
    m = off; off += h * 4;
    l = off; off += h * 4;
    c = off; off += h * 4;
    kseg = off; off += DEC_JR * 4;
    total = off;
  }
};

// MT = ceil(heads / 16) row tiles of the p * vb product.  Both contractions run on the tensor
// cores (mma.sync m16n8k16, bf16 in, fp32 out: with 32 heads a tcgen05 M128 tile would be three
// quarters padding):  dots[rq, jr] = qb (16 x dk) kb^T,  warp w -> the 8 (key, rank) rows 8 w ...;
//                     o[h, dv]   += w (h x 64) vb (64 x dv), warp w -> value columns 16 w ...
template <int MT>
__global__ void __launch_bounds__(DEC_THREADS, MT <= 2 ? 2 : 1)
tpa_fwd_decode_kernel(const Params p, float* part_o, float* part_lse, const int keys_per_split) {
  extern __shared__ uint4 smem_u4[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(smem_u4);
  const int h = p.heads, dk = p.dk, dv = p.dv, rq = p.rank_q, rk = p.rank_k;
  const int KT = DEC_JR / rk;  // keys per tile
  const DecodeSmem L(h, dk, dv, rq, MT);
  __nv_bfloat16* qb16 = reinterpret_cast<__nv_bfloat16*>(smem + L.qb16);  // [16][dk + 8], rows >= rq zero
  __nv_bfloat16* kb16 = reinterpret_cast<__nv_bfloat16*>(smem + L.kb16);  // [JR][dk + 8]
  __nv_bfloat16* vb16 = reinterpret_cast<__nv_bfloat16*>(smem + L.vb16);  // [JR][dv + 8]
  __nv_bfloat16* w16 = reinterpret_cast<__nv_bfloat16*>(smem + L.w16);    // [16 MT][JR + 8] p * va
  float* qaS = reinterpret_cast<float*>(smem + L.qa);    // [rq][h], times sm_scale / (R_q R_k)
  float* kaS = reinterpret_cast<float*>(smem + L.ka);    // [JR][h]
  float* vaS = reinterpret_cast<float*>(smem + L.va);    // [JR][h]
  float* dots = reinterpret_cast<float*>(smem + L.dots); // [JR][rq]
  float* sS = reinterpret_cast<float*>(smem + L.s);      // scratch of the softmax pass (>= 16 h floats)
  float* mS = reinterpret_cast<float*>(smem + L.m);      // [h] running maximum
  float* lS = reinterpret_cast<float*>(smem + L.l);      // [h] running sum
  float* cS = reinterpret_cast<float*>(smem + L.c);      // [h] correction of this tile
  int* ksegS = reinterpret_cast<int*>(smem + L.kseg);    // [KT]

  const int split = blockIdx.x, qi = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;  // fragment coordinates of mma.sync
  const bool causal = (p.flags & TPA_FLAG_CAUSAL) != 0;
  const bool has_seg = p.q_seg != nullptr;
  const __nv_bfloat16* qa = static_cast<const __nv_bfloat16*>(p.qa.ptr) + (int64_t)b * p.qa.stride[0] + (int64_t)qi * p.qa.stride[1];
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(p.qb.ptr) + (int64_t)b * p.qb.stride[0] + (int64_t)qi * p.qb.stride[1];
  const __nv_bfloat16* ka = static_cast<const __nv_bfloat16*>(p.ka.ptr) + (int64_t)b * p.ka.stride[0];
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(p.kb.ptr) + (int64_t)b * p.kb.stride[0];
  const __nv_bfloat16* va = static_cast<const __nv_bfloat16*>(p.va.ptr) + (int64_t)b * p.va.stride[0];
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(p.vb.ptr) + (int64_t)b * p.vb.stride[0];
  const int32_t* kseg_g = has_seg ? p.kv_seg + (int64_t)b * p.kv_seg_bstride : nullptr;
  const int qseg = has_seg ? p.q_seg[(int64_t)b * p.q_seg_bstride + qi] : 0;

  // this CTA's keys, cut at the causal diagonal (tpa/tpa.py:376-379 with global offsets)
  int k_begin = split * keys_per_split;
  int k_end = min(p.lk, k_begin + keys_per_split);
  if (causal) {
    const int64_t last = (int64_t)qi + p.q_offset - p.k_offset;  // last visible local key
    k_end = (int)max((int64_t)k_begin, min((int64_t)k_end, last + 1));
  }

  const float c = p.sm_scale / ((float)rq * (float)rk);
  for (int idx = tid; idx < 16 * L.pk; idx += DEC_THREADS) {
    const int r = idx / L.pk, t = idx - r * L.pk;
    qb16[idx] = (r < rq && t < dk) ? qb[r * p.qb.stride[2] + t] : __float2bfloat16_rn(0.f);
  }
  for (int idx = tid; idx < MT * 16 * L.pw; idx += DEC_THREADS) w16[idx] = __float2bfloat16_rn(0.f);
  for (int idx = tid; idx < rq * h; idx += DEC_THREADS)
    qaS[idx] = c * to_float(qa[(idx / h) * p.qa.stride[2] + idx % h]);
  for (int idx = tid; idx < h; idx += DEC_THREADS) {
    mS[idx] = -CUDART_INF_F;
    lS[idx] = 0.f;
  }
  constexpr int HI = (MT + 1) / 2;  // heads per lane in the softmax pass (lanes over heads)
  float* red = sS;                  // [2][8 warps][h] per-warp maxima, then per-warp sums
  float m_keep[HI], c_keep[HI];     // warp 0: the new maximum and correction of its heads
#pragma unroll
  for (int hi = 0; hi < HI; ++hi) m_keep[hi] = c_keep[hi] = 0.f;
  float acc[MT][2][4];  // [row tile][column tile of 8][fragment]
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][n][e] = 0.f;

  // 64 rows x (dk | dv <= 128: 16 chunks per row) = 4 chunks per thread, x (h <= 64: 8 chunks) = 2
  TileLoad<4, 16> t_kb, t_vb;
  TileLoad<2, 8> t_ka, t_va;
  t_kb.init(p.kb.stride, rk, dk, tid);
  t_vb.init(p.vb.stride, rk, dv, tid);
  t_ka.init(p.ka.stride, rk, h, tid);
  t_va.init(p.va.stride, rk, h, tid);
  auto fetch = [&](int k0) {
    t_kb.fetch(kb, p.kb.stride, k0, k_end);
    t_vb.fetch(vb, p.vb.stride, k0, k_end);
    t_ka.fetch(ka, p.ka.stride, k0, k_end);
    t_va.fetch(va, p.va.stride, k0, k_end);
  };
  if (k_begin < k_end) fetch(k_begin);

  for (int k0 = k_begin; k0 < k_end; k0 += KT) {
    __syncthreads();  // the previous tile's readers are done (and the query factors are written)
    t_kb.store_raw(kb16, L.pk, dk, tid);
    t_vb.store_raw(vb16, L.pv, dv, tid);
    t_ka.store(kaS, h, h, tid);
    t_va.store(vaS, h, h, tid);
    if (has_seg && tid < KT) ksegS[tid] = (k0 + tid < k_end) ? kseg_g[k0 + tid] : 0;
    if (k0 + KT < k_end) fetch(k0 + KT);  // in flight while this tile is computed
    __syncthreads();

    // dots[jr][r] = qb[r, :] . kb[jr, :] for the rows jr = 8 warp ... 8 warp + 7
    {
      float d[4] = {0.f, 0.f, 0.f, 0.f};
      for (int ks = 0; ks < dk; ks += 16) {
        uint32_t a[4], b0, b1;
        a[0] = *reinterpret_cast<const uint32_t*>(qb16 + g * L.pk + ks + 2 * t4);
        a[1] = *reinterpret_cast<const uint32_t*>(qb16 + (g + 8) * L.pk + ks + 2 * t4);
        a[2] = *reinterpret_cast<const uint32_t*>(qb16 + g * L.pk + ks + 8 + 2 * t4);
        a[3] = *reinterpret_cast<const uint32_t*>(qb16 + (g + 8) * L.pk + ks + 8 + 2 * t4);
        ldmatrix_x2(b0, b1, kb16 + (warp * 8 + (lane & 7)) * L.pk + ks + ((lane >> 3) & 1) * 8);
        mma_bf16(d, a, b0, b1);
      }
      const int jr = warp * 8 + 2 * t4;  // d[0] = (rank g, row jr), d[1] = (g, jr + 1), d[2] / d[3]: rank g + 8
      if (g < rq) {
        dots[jr * rq + g] = d[0];
        dots[(jr + 1) * rq + g] = d[1];
      }
      if (g + 8 < rq) {
        dots[jr * rq + g + 8] = d[2];
        dots[(jr + 1) * rq + g + 8] = d[3];
      }
    }
    __syncthreads();

    // Logits, running softmax and w = p * va in one pass, the logits never leaving registers:
    // warp w takes keys w, w + 8, ... (at most 8), lanes over heads.
    //   s[hh][key] = sum_rk ka[jr][hh] * sum_r qa[r][hh] dots[jr][r]; masked entries -inf
    float sv[HI][8];
#pragma unroll
    for (int hi = 0; hi < HI; ++hi) {
      const int hh = min(lane + 32 * hi, h - 1);
#pragma unroll
      for (int i = 0; i < 8; ++i) sv[hi][i] = 0.f;
      for (int q = 0; q < rk; ++q) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = 0.f;
        for (int r = 0; r < rq; ++r) {
          const float a = qaS[r * h + hh];
#pragma unroll
          for (int i = 0; i < 8; ++i) e[i] = fmaf(a, dots[(min(warp + 8 * i, KT - 1) * rk + q) * rq + r], e[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sv[hi][i] = fmaf(kaS[(min(warp + 8 * i, KT - 1) * rk + q) * h + hh], e[i], sv[hi][i]);
      }
      float pmax = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int key = warp + 8 * i;
        bool keep = key < KT && k0 + key < k_end;
        if (has_seg && keep) keep = ksegS[key] == qseg;
        if (!keep) sv[hi][i] = -CUDART_INF_F;
        pmax = fmaxf(pmax, sv[hi][i]);
      }
      if (lane + 32 * hi < h) red[warp * h + hh] = pmax;  // this warp's maximum per head
    }
    __syncthreads();
#pragma unroll
    for (int hi = 0; hi < HI; ++hi) {
      const int hh = lane + 32 * hi;
      if (hh >= h) continue;
      float tmax = red[hh];
#pragma unroll
      for (int w = 1; w < DEC_THREADS / 32; ++w) tmax = fmaxf(tmax, red[w * h + hh]);
      const float m_old = mS[hh], m_new = fmaxf(m_old, tmax);
      const float corr = (m_new == -CUDART_INF_F) ? 1.f : ((m_old == -CUDART_INF_F) ? 0.f : expf(m_old - m_new));
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int key = warp + 8 * i;
        if (key < KT) {
          const float pr = (m_new == -CUDART_INF_F) ? 0.f : expf(sv[hi][i] - m_new);  // exp(-inf) = 0 for masked entries
          psum += pr;
          for (int q = 0; q < rk; ++q) {
            const int jr = key * rk + q;
            w16[hh * L.pw + jr] = __float2bfloat16_rn(pr * vaS[jr * h + hh]);
          }
        }
      }
      red[(DEC_THREADS / 32 + warp) * h + hh] = psum;  // this warp's share of the row sum
      if (warp == 0) {
        cS[hh] = corr;
        m_keep[hi] = m_new;
        c_keep[hi] = corr;
      }
    }
    __syncthreads();
    if (warp == 0) {  // nobody reads mS / lS before the next block-wide sync
#pragma unroll
      for (int hi = 0; hi < HI; ++hi) {
        const int hh = lane + 32 * hi;
        if (hh >= h) continue;
        float psum = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_THREADS / 32; ++w) psum += red[(DEC_THREADS / 32 + w) * h + hh];
        mS[hh] = m_keep[hi];
        lS[hh] = lS[hh] * c_keep[hi] + psum;
      }
    }

    // acc[heads][16 columns of this warp] = acc * corr + w (h x 64) vb (64 x dv)
    if (warp * 16 < dv) {
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const float c0 = (i * 16 + g < h) ? cS[i * 16 + g] : 1.f;
        const float c1 = (i * 16 + g + 8 < h) ? cS[i * 16 + g + 8] : 1.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          acc[i][n][0] *= c0; acc[i][n][1] *= c0;
          acc[i][n][2] *= c1; acc[i][n][3] *= c1;
        }
      }
#pragma unroll
      for (int ks = 0; ks < DEC_JR; ks += 16) {
        // vb rows ks ... ks + 15, columns 16 warp ... + 15: matrices (k 0-7 | 8-15) x (columns 0-7 | 8-15), transposed
        uint32_t bfrag[4];
        ldmatrix_x4_trans(bfrag, vb16 + (ks + ((lane >> 3) & 1) * 8 + (lane & 7)) * L.pv + warp * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          uint32_t a[4];
          const __nv_bfloat16* wr = w16 + (i * 16 + g) * L.pw + ks + 2 * t4;
          a[0] = *reinterpret_cast<const uint32_t*>(wr);
          a[1] = *reinterpret_cast<const uint32_t*>(wr + 8 * L.pw);
          a[2] = *reinterpret_cast<const uint32_t*>(wr + 8);
          a[3] = *reinterpret_cast<const uint32_t*>(wr + 8 * L.pw + 8);
          mma_bf16(acc[i][0], a, bfrag[0], bfrag[1]);
          mma_bf16(acc[i][1], a, bfrag[2], bfrag[3]);
        }
      }
    }
  }
  __syncthreads();

  // normalised partial of this split: 0 / -inf where nothing was visible
  const int64_t rows = (int64_t)p.batch * p.lq * h;
  const int64_t rh0 = ((int64_t)b * p.lq + qi) * h;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int hh = i * 16 + g + half * 8;
      if (hh >= h) continue;
      const float l = lS[hh];
      const bool empty = !(l > 0.f);
      const float inv = empty ? 0.f : 1.f / (l * (float)rk);
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int col = warp * 16 + n * 8 + 2 * t4;
        if (col < dv)
          *reinterpret_cast<float2*>(part_o + ((int64_t)split * rows + rh0 + hh) * dv + col) =
              make_float2(acc[i][n][half * 2] * inv, acc[i][n][half * 2 + 1] * inv);
      }
      if (warp == 0 && t4 == 0) part_lse[(int64_t)split * rows + rh0 + hh] = empty ? -CUDART_INF_F : mS[hh] + logf(l);
    }
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }
inline bool vec_ok(const TpaFactor& f) {
  return aligned16(f.ptr) && f.stride[0] % 8 == 0 && f.stride[1] % 8 == 0 && f.stride[2] % 8 == 0;
}
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t decode_smem_bytes(const Params& p) {
  return (size_t)DecodeSmem(p.heads, p.dk, p.dv, p.rank_q, (p.heads + 15) / 16).total;
}

}  // namespace

// A few query rows against many keys: bf16, vector-loadable factors, h <= 64 and d <= 128.
bool decode_supported(const Params& p) {
  if (p.dtype != TPA_DTYPE_BF16 || p.lq > 8 || p.lk < 256) return false;
  if (p.heads > 64 || p.heads % 8 != 0 || p.dk > 128 || p.dv > 128 || p.dk % 16 != 0 || p.dv % 16 != 0) return false;
  if (p.rank_q > 16 || p.rank_k > 8) return false;
  if (!vec_ok(p.ka) || !vec_ok(p.kb) || !vec_ok(p.va) || !vec_ok(p.vb)) return false;
  if (!(p.flags & TPA_FLAG_STATE_STORE) && !aligned16(p.o)) return false;
  if ((p.flags & (TPA_FLAG_STATE_STORE | TPA_FLAG_STATE_LOAD)) && !aligned16(p.state_o)) return false;
  return decode_smem_bytes(p) <= 200 * 1024;
}

// Measured (h = 32, d = 128, batch 16 x 32768 keys): one row, R_k = 2: 0.41 ms against 3.57 ms for the
// staged tensor-core path; R_k = 4: 0.97 against 3.75; four rows: 1.79 against 3.57 (the rows are
// walked one after the other here, the staged path shares its tiles among them).
bool decode_preferred(const Params& p) { return decode_supported(p) && p.lq <= 6; }

int decode_pick_splits(const Params& p) {
  const int KT = DEC_JR / p.rank_k;
  const int64_t ctas = (int64_t)p.lq * p.batch;
  int splits = (int)(2 * 148 / ctas);                          // two CTAs fit an SM: fill them once, no second wave
  const int max_splits = (p.lk + 4 * KT - 1) / (4 * KT);      // at least four tiles each
  if (splits > max_splits) splits = max_splits;
  if (splits > 2 * 148) splits = 2 * 148;
  return splits < 1 ? 1 : splits;
}

size_t decode_workspace_bytes(const Params& p) {
  return align256((size_t)decode_pick_splits(p) * p.batch * p.lq * p.heads * (p.dv + 1) * sizeof(float));
}

cudaError_t launch_decode(const Params& p, void* workspace, TpaKernelInfo* info, bool dry_run, cudaStream_t stream) {
  const int splits = decode_pick_splits(p);
  const int KT = DEC_JR / p.rank_k;
  int keys_per_split = (p.lk + splits - 1) / splits;
  keys_per_split = (keys_per_split + KT - 1) / KT * KT;  // whole tiles
  const size_t smem = decode_smem_bytes(p);
  dim3 grid(splits, p.lq, p.batch);
  if (info) {
    info->kernel = TPA_KERNEL_DECODE;
    info->block_q = 1;
    info->block_kv = KT;
    info->threads = DEC_THREADS;
    info->grid[0] = grid.x; info->grid[1] = grid.y; info->grid[2] = grid.z;
    info->smem_bytes = (int)smem;
    info->launches = 2;
  }
  if (dry_run) return cudaSuccess;
  float* part_o = static_cast<float*>(workspace);
  float* part_lse = part_o + (size_t)splits * p.batch * p.lq * p.heads * p.dv;
  auto launch = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kern<<<grid, DEC_THREADS, smem, stream>>>(p, part_o, part_lse, keys_per_split);
    return cudaGetLastError();
  };
  cudaError_t e;
  switch ((p.heads + 15) / 16) {
    case 1: e = launch(tpa_fwd_decode_kernel<1>); break;
    case 2: e = launch(tpa_fwd_decode_kernel<2>); break;
    case 3: e = launch(tpa_fwd_decode_kernel<3>); break;
    default: e = launch(tpa_fwd_decode_kernel<4>); break;
  }
  if (e != cudaSuccess) return e;
  count_launch(1);
  return launch_combine_splits(p, part_o, part_lse, splits, stream);
}

}  // namespace tpa
