// TPA forward for a handful of query rows against a long key/value factor cache (decode and
// cross shapes, tpa/tpa_test.py:67-70; bf16 factors).  K and V are never materialised:
//
//   logits  s[h, j] = c * sum_{rq, rk} qa[rq, h] ka[j, rk, h] (qb[rq, :] . kb[j, rk, :])
//           the rank-space form of the reference's `nomat` branch (tpa/tpa.py:333-359):
//           R_q R_k (d + h) multiply-adds per key instead of R_k h d
//   output  o[h, :] = (1 / R_k) sum_{j, rk} (p[h, j] va[j, rk, h]) vb[j, rk, :]
//
// so every factor byte is read from HBM exactly once per query row and nothing else is: the
// staged tensor-core path rebuilds and writes all heads' dense K/V tiles first (h d / (R_k (h+d))
// = 12.8x the factor bytes at h = 32, d = 128, R_k = 2), which is what a single decode row cannot
// amortise.  fp32 math on CUDA cores: measured 740-820 GB/s of factor stream (4.4x the staged
// path for one row), i.e. still bound by its own instruction stream and block-wide syncs, not by HBM.
//
// grid = (key splits, query rows, batch); 256 threads.  A CTA walks its share of the keys in tiles
// of 64 (key, rank) rows, keeps a running (max, sum) per head and the h x dv accumulator in
// registers (warp w owns value columns 16 w ...; lane l heads (h / 8)(l / 4) ... and 4 of those columns), and leaves
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

// NH = heads / 8: lane (hg = lane / 4, c = lane % 4) of warp w accumulates heads NH hg .. NH hg + NH - 1,
// value columns 16 w + 4 c .. + 3 (a warp reads 64 bytes of a vb row and 32 NH bytes of w per step).
template <int NH>
__global__ void __launch_bounds__(DEC_THREADS)
tpa_fwd_decode_kernel(const Params p, float* part_o, float* part_lse, const int keys_per_split) {
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  const int h = p.heads, dk = p.dk, dv = p.dv, rq = p.rank_q, rk = p.rank_k;
  const int KT = DEC_JR / rk;  // keys per tile
  const int ldk = dk + 2;      // row pitch = 2 (mod 32) floats: the 64-bit reads of 32 rows hit every bank once
  float* qbS = smem;                       // [rq][dk]
  float* qaS = qbS + rq * dk;              // [rq][h], times sm_scale / (R_q R_k)
  float* kbS = qaS + rq * h;               // [JR][dk + 2]
  float* vbS = kbS + DEC_JR * ldk;         // [JR][dv]
  float* kaS = vbS + DEC_JR * dv;          // [JR][h]
  float* vaS = kaS + DEC_JR * h;           // [JR][h]
  float* wS = vaS + DEC_JR * h;            // [JR][h] p * va
  float* dotsP = wS + DEC_JR * h;          // [4][JR][rq] partial dots over a quarter of dk
  float* dots = dotsP + 4 * DEC_JR * rq;   // [JR][rq]
  float* sS = dots + DEC_JR * rq;          // [h][JR + 1] logits, then p
  float* mS = sS + h * (DEC_JR + 1);       // [h] running maximum
  float* lS = mS + h;                      // [h] running sum
  float* cS = lS + h;                      // [h] correction of this tile
  int* ksegS = reinterpret_cast<int*>(cS + h);  // [KT]

  const int split = blockIdx.x, qi = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
  for (int idx = tid; idx < rq * dk; idx += DEC_THREADS)
    qbS[idx] = to_float(qb[(idx / dk) * p.qb.stride[2] + idx % dk]);
  for (int idx = tid; idx < rq * h; idx += DEC_THREADS)
    qaS[idx] = c * to_float(qa[(idx / h) * p.qa.stride[2] + idx % h]);
  for (int idx = tid; idx < h; idx += DEC_THREADS) {
    mS[idx] = -CUDART_INF_F;
    lS[idx] = 0.f;
  }
  const int hg = lane >> 2, col0 = warp * 16 + (lane & 3) * 4;
  float acc[NH][4];
#pragma unroll
  for (int i = 0; i < NH; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

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
    t_kb.store(kbS, ldk, dk, tid);
    t_vb.store(vbS, dv, dv, tid);
    t_ka.store(kaS, h, h, tid);
    t_va.store(vaS, h, h, tid);
    if (has_seg && tid < KT) ksegS[tid] = (k0 + tid < k_end) ? kseg_g[k0 + tid] : 0;
    if (k0 + KT < k_end) fetch(k0 + KT);  // in flight while this tile is computed
    __syncthreads();

    // partial dots over a quarter of dk: thread (jr = tid % 64, g = tid / 64), all ranks of q
    {
      const int jr = tid & (DEC_JR - 1), g = tid >> 6;
      const int t0 = g * (dk >> 2), t1 = t0 + (dk >> 2);  // dk % 8 == 0: whole float2 steps
      const float* kr = kbS + jr * ldk;
      for (int r0 = 0; r0 < rq; r0 += 4) {  // four ranks at a time: one k load feeds eight independent FMA chains
        float d[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) d[i][0] = d[i][1] = 0.f;
#pragma unroll 2
        for (int t = t0; t < t1; t += 2) {
          const float2 kv = *reinterpret_cast<const float2*>(kr + t);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 qv = *reinterpret_cast<const float2*>(qbS + min(r0 + i, rq - 1) * dk + t);
            d[i][0] = fmaf(kv.x, qv.x, d[i][0]);
            d[i][1] = fmaf(kv.y, qv.y, d[i][1]);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (r0 + i < rq) dotsP[(g * DEC_JR + jr) * rq + r0 + i] = d[i][0] + d[i][1];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < DEC_JR * rq; idx += DEC_THREADS)
      dots[idx] = (dotsP[idx] + dotsP[DEC_JR * rq + idx]) + (dotsP[2 * DEC_JR * rq + idx] + dotsP[3 * DEC_JR * rq + idx]);
    __syncthreads();

    // logits s[hh][key] = sum_rk ka[jr][hh] * sum_r qa[r][hh] dots[jr][r]; masked entries -inf
    // (warp w takes keys w, w + 8, ..., four of them in flight; lanes over heads)
    for (int kbase = warp; kbase < KT; kbase += 32) {
      for (int hh = lane; hh < h; hh += 32) {
        float sv[4] = {0.f, 0.f, 0.f, 0.f};
        for (int q = 0; q < rk; ++q) {
          float e[4] = {0.f, 0.f, 0.f, 0.f};
          for (int r = 0; r < rq; ++r) {
            const float a = qaS[r * h + hh];
#pragma unroll
            for (int i = 0; i < 4; ++i) e[i] = fmaf(a, dots[(min(kbase + 8 * i, KT - 1) * rk + q) * rq + r], e[i]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) sv[i] = fmaf(kaS[(min(kbase + 8 * i, KT - 1) * rk + q) * h + hh], e[i], sv[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = kbase + 8 * i;
          if (key < KT) {
            bool keep = k0 + key < k_end;
            if (has_seg && keep) keep = ksegS[key] == qseg;
            sS[hh * (DEC_JR + 1) + key] = keep ? sv[i] : -CUDART_INF_F;
          }
        }
      }
    }
    __syncthreads();

    // running softmax per head: warp w takes heads w, w + 8, ... (two at a time, so that their
    // shuffle chains overlap); lanes over the tile's keys
    for (int hh0 = warp; hh0 < h; hh0 += 2 * (DEC_THREADS / 32)) {
      float x0[2], x1[2], tmax[2], psum[2], p0[2], p1[2], corr[2], m_new[2];
      bool on[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int hh = hh0 + u * (DEC_THREADS / 32);
        on[u] = hh < h;
        const float* srow = sS + (on[u] ? hh : hh0) * (DEC_JR + 1);
        x0[u] = lane < KT ? srow[lane] : -CUDART_INF_F;
        x1[u] = lane + 32 < KT ? srow[lane + 32] : -CUDART_INF_F;
        tmax[u] = fmaxf(x0[u], x1[u]);
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1)
#pragma unroll
        for (int u = 0; u < 2; ++u) tmax[u] = fmaxf(tmax[u], __shfl_xor_sync(0xffffffffu, tmax[u], s));
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float m_old = mS[on[u] ? hh0 + u * (DEC_THREADS / 32) : hh0];
        m_new[u] = fmaxf(m_old, tmax[u]);
        p0[u] = p1[u] = 0.f;
        corr[u] = 1.f;
        if (m_new[u] != -CUDART_INF_F) {
          corr[u] = (m_old == -CUDART_INF_F) ? 0.f : expf(m_old - m_new[u]);
          p0[u] = expf(x0[u] - m_new[u]);  // exp(-inf) = 0 for masked entries
          p1[u] = expf(x1[u] - m_new[u]);
        }
        psum[u] = p0[u] + p1[u];
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1)
#pragma unroll
        for (int u = 0; u < 2; ++u) psum[u] += __shfl_xor_sync(0xffffffffu, psum[u], s);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!on[u]) continue;
        const int hh = hh0 + u * (DEC_THREADS / 32);
        float* srow = sS + hh * (DEC_JR + 1);
        if (lane < KT) srow[lane] = p0[u];
        if (lane + 32 < KT) srow[lane + 32] = p1[u];
        if (lane == 0) {
          mS[hh] = m_new[u];
          lS[hh] = lS[hh] * corr[u] + psum[u];
          cS[hh] = corr[u];
        }
      }
    }
    __syncthreads();

    // w[jr][hh] = p[hh][key] * va[jr][hh]
    for (int key = warp; key < KT; key += DEC_THREADS / 32)
      for (int q = 0; q < rk; ++q) {
        const int jr = key * rk + q;
        for (int hh = lane; hh < h; hh += 32) wS[jr * h + hh] = sS[hh * (DEC_JR + 1) + key] * vaS[jr * h + hh];
      }
    __syncthreads();

    // acc[heads of hg][4 columns] = acc * corr + sum_jr w[jr][head] vb[jr][columns]
    if (col0 < dv) {
#pragma unroll
      for (int i = 0; i < NH; ++i) {
        const float corr = cS[hg * NH + i];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] *= corr;
      }
      const int n_jr = KT * rk;
      const float* wp = wS + hg * NH;
      const float* vp = vbS + col0;
#pragma unroll 4
      for (int jr = 0; jr < n_jr; ++jr) {
        const float4 v = *reinterpret_cast<const float4*>(vp + jr * dv);
        float w[NH];
        if constexpr (NH % 4 == 0) {
#pragma unroll
          for (int i = 0; i < NH; i += 4) {
            const float4 w4 = *reinterpret_cast<const float4*>(wp + jr * h + i);
            w[i] = w4.x; w[i + 1] = w4.y; w[i + 2] = w4.z; w[i + 3] = w4.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < NH; ++i) w[i] = wp[jr * h + i];
        }
#pragma unroll
        for (int i = 0; i < NH; ++i) {
          acc[i][0] = fmaf(w[i], v.x, acc[i][0]);
          acc[i][1] = fmaf(w[i], v.y, acc[i][1]);
          acc[i][2] = fmaf(w[i], v.z, acc[i][2]);
          acc[i][3] = fmaf(w[i], v.w, acc[i][3]);
        }
      }
    }
  }
  __syncthreads();

  // normalised partial of this split: 0 / -inf where nothing was visible
  const int64_t rows = (int64_t)p.batch * p.lq * h;
  const int64_t rh0 = ((int64_t)b * p.lq + qi) * h;
#pragma unroll
  for (int i = 0; i < NH; ++i) {
    const int hh = hg * NH + i;
    const float l = lS[hh];
    const bool empty = !(l > 0.f);
    const float inv = empty ? 0.f : 1.f / (l * (float)rk);
    if (col0 < dv)
      *reinterpret_cast<float4*>(part_o + ((int64_t)split * rows + rh0 + hh) * dv + col0) =
          make_float4(acc[i][0] * inv, acc[i][1] * inv, acc[i][2] * inv, acc[i][3] * inv);
    if (warp == 0 && (lane & 3) == 0) part_lse[(int64_t)split * rows + rh0 + hh] = empty ? -CUDART_INF_F : mS[hh] + logf(l);
  }
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }
inline bool vec_ok(const TpaFactor& f) {
  return aligned16(f.ptr) && f.stride[0] % 8 == 0 && f.stride[1] % 8 == 0 && f.stride[2] % 8 == 0;
}
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t decode_smem_bytes(const Params& p) {
  const size_t floats = (size_t)p.rank_q * (p.dk + p.heads) + (size_t)DEC_JR * (p.dk + 2 + p.dv + 3 * p.heads + 5 * p.rank_q) +
                        (size_t)p.heads * (DEC_JR + 1 + 3) + DEC_JR;
  return floats * sizeof(float);
}

}  // namespace

// A few query rows against many keys: bf16, vector-loadable factors, h <= 64 and d <= 128.
bool decode_supported(const Params& p) {
  if (p.dtype != TPA_DTYPE_BF16 || p.lq > 8 || p.lk < 256) return false;
  if (p.heads > 64 || p.heads % 8 != 0 || p.dk > 128 || p.dv > 128 || p.dk % 8 != 0 || p.dv % 8 != 0) return false;
  if (p.rank_q > 16 || p.rank_k > 8) return false;
  if (!vec_ok(p.ka) || !vec_ok(p.kb) || !vec_ok(p.va) || !vec_ok(p.vb)) return false;
  if (!(p.flags & TPA_FLAG_STATE_STORE) && !aligned16(p.o)) return false;
  if ((p.flags & (TPA_FLAG_STATE_STORE | TPA_FLAG_STATE_LOAD)) && !aligned16(p.state_o)) return false;
  return decode_smem_bytes(p) <= 200 * 1024;
}

// Measured (h = 32, d = 128, batch 16 x 32768 keys): one row, R_k = 2: 0.82 ms against 3.57 ms for the
// staged tensor-core path; R_k = 4: 1.69 against 3.75; four rows: 3.44 against 3.57 (the rows are
// walked one after the other here, the staged path shares its tiles among them).
bool decode_preferred(const Params& p) { return decode_supported(p) && p.lq <= 2; }

int decode_pick_splits(const Params& p) {
  const int KT = DEC_JR / p.rank_k;
  const int64_t ctas = (int64_t)p.lq * p.batch;
  int splits = (int)(2 * 148 / ctas);                          // two CTAs fit an SM: fill them once, no second wave
  const int max_splits = (p.lk + 4 * KT - 1) / (4 * KT);      // at least four tiles each
  if (splits > max_splits) splits = max_splits;
  if (splits > 64) splits = 64;
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
  switch (p.heads / 8) {
    case 1: e = launch(tpa_fwd_decode_kernel<1>); break;
    case 2: e = launch(tpa_fwd_decode_kernel<2>); break;
    case 3: e = launch(tpa_fwd_decode_kernel<3>); break;
    case 4: e = launch(tpa_fwd_decode_kernel<4>); break;
    case 5: e = launch(tpa_fwd_decode_kernel<5>); break;
    case 6: e = launch(tpa_fwd_decode_kernel<6>); break;
    case 7: e = launch(tpa_fwd_decode_kernel<7>); break;
    default: e = launch(tpa_fwd_decode_kernel<8>); break;
  }
  if (e != cudaSuccess) return e;
  count_launch(1);
  return launch_combine_splits(p, part_o, part_lse, splits, stream);
}

}  // namespace tpa
