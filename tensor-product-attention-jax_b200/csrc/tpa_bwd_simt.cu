// Generic fp32-math TPA backward (any lengths, heads, dk, dv <= 256, any ranks; fp32 or bf16 I/O).
//
// Replaces _precompute_delta (tpa/tpa.py:965-995) and _bwd_kernel (tpa/tpa.py:546-820):
//
//   delta[i,h] = nansum_t o[i,h,t] do[i,h,t]                       tpa/tpa.py:976-980
//   p  = exp(sm_scale q k^T - lse), masked / NaN entries 0         tpa/tpa.py:662-677
//   dv = p^T do,  dp = do v^T - delta,  ds = p dp sm_scale         tpa/tpa.py:778-786
//   dk = ds^T q,  dq = ds k                                        tpa/tpa.py:789,796
//   da = dX b / R,  db = dX a / R  (per operand X = Q, K, V)       tpa/tpa.py:779-781,790-791,797-799
//
// The reference lets one program own a key/value block and adds its dq contribution with
// atomics (tpa/tpa.py:806-807).  Here the pair computation runs twice instead, once with a
// CTA per 32 keys (accumulating dk, dv over the query tiles) and once with a CTA per 32
// query rows (accumulating dq over the key tiles): no atomics, no zero-fill, and the result
// is bitwise reproducible.  Dense dQ/dK/dV land in fp32 scratch; the factor contraction is a
// separate kernel that sums over ALL heads (the reference's dim-factor blocks ignore the
// head-block index, tpa/tpa.py:929,933, which is only right for num_heads <= block_h).
#include <math_constants.h>

#include "tpa_common.cuh"

namespace tpa {

constexpr int BW_TILE = 32;      // query rows and keys per tile
constexpr int BW_THREADS = 256;  // 8 warps: warp w owns rows (or keys) 4w .. 4w+3
constexpr int BW_RPW = 4;
constexpr int BW_LDP = BW_TILE + 1;

// ------------------------------------------------------------------ delta

template <typename T>
__global__ void __launch_bounds__(256) tpa_bwd_delta_kernel(const T* __restrict__ o,
                                                            const T* __restrict__ d_o,
                                                            float* __restrict__ delta,
                                                            int64_t rows, int dv) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float acc = 0.f;
  for (int t = lane; t < dv; t += 32) {
    const float x = to_float(o[row * dv + t]) * to_float(d_o[row * dv + t]);
    if (x == x) acc += x;  // nansum: rows without a visible key hold NaN
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[row] = acc;
}

// ------------------------------------------------------------------ tile loaders

// dst[r][t] = inv_rank * sum_rho a[row0+r, rho, h] * b[row0+r, rho, t]; zero past row_end / cols.
template <typename T>
__device__ __forceinline__ void bw_rebuild(float* dst, int ld, int row0, int row_end, int cols,
                                           const T* a, const int64_t* as, const T* bfac,
                                           const int64_t* bs, int rank, int h, float inv_rank,
                                           int tid) {
  for (int idx = tid; idx < BW_TILE * ld; idx += BW_THREADS) {
    const int r = idx / ld, t = idx - r * ld;
    const int row = row0 + r;
    float acc = 0.f;
    if (row < row_end && t < cols) {
      const T* ap = a + (int64_t)row * as[1] + h;
      const T* bp = bfac + (int64_t)row * bs[1] + t;
      for (int rho = 0; rho < rank; ++rho)
        acc = fmaf(to_float(ap[rho * as[2]]), to_float(bp[rho * bs[2]]), acc);
    }
    dst[idx] = acc * inv_rank;
  }
}

// dst[r][t] = x[b, row0+r, h, t] of a contiguous [batch, rows, heads, cols] array.
template <typename T>
__device__ __forceinline__ void bw_load_rows(float* dst, int ld, int row0, int row_end, int cols,
                                             const T* x, int64_t batch_off, int heads, int h,
                                             int tid) {
  for (int idx = tid; idx < BW_TILE * ld; idx += BW_THREADS) {
    const int r = idx / ld, t = idx - r * ld;
    const int row = row0 + r;
    float val = 0.f;
    if (row < row_end && t < cols) val = to_float(x[((batch_off + row) * heads + h) * cols + t]);
    dst[idx] = val;
  }
}

// ------------------------------------------------------------------ pair kernel

// KV_OWNER: the CTA owns 32 keys of one head and walks the query tiles (dk, dv).
// otherwise: the CTA owns 32 query rows of one head and walks the key tiles (dq).
template <typename T, int JJ, bool KV_OWNER>
__global__ void __launch_bounds__(BW_THREADS) tpa_bwd_pairs_kernel(const BwdParams bp) {
  const Params& p = bp.f;
  extern __shared__ float smem[];
  constexpr int LD = JJ * 32 + 1;  // +1: rows land in different banks; pad columns are zero
  float* Qs = smem;
  float* Ks = Qs + BW_TILE * LD;
  float* Vs = Ks + BW_TILE * LD;
  float* dOs = Vs + BW_TILE * LD;
  float* Ps = dOs + BW_TILE * LD;    // [32 rows][33]
  float* dSs = Ps + BW_TILE * BW_LDP;
  float* lse_s = dSs + BW_TILE * BW_LDP;
  float* delta_s = lse_s + BW_TILE;
  int* qseg_s = reinterpret_cast<int*>(delta_s + BW_TILE);
  int* kseg_s = qseg_s + BW_TILE;

  const int own0 = blockIdx.x * BW_TILE, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = (p.flags & TPA_FLAG_CAUSAL) != 0;
  const bool has_seg = p.q_seg != nullptr;
  const int dk = p.dk, dv = p.dv;

  const T* qa = static_cast<const T*>(p.qa.ptr) + (int64_t)b * p.qa.stride[0];
  const T* qb = static_cast<const T*>(p.qb.ptr) + (int64_t)b * p.qb.stride[0];
  const T* ka = static_cast<const T*>(p.ka.ptr) + (int64_t)b * p.ka.stride[0];
  const T* kb = static_cast<const T*>(p.kb.ptr) + (int64_t)b * p.kb.stride[0];
  const T* va = static_cast<const T*>(p.va.ptr) + (int64_t)b * p.va.stride[0];
  const T* vb = static_cast<const T*>(p.vb.ptr) + (int64_t)b * p.vb.stride[0];
  const T* d_o = static_cast<const T*>(bp.d_o);
  const int32_t* qseg_g = has_seg ? p.q_seg + (int64_t)b * p.q_seg_bstride : nullptr;
  const int32_t* kseg_g = has_seg ? p.kv_seg + (int64_t)b * p.kv_seg_bstride : nullptr;
  const float inv_rq = 1.f / (float)p.rank_q, inv_rk = 1.f / (float)p.rank_k;

  auto load_q_side = [&](int q0) {
    bw_rebuild<T>(Qs, LD, q0, p.lq, dk, qa, p.qa.stride, qb, p.qb.stride, p.rank_q, h, inv_rq, tid);
    bw_load_rows<T>(dOs, LD, q0, p.lq, dv, d_o, (int64_t)b * p.lq, p.heads, h, tid);
    if (tid < BW_TILE) {
      const int row = q0 + tid;
      const bool live = row < p.lq;
      const int64_t rh = ((int64_t)b * p.lq + row) * p.heads + h;
      lse_s[tid] = live ? p.lse[rh] : -CUDART_INF_F;
      delta_s[tid] = live ? bp.delta[rh] : 0.f;
      qseg_s[tid] = (has_seg && live) ? qseg_g[row] : 0;
    }
  };
  auto load_k_side = [&](int k0) {
    bw_rebuild<T>(Ks, LD, k0, p.lk, dk, ka, p.ka.stride, kb, p.kb.stride, p.rank_k, h, inv_rk, tid);
    bw_rebuild<T>(Vs, LD, k0, p.lk, dv, va, p.va.stride, vb, p.vb.stride, p.rank_k, h, inv_rk, tid);
    if (tid < BW_TILE) kseg_s[tid] = (has_seg && k0 + tid < p.lk) ? kseg_g[k0 + tid] : 0;
  };

  // tiles of the other side that can hold a visible pair (tpa/tpa.py:427-428 for the forward)
  int n_lo = 0, n_hi;
  if (KV_OWNER) {
    n_hi = (p.lq + BW_TILE - 1) / BW_TILE;
    if (causal) {
      const int64_t first = (int64_t)own0 + p.k_offset - p.q_offset;  // first row that sees key own0
      if (first > 0) n_lo = (int)min((int64_t)n_hi, first / BW_TILE);
    }
    load_k_side(own0);
  } else {
    n_hi = (p.lk + BW_TILE - 1) / BW_TILE;
    if (causal) {
      const int64_t kmax = (int64_t)own0 + BW_TILE - 1 + p.q_offset - p.k_offset;  // last visible key
      if (kmax < 0) n_hi = 0;
      else if (kmax / BW_TILE + 1 < n_hi) n_hi = (int)(kmax / BW_TILE) + 1;
    }
    load_q_side(own0);
  }

  float acc0[BW_RPW][JJ], acc1[BW_RPW][JJ];  // KV_OWNER: dk, dv rows; else dq rows (acc1 unused)
#pragma unroll
  for (int i = 0; i < BW_RPW; ++i)
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) acc0[i][jj] = acc1[i][jj] = 0.f;

  for (int n = n_lo; n < n_hi; ++n) {
    const int q0 = KV_OWNER ? n * BW_TILE : own0;
    const int k0 = KV_OWNER ? own0 : n * BW_TILE;
    __syncthreads();  // the previous tile's readers are done
    if (KV_OWNER) load_q_side(q0);
    else load_k_side(k0);
    __syncthreads();

    // s = q k^T and dp = do v^T for rows 4*warp .. +3, key column `lane`
    float s[BW_RPW], dp[BW_RPW];
#pragma unroll
    for (int i = 0; i < BW_RPW; ++i) s[i] = dp[i] = 0.f;
    const float* krow = Ks + lane * LD;
    const float* vrow = Vs + lane * LD;
    const float* qrow = Qs + warp * BW_RPW * LD;
    const float* drow = dOs + warp * BW_RPW * LD;
    for (int t = 0; t < dk; ++t) {
      const float kv = krow[t];
#pragma unroll
      for (int i = 0; i < BW_RPW; ++i) s[i] = fmaf(qrow[i * LD + t], kv, s[i]);
    }
    for (int t = 0; t < dv; ++t) {
      const float vv = vrow[t];
#pragma unroll
      for (int i = 0; i < BW_RPW; ++i) dp[i] = fmaf(drow[i * LD + t], vv, dp[i]);
    }
    const int kc = k0 + lane;
#pragma unroll
    for (int i = 0; i < BW_RPW; ++i) {
      const int r = warp * BW_RPW + i;
      const int row = q0 + r;
      const float lse = lse_s[r];
      bool keep = kc < p.lk && row < p.lq && lse != -CUDART_INF_F;
      if (causal) keep = keep && ((int64_t)row + p.q_offset >= (int64_t)kc + p.k_offset);
      if (has_seg) keep = keep && (qseg_s[r] == kseg_s[lane]);
      const float pr = keep ? expf(s[i] * p.sm_scale - lse) : 0.f;
      Ps[r * BW_LDP + lane] = pr;
      dSs[r * BW_LDP + lane] = pr * (dp[i] - delta_s[r]) * p.sm_scale;
    }
    __syncthreads();

    if (KV_OWNER) {
      // keys 4*warp .. +3, columns lane + 32 jj: dv += p^T do, dk += ds^T q
      for (int i = 0; i < BW_TILE; ++i) {
        float pv[BW_RPW], dsv[BW_RPW];
#pragma unroll
        for (int kk = 0; kk < BW_RPW; ++kk) {
          pv[kk] = Ps[i * BW_LDP + warp * BW_RPW + kk];
          dsv[kk] = dSs[i * BW_LDP + warp * BW_RPW + kk];
        }
#pragma unroll
        for (int jj = 0; jj < JJ; ++jj) {
          const float qv = Qs[i * LD + lane + 32 * jj];
          const float dov = dOs[i * LD + lane + 32 * jj];
#pragma unroll
          for (int kk = 0; kk < BW_RPW; ++kk) {
            acc0[kk][jj] = fmaf(dsv[kk], qv, acc0[kk][jj]);
            acc1[kk][jj] = fmaf(pv[kk], dov, acc1[kk][jj]);
          }
        }
      }
    } else {
      // rows 4*warp .. +3, columns lane + 32 jj: dq += ds k
      for (int c = 0; c < BW_TILE; ++c) {
        float dsv[BW_RPW];
#pragma unroll
        for (int ii = 0; ii < BW_RPW; ++ii) dsv[ii] = dSs[(warp * BW_RPW + ii) * BW_LDP + c];
#pragma unroll
        for (int jj = 0; jj < JJ; ++jj) {
          const float kv = Ks[c * LD + lane + 32 * jj];
#pragma unroll
          for (int ii = 0; ii < BW_RPW; ++ii) acc0[ii][jj] = fmaf(dsv[ii], kv, acc0[ii][jj]);
        }
      }
    }
  }

  const int len = KV_OWNER ? p.lk : p.lq;
#pragma unroll
  for (int i = 0; i < BW_RPW; ++i) {
    const int row = own0 + warp * BW_RPW + i;
    if (row >= len) continue;
    const int64_t rh = ((int64_t)b * len + row) * p.heads + h;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) {
      const int j = lane + 32 * jj;
      if (KV_OWNER) {
        if (j < dk) bp.dk_dense[rh * dk + j] = acc0[i][jj];
        if (j < dv) bp.dv_dense[rh * dv + j] = acc1[i][jj];
      } else {
        if (j < dk) bp.dq_dense[rh * dk + j] = acc0[i][jj];
      }
    }
  }
}

// ------------------------------------------------------------------ factor contraction

// One CTA per (row, batch): da[r,h] = sum_t dX[h,t] b[r,t] / R, db[r,t] = sum_h dX[h,t] a[r,h] / R,
// written (or added) to the concatenated gradient row out[b, row, r, 0:heads | heads:heads+d].
template <typename T, typename G>
__global__ void __launch_bounds__(256) tpa_bwd_contract_kernel(const float* __restrict__ dense,
                                                               TpaFactor a, TpaFactor bf,
                                                               G* __restrict__ out, int rows,
                                                               int rank, int heads, int d,
                                                               int accumulate) {
  extern __shared__ float smem[];
  const int ldx = d + 1;
  float* X = smem;              // [heads][d+1]
  float* A = X + heads * ldx;   // [rank][heads]
  float* B = A + rank * heads;  // [rank][d]
  const int row = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const float* src = dense + ((int64_t)b * rows + row) * heads * d;
  for (int idx = tid; idx < heads * d; idx += blockDim.x) X[(idx / d) * ldx + idx % d] = src[idx];
  const T* ap = static_cast<const T*>(a.ptr) + (int64_t)b * a.stride[0] + (int64_t)row * a.stride[1];
  const T* bp = static_cast<const T*>(bf.ptr) + (int64_t)b * bf.stride[0] + (int64_t)row * bf.stride[1];
  for (int idx = tid; idx < rank * heads; idx += blockDim.x)
    A[idx] = to_float(ap[(idx / heads) * a.stride[2] + idx % heads]);
  for (int idx = tid; idx < rank * d; idx += blockDim.x)
    B[idx] = to_float(bp[(idx / d) * bf.stride[2] + idx % d]);
  __syncthreads();
  const float inv_rank = 1.f / (float)rank;
  G* orow = out + ((int64_t)b * rows + row) * rank * (heads + d);
  for (int idx = tid; idx < rank * heads; idx += blockDim.x) {
    const int r = idx / heads, hh = idx % heads;
    float acc = 0.f;
    for (int t = 0; t < d; ++t) acc = fmaf(X[hh * ldx + t], B[r * d + t], acc);
    G& dst = orow[r * (heads + d) + hh];
    from_float(dst, acc * inv_rank + (accumulate ? to_float(dst) : 0.f));
  }
  for (int idx = tid; idx < rank * d; idx += blockDim.x) {
    const int r = idx / d, t = idx % d;
    float acc = 0.f;
    for (int hh = 0; hh < heads; ++hh) acc = fmaf(X[hh * ldx + t], A[r * heads + hh], acc);
    G& dst = orow[r * (heads + d) + heads + t];
    from_float(dst, acc * inv_rank + (accumulate ? to_float(dst) : 0.f));
  }
}

template <typename T, typename G>
static cudaError_t contract_one(const float* dense, const TpaFactor& a, const TpaFactor& bf, void* out,
                                int batch, int rows, int rank, int heads, int d, bool accumulate,
                                cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)heads * (d + 1) + (size_t)rank * (heads + d));
  auto kern = tpa_bwd_contract_kernel<T, G>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<dim3(rows, batch), 256, smem, stream>>>(dense, a, bf, static_cast<G*>(out), rows, rank,
                                                  heads, d, accumulate ? 1 : 0);
  count_launch(1);
  return cudaGetLastError();
}

cudaError_t launch_bwd_contract(const BwdParams& bp, cudaStream_t stream) {
  const Params& p = bp.f;
  struct Job { const float* dense; const TpaFactor *a, *b; void* out; int rows, rank, d; bool acc; };
  const Job jobs[3] = {
      {bp.dq_dense, &p.qa, &p.qb, bp.dq, p.lq, p.rank_q, p.dk, bp.accumulate_dq},
      {bp.dk_dense, &p.ka, &p.kb, bp.dk, p.lk, p.rank_k, p.dk, bp.accumulate_dkv},
      {bp.dv_dense, &p.va, &p.vb, bp.dv, p.lk, p.rank_k, p.dv, bp.accumulate_dkv}};
  for (const Job& j : jobs) {
    cudaError_t e;
    const bool f32 = p.dtype == TPA_DTYPE_F32, g32 = bp.grad_dtype == TPA_DTYPE_F32;
    if (f32 && g32)
      e = contract_one<float, float>(j.dense, *j.a, *j.b, j.out, p.batch, j.rows, j.rank, p.heads, j.d, j.acc, stream);
    else if (!f32 && g32)
      e = contract_one<__nv_bfloat16, float>(j.dense, *j.a, *j.b, j.out, p.batch, j.rows, j.rank, p.heads, j.d, j.acc, stream);
    else if (!f32 && !g32)
      e = contract_one<__nv_bfloat16, __nv_bfloat16>(j.dense, *j.a, *j.b, j.out, p.batch, j.rows, j.rank, p.heads, j.d, j.acc, stream);
    else
      return cudaErrorInvalidValue;  // fp32 factors with bf16 gradients: rejected by the validator
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// ------------------------------------------------------------------ launchers

template <typename T>
static cudaError_t delta_t(const BwdParams& bp, cudaStream_t stream) {
  const Params& p = bp.f;
  const int64_t rows = (int64_t)p.batch * p.lq * p.heads;
  const int64_t blocks = (rows + 7) / 8;
  tpa_bwd_delta_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(
      static_cast<const T*>(p.o), static_cast<const T*>(bp.d_o), bp.delta, rows, p.dv);
  count_launch(1);
  return cudaGetLastError();
}

cudaError_t launch_bwd_delta(const BwdParams& bp, cudaStream_t stream) {
  return bp.f.dtype == TPA_DTYPE_F32 ? delta_t<float>(bp, stream) : delta_t<__nv_bfloat16>(bp, stream);
}

template <typename T, int JJ>
static cudaError_t pairs_one(const BwdParams& bp, cudaStream_t stream) {
  const Params& p = bp.f;
  constexpr int LD = JJ * 32 + 1;
  const size_t smem = sizeof(float) * ((size_t)4 * BW_TILE * LD + 2 * BW_TILE * BW_LDP + 4 * BW_TILE);
  auto kv = tpa_bwd_pairs_kernel<T, JJ, true>;
  auto qq = tpa_bwd_pairs_kernel<T, JJ, false>;
  cudaError_t e = cudaFuncSetAttribute(kv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(qq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kv<<<dim3((p.lk + BW_TILE - 1) / BW_TILE, p.heads, p.batch), BW_THREADS, smem, stream>>>(bp);
  count_launch(1);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  qq<<<dim3((p.lq + BW_TILE - 1) / BW_TILE, p.heads, p.batch), BW_THREADS, smem, stream>>>(bp);
  count_launch(1);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t pairs_t(const BwdParams& bp, cudaStream_t s) {
  const int d = bp.f.dk > bp.f.dv ? bp.f.dk : bp.f.dv;
  if (d <= 32) return pairs_one<T, 1>(bp, s);
  if (d <= 64) return pairs_one<T, 2>(bp, s);
  if (d <= 128) return pairs_one<T, 4>(bp, s);
  return pairs_one<T, 8>(bp, s);
}

// dense dQ / dK / dV of the whole batch into bp.{dq,dk,dv}_dense (two launches)
cudaError_t launch_bwd_pairs_simt(const BwdParams& bp, cudaStream_t stream) {
  return bp.f.dtype == TPA_DTYPE_F32 ? pairs_t<float>(bp, stream) : pairs_t<__nv_bfloat16>(bp, stream);
}

}  // namespace tpa
