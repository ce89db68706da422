// Generic fp32-math TPA forward (any lq, lk, heads, dk, dv <= 256, any ranks; fp32 or bf16 I/O).
//
// Replaces _fwd_kernel (tpa/tpa.py:245-443) for shapes / precisions the tensor-core kernel
// does not take: one CTA owns 32 query rows of one head of one batch element, walks the
// key/value rows 64 at a time, rebuilds the K and V tiles of its head from the rank factors
// (tpa/tpa.py:364,417), and keeps a running (max, sum, accumulator) per query row.  The
// reference keeps `o` normalised and carries the LSE (tpa/tpa.py:389-424); running
// max / sum is the same function evaluated with one division at the end.
//
// Each warp owns 4 whole query rows, so row reductions are warp shuffles and no two warps
// ever touch the same row: results are bitwise reproducible run to run.
#include <math_constants.h>

#include "tpa_common.cuh"

namespace tpa {

constexpr int SIMT_BQ = 32;
constexpr int SIMT_BK = 64;
constexpr int SIMT_THREADS = 256;
constexpr int SIMT_RPW = 4;  // rows per warp

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ void rebuild_tile(float* dst, int ld, int rows, int row0, int row_end,
                                             int cols, const T* a, const int64_t* as,
                                             const T* bfac, const int64_t* bs, int rank, int h,
                                             float inv_rank, int tid) {
  // dst[r][t] = inv_rank * sum_rho a[row0+r, rho, h] * b[row0+r, rho, t]; zero past row_end/cols.
  // A thread keeps one column (mod 64) and takes four rows at a time: their 2 * rank factor loads
  // are independent and in flight together (one element after the other, each waiting for its
  // own loads, this rebuild was most of the kernel's time at short sequence lengths).  The sum
  // over rho runs in the same order for every element, whatever the grouping.
  constexpr int CW = 64, RS = SIMT_THREADS / CW, U = 4;
  const int tc = tid & (CW - 1), tr = tid / CW;
  for (int t = tc; t < ld; t += CW) {
    const bool col_ok = t < cols;
    for (int r = tr; r < rows; r += RS * U) {
      float acc[U];
      const T* ap[U];
      const T* bp[U];
      bool ok[U];
#pragma unroll
      for (int i = 0; i < U; ++i) {
        const int ri = r + i * RS, row = row0 + ri;
        ok[i] = col_ok && ri < rows && row < row_end;
        const int64_t safe = ok[i] ? row : row0;  // a valid row: the pointers are only read when ok
        ap[i] = a + safe * as[1] + h;
        bp[i] = bfac + safe * bs[1] + (col_ok ? t : 0);
        acc[i] = 0.f;
      }
      for (int rho = 0; rho < rank; ++rho) {
#pragma unroll
        for (int i = 0; i < U; ++i)
          if (ok[i]) acc[i] = fmaf(to_float(ap[i][rho * as[2]]), to_float(bp[i][rho * bs[2]]), acc[i]);
      }
#pragma unroll
      for (int i = 0; i < U; ++i)
        if (r + i * RS < rows) dst[(r + i * RS) * ld + t] = acc[i] * inv_rank;
    }
  }
}

// Rotary embedding of a rebuilt tile in shared memory: columns (2c, 2c + 1) of row r turn by the
// angle in table row pos0 + r.  Rows at or past row_end hold zeros and stay zero.
__device__ __forceinline__ void rope_tile(float* dst, int ld, int rows, int cols, const float* cosr,
                                          const float* sinr, int64_t pos0, int tid) {
  const int half = cols / 2;
  for (int idx = tid; idx < rows * half; idx += SIMT_THREADS) {
    const int r = idx / half, c = idx - r * half;
    const float cs = cosr[(pos0 + r) * half + c], sn = sinr[(pos0 + r) * half + c];
    const float x = dst[r * ld + 2 * c], y = dst[r * ld + 2 * c + 1];
    dst[r * ld + 2 * c] = x * cs - y * sn;
    dst[r * ld + 2 * c + 1] = x * sn + y * cs;
  }
}

template <typename T, int JJ>
__global__ void __launch_bounds__(SIMT_THREADS)
tpa_fwd_simt_kernel(const Params p, const int splits) {
  extern __shared__ float smem[];
  const int dk = p.dk, dv = p.dv;
  const int ldk = dk + 1;       // +1: rows of K land in different banks
  constexpr int ldv = JJ * 32;  // V rows padded to the lane grid, pad is zero
  float* Qs = smem;                     // [BQ][ldk]
  float* Ks = Qs + SIMT_BQ * ldk;       // [BK][ldk]
  float* Vs = Ks + SIMT_BK * ldk;       // [BK][ldv]
  float* Ps = Vs + SIMT_BK * ldv;       // [BQ][BK]
  int* ksegs = reinterpret_cast<int*>(Ps + SIMT_BQ * SIMT_BK);  // [BK]

  // grid.z = batch * splits: with key splits (few row blocks against many keys) this CTA walks only
  // its share of the visible tiles and leaves a partial (o, lse) in its slice of the scratch, which
  // tpa_combine_splits_kernel merges as a ring merges steps; the host has then set STATE_STORE
  const int q0 = blockIdx.x * SIMT_BQ, h = blockIdx.y, b = blockIdx.z / splits, split = blockIdx.z % splits;
  const int64_t split_rows = (int64_t)split * p.batch * p.lq * p.heads;
  float* const st_o = p.state_o + split_rows * p.dv;
  float* const st_lse = p.state_lse + split_rows;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = (p.flags & TPA_FLAG_CAUSAL) != 0;
  const bool has_seg = p.q_seg != nullptr;
  const bool load_state = (p.flags & TPA_FLAG_STATE_LOAD) != 0;
  const bool store_state = (p.flags & TPA_FLAG_STATE_STORE) != 0;

  const T* qa = static_cast<const T*>(p.qa.ptr) + (int64_t)b * p.qa.stride[0];
  const T* qb = static_cast<const T*>(p.qb.ptr) + (int64_t)b * p.qb.stride[0];
  const T* ka = static_cast<const T*>(p.ka.ptr) + (int64_t)b * p.ka.stride[0];
  const T* kb = static_cast<const T*>(p.kb.ptr) + (int64_t)b * p.kb.stride[0];
  const T* va = static_cast<const T*>(p.va.ptr) + (int64_t)b * p.va.stride[0];
  const T* vb = static_cast<const T*>(p.vb.ptr) + (int64_t)b * p.vb.stride[0];
  const int32_t* qseg_g = has_seg ? p.q_seg + (int64_t)b * p.q_seg_bstride : nullptr;
  const int32_t* kseg_g = has_seg ? p.kv_seg + (int64_t)b * p.kv_seg_bstride : nullptr;

  rebuild_tile<T>(Qs, ldk, SIMT_BQ, q0, p.lq, dk, qa, p.qa.stride, qb, p.qb.stride, p.rank_q, h,
                  1.f / (float)p.rank_q, tid);
  const bool rope = p.rope_cos != nullptr;
  if (rope) {
    __syncthreads();
    rope_tile(Qs, ldk, min(SIMT_BQ, p.lq - q0), dk, p.rope_cos, p.rope_sin, q0 + p.rope_q_offset, tid);
  }

  float m[SIMT_RPW], l[SIMT_RPW], acc[SIMT_RPW][JJ];
  int qseg[SIMT_RPW];
  int64_t qpos[SIMT_RPW];
#pragma unroll
  for (int i = 0; i < SIMT_RPW; ++i) {
    const int row = q0 + warp * SIMT_RPW + i;
    const bool live = row < p.lq;
    qpos[i] = (int64_t)row + p.q_offset;
    qseg[i] = (has_seg && live) ? qseg_g[row] : 0;
    m[i] = -CUDART_INF_F;
    l[i] = 0.f;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) acc[i][jj] = 0.f;
    if (load_state && live) {
      const int64_t rh = ((int64_t)b * p.lq + row) * p.heads + h;
      const float prev = st_lse[rh];
      if (prev != -CUDART_INF_F) {
        m[i] = prev;
        l[i] = 1.f;
#pragma unroll
        for (int jj = 0; jj < JJ; ++jj) {
          const int j = lane + 32 * jj;
          if (j < dv) acc[i][jj] = st_o[rh * dv + j];
        }
      }
    }
  }

  // Tiles wholly above the causal diagonal are never visited (tpa/tpa.py:427-428).
  int n_tiles = (p.lk + SIMT_BK - 1) / SIMT_BK;
  if (causal) {
    const int64_t kmax = (int64_t)q0 + SIMT_BQ - 1 + p.q_offset - p.k_offset;  // last visible local key
    if (kmax < 0) n_tiles = 0;
    else if (kmax / SIMT_BK + 1 < n_tiles) n_tiles = (int)(kmax / SIMT_BK) + 1;
  }

  // (with the comparison on part-local key indices the bound above does not apply: every part
  // has visible tiles, and the per-tile test below skips the others)
  if (p.per_part) n_tiles = (p.lk + SIMT_BK - 1) / SIMT_BK;
  const MaskRule rule = mask_rule(p);
  const bool positional = causal || rule.windowed;
  const int64_t q_lo = (int64_t)q0 + p.q_offset, q_hi = q_lo + SIMT_BQ - 1;
  const int64_t span = rule.span;

  int tile_begin = 0, tile_end = n_tiles;
  if (splits > 1) {
    const int chunk = (n_tiles + splits - 1) / splits;
    tile_begin = min(n_tiles, split * chunk);
    tile_end = min(n_tiles, tile_begin + chunk);
  }
  const float inv_rk = 1.f / (float)p.rank_k;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int k0 = tile * SIMT_BK;
    // a tile (it lies in one part: parts are multiples of the tile) no row of the block can see
    const int64_t kp_lo = (int64_t)(p.per_part ? k0 % p.part_len : k0) + p.k_offset, kp_hi = kp_lo + SIMT_BK - 1;
    if (causal && kp_lo > q_hi) continue;
    if (p.window > 0 && (q_lo - kp_hi >= span || (!causal && kp_lo - q_hi >= span))) continue;
    const int part = k0 / p.part_len;
    const int64_t koff = (int64_t)part * p.k_part_stride - (int64_t)part * p.part_len * p.ka.stride[1];
    const int64_t voff = (int64_t)part * p.v_part_stride - (int64_t)part * p.part_len * p.va.stride[1];
    __syncthreads();  // everyone is done with the previous K/V/P tiles (and Q is written)
    rebuild_tile<T>(Ks, ldk, SIMT_BK, k0, p.lk, dk, ka + koff, p.ka.stride, kb + koff, p.kb.stride, p.rank_k, h,
                    inv_rk, tid);
    rebuild_tile<T>(Vs, ldv, SIMT_BK, k0, p.lk, dv, va + voff, p.va.stride, vb + voff, p.vb.stride, p.rank_k, h,
                    inv_rk, tid);
    if (has_seg && tid < SIMT_BK) ksegs[tid] = (k0 + tid < p.lk) ? kseg_g[kseg_offset(p, k0 + tid)] : 0;
    if (rope) {
      __syncthreads();
      rope_tile(Ks, ldk, min(SIMT_BK, p.lk - k0), dk, p.rope_cos, p.rope_sin, k0 + p.rope_k_offset, tid);
    }
    __syncthreads();

    // row position minus the position of the tile's first key, per row of this warp (see MaskRule)
    int rel[SIMT_RPW], phase[SIMT_RPW];
#pragma unroll
    for (int i = 0; i < SIMT_RPW; ++i) {
      rel[i] = clamp_diff(qpos[i] - kp_lo);
      phase[i] = rule.dilated ? diff_phase(qpos[i] - kp_lo, rule.dilation) : 0;
    }

    // logits: this lane owns key columns `lane` and `lane + 32` of the 4 rows of its warp
    float s[SIMT_RPW][2];
#pragma unroll
    for (int i = 0; i < SIMT_RPW; ++i) s[i][0] = s[i][1] = 0.f;
    const float* k0p = Ks + lane * ldk;
    const float* k1p = Ks + (lane + 32) * ldk;
    const float* qp = Qs + warp * SIMT_RPW * ldk;
#pragma unroll 8
    for (int t = 0; t < dk; ++t) {  // unrolled: eight steps' shared-memory loads are in flight together
      const float ka0 = k0p[t], ka1 = k1p[t];
#pragma unroll
      for (int i = 0; i < SIMT_RPW; ++i) {
        const float qv = qp[i * ldk + t];
        s[i][0] = fmaf(qv, ka0, s[i][0]);
        s[i][1] = fmaf(qv, ka1, s[i][1]);
      }
    }

#pragma unroll
    for (int i = 0; i < SIMT_RPW; ++i) {
      float x[2];
      bool keep[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int kc = k0 + lane + 32 * c;
        keep[c] = kc < p.lk;
        if (positional) keep[c] = keep[c] && keep_diff32(rule, rel[i] - (lane + 32 * c));
        if (rule.dilated) keep[c] = keep[c] && keep_dilated(rule, phase[i], lane + 32 * c);
        if (has_seg) keep[c] = keep[c] && (qseg[i] == ksegs[lane + 32 * c]);
        x[c] = keep[c] ? s[i][c] * p.sm_scale : -CUDART_INF_F;
      }
      const float tmax = warp_max(fmaxf(x[0], x[1]));
      const float m_new = fmaxf(m[i], tmax);
      float p0 = 0.f, p1 = 0.f, corr = 1.f;
      if (m_new != -CUDART_INF_F) {
        corr = (m[i] == -CUDART_INF_F) ? 0.f : expf(m[i] - m_new);
        p0 = keep[0] ? expf(x[0] - m_new) : 0.f;
        p1 = keep[1] ? expf(x[1] - m_new) : 0.f;
      }
      const float psum = warp_sum(p0 + p1);
      l[i] = l[i] * corr + psum;
      m[i] = m_new;
#pragma unroll
      for (int jj = 0; jj < JJ; ++jj) acc[i][jj] *= corr;
      Ps[(warp * SIMT_RPW + i) * SIMT_BK + lane] = p0;
      Ps[(warp * SIMT_RPW + i) * SIMT_BK + lane + 32] = p1;
    }
    __syncwarp();

    // acc += P V : this lane owns value columns lane + 32*jj
    const float* pp = Ps + warp * SIMT_RPW * SIMT_BK;
#pragma unroll 8
    for (int c = 0; c < SIMT_BK; ++c) {
      float vv[JJ];
#pragma unroll
      for (int jj = 0; jj < JJ; ++jj) vv[jj] = Vs[c * ldv + lane + 32 * jj];
#pragma unroll
      for (int i = 0; i < SIMT_RPW; ++i) {
        const float pv = pp[i * SIMT_BK + c];
#pragma unroll
        for (int jj = 0; jj < JJ; ++jj) acc[i][jj] = fmaf(pv, vv[jj], acc[i][jj]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < SIMT_RPW; ++i) {
    const int row = q0 + warp * SIMT_RPW + i;
    if (row >= p.lq) continue;
    const int64_t rh = ((int64_t)b * p.lq + row) * p.heads + h;
    const bool empty = !(l[i] > 0.f);
    const float inv = empty ? 0.f : 1.f / l[i];
    const float lse = empty ? -CUDART_INF_F : m[i] + logf(l[i]);
    if (store_state) {
      // partial result for the next ring step: 0 / -inf where nothing was visible yet
      // (the nan_to_num of tpa/ring_tpa.py:85-89)
#pragma unroll
      for (int jj = 0; jj < JJ; ++jj) {
        const int j = lane + 32 * jj;
        if (j < dv) st_o[rh * dv + j] = acc[i][jj] * inv;
      }
      if (lane == 0) st_lse[rh] = lse;
    } else {
      T* op = static_cast<T*>(p.o) + rh * dv;
#pragma unroll
      for (int jj = 0; jj < JJ; ++jj) {
        const int j = lane + 32 * jj;
        // rows that saw no key are NaN (tpa/tpa.py:439, tpa/ring_tpa.py:109)
        if (j < dv) from_float(op[j], empty ? CUDART_NAN_F : acc[i][jj] * inv);
      }
      if (lane == 0 && p.lse != nullptr) p.lse[rh] = lse;
    }
  }
}

// Few row blocks against enough keys leave most of the GPU idle and every CTA latency-bound on a
// serial walk (fp32 c0: 128 CTAs of up to 8 tiles): the key tiles are then split over several CTAs
// per block and the partials merged, as the tensor-core kernel does for decode-like shapes.
int simt_pick_splits(const Params& p) {
  if (p.dv % 4 != 0 || p.kv_parts > 1 || p.has_window()) return 1;
  // the merge kernel moves 16 bytes at a time
  auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (!(p.flags & TPA_FLAG_STATE_STORE) && !aligned16(p.o)) return 1;
  if ((p.flags & (TPA_FLAG_STATE_STORE | TPA_FLAG_STATE_LOAD)) && !aligned16(p.state_o)) return 1;
  const int64_t items = (int64_t)((p.lq + SIMT_BQ - 1) / SIMT_BQ) * p.heads * p.batch;
  const int n_kv = (p.lk + SIMT_BK - 1) / SIMT_BK;
  if (items > 2 * 148 || n_kv < 4) return 1;
  int splits = (int)((4 * 148 + items - 1) / items);
  if (splits > n_kv / 2) splits = n_kv / 2;
  if (splits > 16) splits = 16;
  if ((int64_t)p.batch * splits > 65535) return 1;
  return splits < 2 ? 1 : splits;
}

size_t simt_workspace_bytes(const Params& p) {
  const int splits = simt_pick_splits(p);
  if (splits == 1) return 0;
  const size_t bytes = (size_t)splits * p.batch * p.lq * p.heads * (p.dv + 1) * sizeof(float);
  return (bytes + 255) & ~(size_t)255;
}

template <typename T, int JJ>
static cudaError_t launch_one(const Params& p, void* workspace, TpaKernelInfo* info, bool dry_run,
                              cudaStream_t stream) {
  const int ldk = p.dk + 1, ldv = JJ * 32;
  const size_t smem = sizeof(float) * ((size_t)SIMT_BQ * ldk + (size_t)SIMT_BK * ldk +
                                       (size_t)SIMT_BK * ldv + SIMT_BQ * SIMT_BK + SIMT_BK);
  const int splits = simt_pick_splits(p);
  dim3 grid((p.lq + SIMT_BQ - 1) / SIMT_BQ, p.heads, p.batch * splits);
  if (info) {
    info->kernel = TPA_KERNEL_SIMT;
    info->block_q = SIMT_BQ;
    info->block_kv = SIMT_BK;
    info->threads = SIMT_THREADS;
    info->grid[0] = grid.x;
    info->grid[1] = grid.y;
    info->grid[2] = grid.z;
    info->smem_bytes = (int)smem;
    info->launches = splits > 1 ? 2 : 1;
  }
  if (dry_run) return cudaSuccess;
  // with key splits the kernel stores partials (as a ring step would) into scratch
  Params pk = p;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    part_o = static_cast<float*>(workspace);
    part_lse = part_o + (size_t)splits * p.batch * p.lq * p.heads * p.dv;
    pk.flags = (p.flags & ~(uint32_t)TPA_FLAG_STATE_LOAD) | TPA_FLAG_STATE_STORE;
    pk.state_o = part_o;
    pk.state_lse = part_lse;
  }
  auto kern = tpa_fwd_simt_kernel<T, JJ>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<grid, SIMT_THREADS, smem, stream>>>(pk, splits);
  count_launch(1);
  e = cudaGetLastError();
  if (e != cudaSuccess || splits == 1) return e;
  return launch_combine_splits(p, part_o, part_lse, splits, stream);
}

template <typename T>
static cudaError_t launch_t(const Params& p, void* ws, TpaKernelInfo* info, bool dry, cudaStream_t s) {
  if (p.dv <= 32) return launch_one<T, 1>(p, ws, info, dry, s);
  if (p.dv <= 64) return launch_one<T, 2>(p, ws, info, dry, s);
  if (p.dv <= 128) return launch_one<T, 4>(p, ws, info, dry, s);
  return launch_one<T, 8>(p, ws, info, dry, s);
}

cudaError_t launch_simt(const Params& p, void* workspace, TpaKernelInfo* info, bool dry_run, cudaStream_t stream) {
  if (p.dtype == TPA_DTYPE_F32) return launch_t<float>(p, workspace, info, dry_run, stream);
  return launch_t<__nv_bfloat16>(p, workspace, info, dry_run, stream);
}

}  // namespace tpa
