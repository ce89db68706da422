// Internal declarations shared by the translation units of libtpa_b200.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tpa_b200.h"

namespace tpa {

// Device-side view of one forward call (validated copy of TpaFwdArgs).
struct Params {
  int dtype;
  int batch, lq, lk, rank_q, rank_k, heads, dk, dv;
  TpaFactor qa, qb, ka, kb, va, vb;
  const int32_t* q_seg;
  const int32_t* kv_seg;
  int64_t q_seg_bstride, kv_seg_bstride;
  void* o;
  float* lse;
  float* state_o;
  float* state_lse;
  float sm_scale;
  uint32_t flags;
  int64_t q_offset, k_offset;
  uint32_t* status;  // device status block {flag, where, block, spins} or nullptr
  // keys in parts (kv_parts >= 1, part_len = lk / kv_parts); strides in elements
  int kv_parts, part_len;
  int64_t k_part_stride, v_part_stride, kseg_part_stride;
  bool per_part;      // causal / window comparison on the key's index inside its part
  int window, dilation;  // window 0 = none; dilation >= 1
  const float* rope_cos;
  const float* rope_sin;
  int rope_len;
  int64_t rope_q_offset, rope_k_offset;

  __host__ __device__ __forceinline__ bool has_window() const { return window > 0 || dilation > 1; }
};

// Masking rule shared by the kernels.  With diff = (query row + q_offset) - (key position + k_offset):
// causal keeps diff >= 0; a window keeps |diff| < window * dilation; dilation D keeps diff % D == 0.
// The kernels take the 64-bit difference once per thread and tile (first column of the thread),
// clamp it to +-2^30 -- beyond that every rule has the same answer as at the bound, since
// window * dilation <= 2^29 is enforced on entry -- and work in 32 bits per element.  The
// remainder for dilation is taken from the exact 64-bit value, once, as `phase`.
struct MaskRule {
  bool causal, windowed, dilated;
  int span;      // window * dilation
  int dilation;
};
__host__ __device__ __forceinline__ MaskRule mask_rule(const Params& p) {
  return MaskRule{(p.flags & TPA_FLAG_CAUSAL) != 0, p.window > 0, p.dilation > 1,
                  (int)((int64_t)p.window * p.dilation), p.dilation};
}
__host__ __device__ __forceinline__ int clamp_diff(int64_t d) {
  const int64_t lim = (int64_t)1 << 30;
  return (int)(d > lim ? lim : (d < -lim ? -lim : d));
}
__host__ __device__ __forceinline__ int diff_phase(int64_t d, int dilation) {
  const int r = (int)(d % dilation);
  return r < 0 ? r + dilation : r;
}
// causal and window part of the rule for one element, diff = clamped first-column diff - column
__host__ __device__ __forceinline__ bool keep_diff32(const MaskRule& m, int diff) {
  bool keep = !m.causal || diff >= 0;
  if (m.windowed) keep = keep && diff < m.span && -diff < m.span;
  return keep;
}
// dilation part: column `idx` of a thread whose first column has remainder `phase`
__host__ __device__ __forceinline__ bool keep_dilated(const MaskRule& m, int phase, int idx) {
  return (phase - idx) % m.dilation == 0;
}

// Element offset of key row `kc` of a K or V factor (parts, then rows inside the part).
__host__ __device__ __forceinline__ int64_t key_row_offset(const Params& p, const TpaFactor& f, int64_t part_stride,
                                                           int kc) {
  const int part = kc / p.part_len;
  return (int64_t)part * part_stride + (int64_t)(kc - part * p.part_len) * f.stride[1];
}
__host__ __device__ __forceinline__ int64_t kseg_offset(const Params& p, int kc) {
  const int part = kc / p.part_len;
  return (int64_t)part * p.kseg_part_stride + (kc - part * p.part_len);
}

// Device-side view of one backward call.
struct BwdParams {
  Params f;           // the forward operands; f.o and f.lse are inputs here
  const void* d_o;    // [batch, lq, heads, dv], dtype of the factors
  float* delta;       // scratch [batch, lq, heads]
  float* dq_dense;    // scratch [batch, lq, heads, dk] fp32
  float* dk_dense;    // scratch [batch, lk, heads, dk] fp32
  float* dv_dense;    // scratch [batch, lk, heads, dv] fp32
  void* dq;           // gradients in the concatenated layout [batch, l, rank, heads + d]
  void* dk;
  void* dv;
  int grad_dtype;     // TPA_DTYPE_* of dq / dk / dv
  bool accumulate_dq, accumulate_dkv;
};

cudaError_t launch_bwd_delta(const BwdParams& bp, cudaStream_t stream);
cudaError_t launch_bwd_pairs_simt(const BwdParams& bp, cudaStream_t stream);
cudaError_t launch_bwd_contract(const BwdParams& bp, cudaStream_t stream);
// tensor-core pair passes (bf16, head_dim 64 / 128): `workspace` holds bwd_sm100_workspace_bytes
bool bwd_sm100_supported(const BwdParams& bp);
size_t bwd_sm100_workspace_bytes(const Params& p);
cudaError_t launch_bwd_pairs_sm100(const BwdParams& bp, void* workspace, cudaStream_t stream);
cudaError_t launch_stage_tiles(const Params& p, uint8_t* wq, uint8_t* wk, uint8_t* wv, float qscale,
                               cudaStream_t stream);

// Launchers: enqueue on `stream`, return a cudaError_t.  `info` is filled either way.
// `workspace` holds simt_workspace_bytes(p) (0 unless the key tiles are split over CTAs)
cudaError_t launch_simt(const Params& p, void* workspace, TpaKernelInfo* info, bool dry_run, cudaStream_t stream);
int simt_pick_splits(const Params& p);
size_t simt_workspace_bytes(const Params& p);
bool sm100_supported(const Params& p);
int sm100_pick_variant(const Params& p);  // TPA_KERNEL_SM100_FUSED or TPA_KERNEL_SM100_STAGED
size_t sm100_workspace_bytes(const Params& p, int variant);
cudaError_t launch_sm100(const Params& p, int variant, void* workspace, TpaKernelInfo* info,
                         bool dry_run, cudaStream_t stream);

// few query rows against a long factor cache (tpa_fwd_decode.cu); scratch = per-split partials
bool decode_supported(const Params& p);   // the kernel can run this call
bool decode_preferred(const Params& p);   // ... and is measured faster than the staged path
size_t decode_workspace_bytes(const Params& p);
cudaError_t launch_decode(const Params& p, void* workspace, TpaKernelInfo* info, bool dry_run, cudaStream_t stream);
// merges per-split partial (o, lse) (and the carried state) into the output or the state
cudaError_t launch_combine_splits(const Params& p, const float* part_o, const float* part_lse, int splits,
                                  cudaStream_t stream);

cudaError_t launch_wait_selftest(uint32_t* status, long long budget_cycles, cudaStream_t stream);

void count_launch(int n);
// Records the text of `e` for tpa_last_cuda_error() on this thread and returns TPA_ERR_CUDA.
int fail_cuda(cudaError_t e);

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_float(float& dst, float x) { dst = x; }
__device__ __forceinline__ void from_float(__nv_bfloat16& dst, float x) {
  dst = __float2bfloat16_rn(x);
}

}  // namespace tpa
