// C ABI of libtpa_b200.so: argument validation, kernel choice, status reporting.
// Declarations and the reference interfaces they replace are in include/tpa_b200.h.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>

#include "tpa_common.cuh"

namespace tpa {

static std::atomic<uint64_t> g_launches{0};
static thread_local char g_cuda_error[256] = "";

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int fail_cuda(cudaError_t e) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", cudaGetErrorName(e),
                cudaGetErrorString(e));
  return TPA_ERR_CUDA;
}

static bool factor_ok(const TpaFactor& f) {
  return f.ptr != nullptr && f.stride[1] > 0 && f.stride[2] > 0 && f.stride[0] >= 0;
}

// Mirrors the checks the reference makes at trace time (tpa/tpa.py:474-475, 369-371) plus
// what a C caller can get wrong.
static int validate(const TpaFwdArgs* a, Params* p) {
  if (a == nullptr || a->struct_size != sizeof(TpaFwdArgs)) return TPA_ERR_BAD_ARG;
  if (a->dtype != TPA_DTYPE_F32 && a->dtype != TPA_DTYPE_BF16) return TPA_ERR_UNSUPPORTED;
  if (a->batch <= 0 || a->lq <= 0 || a->lk <= 0 || a->rank_q <= 0 || a->rank_k <= 0 ||
      a->heads <= 0 || a->dk <= 0 || a->dv <= 0)
    return TPA_ERR_BAD_ARG;
  if (!factor_ok(a->qa) || !factor_ok(a->qb) || !factor_ok(a->ka) || !factor_ok(a->kb) ||
      !factor_ok(a->va) || !factor_ok(a->vb))
    return TPA_ERR_BAD_ARG;
  if ((a->q_segment_ids == nullptr) != (a->kv_segment_ids == nullptr)) return TPA_ERR_BAD_ARG;
  const bool store = (a->flags & TPA_FLAG_STATE_STORE) != 0;
  const bool load = (a->flags & TPA_FLAG_STATE_LOAD) != 0;
  if ((store || load) && (a->state_o == nullptr || a->state_lse == nullptr)) return TPA_ERR_BAD_ARG;
  if (!store && a->o == nullptr) return TPA_ERR_BAD_ARG;
  if (a->flags & ~(uint32_t)(TPA_FLAG_CAUSAL | TPA_FLAG_STATE_LOAD | TPA_FLAG_STATE_STORE |
                             TPA_FLAG_REUSE_STAGED_Q | TPA_FLAG_CAUSAL_PER_PART | TPA_FLAG_REUSE_STAGED_KV))
    return TPA_ERR_BAD_ARG;
  const int parts = a->kv_parts > 1 ? a->kv_parts : 1;
  if (a->kv_parts < 0 || a->window < 0 || a->dilation < 0) return TPA_ERR_BAD_ARG;
  if (parts > 1 && (a->lk % parts != 0 || a->k_part_stride <= 0 || a->v_part_stride <= 0)) return TPA_ERR_BAD_ARG;
  if ((a->flags & TPA_FLAG_CAUSAL_PER_PART) && parts == 1) return TPA_ERR_BAD_ARG;
  // the kernels compare clamped 32-bit differences against window * dilation
  if ((int64_t)a->window * (a->dilation > 1 ? a->dilation : 1) > ((int64_t)1 << 29) || a->dilation > (1 << 29))
    return TPA_ERR_UNSUPPORTED;
  if ((a->rope_cos == nullptr) != (a->rope_sin == nullptr)) return TPA_ERR_BAD_ARG;
  if (a->rope_cos != nullptr) {
    // every row the call touches must exist in the tables; pairs of columns need an even dk
    if (a->dk % 2 != 0 || a->rope_q_offset < 0 || a->rope_k_offset < 0 ||
        a->rope_q_offset + a->lq > a->rope_len || a->rope_k_offset + a->lk > a->rope_len)
      return TPA_ERR_BAD_ARG;
  }
  if (a->kernel < TPA_KERNEL_AUTO || a->kernel > TPA_KERNEL_DECODE) return TPA_ERR_BAD_ARG;
  if (a->heads > 65535 || a->batch > 65535) return TPA_ERR_UNSUPPORTED;
  if (a->dk > 256 || a->dv > 256) return TPA_ERR_UNSUPPORTED;
  p->dtype = a->dtype;
  p->batch = a->batch; p->lq = a->lq; p->lk = a->lk;
  p->rank_q = a->rank_q; p->rank_k = a->rank_k;
  p->heads = a->heads; p->dk = a->dk; p->dv = a->dv;
  p->qa = a->qa; p->qb = a->qb; p->ka = a->ka; p->kb = a->kb; p->va = a->va; p->vb = a->vb;
  p->q_seg = a->q_segment_ids; p->kv_seg = a->kv_segment_ids;
  p->q_seg_bstride = a->q_segment_batch_stride; p->kv_seg_bstride = a->kv_segment_batch_stride;
  p->o = a->o; p->lse = a->lse; p->state_o = a->state_o; p->state_lse = a->state_lse;
  p->sm_scale = a->sm_scale; p->flags = a->flags;
  p->q_offset = a->q_offset; p->k_offset = a->k_offset;
  p->status = nullptr;
  p->kv_parts = parts;
  p->part_len = a->lk / parts;
  p->k_part_stride = a->k_part_stride; p->v_part_stride = a->v_part_stride;
  p->kseg_part_stride = a->kv_segment_part_stride;
  p->per_part = (a->flags & TPA_FLAG_CAUSAL_PER_PART) != 0;
  p->window = a->window;
  p->dilation = a->dilation > 1 ? a->dilation : 1;
  p->rope_cos = a->rope_cos; p->rope_sin = a->rope_sin; p->rope_len = a->rope_len;
  p->rope_q_offset = a->rope_q_offset; p->rope_k_offset = a->rope_k_offset;
  return TPA_OK;
}

// Extensions only some kernels implement (parts, window / dilation, rotary embedding).
static bool has_extensions(const Params& p) {
  return p.kv_parts > 1 || p.has_window() || p.rope_cos != nullptr;
}

static int choose(const TpaFwdArgs* a, const Params& p, int* kernel) {
  const bool ext = has_extensions(p);
  if (ext && (a->kernel == TPA_KERNEL_DECODE || a->kernel == TPA_KERNEL_SM100_FUSED)) return TPA_ERR_KERNEL_FORCED;
  // the generic kernel walks keys 64 at a time, the tensor-core kernel 128: parts must be whole tiles
  if (p.kv_parts > 1 && p.part_len % 64 != 0) return TPA_ERR_UNSUPPORTED;
  const bool dec = !ext && decode_supported(p);
  if (a->kernel == TPA_KERNEL_DECODE && !dec) return TPA_ERR_KERNEL_FORCED;
  if (a->kernel == TPA_KERNEL_DECODE || (a->kernel == TPA_KERNEL_AUTO && dec && decode_preferred(p))) {
    *kernel = TPA_KERNEL_DECODE;
    return TPA_OK;
  }
  const bool tc = sm100_supported(p);
  if (a->kernel >= TPA_KERNEL_SM100 && a->kernel <= TPA_KERNEL_SM100_STAGED && !tc) return TPA_ERR_KERNEL_FORCED;
  if (a->kernel == TPA_KERNEL_SIMT || !tc) *kernel = TPA_KERNEL_SIMT;
  else if (a->kernel == TPA_KERNEL_SM100_FUSED || a->kernel == TPA_KERNEL_SM100_STAGED) *kernel = a->kernel;
  else *kernel = sm100_pick_variant(p);
  return TPA_OK;
}

constexpr size_t kStatusBytes = 256;  // status block at the head of every non-empty workspace

static size_t round256(size_t n) { return (n + 255) & ~(size_t)255; }

// ---- the staged forward with bounded scratch: head groups one after the other --------------------
// A caller that passes less than tpa_fwd_workspace_bytes() (but at least tpa_fwd_workspace_bytes_min())
// gets the same result from a workspace that holds the tiles of `hc` heads at a time: for each group
// the staging launch and the attention launch run on that group's heads (the head factors are
// offset pointers, everything else is unchanged), o and lse of the group go to a compact block
// behind the tiles, and a strided device-to-device copy puts them at their heads' place in the
// caller's arrays.  The kernels themselves are the ones every other call uses.
static size_t esize(const Params& p) { return p.dtype == TPA_DTYPE_BF16 ? 2 : 4; }
static Params group_params(const Params& p, int h0, int hc) {
  Params g = p;
  g.heads = hc;
  const size_t es = esize(p);
  g.qa.ptr = static_cast<const char*>(p.qa.ptr) + (size_t)h0 * es;
  g.ka.ptr = static_cast<const char*>(p.ka.ptr) + (size_t)h0 * es;
  g.va.ptr = static_cast<const char*>(p.va.ptr) + (size_t)h0 * es;
  return g;
}
struct GroupLayout {
  size_t o, lse, total;  // offsets behind the status block
};
static GroupLayout group_layout(const Params& p, int hc) {
  GroupLayout l;
  const Params g = group_params(p, 0, hc);
  l.o = round256(sm100_workspace_bytes(g, TPA_KERNEL_SM100_STAGED));
  l.lse = l.o + round256((size_t)p.batch * p.lq * hc * p.dv * esize(p));
  l.total = l.lse + round256((size_t)p.batch * p.lq * hc * sizeof(float));
  return l;
}
// largest head group (a multiple of 8, what one staging CTA rebuilds) whose scratch fits; 0 if none
static int group_heads_for(const Params& p, size_t workspace_bytes) {
  if (p.flags & (TPA_FLAG_STATE_LOAD | TPA_FLAG_STATE_STORE | TPA_FLAG_REUSE_STAGED_Q | TPA_FLAG_REUSE_STAGED_KV))
    return 0;  // carried state and kept tiles belong to the one-pass layout
  int best = 0;  // equal groups only: every group then has the scratch layout that was sized
  for (int hc = 8; hc < p.heads; hc += 8)
    if (p.heads % hc == 0 && kStatusBytes + group_layout(p, hc).total <= workspace_bytes) best = hc;
  return best;
}
static cudaError_t launch_sm100_grouped(const Params& p, int hc, char* ws, cudaStream_t s) {
  const GroupLayout l = group_layout(p, hc);
  const size_t es = esize(p);
  for (int h0 = 0; h0 < p.heads; h0 += hc) {
    Params g = group_params(p, h0, std::min(hc, p.heads - h0));
    g.o = ws + l.o;
    g.lse = p.lse != nullptr ? reinterpret_cast<float*>(ws + l.lse) : nullptr;
    cudaError_t e = launch_sm100(g, TPA_KERNEL_SM100_STAGED, ws, nullptr, false, s);
    if (e != cudaSuccess) return e;
    const size_t rows = (size_t)p.batch * p.lq;
    e = cudaMemcpy2DAsync(static_cast<char*>(p.o) + (size_t)h0 * p.dv * es, (size_t)p.heads * p.dv * es, g.o,
                          (size_t)g.heads * p.dv * es, (size_t)g.heads * p.dv * es, rows, cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) return e;
    if (p.lse != nullptr) {
      e = cudaMemcpy2DAsync(p.lse + h0, (size_t)p.heads * sizeof(float), g.lse, (size_t)g.heads * sizeof(float),
                            (size_t)g.heads * sizeof(float), rows, cudaMemcpyDeviceToDevice, s);
      if (e != cudaSuccess) return e;
    }
  }
  return cudaSuccess;
}

// Scratch of the backward: status block, delta, dense fp32 dQ / dK / dV.
struct BwdLayout {
  size_t delta, dq, dk, dv, tc, total;  // tc: scratch of the tensor-core passes
};
static BwdLayout bwd_layout(const Params& p, bool tensor_cores) {
  BwdLayout l;
  size_t off = kStatusBytes;
  l.delta = off; off += round256(sizeof(float) * (size_t)p.batch * p.lq * p.heads);
  l.dq = off;    off += round256(sizeof(float) * (size_t)p.batch * p.lq * p.heads * p.dk);
  l.dk = off;    off += round256(sizeof(float) * (size_t)p.batch * p.lk * p.heads * p.dk);
  l.dv = off;    off += round256(sizeof(float) * (size_t)p.batch * p.lk * p.heads * p.dv);
  l.tc = off;    off += tensor_cores ? bwd_sm100_workspace_bytes(p) : 0;
  l.total = off;
  return l;
}

static int validate_bwd(const TpaBwdArgs* a, BwdParams* bp) {
  if (a == nullptr || a->struct_size != sizeof(TpaBwdArgs)) return TPA_ERR_BAD_ARG;
  int st = validate(&a->fwd, &bp->f);
  if (st != TPA_OK) return st;
  if (a->fwd.flags & ~(uint32_t)TPA_FLAG_CAUSAL) return TPA_ERR_BAD_ARG;
  if (has_extensions(bp->f)) return TPA_ERR_UNSUPPORTED;  // parts, windows and rotary embedding are forward only
  if (a->fwd.o == nullptr || a->fwd.lse == nullptr || a->d_o == nullptr || a->dq == nullptr ||
      a->dk == nullptr || a->dv == nullptr)
    return TPA_ERR_BAD_ARG;
  if (a->bwd_flags & ~(uint32_t)(TPA_BWD_ACCUMULATE_DQ | TPA_BWD_ACCUMULATE_DKV)) return TPA_ERR_BAD_ARG;
  if (a->grad_dtype != TPA_DTYPE_F32 && a->grad_dtype != a->fwd.dtype) return TPA_ERR_UNSUPPORTED;
  if (a->fwd.kernel >= TPA_KERNEL_SM100_FUSED) return TPA_ERR_KERNEL_FORCED;
  bp->d_o = a->d_o;
  bp->dq = a->dq; bp->dk = a->dk; bp->dv = a->dv;
  bp->grad_dtype = a->grad_dtype;
  bp->accumulate_dq = (a->bwd_flags & TPA_BWD_ACCUMULATE_DQ) != 0;
  bp->accumulate_dkv = (a->bwd_flags & TPA_BWD_ACCUMULATE_DKV) != 0;
  bp->delta = bp->dq_dense = bp->dk_dense = bp->dv_dense = nullptr;
  return TPA_OK;
}

// TPA_OK and whether the tensor-core passes run; SM100 forced on an unsupported shape is an error
static int choose_bwd(const TpaBwdArgs* a, const BwdParams& bp, bool* tensor_cores) {
  const bool tc = bwd_sm100_supported(bp);
  if (a->fwd.kernel == TPA_KERNEL_SM100 && !tc) return TPA_ERR_KERNEL_FORCED;
  *tensor_cores = tc && a->fwd.kernel != TPA_KERNEL_SIMT;
  return TPA_OK;
}

}  // namespace tpa

using namespace tpa;

extern "C" {

int tpa_abi_version(void) { return TPA_B200_ABI_VERSION; }

uint64_t tpa_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* tpa_last_cuda_error(void) { return g_cuda_error; }

const char* tpa_status_string(int status) {
  switch (status) {
    case TPA_OK: return "ok";
    case TPA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size, segment ids given for only one side, or wrong struct_size)";
    case TPA_ERR_UNSUPPORTED: return "unsupported shape or dtype (dtype must be f32/bf16; dk, dv <= 256; heads, batch <= 65535)";
    case TPA_ERR_WORKSPACE: return "workspace missing, misaligned or smaller than tpa_fwd_workspace_bytes()";
    case TPA_ERR_CUDA: return "CUDA runtime error (see tpa_last_cuda_error)";
    case TPA_ERR_KERNEL_FORCED: return "the forced kernel cannot run this shape";
    case TPA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case TPA_ERR_STATIC_SCRATCH: return "the problem needs more scratch than the library's static buffer (TPA_STATIC_SCRATCH_BYTES) holds; use tpa_fwd with a caller workspace";
    default: return "unknown status";
  }
}

size_t tpa_fwd_workspace_bytes(const TpaFwdArgs* args) {
  Params p;
  int kernel;
  if (validate(args, &p) != TPA_OK || choose(args, p, &kernel) != TPA_OK) return 0;
  if (kernel == TPA_KERNEL_SIMT) return simt_workspace_bytes(p) ? kStatusBytes + simt_workspace_bytes(p) : 0;
  if (kernel == TPA_KERNEL_DECODE) return kStatusBytes + decode_workspace_bytes(p);
  return kStatusBytes + sm100_workspace_bytes(p, kernel);
}

size_t tpa_fwd_workspace_bytes_min(const TpaFwdArgs* args) {
  Params p;
  int kernel;
  if (validate(args, &p) != TPA_OK || choose(args, p, &kernel) != TPA_OK) return 0;
  const size_t full = tpa_fwd_workspace_bytes(args);
  if (kernel != TPA_KERNEL_SM100_STAGED || p.heads <= 8 ||
      (p.flags & (TPA_FLAG_STATE_LOAD | TPA_FLAG_STATE_STORE | TPA_FLAG_REUSE_STAGED_Q | TPA_FLAG_REUSE_STAGED_KV)))
    return full;
  // not simply the smallest group: a small group of few row blocks splits its keys over CTAs and
  // keeps the partials in scratch, which can outweigh the tiles it saves
  size_t least = full;
  for (int hc = 8; hc < p.heads; hc += 8)
    if (p.heads % hc == 0) least = std::min(least, kStatusBytes + group_layout(p, hc).total);
  return least;
}

int tpa_query_kernel(const TpaFwdArgs* args, TpaKernelInfo* info) {
  if (info == nullptr) return TPA_ERR_BAD_ARG;
  std::memset(info, 0, sizeof(*info));
  Params p;
  int kernel;
  int st = validate(args, &p);
  if (st != TPA_OK) return st;
  st = choose(args, p, &kernel);
  if (st != TPA_OK) return st;
  cudaError_t e = kernel == TPA_KERNEL_DECODE ? launch_decode(p, nullptr, info, true, nullptr)
                  : kernel != TPA_KERNEL_SIMT ? launch_sm100(p, kernel, nullptr, info, true, nullptr)
                                              : launch_simt(p, nullptr, info, true, nullptr);
  return e == cudaSuccess ? TPA_OK : fail_cuda(e);
}

int tpa_fwd(const TpaFwdArgs* args, void* workspace, size_t workspace_bytes, void* stream) {
  Params p;
  int kernel;
  int st = validate(args, &p);
  if (st != TPA_OK) return st;
  st = choose(args, p, &kernel);
  if (st != TPA_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (kernel != TPA_KERNEL_SIMT) {
    const size_t need = kStatusBytes + (kernel == TPA_KERNEL_DECODE ? decode_workspace_bytes(p)
                                                                     : sm100_workspace_bytes(p, kernel));
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return TPA_ERR_WORKSPACE;
    int group_heads = 0;
    if (workspace_bytes < need) {
      // less scratch than the one-pass layout: the staged kernel can still run head group by head group
      if (kernel == TPA_KERNEL_SM100_STAGED) group_heads = group_heads_for(p, workspace_bytes);
      if (group_heads == 0) return TPA_ERR_WORKSPACE;
    }
    p.status = static_cast<uint32_t*>(workspace);
    e = cudaMemsetAsync(workspace, 0, kStatusBytes, s);
    if (e != cudaSuccess) return fail_cuda(e);
    if (group_heads != 0) {
      e = launch_sm100_grouped(p, group_heads, static_cast<char*>(workspace) + kStatusBytes, s);
      return e == cudaSuccess ? TPA_OK : fail_cuda(e);
    }
    e = kernel == TPA_KERNEL_DECODE
            ? launch_decode(p, static_cast<char*>(workspace) + kStatusBytes, nullptr, false, s)
            : launch_sm100(p, kernel, static_cast<char*>(workspace) + kStatusBytes, nullptr, false, s);
  } else {
    const size_t need = simt_workspace_bytes(p);
    if (need != 0 && (workspace == nullptr || workspace_bytes < kStatusBytes + need ||
                      (reinterpret_cast<uintptr_t>(workspace) & 255) != 0))
      return TPA_ERR_WORKSPACE;
    if (need != 0) {
      e = cudaMemsetAsync(workspace, 0, kStatusBytes, s);
      if (e != cudaSuccess) return fail_cuda(e);
    }
    e = launch_simt(p, need ? static_cast<char*>(workspace) + kStatusBytes : nullptr, nullptr, false, s);
  }
  return e == cudaSuccess ? TPA_OK : fail_cuda(e);
}

size_t tpa_bwd_workspace_bytes(const TpaBwdArgs* args) {
  BwdParams bp;
  bool tc;
  if (validate_bwd(args, &bp) != TPA_OK || choose_bwd(args, bp, &tc) != TPA_OK) return 0;
  return bwd_layout(bp.f, tc).total;
}

int tpa_bwd(const TpaBwdArgs* args, void* workspace, size_t workspace_bytes, void* stream) {
  BwdParams bp;
  int st = validate_bwd(args, &bp);
  if (st != TPA_OK) return st;
  bool tc;
  st = choose_bwd(args, bp, &tc);
  if (st != TPA_OK) return st;
  const BwdLayout l = bwd_layout(bp.f, tc);
  if (workspace == nullptr || workspace_bytes < l.total ||
      (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return TPA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  bp.delta = reinterpret_cast<float*>(ws + l.delta);
  bp.dq_dense = reinterpret_cast<float*>(ws + l.dq);
  bp.dk_dense = reinterpret_cast<float*>(ws + l.dk);
  bp.dv_dense = reinterpret_cast<float*>(ws + l.dv);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(workspace, 0, kStatusBytes, s);
  if (tc) {
    bp.f.status = static_cast<uint32_t*>(workspace);
    if (e == cudaSuccess) e = launch_bwd_pairs_sm100(bp, ws + l.tc, s);
  } else {
    if (e == cudaSuccess) e = launch_bwd_delta(bp, s);
    if (e == cudaSuccess) e = launch_bwd_pairs_simt(bp, s);
  }
  if (e == cudaSuccess) e = launch_bwd_contract(bp, s);
  return e == cudaSuccess ? TPA_OK : fail_cuda(e);
}

int tpa_selftest_wait_timeout(void* workspace, size_t workspace_bytes, int64_t budget_cycles, void* stream) {
  if (workspace == nullptr || workspace_bytes < kStatusBytes || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return TPA_ERR_WORKSPACE;
  if (budget_cycles <= 0 || budget_cycles > (int64_t)1 << 28) return TPA_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(workspace, 0, kStatusBytes, s);
  if (e == cudaSuccess) e = launch_wait_selftest(static_cast<uint32_t*>(workspace), budget_cycles, s);
  return e == cudaSuccess ? TPA_OK : fail_cuda(e);
}

int tpa_read_status(const void* workspace, void* stream, uint32_t detail[4]) {
  uint32_t host[4] = {0, 0, 0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e);
  if (workspace != nullptr) {
    e = cudaMemcpy(host, workspace, sizeof(host), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(e);
  }
  if (detail != nullptr) std::memcpy(detail, host, sizeof(host));
  return host[0] == 0 ? TPA_OK : TPA_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
