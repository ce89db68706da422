/*
 * tpa_b200.h — C ABI of libtpa_b200.so: Tensor Product Attention forward and backward on B200 (sm_100a).
 *
 * The reference (jondeaton/tensor-product-attention-jax) has no FFI of its own; its
 * narrowest seam is the Pallas custom call in tpa/tpa.py:492-543,
 *
 *     (qa, qb, ka, kb, va, vb, q_segment_ids | None, kv_segment_ids | None) -> (o, lse)
 *
 * vmapped over batch by tpa/tpa.py:144-163 and tpa/ring_tpa.py:242-255.  The entry
 * points below are what a jax.ffi (or ctypes / cffi) binding for that seam binds.
 * Everything is plain C: pointers, sizes, element strides.  All pointers are device
 * pointers unless stated otherwise; every call only enqueues work on `stream`
 * (a cudaStream_t passed as void*) and returns without synchronising.  The library
 * never allocates device memory in these calls: outputs and workspace are the caller's.
 */
#ifndef TPA_B200_H_
#define TPA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TPA_B200_ABI_VERSION 2

/* Status codes.  0 = success; negative = the call did nothing. */
enum {
  TPA_OK = 0,
  TPA_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, wrong struct_size            */
  TPA_ERR_UNSUPPORTED = -2,  /* shape/dtype outside what any kernel here handles               */
  TPA_ERR_WORKSPACE = -3,    /* workspace missing or smaller than tpa_fwd_workspace_bytes()    */
  TPA_ERR_CUDA = -4,         /* a CUDA runtime call failed (see tpa_last_cuda_error)           */
  TPA_ERR_KERNEL_FORCED = -5,/* args->kernel forces a kernel that cannot run this shape        */
  TPA_ERR_DEVICE_TIMEOUT = -6,/* a bounded device-side wait ran out (read via tpa_read_status) */
  TPA_ERR_STATIC_SCRATCH = -7 /* tpa_fwd_static_scratch: the problem needs more scratch than
                                 TPA_STATIC_SCRATCH_BYTES                                       */
};

enum { TPA_DTYPE_F32 = 0, TPA_DTYPE_BF16 = 1 };

/* Which kernel runs.  AUTO and SM100 pick the STAGED tensor-core variant when the shape allows
 * (bf16, dk = dv in {64,128}, any lengths, heads % 8 == 0, 16-byte aligned operands; with
 * segment ids lk % 4 == 0),
 * else SIMT.  STAGED rebuilds every tile once into the workspace with a staging kernel and then
 * runs the attention kernel on those tiles; FUSED rebuilds Q/K/V from the factors inside the
 * attention kernel (slower, but needs no scratch beyond the 256-byte status block and, with
 * segment ids or key splits, a few KB). */
enum {
  TPA_KERNEL_AUTO = 0,
  TPA_KERNEL_SIMT = 1,
  TPA_KERNEL_SM100 = 2,
  TPA_KERNEL_SM100_FUSED = 3,
  TPA_KERNEL_SM100_STAGED = 4,
  TPA_KERNEL_DECODE = 5 /* at most 8 query rows against >= 256 keys, bf16, heads <= 64 (a multiple
                           of 8), head dims <= 128 (multiples of 16), 16-byte aligned factors:
                           K and V are never materialised (rank-space logits, tpa/tpa.py:333-359);
                           AUTO picks it for up to six query rows, where it is measured
                           faster than the staged path                                       */
};

/* flags */
enum {
  TPA_FLAG_CAUSAL = 1,      /* keep key j for query i iff i + q_offset >= j + k_offset
                               (tpa/tpa.py:376-379 with both offsets 0)                        */
  TPA_FLAG_STATE_LOAD = 2,  /* start from the partial result in state_o / state_lse
                               (the carry of tpa/ring_tpa.py:69-71) instead of (0, -inf)       */
  TPA_FLAG_STATE_STORE = 4, /* write the merged partial back to state_o / state_lse
                               (tpa/ring_tpa.py:82-91) instead of the final o / lse            */
  TPA_FLAG_REUSE_STAGED_Q = 8,/* the workspace is the one the previous call used, with the same
                               q operand, sm_scale, ranks, heads, batch and lq (the ring scan keeps
                               q fixed, tpa/ring_tpa.py:73-79): the STAGED variant then skips
                               re-staging Q.  The staged Q tiles sit right behind the status block
                               whatever the keys are, so k, v and lk may differ from the previous
                               call's.  Ignored by the other kernels.                          */
  TPA_FLAG_REUSE_STAGED_KV = 32,/* likewise for the K and V tiles: same k, v operands, ranks, lk and
                               lq as the previous call on this workspace (two query chunks of
                               one rank against the same gathered keys); STAGED only          */
  TPA_FLAG_CAUSAL_PER_PART = 16 /* with kv_parts > 1: the causal (and window) comparison uses the
                               key's index inside its own part, not in the whole key array.
                               This is what the reference's ring computes with causal=True: no
                               shard offset reaches its block kernel, so every visiting shard
                               is masked on shard-local indices (tpa/ring_tpa.py:73-79,
                               tpa/tpa.py:376-379).  One call with the N shards as N parts then
                               equals the N steps of the scan plus their merges.               */
};

/* One factor operand: `ptr[b*stride[0] + l*stride[1] + r*stride[2] + c]`, c contiguous.
 * The reference passes the concatenated arrays q[b,l,r,h+d]; A = base, B = base + h
 * (tpa/tpa.py:477-479), both with stride {l*r*(h+d), r*(h+d), h+d} — zero copy. */
typedef struct TpaFactor {
  const void* ptr;
  int64_t stride[3]; /* elements: batch, row (token), rank */
} TpaFactor;

/* Replaces the operand list of the custom call at tpa/tpa.py:492-543 (plus the batch
 * vmap of tpa/tpa.py:144-163).  Zero-initialise, then fill. */
typedef struct TpaFwdArgs {
  uint32_t struct_size; /* = sizeof(TpaFwdArgs) */
  int32_t dtype;        /* TPA_DTYPE_*: element type of the factors and of `o`            */
  int32_t batch, lq, lk;
  int32_t rank_q, rank_k; /* rank of v must equal rank of k (tpa/tpa.py:474-475)           */
  int32_t heads, dk, dv;
  TpaFactor qa, qb;     /* [batch, lq, rank_q, heads], [batch, lq, rank_q, dk]             */
  TpaFactor ka, kb;     /* [batch, lk, rank_k, heads], [batch, lk, rank_k, dk]             */
  TpaFactor va, vb;     /* [batch, lk, rank_k, heads], [batch, lk, rank_k, dv]             */
  const int32_t* q_segment_ids;  /* [batch, lq] or NULL                                    */
  const int32_t* kv_segment_ids; /* [batch, lk] or NULL; both or neither (tpa/tpa.py:369-371) */
  int64_t q_segment_batch_stride;  /* elements; 0 = one row shared by the batch            */
  int64_t kv_segment_batch_stride;
  void* o;              /* [batch, lq, heads, dv] contiguous, dtype; rows with no visible
                           key are NaN (tpa/tpa.py:439).  Unused with STATE_STORE.         */
  float* lse;           /* [batch, lq, heads] fp32 natural-log LSE of the scaled masked
                           logits (tpa/tpa.py:443), -inf for empty rows; may be NULL       */
  float* state_o;       /* [batch, lq, heads, dv] fp32 normalised partial output           */
  float* state_lse;     /* [batch, lq, heads] fp32 partial LSE                             */
  float sm_scale;       /* tpa/tpa.py:367                                                  */
  uint32_t flags;       /* TPA_FLAG_*                                                      */
  int64_t q_offset, k_offset; /* global positions of local row 0 (causal comparison only)  */
  int32_t kernel;       /* TPA_KERNEL_*                                                    */
  int32_t reserved;
  /* ---- everything below may stay zero: the call is then exactly the reference's ---------- */
  int32_t kv_parts;     /* 0 or 1: k and v are one array.  P > 1: the lk keys are P parts of
                           lk / P rows each (the visiting shards of a ring, gathered in one
                           buffer, tpa/ring_tpa.py:96): part p of a factor starts
                           p * {k,v}_part_stride elements after part 0, key index = p * lk/P +
                           row.  Staged tensor-core variant and the generic kernel only; lk / P
                           must be a multiple of 128.                                        */
  int32_t window;       /* > 0: sliding-window attention, planned in the reference
                           (tpa/ring_tpa.py:5-7, tpa/tpa.py:31-32) but not written there.  With
                           diff = (i + q_offset) - (j + k_offset): key j is kept for query i iff
                           diff < window * dilation, diff % dilation == 0 and (causal: diff >= 0;
                           not causal: -diff < window * dilation), i.e. `window` keys at stride
                           `dilation` behind the query (and as many ahead when not causal).   */
  int32_t dilation;     /* 0 or 1: none; D > 1: only every D-th position (see window); may be
                           used without a window                                             */
  int32_t rope_len;     /* rows of rope_cos / rope_sin                                       */
  int64_t k_part_stride, v_part_stride;   /* elements, kv_parts > 1                          */
  int64_t kv_segment_part_stride;         /* elements of kv_segment_ids between parts        */
  /* Rotary position embedding of the dim factors of q and k (the step before this path in a
   * TPA model; the reference has none, its README links the paper only).  rope_cos / rope_sin:
   * fp32 [rope_len, dk / 2].  Pairs of adjacent columns (2c, 2c + 1) of every rank row of B_Q
   * at query row i are rotated by the angle whose cos / sin are in row i + rope_q_offset,
   * column c; B_K at key index j likewise with j + rope_k_offset:
   * (x, y) -> (x cos - y sin, x sin + y cos).  Rotation commutes with the rank sum, so it is
   * applied once to each rebuilt Q and K row.  NULL: no rotation.  Forward only.            */
  const float* rope_cos;
  const float* rope_sin;
  int64_t rope_q_offset, rope_k_offset;
} TpaFwdArgs;

typedef struct TpaKernelInfo {
  int32_t kernel;       /* TPA_KERNEL_SIMT, TPA_KERNEL_SM100_FUSED, TPA_KERNEL_SM100_STAGED or
                           TPA_KERNEL_DECODE                                                */
  int32_t block_q, block_kv; /* tile sizes the kernel will use                             */
  int32_t threads;      /* threads per CTA                                                 */
  int32_t grid[3];
  int32_t smem_bytes;   /* dynamic shared memory per CTA                                   */
  int32_t launches;     /* kernel launches one tpa_fwd call makes for these arguments      */
} TpaKernelInfo;

/* Forward pass.  Replaces pl.pallas_call(_fwd_kernel ...) at tpa/tpa.py:492-543 for the
 * whole batch.  `workspace` must hold tpa_fwd_workspace_bytes(args) bytes (may be NULL
 * when that is 0) and be 256-byte aligned; its first 256 bytes are reserved for a device status
 * block, of which the first 16 are used (see tpa_read_status). */
int tpa_fwd(const TpaFwdArgs* args, void* workspace, size_t workspace_bytes, void* stream);

/* Same forward pass for callers that cannot allocate the workspace: an XLA custom-call
 * handler (device memory is owned, and mostly pre-reserved, by XLA's allocator) or an embedder
 * with a fixed device-memory budget.  No counterpart in the reference.  Runs the STAGED
 * tensor-core variant (bf16, head_dim 64/128; other shapes return TPA_ERR_KERNEL_FORCED) with
 * its scratch in a static device array inside the library: what tpa_fwd_workspace_bytes reports
 * for TPA_KERNEL_SM100_STAGED (about 256 + (lq + 2*lk) * batch * heads * dk * 2 bytes, lengths
 * rounded up to 128) must fit TPA_STATIC_SCRATCH_BYTES, else
 * TPA_ERR_STATIC_SCRATCH and nothing is launched.  Allocates nothing.  The first call on each
 * device (with that device current) looks the array's address up once: make it at start-up,
 * before any stream capture begins.  Calls on one GPU share the array: do not let two of
 * them overlap.  Every GPU that loads the library holds TPA_STATIC_SCRATCH_BYTES until exit. */
#define TPA_STATIC_SCRATCH_BYTES (64u << 20)
int tpa_fwd_static_scratch(const TpaFwdArgs* args, void* stream);

/* tpa_read_status for tpa_fwd_static_scratch (no counterpart in the reference): the status block
 * of that entry point is the head of the library's static array, whose address no caller holds.
 * Synchronises `stream`, reads the block of the current device and returns TPA_OK or
 * TPA_ERR_DEVICE_TIMEOUT; `detail` as for tpa_read_status.  Allocates nothing. */
int tpa_read_status_static_scratch(void* stream, uint32_t detail[4]);

/* Backward pass: gradients of the forward result with respect to the three concatenated
 * factor arrays.  Replaces _tpa_bwd / _bwd (tpa/tpa.py:168-217, 823-962): _precompute_delta
 * (tpa/tpa.py:965-995), the custom call pl.pallas_call(_bwd_kernel ...) at tpa/tpa.py:882-956
 * and the concatenation of the factor gradients (tpa/tpa.py:958-960), for the whole batch.
 *
 * `fwd` holds the forward call's operands unchanged; fwd.o and fwd.lse are the forward's
 * RESULTS and are read here (the residuals of tpa/tpa.py:165); of fwd.flags only
 * TPA_FLAG_CAUSAL is allowed; fwd.kernel is TPA_KERNEL_AUTO, TPA_KERNEL_SIMT (fp32 math, any
 * shape the forward accepts) or TPA_KERNEL_SM100 (tcgen05 pair passes; same shapes as the
 * tensor-core forward, plus d_o 16-byte aligned; AUTO picks them whenever they apply).
 * A query row that saw no key (lse = -inf, o = NaN) contributes nothing, as in the reference
 * (p = 0 after tpa/tpa.py:676-677, delta by nansum).  The dim-factor gradients sum over all
 * heads. */
enum {
  TPA_BWD_ACCUMULATE_DQ = 1,  /* add to dq instead of overwriting it                        */
  TPA_BWD_ACCUMULATE_DKV = 2  /* add to dk and dv (a ring step's travelling accumulators,
                                 tpa/ring_tpa.py:115-172)                                    */
};

typedef struct TpaBwdArgs {
  uint32_t struct_size; /* = sizeof(TpaBwdArgs) */
  int32_t grad_dtype;   /* TPA_DTYPE_* of dq/dk/dv: fwd.dtype, or TPA_DTYPE_F32             */
  TpaFwdArgs fwd;
  const void* d_o;      /* [batch, lq, heads, dv] contiguous, fwd.dtype                      */
  void* dq;             /* [batch, lq, rank_q, heads + dk] contiguous, grad_dtype            */
  void* dk;             /* [batch, lk, rank_k, heads + dk]                                   */
  void* dv;             /* [batch, lk, rank_k, heads + dv]                                   */
  uint32_t bwd_flags;   /* TPA_BWD_*                                                        */
  int32_t reserved;
} TpaBwdArgs;

/* `workspace`: tpa_bwd_workspace_bytes(args) bytes, 256-byte aligned (dense fp32 dQ, dK, dV
 * of the whole batch, delta and, for the tensor-core passes, the staged bf16 Q, K, V, dO tiles).
 * Six launches (SIMT) or eight (tensor cores); enqueue-only.  The first 256 bytes are reserved for
 * the device status block that tpa_read_status reads (16 bytes used). */
int tpa_bwd(const TpaBwdArgs* args, void* workspace, size_t workspace_bytes, void* stream);
size_t tpa_bwd_workspace_bytes(const TpaBwdArgs* args);

/* Bytes of scratch tpa_fwd needs for these arguments (0 is possible). */
size_t tpa_fwd_workspace_bytes(const TpaFwdArgs* args);

/* The least scratch tpa_fwd accepts for these arguments (no counterpart in the reference, whose Pallas
 * call owns its scratch).  The staged tensor-core kernel keeps the rebuilt Q, K, V tiles of every head
 * in the workspace (c3 on one GPU: 3.2 GB), which is the fast layout; given anything from this many
 * bytes upwards it instead works through the heads in groups (multiples of 8) whose tiles fit, one
 * group's staging and attention launches after the other's, at the price of a tail of idle SMs per
 * group and a strided copy of o and lse.  Same results.  Equal to tpa_fwd_workspace_bytes() where
 * grouping does not apply (other kernels, up to 8 heads, carried state, kept tiles). */
size_t tpa_fwd_workspace_bytes_min(const TpaFwdArgs* args);

/* Which kernel, tiles and grid tpa_fwd would use; TPA_OK or the error tpa_fwd would return. */
int tpa_query_kernel(const TpaFwdArgs* args, TpaKernelInfo* info);

/* Synchronises `stream`, reads the status block at the start of `workspace` and returns
 * TPA_OK or TPA_ERR_DEVICE_TIMEOUT.  `detail` (host, may be NULL) receives the raw
 * device words {flag, where, block, spins}. */
int tpa_read_status(const void* workspace, void* stream, uint32_t detail[4]);

/* Self-test of the bounded device-side waits (no counterpart in the reference): launches one warp
 * that waits on a barrier nothing ever signals, with a budget of `budget_cycles` SM cycles (at most
 * 2^28) instead of the kernels' 2^28.  The wait runs out, the kernel ends normally and the status
 * block at the head of `workspace` (>= 256 bytes, 256-byte aligned) then reads
 * {1, 0x7e57, block, spins}: tpa_read_status returns TPA_ERR_DEVICE_TIMEOUT.  Nothing faults or
 * stays waiting; the context remains usable. */
int tpa_selftest_wait_timeout(void* workspace, size_t workspace_bytes, int64_t budget_cycles, void* stream);

/* Human-readable text for a status code (static storage). */
const char* tpa_status_string(int status);

/* Text of the last CUDA error this library saw on the calling thread (static storage). */
const char* tpa_last_cuda_error(void);

/* Number of kernel launches this library has issued in this process. */
uint64_t tpa_launch_count(void);

int tpa_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TPA_B200_H_ */
