"""Tensor Product Attention: the reference's call signatures over libtpa_b200.so.

Mirrors tpa/tpa.py of jondeaton/tensor-product-attention-jax:

    BlockSizes   tpa/tpa.py:35-70
    tpa()        tpa/tpa.py:73-121    (differentiable: torch autograd plays custom_vjp)
    _tpa_fwd()   tpa/tpa.py:124-165
    _tpa_bwd()   tpa/tpa.py:168-214
    _fwd()       tpa/tpa.py:446-543   (the forward custom call this library replaces)
    _bwd()       tpa/tpa.py:823-962   (the backward custom call and its delta pre-pass)

Arrays are torch tensors.  CUDA tensors are used in place (zero copy: the head factor
A = x[..., :h] and the dim factor B = x[..., h:] are passed as pointer + strides).  Host
arrays (numpy arrays or CPU torch tensors) are copied to the current CUDA device, run
there, and the result is copied back — there is no CPU implementation.
"""

from __future__ import annotations

import ctypes as C
import dataclasses

import numpy as np
import torch

from . import _capi

__all__ = ["BlockSizes", "tpa", "fwd_device", "bwd_device"]


@dataclasses.dataclass
class BlockSizes:
    """Tile-size request, kept for signature compatibility (tpa/tpa.py:35-70).

    The divisibility rule of the reference launcher is enforced with these values
    (tpa/tpa.py:485-490); the kernels choose their own tiles.
    """

    block_q: int = 128
    block_kv: int = 128
    block_h: int = 4


_DTYPES = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}
_workspaces: dict = {}
# what the Q tiles staged in a workspace were made from: key as _workspaces, value = signature
_staged_q: dict = {}


def _workspace(device, nbytes, kind=None):
    """Per-(device, stream) scratch buffer, grown on demand and reused across calls.  The
    backward keeps its own (`kind="bwd"`) so that it never overwrites staged forward tiles."""
    if nbytes == 0:
        return None
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    if kind is not None:
        key += (kind,)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def device_status(device=None):
    """Synchronise and read the status block of the last tensor-core launch on the current
    stream of `device`: (status code, [flag, where, block, spins])."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    stream = torch.cuda.current_stream(device).cuda_stream
    ws = _workspaces.get((device, stream))
    detail = (C.c_uint32 * 4)()
    st = _capi.lib.tpa_read_status(ws.data_ptr() if ws is not None else None, C.c_void_p(stream), C.byref(detail))
    return st, list(detail)


def device_status_bwd(device=None):
    """device_status for the backward's scratch (it keeps its own buffer)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    stream = torch.cuda.current_stream(device).cuda_stream
    ws = _workspaces.get((device, stream, "bwd"))
    detail = (C.c_uint32 * 4)()
    st = _capi.lib.tpa_read_status(ws.data_ptr() if ws is not None else None, C.c_void_p(stream), C.byref(detail))
    return st, list(detail)


def _factor(x, col0):
    f = _capi.TpaFactor()
    f.ptr = x.data_ptr() + col0 * x.element_size()
    f.stride[0], f.stride[1], f.stride[2] = x.stride(0), x.stride(1), x.stride(2)
    return f


def _check_shapes(q, k, v, num_heads, kv_parts=1):
    """(b, lq, lk, rank_q, rank_k, dk, dv).  With `kv_parts` > 1, k and v are
    [parts, b, lk / parts, r, h + d] and lk counts the keys of all parts."""
    if kv_parts > 1:
        if k.ndim != 5 or v.ndim != 5 or k.shape[0] != kv_parts or v.shape[0] != kv_parts:
            raise AssertionError(f"expected [{kv_parts}, b, l, r, h+d] key / value parts, got {k.shape}, {v.shape}")
        kshape = (k.shape[1], kv_parts * k.shape[2]) + tuple(k.shape[3:])
        vshape = (v.shape[1], kv_parts * v.shape[2]) + tuple(v.shape[3:])
    else:
        kshape, vshape = tuple(k.shape), tuple(v.shape)
    if q.ndim != 4 or len(kshape) != 4 or len(vshape) != 4:
        raise AssertionError(f"expected [b, l, r, h+d] factors, got {q.shape}, {k.shape}, {v.shape}")
    b, lq, rank_q, h_dk = q.shape
    _, lk, rank_k, h_dv = vshape
    # tpa/tpa.py:474-475: rank is read from v and k must match it
    if kshape != (b, lk, rank_k, h_dk):
        raise AssertionError(tuple(k.shape))
    if vshape[0] != b:
        raise AssertionError(tuple(v.shape))
    dk, dv = h_dk - num_heads, h_dv - num_heads
    if dk <= 0 or dv <= 0:
        raise AssertionError((h_dk, h_dv, num_heads))
    return b, lq, lk, rank_q, rank_k, dk, dv


def _fill_operands(a, q, k, v, num_heads, q_segment_ids, kv_segment_ids, kv_parts=1):
    """Shapes, dtype, factor pointers and segment ids of a TpaFwdArgs; returns tensors to keep alive.

    `kv_parts` > 1: k and v are [parts, b, lk / parts, r, h + d] (the shards of a ring gathered in
    one buffer) and the key ids [parts, b, lk / parts]."""
    b, lq, lk, rank_q, rank_k, dk, dv = _check_shapes(q, k, v, num_heads, kv_parts)
    a.struct_size = C.sizeof(_capi.TpaFwdArgs)
    a.dtype = _DTYPES[q.dtype]
    a.batch, a.lq, a.lk = b, lq, lk
    a.rank_q, a.rank_k = rank_q, rank_k
    a.heads, a.dk, a.dv = num_heads, dk, dv
    a.qa, a.qb = _factor(q, 0), _factor(q, num_heads)
    if kv_parts > 1:
        a.ka, a.kb = _factor(k[0], 0), _factor(k[0], num_heads)
        a.va, a.vb = _factor(v[0], 0), _factor(v[0], num_heads)
        a.kv_parts = kv_parts
        a.k_part_stride, a.v_part_stride = k.stride(0), v.stride(0)
    else:
        a.ka, a.kb = _factor(k, 0), _factor(k, num_heads)
        a.va, a.vb = _factor(v, 0), _factor(v, num_heads)
    keep = []
    if q_segment_ids is not None:
        qs = q_segment_ids.to(device=q.device, dtype=torch.int32)
        ks = kv_segment_ids.to(device=q.device, dtype=torch.int32)
        # a 1-D id row is shared by the whole batch (vmap in_axes None, tpa/tpa.py:155-161)
        qs = qs.contiguous()
        ks = ks.contiguous()
        if kv_parts > 1:
            if tuple(ks.shape) != (kv_parts, b, lk // kv_parts) or qs.shape[-1] != lq:
                raise AssertionError((tuple(qs.shape), tuple(ks.shape)))
            a.kv_segment_part_stride = ks.stride(0)
            a.kv_segment_batch_stride = ks.stride(1)
        else:
            if qs.shape[-1] != lq or ks.shape[-1] != lk:
                raise AssertionError((tuple(qs.shape), tuple(ks.shape)))
            a.kv_segment_batch_stride = lk if ks.ndim == 2 else 0
        a.q_segment_ids, a.kv_segment_ids = qs.data_ptr(), ks.data_ptr()
        a.q_segment_batch_stride = lq if qs.ndim == 2 else 0
        keep += [qs, ks]
    return keep


def _check_operands(q, k, v, q_segment_ids, kv_segment_ids):
    if not q.is_cuda:
        raise RuntimeError("tpa_b200 needs a CUDA device: there is no CPU implementation")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError(f"dtype {q.dtype}/{k.dtype}/{v.dtype}: float32 or bfloat16 factors only")
    for x in (q, k, v):
        if x.stride(-1) != 1:
            raise ValueError("the last (h+d) axis of the factors must be contiguous")
    if (q_segment_ids is None) != (kv_segment_ids is None):
        raise AssertionError("segment ids must be given for both sides or neither")  # tpa/tpa.py:369-371


def fwd_device(
    q,
    k,
    v,
    num_heads,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale=1.0,
    causal=False,
    *,
    q_offset=0,
    k_offset=0,
    state=None,
    load_state=False,
    store_state=False,
    out=None,
    lse=None,
    want_lse=True,
    kernel="auto",
    reuse_staged_q=False,
    reuse_staged_kv=False,
    kv_parts=1,
    per_part=False,
    window=0,
    dilation=1,
    rope=None,
    rope_q_offset=0,
    rope_k_offset=0,
    workspace_limit=None,
):
    """One tpa_fwd call on CUDA tensors; returns (o, lse_fp32).

    `workspace_limit` (bytes): give the call at most this much scratch.  The staged tensor-core
    kernel then works through the heads in groups whose tiles fit (tpa_fwd_workspace_bytes_min is
    the least it accepts); same result, some speed for memory.

    Beyond the reference (all off by default): `kv_parts` > 1 takes k, v as
    [parts, b, lk / parts, r, h + d] and key ids as [parts, b, lk / parts] -- the shards of a ring
    gathered in one buffer -- and `per_part` compares positions on part-local key indices, which
    makes one call equal the reference's whole ring scan (tpa/ring_tpa.py:60-112); `window` /
    `dilation` are the sliding-window and dilated masks the reference plans
    (tpa/ring_tpa.py:5-7); `rope=(cos, sin)` (fp32 [positions, dk / 2]) rotates the dim factors
    of q and k, row i by table row i + rope_q_offset (keys: + rope_k_offset).

    `reuse_staged_q=True` promises that the previous call on this stream had the same q,
    shapes and scale (ring steps): the staged variant then keeps its Q tiles.

    `state = (state_o fp32 [b,lq,h,dv], state_lse fp32 [b,lq,h])` with `load_state` /
    `store_state` is the carry of the ring scan (tpa/ring_tpa.py:69-91): a call with
    `store_state=True` writes the merged partial into `state` and returns (None, None).
    Work is enqueued on the current stream of q's device.
    """
    _check_operands(q, k, v, q_segment_ids, kv_segment_ids)
    b, lq, lk, rank_q, rank_k, dk, dv = _check_shapes(q, k, v, num_heads, kv_parts)

    a = _capi.TpaFwdArgs()
    keep = _fill_operands(a, q, k, v, num_heads, q_segment_ids, kv_segment_ids, kv_parts)
    flags = _capi.FLAG_CAUSAL if causal else 0
    if per_part:
        flags |= _capi.FLAG_CAUSAL_PER_PART
    a.window, a.dilation = int(window), int(dilation)
    if rope is not None:
        cos, sin = rope
        for t in (cos, sin):
            if t.dtype != torch.float32 or not t.is_contiguous() or t.device != q.device or t.shape != cos.shape:
                raise ValueError("rope tables: two contiguous fp32 [positions, dk / 2] tensors on q's device")
        if cos.ndim != 2 or cos.shape[1] * 2 != dk:
            raise ValueError(f"rope tables must be [positions, {dk // 2}], got {tuple(cos.shape)}")
        a.rope_cos, a.rope_sin, a.rope_len = cos.data_ptr(), sin.data_ptr(), cos.shape[0]
        a.rope_q_offset, a.rope_k_offset = int(rope_q_offset), int(rope_k_offset)
        keep += [cos, sin]
    if load_state:
        flags |= _capi.FLAG_STATE_LOAD
    if store_state:
        flags |= _capi.FLAG_STATE_STORE
    if reuse_staged_q:
        flags |= _capi.FLAG_REUSE_STAGED_Q
    if reuse_staged_kv:
        flags |= _capi.FLAG_REUSE_STAGED_KV
    if load_state or store_state:
        so, sl = state
        assert so.dtype == torch.float32 and sl.dtype == torch.float32
        assert so.is_contiguous() and sl.is_contiguous()
        assert tuple(so.shape) == (b, lq, num_heads, dv) and tuple(sl.shape) == (b, lq, num_heads)
        a.state_o, a.state_lse = so.data_ptr(), sl.data_ptr()
    if not store_state:
        if out is None:
            out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=q.device)
        assert out.is_contiguous() and out.dtype == q.dtype
        a.o = out.data_ptr()
        if lse is None and want_lse:
            lse = torch.empty((b, lq, num_heads), dtype=torch.float32, device=q.device)
        if lse is not None:
            assert lse.is_contiguous() and lse.dtype == torch.float32
            a.lse = lse.data_ptr()
    a.sm_scale = float(sm_scale)
    a.flags = flags
    a.q_offset, a.k_offset = int(q_offset), int(k_offset)
    a.kernel = _capi.KERNELS[kernel]

    with torch.cuda.device(q.device):
        nbytes = _capi.lib.tpa_fwd_workspace_bytes(C.byref(a))
        if workspace_limit is not None and workspace_limit < nbytes:
            nbytes = max(_capi.lib.tpa_fwd_workspace_bytes_min(C.byref(a)), int(workspace_limit))
        ws = _workspace(q.device, nbytes)
        stream = torch.cuda.current_stream(q.device).cuda_stream
        # TPA_FLAG_REUSE_STAGED_Q / _KV are promises about the workspace's contents; keep them only
        # when the last call on this stream ran the staged kernel into this very buffer from the
        # same operand, shapes and scale (another call on the stream, a regrown buffer or a call
        # that another kernel took silently voids the promise).  The staged Q tiles sit at the
        # head of the workspace whatever the keys are, so they survive a change of k and v.
        info = _capi.TpaKernelInfo()
        staged = (_capi.lib.tpa_query_kernel(C.byref(a), C.byref(info)) == 0
                  and _capi.KERNEL_NAMES.get(info.kernel) == "sm100_staged")
        ws_ptr = ws.data_ptr() if ws is not None else 0
        rope_sig = None if rope is None else (rope[0].data_ptr(), rope[1].data_ptr(), rope_q_offset, rope_k_offset)
        sig_q = (q.data_ptr(), q._version, tuple(q.shape), tuple(q.stride()), q.dtype, num_heads, float(sm_scale), rank_k,
                 ws_ptr, rope_sig) if staged else None
        sig_kv = (k.data_ptr(), v.data_ptr(), k._version, v._version, tuple(k.shape), tuple(v.shape), tuple(k.stride()),
                  tuple(v.stride()), q.dtype, num_heads, lq, kv_parts, bool(per_part), ws_ptr, rope_sig) if staged else None
        key = (q.device, stream)
        last_q, last_kv = _staged_q.get(key, (None, None))
        if reuse_staged_q and (sig_q is None or last_q != sig_q):
            a.flags &= ~_capi.FLAG_REUSE_STAGED_Q
        if reuse_staged_kv and (sig_kv is None or last_kv != sig_kv):
            a.flags &= ~_capi.FLAG_REUSE_STAGED_KV
        _staged_q[key] = (sig_q, sig_kv)
        st = _capi.lib.tpa_fwd(
            C.byref(a), ws.data_ptr() if ws is not None else None, nbytes, C.c_void_p(stream)
        )
    _capi.check(st)
    del keep
    if store_state:
        return None, None
    return out, lse


def bwd_device(
    q,
    k,
    v,
    num_heads,
    q_segment_ids,
    kv_segment_ids,
    sm_scale,
    causal,
    o,
    lse,
    do,
    *,
    q_offset=0,
    k_offset=0,
    grad_dtype=None,
    out=None,
    accumulate_dq=False,
    accumulate_dkv=False,
    kernel="auto",
):
    """One tpa_bwd call on CUDA tensors; returns (dq, dk, dv) shaped like q, k, v.

    `kernel`: "auto" (tensor cores when the shape allows, as for the forward), "simt" or "sm100".

    `o` and `lse` (fp32) are the forward's results, `do[b, lq, h, dv]` the incoming gradient.
    `grad_dtype` is q's dtype (default) or torch.float32; `out = (dq, dk, dv)` supplies the
    gradient buffers, which `accumulate_dq` / `accumulate_dkv` add to instead of overwriting
    (the travelling dk, dv of a ring backward, tpa/ring_tpa.py:115-172).
    """
    _check_operands(q, k, v, q_segment_ids, kv_segment_ids)
    b, lq, lk, rank_q, rank_k, dk, dv = _check_shapes(q, k, v, num_heads)
    grad_dtype = q.dtype if grad_dtype is None else grad_dtype
    if grad_dtype not in (q.dtype, torch.float32):
        raise NotImplementedError(f"gradient dtype {grad_dtype} for {q.dtype} factors")
    a = _capi.TpaBwdArgs()
    a.struct_size = C.sizeof(_capi.TpaBwdArgs)
    a.grad_dtype = _DTYPES[grad_dtype]
    keep = _fill_operands(a.fwd, q, k, v, num_heads, q_segment_ids, kv_segment_ids)
    o, do = o.contiguous(), do.contiguous()
    lse = lse.to(torch.float32).contiguous()
    if tuple(o.shape) != (b, lq, num_heads, dv) or tuple(do.shape) != tuple(o.shape):
        raise AssertionError((tuple(o.shape), tuple(do.shape)))
    if tuple(lse.shape) != (b, lq, num_heads) or o.dtype != q.dtype or do.dtype != q.dtype:
        raise AssertionError((tuple(lse.shape), o.dtype, do.dtype))
    a.fwd.o, a.fwd.lse, a.d_o = o.data_ptr(), lse.data_ptr(), do.data_ptr()
    a.fwd.sm_scale = float(sm_scale)
    a.fwd.flags = _capi.FLAG_CAUSAL if causal else 0
    a.fwd.q_offset, a.fwd.k_offset = int(q_offset), int(k_offset)
    a.fwd.kernel = _capi.KERNELS[kernel]
    if out is None:
        if accumulate_dq or accumulate_dkv:
            raise ValueError("accumulating needs the buffers to add to (out=(dq, dk, dv))")
        out = tuple(torch.empty(x.shape, dtype=grad_dtype, device=q.device) for x in (q, k, v))
    for g, x in zip(out, (q, k, v)):
        assert g.is_contiguous() and g.dtype == grad_dtype and tuple(g.shape) == tuple(x.shape)
    a.dq, a.dk, a.dv = (g.data_ptr() for g in out)
    a.bwd_flags = (_capi.BWD_ACCUMULATE_DQ if accumulate_dq else 0) | (
        _capi.BWD_ACCUMULATE_DKV if accumulate_dkv else 0
    )
    with torch.cuda.device(q.device):
        nbytes = _capi.lib.tpa_bwd_workspace_bytes(C.byref(a))
        ws = _workspace(q.device, nbytes, "bwd")
        stream = torch.cuda.current_stream(q.device).cuda_stream
        st = _capi.lib.tpa_bwd(C.byref(a), ws.data_ptr() if ws is not None else None, nbytes, C.c_void_p(stream))
    _capi.check(st)
    del keep
    return out


def query_kernel(q, k, v, num_heads, kernel="auto", causal=False, segments=False):
    """Which kernel / tiles / grid a call with these operands would use (tpa_query_kernel)."""
    b, lq, lk, rank_q, rank_k, dk, dv = _check_shapes(q, k, v, num_heads)
    a = _capi.TpaFwdArgs()
    a.struct_size = C.sizeof(_capi.TpaFwdArgs)
    a.dtype = _DTYPES[q.dtype]
    a.batch, a.lq, a.lk, a.rank_q, a.rank_k = b, lq, lk, rank_q, rank_k
    a.heads, a.dk, a.dv = num_heads, dk, dv
    a.qa, a.qb = _factor(q, 0), _factor(q, num_heads)
    a.ka, a.kb = _factor(k, 0), _factor(k, num_heads)
    a.va, a.vb = _factor(v, 0), _factor(v, num_heads)
    a.o = 4096  # any aligned non-null value: nothing is dereferenced by the query
    if segments:
        a.q_segment_ids = a.kv_segment_ids = 4096
    a.flags = _capi.FLAG_CAUSAL if causal else 0
    a.kernel = _capi.KERNELS[kernel]
    info = _capi.TpaKernelInfo()
    _capi.check(_capi.lib.tpa_query_kernel(C.byref(a), C.byref(info)))
    return {
        "kernel": _capi.KERNEL_NAMES[info.kernel],
        "block_q": info.block_q,
        "block_kv": info.block_kv,
        "threads": info.threads,
        "grid": tuple(info.grid),
        "smem_bytes": info.smem_bytes,
        "launches": info.launches,
    }


def _to_device(x, device):
    """Host array -> CUDA tensor (through pinned memory when the source is pinned)."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    return x.to(device, non_blocking=x.is_pinned() if not x.is_cuda else False)


def _tpa_fwd_checks(q, k, block_sizes):
    """The divisibility rule of the reference launcher (tpa/tpa.py:485-490)."""
    if block_sizes is None:
        block_sizes = BlockSizes()
    lq, lk = q.shape[1], k.shape[1]
    block_q = min(block_sizes.block_q, lq)
    block_kv = min(block_sizes.block_kv, lk)
    if lq % block_q != 0:
        raise AssertionError((lq, block_q))
    if lk % block_kv != 0:
        raise AssertionError((lk, block_kv))


def _tpa_fwd(
    q,
    k,
    v,
    num_heads,
    q_segment_ids,
    kv_segment_ids,
    sm_scale,
    causal,
    block_sizes,
    nomat,
    debug,
    interpret,
):
    """Batch forward returning (o, residuals) as tpa/tpa.py:124-165 does.

    residuals = (q, k, v, q_segment_ids, kv_segment_ids, o, l) with l[b, lq, h] the LSE
    in q's dtype.  `nomat`, `debug` and `interpret` are accepted and have no effect: the
    non-materialising strategy (tpa/tpa.py:333-359) gives the same result by construction
    and the other two are Pallas debugging switches.
    """
    del nomat, debug, interpret
    _tpa_fwd_checks(q, k, block_sizes)
    o, l = fwd_device(q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal)
    l = l.to(q.dtype)
    return o, (q, k, v, q_segment_ids, kv_segment_ids, o, l)


def _tpa_bwd(num_heads, sm_scale, causal, block_sizes, nomat, debug, interpret, residuals, do):
    """Backward of the batch forward, same arguments and result as tpa/tpa.py:168-214:
    (dq, dk, dv, None, None) for residuals = (q, k, v, q_segment_ids, kv_segment_ids, o, l)."""
    del block_sizes, nomat, debug, interpret
    q, k, v, q_segment_ids, kv_segment_ids, o, l = residuals
    dq, dk, dv = bwd_device(q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal, o, l, do)
    return dq, dk, dv, None, None


def _bwd(q, k, v, q_segment_ids, kv_segment_ids, o, l, do, num_heads, sm_scale, causal,
         block_sizes=None, nomat=False, debug=False, interpret=False):
    """Per-batch-element backward (dq, dk, dv) as tpa/tpa.py:823-962."""
    dq, dk, dv, _, _ = _tpa_bwd(
        num_heads, sm_scale, causal, block_sizes, nomat, debug, interpret,
        (q[None], k[None], v[None],
         None if q_segment_ids is None else q_segment_ids[None],
         None if kv_segment_ids is None else kv_segment_ids[None], o[None], l[None]),
        do[None],
    )
    return dq[0], dk[0], dv[0]


class _TpaFunction(torch.autograd.Function):
    """What jax.custom_vjp + tpa.defvjp(_tpa_fwd, _tpa_bwd) is in the reference (tpa/tpa.py:73,217):
    the forward keeps (o, fp32 lse) as residuals, the backward is tpa_bwd."""

    @staticmethod
    def forward(ctx, q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal):
        o, lse = fwd_device(q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.segments = (q_segment_ids, kv_segment_ids)
        ctx.meta = (num_heads, sm_scale, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        num_heads, sm_scale, causal = ctx.meta
        dq, dk, dv = bwd_device(q, k, v, num_heads, *ctx.segments, sm_scale, causal, o, lse, do)
        return dq, dk, dv, None, None, None, None, None


_copy_streams: dict = {}
_HOST_CHUNKS = 4  # chunks of the host-array path (batch elements, or query-row blocks of one); eight measured no better


def _tpa_host_pipelined(q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal, out):
    """Host arrays in, host array out, with the copies overlapped with the kernels.

    K, V (and the ids) go up first, the query rows follow in chunks on a copy stream; each chunk is
    one tpa_fwd call (the K / V tiles staged by the first call are kept) and its rows of the
    result go down on a second copy stream while the next chunk computes.  Copies are
    asynchronous where the host arrays are pinned.  Returns a CPU tensor (`out` if given)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    as_t = lambda x: torch.from_numpy(x) if isinstance(x, np.ndarray) else x  # noqa: E731
    q, k, v = as_t(q), as_t(k), as_t(v)
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError(f"dtype {q.dtype}/{k.dtype}/{v.dtype}: float32 or bfloat16 factors only")
    b, lq = q.shape[:2]
    dv = v.shape[-1] - num_heads
    if out is None:
        out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype)
    if tuple(out.shape) != (b, lq, num_heads, dv) or out.dtype != q.dtype or out.is_cuda:
        raise ValueError(f"out must be a CPU tensor of shape {(b, lq, num_heads, dv)} and dtype {q.dtype}")
    # Chunks: whole batch elements when there are enough of them (their K / V go up chunk by chunk
    # too), else blocks of query rows of the one batch element (K / V tiles staged once, kept).
    n = _HOST_CHUNKS
    nb_ = max([m for m in range(1, n + 1) if b % m == 0])  # batch chunks: the largest divisor of b up to n
    if nb_ > 1:
        n = nb_
        plan = [(slice(c * (b // n), (c + 1) * (b // n)), slice(0, lq)) for c in range(n)]
        by_batch = True
    elif b == 1 and lq >= n * 1024 and lq % (n * 256) == 0:
        rows = lq // n
        # for a causal call the last rows cost the most: they go first, so that the shortest
        # chunk is the one whose way down is not hidden behind a next one
        order = range(n - 1, -1, -1) if causal else range(n)
        plan = [(slice(0, 1), slice(c * rows, (c + 1) * rows)) for c in order]
        by_batch = False
    else:
        plan = [(slice(0, b), slice(0, lq))]
        by_batch = True
    main = torch.cuda.current_stream(dev)
    up, down = _copy_streams.get(dev) or _copy_streams.setdefault(dev, (torch.cuda.Stream(dev), torch.cuda.Stream(dev)))
    up.wait_stream(main)
    down.wait_stream(main)
    put = lambda x: x.to(dev, non_blocking=x.is_pinned())  # noqa: E731
    ids2 = lambda x: None if x is None else as_t(x)  # noqa: E731
    hqs, hks = ids2(q_segment_ids), ids2(kv_segment_ids)
    ops, ready, keep = [], [], []
    with torch.cuda.stream(up):
        dqs = None if hqs is None else hqs.to(dev)
        dks = None if hks is None else hks.to(dev)
        if not by_batch:
            dk, dv_ = put(k), put(v)
        for bs, rs in plan:
            if by_batch:
                dk, dv_ = put(k[bs]), put(v[bs])
            dq = put(q[bs, rs])
            e = torch.cuda.Event()
            e.record(up)
            ops.append((dq, dk, dv_))
            ready.append(e)
    o_dev = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=dev)
    for i, (bs, rs) in enumerate(plan):
        main.wait_event(ready[i])
        dq, dk, dv_ = ops[i]
        # a 1-D id row is shared by the whole batch; a 2-D one is cut like its array
        cut = lambda x, r: None if x is None else (x[r] if x.ndim == 1 else x[bs, r]).contiguous()  # noqa: E731
        fwd_device(dq, dk, dv_, num_heads, cut(dqs, rs), cut(dks, slice(None)), sm_scale, causal, q_offset=rs.start,
                   out=o_dev[bs, rs], want_lse=False, reuse_staged_kv=(not by_batch) and i > 0)
        done = torch.cuda.Event()
        done.record(main)
        down.wait_event(done)
        with torch.cuda.stream(down):
            out[bs, rs].copy_(o_dev[bs, rs], non_blocking=out.is_pinned())
    for ts in ops:  # allocated on one stream, used on another: keep the allocator from recycling them early
        for t in ts:
            t.record_stream(main)
    for t in (dqs, dks):
        if t is not None:
            t.record_stream(main)
    o_dev.record_stream(down)
    down.synchronize()  # the result is a host array: complete on return
    return out


def tpa(
    q,
    k,
    v,
    num_heads: int,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale: float = 1.0,
    causal: bool = False,
    block_sizes: BlockSizes | None = None,
    nomat: bool = False,
    debug: bool = False,
    interpret: bool = False,
    *,
    out=None,
):
    """Tensor Product Attention forward; same arguments as tpa/tpa.py:73-121.

    q[b, lq, rq, h+dk], k[b, lk, rk, h+dk], v[b, lk, rk, h+dv] hold the head factor in
    [..., :h] and the dim factor in [..., h:]; Q, K, V are rank means of their outer
    products.  Returns o[b, lq, h, dv] in q's dtype; rows whose every key is masked are NaN.
    Host inputs (numpy / CPU tensors) are copied to the current CUDA device and the
    result comes back as the same kind of host array; the copies overlap with the kernels
    (see _tpa_host_pipelined), fully so when the host arrays are pinned.  `out` (keyword only,
    not in the reference) is a CPU tensor to receive the result of a host-array call, e.g. a
    pinned buffer that is reused from call to call.
    """
    host_kind = None
    if isinstance(q, np.ndarray):
        host_kind = "numpy"
    elif not q.is_cuda:
        host_kind = "torch"
    if out is not None and host_kind is None:
        raise ValueError("out= is for host-array calls; a call on CUDA tensors returns a new CUDA tensor")
    if host_kind is not None:
        if not torch.cuda.is_available():
            raise RuntimeError("tpa_b200 needs a CUDA device: there is no CPU implementation")
        _tpa_fwd_checks(q, k, block_sizes)
        o = _tpa_host_pipelined(q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal, out)
        if host_kind == "numpy":
            return o.float().numpy() if o.dtype == torch.bfloat16 else o.numpy()
        return o
    if host_kind is None and torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        _tpa_fwd_checks(q, k, block_sizes)
        return _TpaFunction.apply(q, k, v, num_heads, q_segment_ids, kv_segment_ids, sm_scale, causal)
    o, _ = _tpa_fwd(
        q,
        k,
        v,
        num_heads=num_heads,
        q_segment_ids=q_segment_ids,
        kv_segment_ids=kv_segment_ids,
        sm_scale=sm_scale,
        causal=causal,
        block_sizes=block_sizes,
        nomat=nomat,
        debug=debug,
        interpret=interpret,
    )
    return o


def _fwd(
    q,
    k,
    v,
    q_segment_ids,
    kv_segment_ids,
    num_heads,
    sm_scale,
    causal,
    block_sizes,
    nomat=False,
    debug=False,
    interpret=False,
):
    """Per-batch-element forward (o[lq,h,dv], lse[lq,h]) as tpa/tpa.py:446-543."""
    o, res = _tpa_fwd(
        q[None],
        k[None],
        v[None],
        num_heads,
        None if q_segment_ids is None else q_segment_ids[None],
        None if kv_segment_ids is None else kv_segment_ids[None],
        sm_scale,
        causal,
        block_sizes,
        nomat,
        debug,
        interpret,
    )
    return o[0], res[-1][0]
