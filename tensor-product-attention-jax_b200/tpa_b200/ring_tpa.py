"""Ring (sequence-parallel) Tensor Product Attention forward, one process per GPU.

Mirrors tpa/ring_tpa.py of jondeaton/tensor-product-attention-jax for the forward path:

    _rotate_block()            tpa/ring_tpa.py:24-38    -> grouped NCCL send/recv to rank+1
    _ring_tpa_fwd()            tpa/ring_tpa.py:41-112   -> ring_tpa() below (steps + merge)
    ring_tpa()                 tpa/ring_tpa.py:209-287
    ring_tp_self_attention()   tpa/ring_tpa.py:290-338

The reference runs under shard_map with a named mesh axis; here every rank of a
torch.distributed process group holds one contiguous length shard and `axis_name`
names (or is) that group.  Only the compact K/V factors and the key segment ids travel
(tpa/ring_tpa.py:96).  The (o, lse) merge of tpa/ring_tpa.py:82-91 is not a separate
pass: each step's kernel starts from the carried partial and writes the merged one.
The transfer for step s+1 is issued on a side stream before step s computes.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import tpa as _tpa

__all__ = ["ring_tpa", "ring_tp_self_attention", "register_axis"]

_AXES: dict = {}
_side_streams: dict = {}

MASK_MODES = ("reference_local", "global")


def register_axis(name: str, group) -> None:
    """Bind a mesh-axis name (the reference's `axis_name`) to a process group."""
    _AXES[name] = group


def _group_of(axis_name):
    if axis_name is None or isinstance(axis_name, str):
        return _AXES.get(axis_name, None)  # None = the default (world) group
    return axis_name


def _rotate_block(tensors, recv_into, group, rank, size):
    """Send `tensors` to rank+1 and receive the same shapes from rank-1 (tpa/ring_tpa.py:24-38).

    Returns the outstanding requests; the caller waits on them.
    """
    dst = dist.get_global_rank(group, (rank + 1) % size) if group is not None else (rank + 1) % size
    src = dist.get_global_rank(group, (rank - 1) % size) if group is not None else (rank - 1) % size
    ops = []
    for t, r in zip(tensors, recv_into):
        ops.append(dist.P2POp(dist.isend, t, dst, group))
        ops.append(dist.P2POp(dist.irecv, r, src, group))
    return dist.batch_isend_irecv(ops)


def _device_block(q, k, v, qs, ks, num_heads, sm_scale, causal, q_offset, k_offset, state,
                  load_state, store_state, out):
    return _tpa.fwd_device(
        q, k, v, num_heads, qs, ks, sm_scale, causal, q_offset=q_offset, k_offset=k_offset,
        state=state, load_state=load_state, store_state=store_state, out=out, want_lse=False,
        reuse_staged_q=load_state,  # q and the workspace are those of the previous step
    )[0]


def ring_tpa(
    q,
    k,
    v,
    q_segment_ids,
    kv_segment_ids,
    axis_name,
    num_heads: int,
    sm_scale: float = 1.0,
    causal: bool = False,
    impl: str = "pallas",
    debug: bool = False,
    interpret: bool = False,
    *,
    mask_mode: str = "reference_local",
    _block_fn=None,
):
    """Ring TPA forward on this rank's shard; arguments as tpa/ring_tpa.py:209-222.

    q[b, l/N, rq, h+dk], k, v, and the two int32 id arrays are this rank's contiguous
    shard; returns this rank's o[b, l/N, h, dv].  `impl="pallas"` is the reference's name
    for its kernel path and selects the CUDA kernels here; "xla" raises NotImplementedError
    and anything else ValueError, as in the reference (tpa/ring_tpa.py:237-273).

    `mask_mode` (keyword only; not in the reference) chooses what `causal=True` means:
    "reference_local" masks on shard-local indices at every step, which is what the
    reference computes because no shard offset reaches its block kernel
    (tpa/ring_tpa.py:73-79, tpa/tpa.py:376-379); "global" masks on positions in the whole
    sequence, i.e. equals tpa(causal=True) on the unsharded input.
    """
    del debug, interpret
    if impl == "xla":
        raise NotImplementedError()
    if impl not in ("pallas", "cuda"):
        raise ValueError(f"Unknown implementaiton: {impl}")
    if mask_mode not in MASK_MODES:
        raise ValueError(f"mask_mode must be one of {MASK_MODES}")
    block = _block_fn or _device_block
    if _block_fn is None and not q.is_cuda:
        raise RuntimeError("tpa_b200 needs a CUDA device: there is no CPU implementation")

    group = _group_of(axis_name)
    if dist.is_available() and dist.is_initialized():
        size, rank = dist.get_world_size(group), dist.get_rank(group)
    else:
        size, rank = 1, 0

    b, lq = q.shape[:2]
    lk = k.shape[1]
    dv = v.shape[-1] - num_heads
    # tpa/ring_tpa.py:64
    if tuple(k.shape) != (b, lk, v.shape[2], q.shape[-1]):
        raise AssertionError(tuple(k.shape))
    kseg = kv_segment_ids.to(torch.int32).contiguous()
    qseg = q_segment_ids.to(torch.int32).contiguous()

    use_streams = q.is_cuda
    out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=q.device)
    state = None
    if size > 1:
        state = (
            torch.empty((b, lq, num_heads, dv), dtype=torch.float32, device=q.device),
            torch.empty((b, lq, num_heads), dtype=torch.float32, device=q.device),
        )
    cur = [k.contiguous(), v.contiguous(), kseg]
    spare = [[torch.empty_like(t) for t in cur] for _ in range(min(2, size - 1))]

    if use_streams:
        main = torch.cuda.current_stream(q.device)
        side = _side_streams.get(q.device)
        if side is None:
            side = _side_streams[q.device] = torch.cuda.Stream(q.device)
        ready = torch.cuda.Event()
        ready.record(main)  # inputs are ready on the main stream

    # Steps that see nothing under a global causal mask are not launched, but their K/V
    # still moves on so that later ranks get it.
    def visible(src):
        return not (causal and mask_mode == "global" and src * lk > rank * lq + lq - 1)

    steps = [s for s in range(size)]
    last_compute = max(s for s in steps if visible((rank - s) % size))
    started = False
    for s in steps:
        src = (rank - s) % size
        reqs = None
        if s < size - 1:
            nxt = spare[s % 2]
            if use_streams:
                side.wait_event(ready)  # the buffer being overwritten is no longer read
                with torch.cuda.stream(side):
                    reqs = _rotate_block(cur, nxt, group, rank, size)
            else:
                reqs = _rotate_block(cur, nxt, group, rank, size)
        if visible(src):
            q_off, k_off = (rank * lq, src * lk) if mask_mode == "global" else (0, 0)
            block(
                q, cur[0], cur[1], qseg, cur[2], num_heads, sm_scale, causal, q_off, k_off, state,
                started, s != last_compute, out,
            )
            started = True
        if s < size - 1:
            if use_streams:
                ready = torch.cuda.Event()
                ready.record(main)  # step s has finished reading `cur`
                with torch.cuda.stream(side):
                    for r in reqs:
                        r.wait()
                    arrived = torch.cuda.Event()
                    arrived.record(side)
                main.wait_event(arrived)
            else:
                for r in reqs:
                    r.wait()
            cur = nxt
    return out


def ring_tp_self_attention(
    q,
    k,
    v,
    q_segment_ids,
    kv_segment_ids,
    mesh,
    pspec,
    num_heads: int,
    sm_scale: float = 1.0,
    causal: bool = False,
    impl: str = "pallas",
    debug: bool = False,
    interpret: bool = False,
    *,
    mask_mode: str = "reference_local",
    gather_output: bool = False,
    _block_fn=None,
):
    """Ring self-attention over whole-sequence arrays; arguments as tpa/ring_tpa.py:290-304.

    Every rank passes the same whole-sequence arrays; this rank's contiguous slice of the
    length axis is cut out (what shard_map does with `in_specs=pspec`,
    tpa/ring_tpa.py:317-338), ring_tpa runs on it, and the rank's slice of the output is
    returned — the addressable shard of the reference's sharded result.  With
    `gather_output=True` the slices are all-gathered into the whole [b, l, h, dv] array.

    `mesh` is a process group, a {axis name: group} dict, or None for the default group;
    `pspec[1]` names the axis the length dimension is sharded over, as in the reference.
    """
    axis = pspec[1]
    if isinstance(mesh, dict):
        group = mesh[axis]
    else:
        group = mesh if mesh is not None else _group_of(axis)
    if dist.is_available() and dist.is_initialized():
        size, rank = dist.get_world_size(group), dist.get_rank(group)
    else:
        size, rank = 1, 0
    length = q.shape[1]
    if length % size != 0:
        raise AssertionError((length, size))
    per = length // size
    sl = slice(rank * per, (rank + 1) * per)
    o = ring_tpa(
        q[:, sl], k[:, sl], v[:, sl], q_segment_ids[:, sl], kv_segment_ids[:, sl],
        axis_name=group, num_heads=num_heads, sm_scale=sm_scale, causal=causal, impl=impl,
        debug=debug, interpret=interpret, mask_mode=mask_mode, _block_fn=_block_fn,
    )
    if not gather_output or size == 1:
        return o
    parts = [torch.empty_like(o) for _ in range(size)]
    dist.all_gather(parts, o, group=group)
    return torch.cat(parts, dim=1)
