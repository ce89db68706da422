"""Ring (sequence-parallel) Tensor Product Attention, one process per GPU.

Mirrors tpa/ring_tpa.py of jondeaton/tensor-product-attention-jax:

    _rotate_block()            tpa/ring_tpa.py:24-38    -> grouped NCCL send/recv to rank+1
    _ring_tpa_fwd()            tpa/ring_tpa.py:41-112   -> ring_tpa() below (steps + merge)
    _ring_tpa_bwd()            tpa/ring_tpa.py:115-172  -> ring_tpa_bwd() below
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

__all__ = ["ring_tpa", "ring_tpa_bwd", "ring_tp_self_attention", "register_axis"]

_AXES: dict = {}
_side_streams: dict = {}
# Set to a list to have _ring_overlapped append, per call, its CUDA events (entry, own shard done,
# all hops arrived, visiting shards done) and operands; None (default) records nothing.
_timing = None

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
                  load_state, store_state, out, reuse_q=True, lse=None):
    return _tpa.fwd_device(
        q, k, v, num_heads, qs, ks, sm_scale, causal, q_offset=q_offset, k_offset=k_offset,
        state=state, load_state=load_state, store_state=store_state, out=out, lse=lse, want_lse=False,
        # q and the workspace are those of the previous step (not so when two query chunks alternate)
        reuse_staged_q=load_state and reuse_q,
    )[0]


def _device_block_fresh_q(*args):
    return _device_block(*args, reuse_q=False)


def _zigzag_owner(chunk, size):
    """Rank that computes `chunk` (of 2 * size equal chunks of the whole sequence)."""
    return chunk if chunk < size else 2 * size - 1 - chunk


def _exchange_chunks(send, recv, group, rank):
    """send/recv: lists of (peer rank in group, [tensors]); peers in increasing chunk order on
    both sides, so that the pairwise send/recv order matches.  Local moves are plain copies."""
    ops, copies = [], []
    to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    local_src = [ts for peer, ts in send if peer == rank]
    local_dst = [ts for peer, ts in recv if peer == rank]
    for src, dst in zip(local_src, local_dst):
        copies += list(zip(dst, src))
    for peer, ts in send:
        if peer != rank:
            ops += [dist.P2POp(dist.isend, t.contiguous(), to_global(peer), group) for t in ts]
    for peer, ts in recv:
        if peer != rank:
            ops += [dist.P2POp(dist.irecv, t, to_global(peer), group) for t in ts]
    reqs = dist.batch_isend_irecv(ops) if ops else []
    for d, s_ in copies:
        d.copy_(s_)
    for r in reqs:
        r.wait()


def _ring_global_zigzag(q, k, v, qseg, kseg, group, size, rank, num_heads, sm_scale, block):
    """Causal attention over the whole sequence with balanced ranks.

    Contiguous shards make rank r do r + 1 of the N key blocks.  Here the sequence is cut into
    2N chunks and rank r computes the queries of chunks r and 2N-1-r (one early, one late):
    the rank's shard is first re-dealt that way (q, k, v and ids; the factors are small), the
    K/V factors of both chunks ring-rotate as usual, every step costs two chunk-by-chunk
    blocks on every rank, and the two output chunks travel back to the ranks that own those
    rows.  Same result as tpa(causal=True) on the unsharded input.
    """
    b, lq = q.shape[:2]
    if lq % 2 != 0 or k.shape[1] != lq:
        raise AssertionError("the balanced global mask needs equal, even shard lengths")
    c = lq // 2
    dv = v.shape[-1] - num_heads
    mine = [2 * rank, 2 * rank + 1]                 # chunks this rank holds on entry
    want = [rank, 2 * size - 1 - rank]              # chunks it computes (early, late)
    holder = lambda ch: ch // 2                     # noqa: E731  rank that holds chunk `ch` on entry

    def halves(x):
        return [x[:, :c], x[:, c:]]

    src = {ch: [h[i] for h in map(halves, (q, k, v, qseg, kseg))] for i, ch in enumerate(mine)}
    got = {ch: [torch.empty_like(t) for t in src[mine[0]]] for ch in want}
    send = sorted(((_zigzag_owner(ch, size), ch) for ch in mine), key=lambda x: x[1])
    recv = sorted(((holder(ch), ch) for ch in want), key=lambda x: x[1])
    _exchange_chunks([(peer, src[ch]) for peer, ch in send], [(peer, got[ch]) for peer, ch in recv],
                     group, rank)
    (q_e, k_e, v_e, qs_e, ks_e), (q_l, k_l, v_l, qs_l, ks_l) = got[want[0]], got[want[1]]

    dev, f32 = q.device, torch.float32
    out_e = torch.empty((b, c, num_heads, dv), dtype=q.dtype, device=dev)
    out_l = torch.empty_like(out_e)
    st_e = (torch.empty((b, c, num_heads, dv), dtype=f32, device=dev), torch.empty((b, c, num_heads), dtype=f32, device=dev))
    st_l = (torch.empty_like(st_e[0]), torch.empty_like(st_e[1]))
    cur = [torch.cat([k_e, k_l], 1), torch.cat([v_e, v_l], 1), torch.cat([ks_e, ks_l], 1)]
    spare = [[torch.empty_like(t) for t in cur] for _ in range(min(2, size - 1))]
    use_streams = q.is_cuda
    if use_streams:
        main = torch.cuda.current_stream(dev)
        side = _side_streams.get(dev) or _side_streams.setdefault(dev, torch.cuda.Stream(dev))
        ready = torch.cuda.Event()
        ready.record(main)
    started_e = started_l = False
    for s in range(size):
        origin = (rank - s) % size  # the rank whose chunks (origin, 2N-1-origin) are visiting
        reqs = None
        if s < size - 1:
            nxt = spare[s % 2]
            if use_streams:
                side.wait_event(ready)
                with torch.cuda.stream(side):
                    reqs = _rotate_block(cur, nxt, group, rank, size)
            else:
                reqs = _rotate_block(cur, nxt, group, rank, size)
        kk, vv, ss = cur
        # late queries: the visiting early chunk is always wholly visible, the late one iff
        # origin > rank (wholly) or origin == rank (diagonal)
        last_l = s == size - 1
        if origin > rank:
            block(q_l, kk, vv, qs_l, ss, num_heads, sm_scale, False, 0, 0, st_l, started_l, not last_l, out_l)
        elif origin < rank:
            block(q_l, kk[:, :c], vv[:, :c], qs_l, ss[:, :c], num_heads, sm_scale, False, 0, 0, st_l,
                  started_l, not last_l, out_l)
        else:  # positions: early chunk just before the late one, so that it stays wholly visible
            block(q_l, kk, vv, qs_l, ss, num_heads, sm_scale, True, (2 * size - 1 - rank) * c,
                  (2 * size - 2 - rank) * c, st_l, started_l, not last_l, out_l)
        started_l = True
        # early queries: only early chunks of ranks <= this one (steps 0..rank)
        if origin <= rank:
            block(q_e, kk[:, :c], vv[:, :c], qs_e, ss[:, :c], num_heads, sm_scale, origin == rank,
                  rank * c, origin * c, st_e, started_e, s != rank, out_e)
            started_e = True
        if s < size - 1:
            if use_streams:
                ready = torch.cuda.Event()
                ready.record(main)
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
    # the two output chunks go back to the ranks that own those rows
    out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=dev)
    back_send = sorted(((holder(ch), ch, o) for ch, o in zip(want, (out_e, out_l))), key=lambda x: x[1])
    back_recv = sorted(((_zigzag_owner(ch, size), ch, o) for ch, o in zip(mine, halves(out))), key=lambda x: x[1])
    tmp = [torch.empty_like(out_e) for _ in back_recv]
    _exchange_chunks([(peer, [o]) for peer, _, o in back_send], [(peer, [t]) for (peer, _, _), t in zip(back_recv, tmp)],
                     group, rank)
    for (_, _, dst), t in zip(back_recv, tmp):
        dst.copy_(t)
    return out


def _gather_ring(k, v, kseg, group, size, rank):
    """All N K/V factor shards (and key ids) of the ring in one buffer per array, in sequence order:
    [N, b, l, r, h + d] with slot s = the shard of rank s.

    The same N - 1 neighbour hops as the scan of tpa/ring_tpa.py:69-106 -- at hop t every rank sends
    on what it received at hop t - 1 and receives the shard that started t ranks behind it -- but
    they do not wait for compute: all are queued at entry on the side stream, into their own
    slots, and the attention then runs as one call over the N parts.  Only the compact factors
    travel (tpa/ring_tpa.py:96).  Returns the buffers; on CUDA the current stream has been made
    to wait for the last hop."""
    kbuf = torch.empty((size,) + tuple(k.shape), dtype=k.dtype, device=k.device)
    vbuf = torch.empty((size,) + tuple(v.shape), dtype=v.dtype, device=v.device)
    sbuf = torch.empty((size,) + tuple(kseg.shape), dtype=kseg.dtype, device=kseg.device)
    kbuf[rank].copy_(k)
    vbuf[rank].copy_(v)
    sbuf[rank].copy_(kseg)
    if size == 1:
        return kbuf, vbuf, sbuf
    use_streams = k.is_cuda
    if use_streams:
        main = torch.cuda.current_stream(k.device)
        side = _side_streams.get(k.device) or _side_streams.setdefault(k.device, torch.cuda.Stream(k.device))
        side.wait_stream(main)  # the local shard is in its slot
        ctx = torch.cuda.stream(side)
    else:
        import contextlib
        ctx = contextlib.nullcontext()
    with ctx:
        for hop in range(1, size):
            have, want = (rank - hop + 1) % size, (rank - hop) % size
            reqs = _rotate_block([kbuf[have], vbuf[have], sbuf[have]], [kbuf[want], vbuf[want], sbuf[want]],
                                 group, rank, size)
            # the next hop forwards what this one receives
            for r in reqs:
                r.wait()
    if use_streams:
        main.wait_stream(side)
    return kbuf, vbuf, sbuf


def _device_parts(q, kbuf, vbuf, qs, sbuf, num_heads, sm_scale, causal, per_part, q_offset, out, lse, reuse_kv=False,
                  state=None, load_state=False, store_state=False, reuse_q=False):
    """One tpa_fwd call over gathered key parts [parts, b, l, ...] (the whole ring for this rank's
    rows, or a share of it that starts from / leaves a carried partial in `state`)."""
    parts = kbuf.shape[0]
    if parts == 1:  # one shard: the plain call
        kbuf, vbuf, sbuf = kbuf[0], vbuf[0], sbuf[0]
    return _tpa.fwd_device(q, kbuf, vbuf, num_heads, qs, sbuf, sm_scale, causal, q_offset=q_offset, out=out, lse=lse,
                           want_lse=lse is not None, kv_parts=parts, per_part=per_part and parts > 1,
                           reuse_staged_kv=reuse_kv, reuse_staged_q=reuse_q, state=state, load_state=load_state,
                           store_state=store_state)


def _ring_overlapped(q, k, v, qseg, kseg, group, size, rank, num_heads, sm_scale, causal, return_lse, parts_fn):
    """The reference's ring (every visiting shard under its own shard-local mask, tpa/ring_tpa.py:73-79)
    as two attention calls: the rank's own shard at once, while all N - 1 hops are under way on the
    side stream, then the N - 1 visiting shards in one call that starts from the first call's
    partial (o, lse) -- the carry of tpa/ring_tpa.py:69-71, used once.  The hops are the scan's
    neighbour sends (at hop t a rank forwards what it received at hop t - 1) into slots in arrival
    order; with a shard-local mask the order of the shards does not matter."""
    b, lq = q.shape[:2]
    dv = v.shape[-1] - num_heads
    dev = q.device
    out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=dev)
    lse = torch.empty((b, lq, num_heads), dtype=torch.float32, device=dev) if return_lse else None
    timing = _timing is not None and q.is_cuda
    if timing:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
    if size == 1:
        parts_fn(q, k[None], v[None], qseg, kseg[None], num_heads, sm_scale, causal, False, 0, out, lse, False)
        return (out, lse) if return_lse else out
    kbuf = torch.empty((size - 1,) + tuple(k.shape), dtype=k.dtype, device=dev)
    vbuf = torch.empty((size - 1,) + tuple(v.shape), dtype=v.dtype, device=dev)
    sbuf = torch.empty((size - 1,) + tuple(kseg.shape), dtype=kseg.dtype, device=dev)
    use_streams = q.is_cuda
    if use_streams:
        main = torch.cuda.current_stream(dev)
        side = _side_streams.get(dev) or _side_streams.setdefault(dev, torch.cuda.Stream(dev))
        side.wait_stream(main)  # k, v and the ids are ready, the buffers exist
        ctx = torch.cuda.stream(side)
    else:
        import contextlib
        ctx = contextlib.nullcontext()
    with ctx:
        for hop in range(1, size):
            have = [k, v, kseg] if hop == 1 else [kbuf[hop - 2], vbuf[hop - 2], sbuf[hop - 2]]
            for r in _rotate_block(have, [kbuf[hop - 1], vbuf[hop - 1], sbuf[hop - 1]], group, rank, size):
                r.wait()  # the next hop forwards what this one receives
    state = (torch.empty((b, lq, num_heads, dv), dtype=torch.float32, device=dev),
             torch.empty((b, lq, num_heads), dtype=torch.float32, device=dev))
    parts_fn(q, k[None], v[None], qseg, kseg[None], num_heads, sm_scale, causal, False, 0, None, None, False,
             state=state, store_state=True)
    if timing:
        ev[1].record()
    if use_streams:
        main.wait_stream(side)
    if timing:
        ev[2].record()
    parts_fn(q, kbuf, vbuf, qseg, sbuf, num_heads, sm_scale, causal, causal, 0, out, lse, False,
             state=state, load_state=True, reuse_q=True)
    if timing:
        ev[3].record()
        _timing.append({"events": ev, "operands": (q, kbuf, vbuf, qseg, sbuf, state)})
    return (out, lse) if return_lse else out


def _parts_supported(q, k):
    """The one-call path needs key parts of whole 64-row tiles (128 on tensor cores, else the generic
    kernel takes them) -- the same on every rank, because shapes are."""
    return k.shape[1] % 64 == 0


def _ring_one_call(q, k, v, qseg, kseg, group, size, rank, num_heads, sm_scale, causal, mask_mode, return_lse, parts_fn):
    """Ring forward as gather + one attention call (two for the balanced global mask); the
    reference's shard-local mask and the unmasked ring go through _ring_overlapped instead."""
    if not (causal and mask_mode == "global"):
        return _ring_overlapped(q, k, v, qseg, kseg, group, size, rank, num_heads, sm_scale, causal, return_lse, parts_fn)
    b, lq = q.shape[:2]
    lk = k.shape[1]
    dv = v.shape[-1] - num_heads
    dev = q.device
    want_lse = return_lse
    if causal and mask_mode == "global" and size > 1 and lq == lk and lq % 2 == 0:
        # balanced: this rank computes sequence chunks `rank` and 2N-1-rank (see _ring_global_zigzag);
        # the keys are the gathered shards in sequence order, compared on global positions
        c = lq // 2
        mine, want = [2 * rank, 2 * rank + 1], [rank, 2 * size - 1 - rank]
        holder = lambda ch: ch // 2  # noqa: E731
        src = {ch: [q[:, i * c:(i + 1) * c], qseg[:, i * c:(i + 1) * c]] for i, ch in enumerate(mine)}
        got = {ch: [torch.empty_like(t) for t in src[mine[0]]] for ch in want}
        send = sorted(((_zigzag_owner(ch, size), ch) for ch in mine), key=lambda x: x[1])
        recv = sorted(((holder(ch), ch) for ch in want), key=lambda x: x[1])
        _exchange_chunks([(peer, src[ch]) for peer, ch in send], [(peer, got[ch]) for peer, ch in recv], group, rank)
        kbuf, vbuf, sbuf = _gather_ring(k, v, kseg, group, size, rank)
        outs, lses = [], []
        n_parts = want[1] // 2 + 1  # shards the late chunk can see; the early one sees a prefix of them
        for i, ch in enumerate((want[1], want[0])):  # late chunk first: it stages every tile both need
            o_c = torch.empty((b, c, num_heads, dv), dtype=q.dtype, device=dev)
            l_c = torch.empty((b, c, num_heads), dtype=torch.float32, device=dev) if want_lse else None
            parts_fn(got[ch][0], kbuf[:n_parts], vbuf[:n_parts], got[ch][1], sbuf[:n_parts], num_heads, sm_scale, True,
                     False, ch * c, o_c, l_c, i == 1)
            outs.append(o_c)
            lses.append(l_c)
        out_l, out_e = outs
        out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=dev)
        lse = torch.empty((b, lq, num_heads), dtype=torch.float32, device=dev) if want_lse else None
        pieces = [[out_e], [out_l]] if not want_lse else [[out_e, lses[1]], [out_l, lses[0]]]
        dsts = [[out[:, :c]], [out[:, c:]]] if not want_lse else [[out[:, :c], lse[:, :c]], [out[:, c:], lse[:, c:]]]
        back_send = sorted(((holder(ch), ch, ts) for ch, ts in zip(want, pieces)), key=lambda x: x[1])
        back_recv = sorted(((_zigzag_owner(ch, size), ch, ts) for ch, ts in zip(mine, dsts)), key=lambda x: x[1])
        tmp = [[torch.empty_like(t) for t in pieces[0]] for _ in back_recv]
        _exchange_chunks([(peer, ts) for peer, _, ts in back_send], [(peer, t) for (peer, _, _), t in zip(back_recv, tmp)],
                         group, rank)
        for (_, _, ds), ts in zip(back_recv, tmp):
            for d_, t in zip(ds, ts):
                d_.copy_(t)
        return (out, lse) if return_lse else out

    kbuf, vbuf, sbuf = _gather_ring(k, v, kseg, group, size, rank)
    out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=dev)
    lse = torch.empty((b, lq, num_heads), dtype=torch.float32, device=dev) if want_lse else None
    if causal and mask_mode == "global":
        # contiguous shards, global positions: only the shards up to this rank's own are visible
        n_parts = min(size, (rank * lq + lq - 1) // lk + 1)
        parts_fn(q, kbuf[:n_parts], vbuf[:n_parts], qseg, sbuf[:n_parts], num_heads, sm_scale, True, False, rank * lq,
                 out, lse, False)
    else:
        # the reference's ring: every visiting shard is masked on shard-local indices
        parts_fn(q, kbuf, vbuf, qseg, sbuf, num_heads, sm_scale, causal, causal and size > 1, 0, out, lse, False)
    return (out, lse) if return_lse else out


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
    return_lse: bool = False,
    one_call: bool | None = None,
    _block_fn=None,
    _parts_fn=None,
):
    """Ring TPA forward on this rank's shard; arguments as tpa/ring_tpa.py:209-222.

    Differentiable: when q, k or v requires grad the call goes through torch autograd with
    ring_tpa_bwd as its backward (the custom_vjp of tpa/ring_tpa.py:175-206).
    `return_lse=True` (keyword only) also returns the fp32 LSE of the whole ring, [b, l/N, h].

    q[b, l/N, rq, h+dk], k, v, and the two int32 id arrays are this rank's contiguous
    shard; returns this rank's o[b, l/N, h, dv].  `impl="pallas"` is the reference's name
    for its kernel path and selects the CUDA kernels here; "xla" raises NotImplementedError
    and anything else ValueError, as in the reference (tpa/ring_tpa.py:237-273).

    `one_call` (keyword only): None picks the one-call path whenever the shard length allows,
    False forces the step-by-step scan with carried state.

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
    if (_block_fn is None and _parts_fn is None and not return_lse and torch.is_grad_enabled()
            and (q.requires_grad or k.requires_grad or v.requires_grad)):
        return _RingTpaFunction.apply(q, k, v, q_segment_ids, kv_segment_ids, axis_name, num_heads,
                                      sm_scale, causal, mask_mode)
    block = _block_fn or _device_block
    if _block_fn is None and _parts_fn is None and not q.is_cuda:
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

    # Default: all hops are queued at entry and the attention runs as ONE call over the gathered
    # shards (no per-step launch, no carried state in HBM).  The step-by-step scan below remains
    # for shard lengths the one-call kernels do not take and on request (`one_call=False`).
    if one_call is None:
        one_call = _parts_fn is not None or (_block_fn is None and _parts_supported(q, k))
    if one_call:
        if _parts_fn is None and not _parts_supported(q, k):
            raise ValueError("one_call=True needs shard lengths that are multiples of 64")
        return _ring_one_call(q, k.contiguous(), v.contiguous(), qseg, kseg, group, size, rank, num_heads, sm_scale,
                              causal, mask_mode, return_lse, _parts_fn or _device_parts)

    # (the balanced exchange does not carry the LSE back; with return_lse the contiguous walk runs)
    if causal and mask_mode == "global" and size > 1 and lq == lk and lq % 2 == 0 and not return_lse:
        zz_block = _device_block_fresh_q if _block_fn is None else _block_fn
        return _ring_global_zigzag(q, k.contiguous(), v.contiguous(), qseg, kseg, group, size, rank,
                                   num_heads, sm_scale, zz_block)

    use_streams = q.is_cuda
    out = torch.empty((b, lq, num_heads, dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((b, lq, num_heads), dtype=torch.float32, device=q.device) if return_lse else None
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
            extra = {"lse": lse} if (return_lse and s == last_compute) else {}
            block(
                q, cur[0], cur[1], qseg, cur[2], num_heads, sm_scale, causal, q_off, k_off, state,
                started, s != last_compute, out, **extra,
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
    return (out, lse) if return_lse else out


def _device_bwd_block(q, k, v, qs, ks, num_heads, sm_scale, causal, q_offset, k_offset, o, lse, do,
                      grads, accumulate_dq):
    """One ring step of the backward: dq (+)= , travelling dk, dv += (fp32 buffers in `grads`)."""
    _tpa.bwd_device(q, k, v, num_heads, qs, ks, sm_scale, causal, o, lse, do, q_offset=q_offset,
                    k_offset=k_offset, grad_dtype=torch.float32, out=grads,
                    accumulate_dq=accumulate_dq, accumulate_dkv=True)


def _ring_bwd_global_zigzag(q, k, v, qseg, kseg, o, lse, do, group, size, rank, num_heads, sm_scale, block):
    """Backward of causal attention over the whole sequence with balanced ranks.

    With contiguous shards rank r would run r + 1 of the N key blocks (efficiency bound 0.53 at
    N = 8).  As in the forward (_ring_global_zigzag), the sequence is cut into 2N chunks and rank
    r takes chunks r (early) and 2N-1-r (late): the rows of q, o, lse, do and their ids, and the
    K/V factors of those chunks, are re-dealt that way first.  The K/V chunks of every rank then
    ring-rotate together with their fp32 dk / dv accumulators (tpa/ring_tpa.py:147-160); each
    step costs two chunk-by-chunk block backwards on every rank (late queries against the
    visiting early chunk always; against the visiting late chunk, or the early queries against
    the visiting early chunk, as positions allow).  After N rotations the accumulators are back
    with the rank that dealt them, and dq, dk, dv travel back to the ranks that own those rows.
    """
    b, lq = q.shape[:2]
    if lq % 2 != 0 or k.shape[1] != lq:
        raise AssertionError("the balanced global mask needs equal, even shard lengths")
    c = lq // 2
    f32 = torch.float32
    mine = [2 * rank, 2 * rank + 1]            # chunks this rank holds on entry
    want = [rank, 2 * size - 1 - rank]         # chunks it works on (early, late)
    holder = lambda ch: ch // 2                # noqa: E731  rank that holds chunk `ch` on entry

    def halves(x):
        return [x[:, :c].contiguous(), x[:, c:].contiguous()]

    per_row = (q, k, v, qseg, kseg, o, lse, do)
    src = {ch: [h[i] for h in map(halves, per_row)] for i, ch in enumerate(mine)}
    got = {ch: [torch.empty_like(t) for t in src[mine[0]]] for ch in want}
    send = sorted(((_zigzag_owner(ch, size), ch) for ch in mine), key=lambda x: x[1])
    recv = sorted(((holder(ch), ch) for ch in want), key=lambda x: x[1])
    _exchange_chunks([(peer, src[ch]) for peer, ch in send], [(peer, got[ch]) for peer, ch in recv], group, rank)
    (q_e, k_e, v_e, qs_e, ks_e, o_e, l_e, do_e), (q_l, k_l, v_l, qs_l, ks_l, o_l, l_l, do_l) = got[want[0]], got[want[1]]

    dq_e = torch.zeros(q_e.shape, dtype=f32, device=q.device)
    dq_l = torch.zeros(q_l.shape, dtype=f32, device=q.device)
    # the travelling bundle: factors and ids of (early, late) chunk, and their gradient accumulators
    cur = [k_e, v_e, ks_e, k_l, v_l, ks_l]
    acc = [torch.zeros(t.shape, dtype=f32, device=q.device) for t in (k_e, v_e, k_l, v_l)]
    spare = [torch.empty_like(t) for t in cur]
    acc_spare = [torch.empty_like(t) for t in acc]
    started_e = started_l = False
    pos_e, pos_l = rank * c, (2 * size - 1 - rank) * c          # positions of this rank's query chunks
    for s in range(size):
        origin = (rank - s) % size  # the rank whose chunks (origin, 2N-1-origin) are visiting
        ke, ve, se, kl, vl, sl = cur
        # late queries against the visiting early chunk: always wholly visible
        block(q_l, ke, ve, qs_l, se, num_heads, sm_scale, False, 0, 0, o_l, l_l, do_l, (dq_l, acc[0], acc[1]), started_l)
        started_l = True
        if origin > rank:      # ... and against the visiting late chunk, which lies before theirs
            block(q_l, kl, vl, qs_l, sl, num_heads, sm_scale, False, 0, 0, o_l, l_l, do_l, (dq_l, acc[2], acc[3]), True)
        elif origin == rank:   # their own chunk: the diagonal
            block(q_l, kl, vl, qs_l, sl, num_heads, sm_scale, True, pos_l, pos_l, o_l, l_l, do_l, (dq_l, acc[2], acc[3]), True)
        # early queries see early chunks of ranks <= this one only
        if origin <= rank:
            block(q_e, ke, ve, qs_e, se, num_heads, sm_scale, origin == rank, pos_e, origin * c, o_e, l_e, do_e,
                  (dq_e, acc[0], acc[1]), started_e)
            started_e = True
        if size > 1:  # factors and accumulators move on together, every step, so that they end at home
            for r in _rotate_block(cur + acc, spare + acc_spare, group, rank, size):
                r.wait()
            cur, spare = spare, cur
            acc, acc_spare = acc_spare, acc
    # home again: acc holds the gradients of this rank's (early, late) K/V chunks; everything goes
    # back to the ranks that own those rows
    outs = {want[0]: [dq_e, acc[0], acc[1]], want[1]: [dq_l, acc[2], acc[3]]}
    back_send = sorted(((holder(ch), ch, ts) for ch, ts in outs.items()), key=lambda x: x[1])
    back_recv = sorted(((_zigzag_owner(ch, size), ch) for ch in mine), key=lambda x: x[1])
    tmp = {ch: [torch.empty_like(t) for t in outs[want[0]]] for _, ch in back_recv}
    _exchange_chunks([(peer, ts) for peer, _, ts in back_send], [(peer, tmp[ch]) for peer, ch in back_recv], group, rank)
    dq = torch.cat([tmp[mine[0]][0], tmp[mine[1]][0]], 1).to(q.dtype)
    dk = torch.cat([tmp[mine[0]][1], tmp[mine[1]][1]], 1).to(k.dtype)
    dv = torch.cat([tmp[mine[0]][2], tmp[mine[1]][2]], 1).to(v.dtype)
    return dq, dk, dv


def ring_tpa_bwd(
    q,
    k,
    v,
    q_segment_ids,
    kv_segment_ids,
    o,
    lse,
    do,
    axis_name,
    num_heads: int,
    sm_scale: float = 1.0,
    causal: bool = False,
    *,
    mask_mode: str = "reference_local",
    _block_fn=None,
):
    """Ring TPA backward on this rank's shard (_ring_tpa_bwd, tpa/ring_tpa.py:115-172).

    `o`, `lse` are the ring forward's results for this rank's rows (lse of the whole ring, fp32),
    `do` the incoming gradient.  Every step runs the block backward against the visiting K/V
    shard, adds into the local dq and into the dk / dv accumulators that travel with that shard
    (tpa/ring_tpa.py:147-160); after N rotations the accumulators are home again.  Gradients are
    accumulated in fp32 and returned in the dtype of q, k, v.  The K/V factors of the next step
    move on a side stream while the current step computes; the accumulators can only follow it.
    """
    if mask_mode not in MASK_MODES:
        raise ValueError(f"mask_mode must be one of {MASK_MODES}")
    block = _block_fn or _device_bwd_block
    if _block_fn is None and not q.is_cuda:
        raise RuntimeError("tpa_b200 needs a CUDA device: there is no CPU implementation")
    group = _group_of(axis_name)
    if dist.is_available() and dist.is_initialized():
        size, rank = dist.get_world_size(group), dist.get_rank(group)
    else:
        size, rank = 1, 0
    lq, lk = q.shape[1], k.shape[1]
    kseg = kv_segment_ids.to(torch.int32).contiguous()
    qseg = q_segment_ids.to(torch.int32).contiguous()
    f32 = torch.float32
    if causal and mask_mode == "global" and size > 1 and lq == lk and lq % 2 == 0:
        return _ring_bwd_global_zigzag(q, k.contiguous(), v.contiguous(), qseg, kseg, o, lse.to(f32), do, group, size,
                                       rank, num_heads, sm_scale, block)
    dq = torch.zeros(q.shape, dtype=f32, device=q.device)
    cur = [k.contiguous(), v.contiguous(), kseg]
    acc = [torch.zeros(k.shape, dtype=f32, device=q.device), torch.zeros(v.shape, dtype=f32, device=q.device)]
    spare = [[torch.empty_like(t) for t in cur] for _ in range(min(2, size - 1))]
    acc_spare = [torch.empty_like(t) for t in acc] if size > 1 else None
    use_streams = q.is_cuda
    if use_streams:
        main = torch.cuda.current_stream(q.device)
        side = _side_streams.get(q.device) or _side_streams.setdefault(q.device, torch.cuda.Stream(q.device))
        ready = torch.cuda.Event()
        ready.record(main)

    def visible(src):
        return not (causal and mask_mode == "global" and src * lk > rank * lq + lq - 1)

    started = False
    for s in range(size):
        src = (rank - s) % size
        reqs = None
        if s < size - 1:  # the factors of the next step leave while this step computes
            nxt = spare[s % 2]
            if use_streams:
                side.wait_event(ready)
                with torch.cuda.stream(side):
                    reqs = _rotate_block(cur, nxt, group, rank, size)
            else:
                reqs = _rotate_block(cur, nxt, group, rank, size)
        if visible(src):
            q_off, k_off = (rank * lq, src * lk) if mask_mode == "global" else (0, 0)
            block(q, cur[0], cur[1], qseg, cur[2], num_heads, sm_scale, causal, q_off, k_off, o, lse, do,
                  (dq, acc[0], acc[1]), started)
            started = True
        if size > 1:
            if s < size - 1:
                if use_streams:
                    ready = torch.cuda.Event()
                    ready.record(main)
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
            # the accumulators follow their shard (every step, so that they end at home)
            for r in _rotate_block(acc, acc_spare, group, rank, size):
                r.wait()
            acc, acc_spare = acc_spare, acc
    return dq.to(q.dtype), acc[0].to(k.dtype), acc[1].to(v.dtype)


class _RingTpaFunction(torch.autograd.Function):
    """custom_vjp of the reference (tpa/ring_tpa.py:175-206): forward keeps (o, lse of the ring)."""

    @staticmethod
    def forward(ctx, q, k, v, q_segment_ids, kv_segment_ids, axis_name, num_heads, sm_scale, causal, mask_mode):
        o, lse = ring_tpa(q, k, v, q_segment_ids, kv_segment_ids, axis_name, num_heads, sm_scale, causal,
                          mask_mode=mask_mode, return_lse=True)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.rest = (q_segment_ids, kv_segment_ids, axis_name, num_heads, sm_scale, causal, mask_mode)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        qs, ks, axis_name, num_heads, sm_scale, causal, mask_mode = ctx.rest
        dq, dk, dv = ring_tpa_bwd(q, k, v, qs, ks, o, lse, do.contiguous(), axis_name, num_heads, sm_scale,
                                  causal, mask_mode=mask_mode)
        return (dq, dk, dv) + (None,) * 7


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
    one_call: bool | None = None,
    _block_fn=None,
    _parts_fn=None,
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
        debug=debug, interpret=interpret, mask_mode=mask_mode, one_call=one_call, _block_fn=_block_fn,
        _parts_fn=_parts_fn,
    )
    if not gather_output or size == 1:
        return o
    parts = [torch.empty_like(o) for _ in range(size)]
    dist.all_gather(parts, o, group=group)
    return torch.cat(parts, dim=1)
