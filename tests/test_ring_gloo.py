"""Host logic of the ring path on CPU: 2 and 4 gloo ranks, the device kernel replaced by an
oracle-backed block with the same state contract (test-only hook `_block_fn`, the step-by-step
scan) or by an oracle-backed call over gathered key parts (`_parts_fn`, the one-call path)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, PKG_DIR  # noqa: F401  (puts the package on sys.path)
from oracle import tpa_oracle as orc


def oracle_block(q, k, v, qs, ks, num_heads, sm_scale, causal, q_off, k_off, state, load, store, out, lse=None):
    """CPU stand-in for one tpa_fwd call with the TPA_FLAG_STATE_* contract."""
    o_, l_ = orc.tpa_reference(q.numpy(), k.numpy(), v.numpy(), num_heads, qs.numpy(), ks.numpy(),
                               sm_scale=sm_scale, causal=causal, q_offset=q_off, k_offset=k_off,
                               return_lse=True)
    o_ = np.nan_to_num(o_, nan=0.0)
    if load:
        so, sl = state[0].numpy().astype(np.float64), state[1].numpy().astype(np.float64)
        ln = orc.lse_accum(sl, l_)
        with np.errstate(invalid="ignore"):
            o_ = np.nan_to_num(so * np.exp(sl - ln)[..., None]) + np.nan_to_num(o_ * np.exp(l_ - ln)[..., None])
        l_ = ln
    if store:
        state[0].copy_(torch.from_numpy(o_).float())
        state[1].copy_(torch.from_numpy(l_).float())
    else:
        o_ = np.where(np.isneginf(l_)[..., None], np.nan, o_)
        out.copy_(torch.from_numpy(o_).to(out.dtype))
        if lse is not None:
            lse.copy_(torch.from_numpy(l_).float())


def oracle_parts(q, kbuf, vbuf, qs, sbuf, num_heads, sm_scale, causal, per_part, q_off, out, lse, reuse_kv,
                 state=None, load_state=False, store_state=False, reuse_q=False):
    """CPU stand-in for one tpa_fwd call over gathered key parts [parts, b, l, ...], with the
    carried partial of a ring step when asked for."""
    n, b, l = kbuf.shape[:3]
    cat = lambda x: x.transpose(0, 1).reshape(b, n * l, *x.shape[3:]).numpy()  # noqa: E731  parts side by side
    o_, l_ = orc.tpa_reference(q.numpy(), cat(kbuf), cat(vbuf), num_heads, qs.numpy(), cat(sbuf), sm_scale=sm_scale,
                               causal=causal, q_offset=q_off, kv_parts=n, per_part=per_part and n > 1, return_lse=True)
    if load_state or store_state:
        o_ = np.nan_to_num(o_, nan=0.0)
        if load_state:
            so, sl = state[0].numpy().astype(np.float64), state[1].numpy().astype(np.float64)
            ln = orc.lse_accum(sl, l_)
            with np.errstate(invalid="ignore"):
                o_ = np.nan_to_num(so * np.exp(sl - ln)[..., None]) + np.nan_to_num(o_ * np.exp(l_ - ln)[..., None])
            l_ = ln
        if store_state:
            state[0].copy_(torch.from_numpy(o_).float())
            state[1].copy_(torch.from_numpy(l_).float())
            return
        o_ = np.where(np.isneginf(l_)[..., None], np.nan, o_)
    out.copy_(torch.from_numpy(o_).to(out.dtype))
    if lse is not None:
        lse.copy_(torch.from_numpy(l_).float())


def oracle_bwd_block(q, k, v, qs, ks, num_heads, sm_scale, causal, q_off, k_off, o, lse, do, grads, accumulate_dq):
    """CPU stand-in for one tpa_bwd call (fp32 gradients, dk / dv always accumulate)."""
    g = orc.tpa_bwd_block(q.numpy(), k.numpy(), v.numpy(), do.numpy(), o.numpy(), lse.numpy(), num_heads,
                          qs.numpy(), ks.numpy(), sm_scale, causal, np.float64, q_off, k_off)
    for buf, new, acc in zip(grads, g, (accumulate_dq, True, True)):
        new = torch.from_numpy(new).to(buf.dtype)
        buf.copy_(buf + new if acc else new)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    import sys
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    import tpa_b200

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        seed, b, l, rq, rk, h, dk, dv, seg, sm, causal, mode, path = case
        q, k, v = orc.make_factors(seed, b, l, l, rq, rk, h, dk, dv)
        ids = orc.segment_ids(b, l, seg) if seg else np.zeros((b, l), np.int32)
        tq, tk, tv, tid = (torch.from_numpy(x) for x in (q, k, v, ids))
        hook = {"_block_fn": oracle_block} if path == "scan" else {"_parts_fn": oracle_parts}
        o = tpa_b200.ring_tpa.ring_tp_self_attention(
            tq, tk, tv, tid, tid, mesh=None, pspec=(None, "sp", None, None), num_heads=h,
            sm_scale=sm, causal=causal, mask_mode=mode, gather_output=True, **hook)
        if rank == 0:
            ref = orc.ring_tpa_reference(q, k, v, ids, ids, h, world, sm_scale=sm, causal=causal,
                                         mask_mode=mode)
            ret["err"] = float(np.nanmax(np.abs(o.numpy() - ref)))
            ret["nan_equal"] = bool(np.array_equal(np.isnan(o.numpy()), np.isnan(ref)))
            ret["shape"] = tuple(o.shape)
    finally:
        dist.destroy_process_group()


CASES = [
    # seed, b, l, rq, rk, h, dk, dv, seg, sm_scale, causal, mask_mode
    (21, 2, 64, 2, 2, 2, 8, 8, 42, 1.0, False, "reference_local"),
    (22, 1, 128, 3, 2, 4, 8, 4, None, 0.3, True, "reference_local"),
    (23, 1, 128, 3, 2, 4, 8, 4, 50, 0.3, True, "global"),
]


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("path", ["scan", "one_call"])
@pytest.mark.parametrize("case", CASES)
def test_ring_host_logic_gloo(world, case, path):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), case + (path,), ret), nprocs=world, join=True)
    assert ret["shape"] == (case[1], case[2], case[5], case[7])
    assert ret["nan_equal"]
    assert ret["err"] < 1e-5, ret["err"]


def _bwd_worker(rank, world, port, case, ret):
    import sys
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    import tpa_b200

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        seed, b, l, rq, rk, h, dk, dv, seg, sm, causal, mode = case
        q, k, v = orc.make_factors(seed, b, l, l, rq, rk, h, dk, dv)
        ids = orc.segment_ids(b, l, seg) if seg else np.zeros((b, l), np.int32)
        do = np.random.default_rng(seed).standard_normal((b, l, h, dv)).astype(np.float32)
        sh = slice(rank * (l // world), (rank + 1) * (l // world))
        tq, tk, tv, tid, tdo = (torch.from_numpy(np.ascontiguousarray(x[:, sh])) for x in (q, k, v, ids, do))
        o, lse = tpa_b200.ring_tpa.ring_tpa(tq, tk, tv, tid, tid, None, h, sm_scale=sm, causal=causal,
                                            mask_mode=mode, return_lse=True, _block_fn=oracle_block)
        # the one-call path must hand the backward the same residuals (balanced exchange included)
        o1, lse1 = tpa_b200.ring_tpa.ring_tpa(tq, tk, tv, tid, tid, None, h, sm_scale=sm, causal=causal,
                                              mask_mode=mode, return_lse=True, _parts_fn=oracle_parts)
        assert torch.allclose(o, o1, atol=1e-5, equal_nan=True) and torch.allclose(lse, lse1, atol=1e-5)
        grads = tpa_b200.ring_tpa.ring_tpa_bwd(tq, tk, tv, tid, tid, o, lse, tdo, None, h, sm_scale=sm,
                                               causal=causal, mask_mode=mode, _block_fn=oracle_bwd_block)
        full = []
        for g in grads:
            parts = [torch.empty_like(g) for _ in range(world)]
            dist.all_gather(parts, g.contiguous())
            full.append(torch.cat(parts, 1).numpy())
        if rank == 0:
            ref = orc.ring_tpa_bwd_reference(q, k, v, ids, ids, do, h, world, sm, causal, mode)
            ret["err"] = max(float(np.max(np.abs(a - r))) for a, r in zip(full, ref))
            ret["scale"] = max(float(np.max(np.abs(r))) for r in ref)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", CASES)
def test_ring_backward_host_logic_gloo(world, case):
    """dq stays, dk / dv travel with their shard and come home after N rotations (tpa/ring_tpa.py:147-160)."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_bwd_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert ret["err"] < 1e-5 * max(1.0, ret["scale"]), (ret["err"], ret["scale"])
