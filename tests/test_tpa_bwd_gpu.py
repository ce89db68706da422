"""GPU parity of the backward (tpa_bwd through the C ABI) against fixtures made by the
reference's own _tpa_bwd and against the oracle.

Tolerances: the reference's own atol = 1e-3, rtol = 1e-2 (tpa/tpa_test.py:203-205) on its
24-shape matrix, where a 20x tighter bound is also asserted; fp32 elsewhere 1e-4 relative to
the largest gradient entry; bf16 (inputs rounded to bf16, fp32 oracle) 3e-2 of the largest entry.
"""

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import tpa_oracle as orc

import tpa_b200
from tpa_b200 import _capi

pytestmark = pytest.mark.gpu

BWD = load_golden("bwd_matrix")


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def _do(seed, shape):
    return np.random.Generator(np.random.Philox(key=seed + 5000)).standard_normal(shape, dtype=np.float32)


def _rel(got, want):
    return float(np.max(np.abs(got - want)) / max(1e-6, np.max(np.abs(want))))


@pytest.mark.parametrize("case", sorted(BWD))
def test_reference_backward_matrix(case):
    """The 24 shapes of tpa/tpa_test.py:128-140 against gradients from the reference's kernel."""
    g = BWD[case]
    seed, b, lq, lk, rq, rk, h, dk, dv, seg = (int(x) for x in g["meta"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="normal")
    do = _do(seed, (b, lq, h, dv))
    qs = dev(orc.segment_ids(b, lq, seg)) if seg else None
    ks = dev(orc.segment_ids(b, lk, seg)) if seg else None
    n0 = _capi.lib.tpa_launch_count()
    _, res = tpa_b200.tpa._tpa_fwd(dev(q), dev(k), dev(v), h, qs, ks, 1.0, False, None, False, False, True)
    grads = tpa_b200.tpa._tpa_bwd(h, 1.0, False, None, False, False, True, res, dev(do))
    assert _capi.lib.tpa_launch_count() == n0 + 1 + 6  # forward + delta, 2 pair passes, 3 contractions
    assert grads[3] is None and grads[4] is None
    for name, got in zip(("dq", "dk", "dv"), grads[:3]):
        got = got.cpu().numpy()
        np.testing.assert_allclose(got, g[name], atol=1e-3, rtol=1e-2)
        assert np.max(np.abs(got - g[name]) / (1e-3 + 1e-2 * np.abs(g[name]))) < 0.05


CASES = [
    # b, lq, lk, rq, rk, h, dk, dv, seg_q, seg_k, causal, q_off, k_off, scale
    (1, 64, 64, 2, 2, 8, 16, 16, 0, 0, True, 0, 0, 0.25),
    (2, 100, 77, 3, 2, 6, 24, 40, 0, 0, False, 0, 0, 0.2),       # ragged tiles, dk != dv, 6 heads
    (2, 96, 160, 2, 3, 5, 32, 32, 37, 37, True, 0, 0, 0.18),     # packed + causal
    (1, 128, 128, 1, 1, 4, 8, 8, 16, 48, True, 0, 0, 0.35),      # rows that see no key (ids differ)
    (1, 96, 64, 2, 2, 4, 64, 64, 0, 0, True, 32, 0, 0.125),      # offsets: later query block
    (1, 64, 96, 2, 2, 4, 64, 64, 0, 0, True, 0, 40, 0.125),      # offsets: some rows see nothing
    (1, 40, 300, 4, 4, 2, 128, 128, 0, 0, False, 0, 0, 0.09),
    (1, 33, 65, 2, 2, 3, 200, 136, 0, 0, True, 40, 0, 0.07),     # head_dim > 128
]


@pytest.mark.parametrize("case", CASES)
def test_backward_against_oracle_fp32(case):
    b, lq, lk, rq, rk, h, dk, dv, sq, sk, causal, q_off, k_off, scale = case
    q, k, v = orc.make_factors(11, b, lq, lk, rq, rk, h, dk, dv)
    do = _do(11, (b, lq, h, dv))
    qs = orc.segment_ids(b, lq, sq) if sq else None
    ks = orc.segment_ids(b, lk, sk) if sk else None
    want = orc.tpa_bwd_reference(q, k, v, do, h, qs, ks, scale, causal, q_offset=q_off, k_offset=k_off)
    tq, tk, tv = dev(q), dev(k), dev(v)
    dqs, dks = (None if qs is None else dev(qs)), (None if ks is None else dev(ks))
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, dqs, dks, scale, causal, q_offset=q_off, k_offset=k_off)
    got = tpa_b200.tpa.bwd_device(tq, tk, tv, h, dqs, dks, scale, causal, o, lse, dev(do),
                                  q_offset=q_off, k_offset=k_off)
    for g, w in zip(got, want):
        g = g.cpu().numpy()
        assert np.isfinite(g).all()
        assert _rel(g, w) < 1e-4


@pytest.mark.parametrize("causal", [False, True])
def test_backward_bf16_and_accumulation(causal):
    b, lq, lk, rq, rk, h, d = 2, 160, 224, 3, 2, 8, 64
    q, k, v = orc.make_factors(5, b, lq, lk, rq, rk, h, d, d)
    tq, tk, tv = (dev(x, torch.bfloat16) for x in (q, k, v))
    do = dev(_do(5, (b, lq, h, d)), torch.bfloat16)
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, causal)
    f = lambda t: t.float().cpu().numpy()
    want = orc.tpa_bwd_reference(f(tq), f(tk), f(tv), f(do), h, None, None, d**-0.5, causal)
    got = tpa_b200.tpa.bwd_device(tq, tk, tv, h, None, None, d**-0.5, causal, o, lse, do, kernel="simt")
    for g, w in zip(got, want):
        assert g.dtype == torch.bfloat16
        assert _rel(f(g), w) < 3e-2
    # fp32 gradients, added twice onto a known start
    bufs = tuple(torch.full(x.shape, 0.5, dtype=torch.float32, device="cuda") for x in (tq, tk, tv))
    for _ in range(2):
        tpa_b200.tpa.bwd_device(tq, tk, tv, h, None, None, d**-0.5, causal, o, lse, do, kernel="simt",
                                grad_dtype=torch.float32, out=bufs, accumulate_dq=True, accumulate_dkv=True)
    for g, w in zip(bufs, want):
        assert _rel((f(g) - 0.5) / 2, w) < 2e-2
    # overwriting ignores what the buffers held
    tpa_b200.tpa.bwd_device(tq, tk, tv, h, None, None, d**-0.5, causal, o, lse, do, kernel="simt",
                            grad_dtype=torch.float32, out=bufs)
    for g, w in zip(bufs, want):
        assert _rel(f(g), w) < 2e-2


def test_autograd_through_tpa():
    """tpa() is differentiable like the reference's custom_vjp wrapper (tpa/tpa.py:73,217)."""
    b, lq, lk, rq, rk, h, dk, dv = 2, 128, 256, 2, 2, 4, 16, 24
    q, k, v = orc.make_factors(9, b, lq, lk, rq, rk, h, dk, dv)
    qs, ks = orc.segment_ids(b, lq, 50), orc.segment_ids(b, lk, 50)  # rows past the last key id are empty
    w = _do(9, (b, lq, h, dv))
    tq, tk, tv = (dev(x).requires_grad_() for x in (q, k, v))
    o = tpa_b200.tpa.tpa(tq, tk, tv, h, dev(qs), dev(ks), sm_scale=0.3, causal=True)
    torch.nansum(o * dev(w)).backward()
    do = np.where(np.isnan(o.detach().cpu().numpy()), 0.0, w).astype(np.float32)
    want = orc.tpa_bwd_reference(q, k, v, do, h, qs, ks, 0.3, True)
    for t, wnt in zip((tq, tk, tv), want):
        assert _rel(t.grad.cpu().numpy(), wnt) < 1e-4


def test_backward_rejects_bad_arguments():
    q, k, v = (dev(x) for x in orc.make_factors(1, 1, 32, 32, 1, 1, 2, 8, 8))
    o, lse = tpa_b200.tpa.fwd_device(q, k, v, 2)
    with pytest.raises(AssertionError):
        tpa_b200.tpa.bwd_device(q, k, v, 2, None, None, 1.0, False, o, lse, o[:, :16])
    with pytest.raises(NotImplementedError):
        tpa_b200.tpa.bwd_device(q, k, v, 2, None, None, 1.0, False, o, lse, o, grad_dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        tpa_b200.tpa.bwd_device(q, k, v, 2, None, None, 1.0, False, o, lse, o, accumulate_dq=True)


TC_CASES = [
    # b, lq, lk, rq, rk, h, d, seg_q, seg_k, causal, q_off, k_off
    (1, 128, 128, 2, 2, 8, 128, 0, 0, False, 0, 0),
    (1, 256, 256, 2, 2, 8, 64, 0, 0, True, 0, 0),
    (2, 384, 640, 3, 2, 8, 128, 0, 0, False, 0, 0),
    (1, 512, 512, 6, 2, 16, 128, 0, 0, True, 0, 0),
    (1, 300, 200, 2, 4, 8, 128, 0, 0, False, 0, 0),       # ragged last tiles
    (2, 130, 260, 2, 2, 8, 64, 0, 0, True, 200, 0),       # ragged + offsets
    (1, 256, 384, 2, 2, 8, 128, 0, 0, True, 128, 0),      # later query block of a ring
    (1, 256, 256, 2, 2, 8, 128, 0, 0, True, 0, 100),      # rows that see no key
    (1, 384, 512, 2, 2, 8, 128, 100, 100, True, 0, 0),    # packed sequences
    (1, 256, 256, 1, 1, 8, 64, 32, 96, False, 0, 0),      # ids that leave rows empty
]


@pytest.mark.parametrize("case", TC_CASES)
def test_tensor_core_backward(case):
    """tcgen05 pair passes against the fp32 oracle on bf16-rounded inputs, and against the
    SIMT passes on the same inputs."""
    b, lq, lk, rq, rk, h, d, sq, sk, causal, q_off, k_off = case
    q, k, v = orc.make_factors(21, b, lq, lk, rq, rk, h, d, d)
    tq, tk, tv = (dev(x, torch.bfloat16) for x in (q, k, v))
    do = dev(_do(21, (b, lq, h, d)), torch.bfloat16)
    qs = orc.segment_ids(b, lq, sq) if sq else None
    ks = orc.segment_ids(b, lk, sk) if sk else None
    dqs, dks = (None if qs is None else dev(qs)), (None if ks is None else dev(ks))
    scale = d**-0.5
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, dqs, dks, scale, causal, q_offset=q_off, k_offset=k_off)
    f = lambda t: t.float().cpu().numpy()
    want = orc.tpa_bwd_reference(f(tq), f(tk), f(tv), f(do), h, qs, ks, scale, causal,
                                 q_offset=q_off, k_offset=k_off)
    n0 = _capi.lib.tpa_launch_count()
    got = tpa_b200.tpa.bwd_device(tq, tk, tv, h, dqs, dks, scale, causal, o, lse, do, q_offset=q_off,
                                  k_offset=k_off, kernel="sm100", grad_dtype=torch.float32)
    assert _capi.lib.tpa_launch_count() == n0 + 8
    st, detail = tpa_b200.tpa.device_status_bwd()
    assert st == 0, detail
    simt = tpa_b200.tpa.bwd_device(tq, tk, tv, h, dqs, dks, scale, causal, o, lse, do, q_offset=q_off,
                                   k_offset=k_off, kernel="simt", grad_dtype=torch.float32)
    for name, g, s_, w in zip(("dq", "dk", "dv"), got, simt, want):
        g, s_ = f(g), f(s_)
        assert np.isfinite(g).all(), name
        assert _rel(g, w) < 3e-2, (name, _rel(g, w))
        assert _rel(g, s_) < 2e-2, (name, _rel(g, s_))
    # bitwise reproducible
    again = tpa_b200.tpa.bwd_device(tq, tk, tv, h, dqs, dks, scale, causal, o, lse, do, q_offset=q_off,
                                    k_offset=k_off, kernel="sm100", grad_dtype=torch.float32)
    for g, a in zip(got, again):
        assert torch.equal(g, a)
