"""The CPU oracle against fixtures produced by the reference's own source (tests/golden/make_golden.py).

Tolerance is the reference's own: rtol = atol = 1e-3 (tpa/tpa_test.py:125,
tpa/ring_tpa_test.py:138).  A tighter 2e-5 bound is also asserted because both
sides are numpy evaluations of the same formulas.
"""

import numpy as np
import pytest

from conftest import load_golden
from oracle import tpa_oracle as orc

FWD = load_golden("fwd_matrix")
RING = load_golden("ring_matrix")
EXTRA = load_golden("extra")
BWD = load_golden("bwd_matrix")


def _close(a, b, tight=2e-5):
    np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-3, equal_nan=True)
    assert np.array_equal(np.isnan(a), np.isnan(b))
    assert np.nanmax(np.abs(a - b)) <= tight


@pytest.mark.parametrize("case", sorted(FWD))
def test_forward_matrix(case):
    g = FWD[case]
    seed, b, lq, lk, rq, rk, h, dk, dv, seg = (int(x) for x in g["meta"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="uniform")
    qs = orc.segment_ids(b, lq, seg) if seg else None
    ks = orc.segment_ids(b, lk, seg) if seg else None
    o, l = orc.tpa_reference(q, k, v, h, qs, ks, return_lse=True)
    _close(o, g["o"])
    _close(l, g["lse"])
    ob, lb = orc.tpa_fwd_blockwise(q, k, v, h, qs, ks)
    _close(ob, g["o"])
    _close(lb, g["lse"])


@pytest.mark.parametrize("case", sorted(RING))
def test_ring_matrix(case):
    g = RING[case]
    seed, b, lq, lk, rq, rk, h, dk, dv, seg, n = (int(x) for x in g["meta"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="uniform")
    qs, ks = orc.segment_ids(b, lq, seg), orc.segment_ids(b, lk, seg)
    o = orc.ring_tpa_reference(q, k, v, qs, ks, h, n)
    _close(o, g["o"])
    # non-causal: the ring equals the unsharded definition
    _close(orc.tpa_reference(q, k, v, h, qs, ks), g["o"])


@pytest.mark.parametrize("case", ["c0_causal", "causal_seg", "peaky", "empty_rows"])
def test_untested_by_reference_forward(case):
    g = EXTRA[case]
    seed, b, lq, lk, rq, rk, h, dk, dv, sq, sk, causal, dist = (int(x) for x in g["meta"])
    sm = float(g["sm_scale"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist=["normal", "uniform"][dist])
    qs = orc.segment_ids(b, lq, sq) if sq else None
    ks = orc.segment_ids(b, lk, sk) if sk else None
    o, l = orc.tpa_reference(q, k, v, h, qs, ks, sm_scale=sm, causal=bool(causal), return_lse=True)
    _close(o, g["o"])
    _close(l, g["lse"])
    ob, lb = orc.tpa_fwd_blockwise(q, k, v, h, qs, ks, sm_scale=sm, causal=bool(causal))
    _close(ob, g["o"])
    _close(lb, g["lse"])
    if case == "empty_rows":
        assert np.isnan(g["o"]).any() and np.isneginf(g["lse"]).any()
    # the torch variant used for large cases and the CPU baseline agrees too
    ot = orc.tpa_reference_torch(q, k, v, h, qs, ks, sm_scale=sm, causal=bool(causal)).numpy()
    _close(ot, g["o"], tight=1e-4)


@pytest.mark.parametrize("case", ["ring_causal_n4", "ring_causal_n8_seg"])
def test_ring_causal_is_shard_local_in_the_reference(case):
    g = EXTRA[case]
    seed, b, l, _, rq, rk, h, dk, dv, seg, n, causal = (int(x) for x in g["meta"])
    sm = float(g["sm_scale"])
    q, k, v = orc.make_factors(seed, b, l, l, rq, rk, h, dk, dv, dist="normal")
    qs = orc.segment_ids(b, l, seg) if seg else np.zeros((b, l), np.int32)
    o = orc.ring_tpa_reference(q, k, v, qs, qs, h, n, sm_scale=sm, causal=True,
                               mask_mode="reference_local")
    _close(o, g["o"])
    # and global causal is a different function (it equals the unsharded causal forward)
    og = orc.ring_tpa_reference(q, k, v, qs, qs, h, n, sm_scale=sm, causal=True, mask_mode="global")
    _close(og, orc.tpa_reference(q, k, v, h, qs, qs, sm_scale=sm, causal=True), tight=1e-9)
    assert np.nanmax(np.abs(og - g["o"])) > 1e-2


def _bwd_inputs(g):
    seed, b, lq, lk, rq, rk, h, dk, dv, seg = (int(x) for x in g["meta"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="normal")
    do = np.random.Generator(np.random.Philox(key=seed + 5000)).standard_normal((b, lq, h, dv), dtype=np.float32)
    qs = orc.segment_ids(b, lq, seg) if seg else None
    ks = orc.segment_ids(b, lk, seg) if seg else None
    return q, k, v, do, h, qs, ks


@pytest.mark.parametrize("case", sorted(BWD))
def test_backward_matrix(case):
    """Oracle gradients against the reference's own _tpa_bwd; tolerance of tpa/tpa_test.py:203-205."""
    g = BWD[case]
    q, k, v, do, h, qs, ks = _bwd_inputs(g)
    grads = orc.tpa_bwd_reference(q, k, v, do, h, qs, ks)
    for name, got in zip(("dq", "dk", "dv"), grads):
        np.testing.assert_allclose(got, g[name], atol=1e-3, rtol=1e-2)
        assert np.max(np.abs(got - g[name]) / (1e-3 + 1e-2 * np.abs(g[name]))) < 0.05


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("seg", [None, 9])
def test_backward_oracle_is_the_autograd_of_the_definition(causal, seg):
    """jax.grad of reference() is what tpa/tpa_test.py:196 compares with; torch autograd of the
    same definition stands in for it (causal and multi-head cases included)."""
    import torch

    b, lq, lk, h, dk, dv = 2, 24, 40, 6, 8, 10
    q, k, v = orc.make_factors(3, b, lq, lk, 3, 2, h, dk, dv)
    do = np.random.default_rng(0).standard_normal((b, lq, h, dv))
    qs = orc.segment_ids(b, lq, seg) if seg else None
    ks = orc.segment_ids(b, lk, seg) if seg else None
    grads = orc.tpa_bwd_reference(q, k, v, do, h, qs, ks, 0.3, causal)
    tq, tk, tv = (torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (q, k, v))
    o = orc.tpa_reference_torch(tq, tk, tv, h, None if qs is None else torch.tensor(qs),
                                None if ks is None else torch.tensor(ks), 0.3, causal)
    loss = (torch.nan_to_num(o) * torch.tensor(do, dtype=o.dtype)).sum()
    want = torch.autograd.grad(loss, (tq, tk, tv))
    for got, w in zip(grads, want):
        np.testing.assert_allclose(got, w.numpy(), atol=2e-5, rtol=1e-4)


# --------------------------------------------------------------------------- extensions of the definition


def test_parts_with_part_local_mask_equal_the_ring_definition():
    """One call whose keys are the N shards as N parts, compared on part-local indices, is the
    reference's ring with causal=True (shard-local mask at every step, tpa/ring_tpa.py:73-91)."""
    n, b, l, h, d = 4, 2, 64, 2, 8
    q, k, v = orc.make_factors(7, b, l * n, l * n, 3, 2, h, d, d)
    ids = orc.segment_ids(b, l * n, 24)
    ring = orc.ring_tpa_reference(q, k, v, ids, ids, h, n, sm_scale=0.3, causal=True, mask_mode="reference_local")
    for r in range(n):
        sl = slice(r * l, (r + 1) * l)
        o = orc.tpa_reference(q[:, sl], k, v, h, ids[:, sl], ids, sm_scale=0.3, causal=True, kv_parts=n, per_part=True)
        np.testing.assert_allclose(o, ring[:, sl], rtol=1e-12, atol=1e-12, equal_nan=True)


def test_window_and_dilation_masks_by_brute_force():
    for causal in (False, True):
        for window, dilation in ((0, 3), (5, 1), (4, 2)):
            keep = orc.position_mask(np.arange(40) + 7, np.arange(50) + 2, causal, window, dilation)
            for i in range(40):
                for j in range(50):
                    diff = (i + 7) - (j + 2)
                    want = (not causal or diff >= 0) and diff % dilation == 0
                    if window:
                        want = want and abs(diff) < window * dilation
                    assert keep[i, j] == want, (causal, window, dilation, i, j)
    # a causal window of w keeps exactly min(w, i + 1) keys for row i
    keep = orc.position_mask(np.arange(30), np.arange(30), True, 6, 1)
    assert [int(r.sum()) for r in keep] == [min(6, i + 1) for i in range(30)]


def test_rope_on_the_dim_factors_is_rope_on_the_rebuilt_rows():
    """Rotating B before the rank sum equals rotating Q and K rows after it, and the logits then
    depend on relative position only (the defining property of the rotary embedding)."""
    b, l, h, d = 1, 12, 3, 16
    q, k, v = orc.make_factors(11, b, l, l, 4, 2, h, d, d, dtype=np.float64)
    cos, sin = orc.rope_tables(64, d, dtype=np.float64)
    q_, k_, _ = orc.materialize(q, k, v, h)
    qr, kr, _ = orc.materialize(orc.apply_rope(q, h, cos, sin, 5), orc.apply_rope(k, h, cos, sin, 5), v, h)

    def rot(x, off):
        out = x.copy()
        c, s_ = cos[off:off + l][None, :, None, :], sin[off:off + l][None, :, None, :]
        out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s_
        out[..., 1::2] = x[..., 0::2] * s_ + x[..., 1::2] * c
        return out

    np.testing.assert_allclose(qr, rot(q_, 5), atol=1e-12)
    np.testing.assert_allclose(kr, rot(k_, 5), atol=1e-12)
    # shift both offsets: q.k of the same (row, key) pair is unchanged
    q2, k2, _ = orc.materialize(orc.apply_rope(q, h, cos, sin, 20), orc.apply_rope(k, h, cos, sin, 20), v, h)
    np.testing.assert_allclose(np.einsum("bqhd,bkhd->bhqk", qr, kr), np.einsum("bqhd,bkhd->bhqk", q2, k2), atol=1e-10)
    # the head factor is untouched
    assert np.array_equal(orc.apply_rope(q, h, cos, sin, 3)[..., :h], q[..., :h])
