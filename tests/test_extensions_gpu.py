"""GPU parity of what this library adds around the reference's forward: key parts (a whole ring in
one call), sliding-window / dilated masks, rotary embedding of the dim factors.  Each against the
CPU oracle's definition of the same thing (oracle/tpa_oracle.py: position_mask, key_positions,
apply_rope), through the C ABI.  fp32: max-abs <= 1e-5; bf16: max-abs <= 2e-2, mean-abs <= 5e-3.
"""

import numpy as np
import pytest
import torch

from oracle import tpa_oracle as orc

import tpa_b200
from tpa_b200 import _capi

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def no_device_timeout():
    yield
    st, detail = tpa_b200.tpa.device_status()
    assert st == 0, (st, [hex(x) for x in detail])


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def _cmp(o, ref, dtype):
    o = o.float().cpu().numpy()
    assert np.array_equal(np.isnan(o), np.isnan(ref))
    diff = np.abs(np.nan_to_num(o) - np.nan_to_num(ref))
    if dtype == torch.float32:
        assert diff.max() <= 1e-5, float(diff.max())
    else:
        assert diff.max() <= 2e-2 and diff.mean() <= 5e-3, (float(diff.max()), float(diff.mean()))


def _parts(x, n):
    """[b, n * l, ...] -> [n, b, l, ...] contiguous: the shards of a ring gathered in one buffer."""
    b, t = x.shape[:2]
    return x.reshape(b, n, t // n, *x.shape[2:]).transpose(0, 1).contiguous()


@pytest.mark.parametrize("dtype,kernel,d", [(torch.float32, "simt", 32), (torch.bfloat16, "simt", 64),
                                            (torch.bfloat16, "sm100_staged", 64), (torch.bfloat16, "sm100_staged", 128)])
@pytest.mark.parametrize("n,seg,causal", [(4, 0, True), (8, 200, True), (2, 0, False), (3, 150, True)])
def test_whole_ring_in_one_call(dtype, kernel, d, n, seg, causal):
    """N key parts with the part-local mask = the N steps of the reference's ring scan and their
    merges (tpa/ring_tpa.py:60-112), for every rank's query shard."""
    b, l, h, rq, rk = 2, 256, 8, 3, 2
    t = n * l
    q, k, v = orc.make_factors(61, b, t, t, rq, rk, h, d, d)
    tq, tk, tv = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    q, k, v = (x.float().cpu().numpy() for x in (tq, tk, tv))
    ids = orc.segment_ids(b, t, seg) if seg else np.zeros((b, t), np.int32)
    ref = orc.ring_tpa_reference(q, k, v, ids, ids, h, n, sm_scale=d**-0.5, causal=causal, mask_mode="reference_local",
                                 dtype=np.float32)
    kp, vp, idp = _parts(tk, n), _parts(tv, n), _parts(dev(ids), n)
    for r in (0, n - 1):
        sl = slice(r * l, (r + 1) * l)
        o, lse = tpa_b200.tpa.fwd_device(tq[:, sl].contiguous(), kp, vp, h, dev(ids)[:, sl].contiguous(), idp, d**-0.5, causal,
                                         kv_parts=n, per_part=True, kernel=kernel)
        _cmp(o, ref[:, sl], dtype)
        assert torch.isfinite(lse).all()


@pytest.mark.parametrize("dtype,kernel,d", [(torch.float32, "simt", 32), (torch.bfloat16, "sm100_staged", 64),
                                            (torch.bfloat16, "sm100_staged", 128)])
@pytest.mark.parametrize("n,seg,causal", [(4, 0, True), (8, 200, True), (3, 0, False)])
def test_ring_as_own_shard_then_visiting_parts(dtype, kernel, d, n, seg, causal):
    """What ring_tpa does on every rank: the rank's own shard first (the partial (o, lse) stays as
    carried state), then the N - 1 visiting shards in ONE call as key parts that starts from that
    state -- in arrival order, which the shard-local mask makes irrelevant.  Equals the N steps of
    the reference's scan (tpa/ring_tpa.py:60-112)."""
    b, l, h, rq, rk = 2, 256, 8, 3, 2
    t = n * l
    q, k, v = orc.make_factors(67, b, t, t, rq, rk, h, d, d)
    tq, tk, tv = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    q, k, v = (x.float().cpu().numpy() for x in (tq, tk, tv))
    ids = orc.segment_ids(b, t, seg) if seg else np.zeros((b, t), np.int32)
    ref = orc.ring_tpa_reference(q, k, v, ids, ids, h, n, sm_scale=d**-0.5, causal=causal, mask_mode="reference_local",
                                 dtype=np.float32)
    tid = dev(ids)
    for r in (0, n // 2, n - 1):
        sl = slice(r * l, (r + 1) * l)
        order = [(r - hop) % n for hop in range(1, n)]  # the shards in the order the hops deliver them
        kp = torch.stack([tk[:, s * l:(s + 1) * l] for s in order]).contiguous()
        vp = torch.stack([tv[:, s * l:(s + 1) * l] for s in order]).contiguous()
        ip = torch.stack([tid[:, s * l:(s + 1) * l] for s in order]).contiguous()
        qr, idr = tq[:, sl].contiguous(), tid[:, sl].contiguous()
        state = (torch.empty((b, l, h, d), dtype=torch.float32, device="cuda"),
                 torch.empty((b, l, h), dtype=torch.float32, device="cuda"))
        tpa_b200.tpa.fwd_device(qr, tk[:, sl].contiguous(), tv[:, sl].contiguous(), h, idr, idr, d**-0.5, causal,
                                state=state, store_state=True, kernel=kernel)
        o, lse = tpa_b200.tpa.fwd_device(qr, kp, vp, h, idr, ip, d**-0.5, causal, kv_parts=n - 1, per_part=causal,
                                         state=state, load_state=True, reuse_staged_q=True, kernel=kernel)
        _cmp(o, ref[:, sl], dtype)
        assert torch.isfinite(lse).all()


@pytest.mark.parametrize("kernel,dtype", [("simt", torch.float32), ("sm100_staged", torch.bfloat16)])
def test_parts_in_sequence_order_equal_one_array(kernel, dtype):
    """Without the part-local flag the parts are just the key array cut in pieces: same result as
    the plain call, causal on positions in the whole sequence (the ring's "global" mask)."""
    b, l, n, h, d = 1, 384, 3, 8, 64
    q, k, v = orc.make_factors(62, b, l, n * l, 2, 2, h, d, d)
    tq, tk, tv = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    want, wl = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, 0.2, True, q_offset=2 * l, kernel=kernel)
    got, gl = tpa_b200.tpa.fwd_device(tq, _parts(tk, n), _parts(tv, n), h, None, None, 0.2, True, q_offset=2 * l,
                                      kv_parts=n, kernel=kernel)
    # the same tiles in the same order on the tensor-core path; the generic kernel may split the keys
    # of the plain call over CTAs and merge partials, which rounds differently
    if kernel == "simt":
        assert (want - got).abs().max() <= 1e-6 and (wl - gl).abs().max() <= 1e-5
    else:
        assert torch.equal(want, got) and torch.equal(wl, gl)


WINDOWS = [  # lq, lk, causal, window, dilation, q_off, k_off
    (512, 512, True, 100, 1, 0, 0),
    (512, 512, False, 64, 1, 0, 0),
    (300, 700, True, 128, 1, 400, 0),
    (384, 384, True, 33, 4, 0, 0),
    (256, 640, False, 50, 3, 100, 37),
    (256, 256, True, 0, 5, 0, 0),
    (640, 640, True, 1, 1, 0, 0),
]


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "simt"), (torch.bfloat16, "sm100_staged")])
@pytest.mark.parametrize("case", WINDOWS)
def test_sliding_window_and_dilation(dtype, kernel, case):
    lq, lk, causal, window, dilation, q_off, k_off = case
    b, h, d = 2, 8, 64
    q, k, v = orc.make_factors(63, b, lq, lk, 3, 2, h, d, d)
    tq, tk, tv = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    q, k, v = (x.float().cpu().numpy() for x in (tq, tk, tv))
    ref, lref = orc.tpa_reference(q, k, v, h, sm_scale=d**-0.5, causal=causal, q_offset=q_off, k_offset=k_off,
                                  window=window, dilation=dilation, return_lse=True, dtype=np.float32)
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, causal, q_offset=q_off, k_offset=k_off,
                                     window=window, dilation=dilation, kernel=kernel)
    _cmp(o, ref, dtype)
    fin = np.isfinite(lref)
    assert np.array_equal(np.isfinite(lse.cpu().numpy()), fin)
    assert np.abs(lse.cpu().numpy()[fin] - lref[fin]).max() <= (1e-4 if dtype == torch.float32 else 2e-2)


def test_window_walks_only_its_own_tiles():
    """A causal window of 1024 over 16384 tokens walks 11 key tiles per row block instead of 65 on average."""
    b, t, h, d = 1, 16384, 8, 128
    q, k, v = orc.make_factors(64, b, t, t, 2, 2, h, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)

    def run(window):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True, window=window)
        e0.record()
        for _ in range(10):
            tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True, window=window)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    assert run(1024) < 0.5 * run(0)


@pytest.mark.parametrize("dtype,kernel,d", [(torch.float32, "simt", 32), (torch.bfloat16, "sm100_staged", 64),
                                            (torch.bfloat16, "sm100_staged", 128), (torch.bfloat16, "auto", 128)])
@pytest.mark.parametrize("lq,lk,q_off,k_off", [(256, 256, 0, 0), (130, 500, 370, 0), (1, 1024, 1023, 0)])
def test_rotary_embedding_of_the_dim_factors(dtype, kernel, d, lq, lk, q_off, k_off):
    """rope=(cos, sin): B_Q row i turns by the angle of position i + q_off, B_K row j by j + k_off;
    against the oracle run on factors rotated on the CPU."""
    b, h = 2, 8
    q, k, v = orc.make_factors(65, b, lq, lk, 3, 2, h, d, d)
    tq, tk, tv = dev(q * 6.0, dtype), dev(k, dtype), dev(v, dtype)  # logits large enough for positions to matter
    q, k, v = (x.float().cpu().numpy() for x in (tq, tk, tv))
    cos, sin = orc.rope_tables(1100, d)
    ref = orc.tpa_reference(orc.apply_rope(q, h, cos, sin, q_off), orc.apply_rope(k, h, cos, sin, k_off), v, h,
                            sm_scale=d**-0.5, causal=True, q_offset=q_off, k_offset=k_off, dtype=np.float32)
    o, _ = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True, q_offset=q_off, k_offset=k_off,
                                   rope=(dev(cos), dev(sin)), rope_q_offset=q_off, rope_k_offset=k_off, kernel=kernel)
    _cmp(o, ref, dtype)
    # and it is not a no-op
    plain, _ = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True, q_offset=q_off, k_offset=k_off, kernel=kernel)
    if lk > 1 and lq > 1:
        assert (plain.float() - o.float()).abs().max() > 1e-3


def test_extensions_are_refused_where_not_implemented():
    b, l, h, d = 1, 512, 8, 64
    q, k, v = orc.make_factors(66, b, l, l, 2, 2, h, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    with pytest.raises(ValueError):  # the in-kernel-rebuild variant has no window
        tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, 1.0, True, window=64, kernel="sm100_fused")
    with pytest.raises(ValueError):  # rope tables too short for the rows of the call
        cos, sin = orc.rope_tables(100, d)
        tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, 1.0, True, rope=(dev(cos), dev(sin)))
    # a single decode row with a window goes to a kernel that implements it
    o, _ = tpa_b200.tpa.fwd_device(tq[:, -1:].contiguous(), tk, tv, h, None, None, d**-0.5, True, q_offset=l - 1, window=100)
    f = lambda x: x.float().cpu().numpy()  # noqa: E731
    ref = orc.tpa_reference(f(tq[:, -1:]), f(tk), f(tv), h, sm_scale=d**-0.5, causal=True, q_offset=l - 1, window=100,
                            dtype=np.float32)
    _cmp(o, ref, torch.bfloat16)

