"""GPU parity: the CUDA path, called through the C ABI, against the golden fixtures and the oracle.

Tolerances: fp32 max-abs <= 1e-5 on the benchmark's fp32 configuration and
rtol = atol = 1e-3 (tpa/tpa_test.py:125) on the reference's own test matrix, where the
tighter 2e-5 bound is also asserted; bf16 max-abs <= 2e-2 and mean-abs <= 5e-3.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import tpa_oracle as orc

import tpa_b200
from tpa_b200 import _capi

pytestmark = pytest.mark.gpu

FWD = load_golden("fwd_matrix")
RING = load_golden("ring_matrix")
EXTRA = load_golden("extra")


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def assert_close(a, b, tight=2e-5):
    np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-3, equal_nan=True)
    assert np.array_equal(np.isnan(a), np.isnan(b))
    assert np.nanmax(np.abs(a - b)) <= tight


def test_extension_loaded_and_counts_launches():
    n0 = _capi.lib.tpa_launch_count()
    q, k, v = orc.make_factors(1, 1, 8, 8, 1, 1, 1, 4, 6)
    tpa_b200.tpa.tpa(dev(q), dev(k), dev(v), num_heads=1)
    torch.cuda.synchronize()
    assert _capi.lib.tpa_launch_count() == n0 + 1


@pytest.mark.parametrize("nomat", [False, True])
@pytest.mark.parametrize("case", sorted(FWD))
def test_reference_forward_matrix(case, nomat):
    """The 48 cases of tpa/tpa_test.py:60-125 against outputs of the reference's kernel."""
    g = FWD[case]
    seed, b, lq, lk, rq, rk, h, dk, dv, seg = (int(x) for x in g["meta"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="uniform")
    qs = dev(orc.segment_ids(b, lq, seg)) if seg else None
    ks = dev(orc.segment_ids(b, lk, seg)) if seg else None
    o, res = tpa_b200.tpa._tpa_fwd(dev(q), dev(k), dev(v), h, qs, ks, 1.0, False, None, nomat, False, True)
    assert o.shape == (b, lq, h, dv)
    assert_close(o.cpu().numpy(), g["o"])
    assert_close(res[-1].cpu().numpy(), g["lse"])


@pytest.mark.parametrize("case", ["c0_causal", "causal_seg", "peaky", "empty_rows"])
def test_causal_scale_and_empty_rows(case):
    g = EXTRA[case]
    seed, b, lq, lk, rq, rk, h, dk, dv, sq, sk, causal, dist = (int(x) for x in g["meta"])
    sm = float(g["sm_scale"])
    q, k, v = orc.make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist=["normal", "uniform"][dist])
    qs = dev(orc.segment_ids(b, lq, sq)) if sq else None
    ks = dev(orc.segment_ids(b, lk, sk)) if sk else None
    o, res = tpa_b200.tpa._tpa_fwd(dev(q), dev(k), dev(v), h, qs, ks, sm, bool(causal), None, False, False, False)
    o = o.cpu().numpy()
    # fp32 bound of the benchmark: max-abs <= 1e-5 against the reference's output
    assert np.nanmax(np.abs(o - g["o"])) <= 1e-5
    assert np.array_equal(np.isnan(o), np.isnan(g["o"]))
    assert_close(res[-1].cpu().numpy(), g["lse"])
    # against the fp64 oracle as well
    ref = orc.tpa_reference(q, k, v, h, None if qs is None else qs.cpu().numpy(),
                            None if ks is None else ks.cpu().numpy(), sm_scale=sm, causal=bool(causal))
    assert np.nanmax(np.abs(o - ref)) <= 1e-5


def test_host_arrays_round_trip():
    """numpy in -> numpy out through the public call (copies inside the call)."""
    q, k, v = orc.make_factors(5, 2, 128, 128, 2, 2, 4, 16, 16)
    o = tpa_b200.tpa.tpa(q, k, v, num_heads=4, sm_scale=0.25, causal=True)
    assert isinstance(o, np.ndarray)
    assert np.max(np.abs(o - orc.tpa_reference(q, k, v, 4, sm_scale=0.25, causal=True))) <= 1e-5


@pytest.mark.parametrize("b,t,seg,causal,pinned", [(1, 4096, 0, True, True), (1, 4096, 700, True, False),
                                                   (4, 1024, 0, False, True), (8, 512, 100, True, True),
                                                   (3, 512, 0, True, True)])
def test_host_arrays_pipelined(b, t, seg, causal, pinned):
    """Host tensors through tpa(): the call moves them in chunks (query-row blocks of one batch
    element, or batch elements) while it computes, and gives the device call's result (to bf16
    rounding: a chunk of few rows may split its keys over CTAs and merge partials)."""
    h, d = 8, 64
    q, k, v = orc.make_factors(6, b, t, t, 3, 2, h, d, d)
    hq, hk, hv = (torch.from_numpy(x).bfloat16() for x in (q, k, v))
    ids = torch.from_numpy(orc.segment_ids(b, t, seg)) if seg else None
    if pinned:
        hq, hk, hv = hq.pin_memory(), hk.pin_memory(), hv.pin_memory()
    out = torch.empty((b, t, h, d), dtype=torch.bfloat16)
    out = out.pin_memory() if pinned else out
    got = tpa_b200.tpa.tpa(hq, hk, hv, h, ids, ids, sm_scale=d**-0.5, causal=causal, out=out)
    assert got is out and not got.is_cuda
    dq, dk, dv_ = hq.cuda(), hk.cuda(), hv.cuda()
    did = None if ids is None else ids.cuda()
    want = tpa_b200.tpa.tpa(dq, dk, dv_, h, did, did, sm_scale=d**-0.5, causal=causal)
    assert torch.equal(torch.isnan(got), torch.isnan(want.cpu()))
    assert (torch.nan_to_num(got.float()) - torch.nan_to_num(want.float().cpu())).abs().max() <= 2e-3
    fresh = tpa_b200.tpa.tpa(hq, hk, hv, h, ids, ids, sm_scale=d**-0.5, causal=causal)  # no out=: a new host tensor
    assert torch.equal(torch.nan_to_num(fresh.float()), torch.nan_to_num(got.float()))
    with pytest.raises(ValueError):
        tpa_b200.tpa.tpa(dq, dk, dv_, h, sm_scale=1.0, out=out)


@pytest.mark.parametrize("shape", [(1, 100, 77, 3, 2, 3, 7, 9), (2, 33, 200, 1, 5, 5, 20, 130), (1, 64, 64, 2, 2, 2, 256, 256)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_shapes_low_level(shape, causal):
    """Lengths that are not multiples of any tile, dv > 128, offsets: the C entry point itself."""
    b, lq, lk, rq, rk, h, dk, dv = shape
    q, k, v = orc.make_factors(31, b, lq, lk, rq, rk, h, dk, dv)
    qo, ko = (37, 5) if causal else (0, 0)
    o, l = tpa_b200.tpa.fwd_device(dev(q), dev(k), dev(v), h, None, None, 0.4, causal, q_offset=qo, k_offset=ko)
    ref, lref = orc.tpa_reference(q, k, v, h, sm_scale=0.4, causal=causal, q_offset=qo, k_offset=ko, return_lse=True)
    assert_close(o.cpu().numpy(), ref)
    assert_close(l.cpu().numpy(), lref)


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "simt"), (torch.bfloat16, "simt"),
                                          (torch.bfloat16, "sm100_fused"), (torch.bfloat16, "sm100_staged")])
@pytest.mark.parametrize("mode", ["reference_local", "global"])
def test_state_chaining_equals_ring_oracle(dtype, kernel, mode):
    """N ring steps emulated on one GPU through TPA_FLAG_STATE_LOAD/STORE vs the ring oracle."""
    n, b, l, rq, rk, h, d = 4, 1, 1024, 3, 2, 8, 64
    q, k, v = orc.make_factors(41, b, l, l, rq, rk, h, d, d)
    tq, tk, tv = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    q, k, v = (t.float().cpu().numpy() for t in (tq, tk, tv))
    ids = np.zeros((b, l), np.int32)
    ref = orc.ring_tpa_reference(q, k, v, ids, ids, h, n, sm_scale=d**-0.5, causal=True, mask_mode=mode)
    per = l // n
    out = torch.empty(b, l, h, d, dtype=dtype, device="cuda")
    for r in range(n):
        sl = slice(r * per, (r + 1) * per)
        state = (torch.empty(b, per, h, d, device="cuda"), torch.empty(b, per, h, device="cuda"))
        steps = [s for s in range(n) if not (mode == "global" and (r - s) % n > r)]
        for i, s in enumerate(steps):
            src = (r - s) % n
            ks = slice(src * per, (src + 1) * per)
            off = (r * per, src * per) if mode == "global" else (0, 0)
            o_r = torch.empty(b, per, h, d, dtype=dtype, device="cuda")
            tpa_b200.tpa.fwd_device(tq[:, sl], tk[:, ks], tv[:, ks], h, None, None, d**-0.5, True,
                                    q_offset=off[0], k_offset=off[1], state=state, load_state=i > 0,
                                    store_state=i < len(steps) - 1, out=o_r, kernel=kernel)
        out[:, sl] = o_r
    diff = np.abs(out.float().cpu().numpy() - ref)
    if dtype == torch.float32:
        assert diff.max() <= 1e-5
    else:
        assert diff.max() <= 2e-2 and diff.mean() <= 5e-3


def test_bitwise_reproducible():
    q, k, v = orc.make_factors(3, 2, 256, 256, 6, 2, 8, 64, 64)
    a = tpa_b200.tpa.tpa(dev(q), dev(k), dev(v), num_heads=8, sm_scale=0.125, causal=True)
    b = tpa_b200.tpa.tpa(dev(q), dev(k), dev(v), num_heads=8, sm_scale=0.125, causal=True)
    assert torch.equal(a, b)


# --------------------------------------------------------------------------- bf16 configurations


@pytest.fixture(autouse=True)
def no_device_timeout():
    """After every test: no bounded device-side wait may have run out."""
    yield
    st, detail = tpa_b200.tpa.device_status()
    assert st == 0, (st, [hex(x) for x in detail])


@pytest.mark.parametrize("kernel", ["sm100_fused", "sm100_staged"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("t", [128, 256, 384, 1024])
@pytest.mark.parametrize("causal", [False, True])
def test_sm100_small(d, t, causal, kernel):
    """Both tensor-core variants on one to a few tiles, all rows checked, LSE included."""
    q, k, v = orc.make_factors(50 + t + d, 2, t, t, 3, 2, 8, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    assert tpa_b200.tpa.query_kernel(tq, tk, tv, 8, causal=causal)["kernel"] == "sm100_staged"
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, 8, None, None, d**-0.5, causal, kernel=kernel)
    ref, lref = orc.tpa_reference_torch(tq.float().cpu(), tk.float().cpu(), tv.float().cpu(), 8,
                                        sm_scale=d**-0.5, causal=causal, return_lse=True)
    diff = (o.float().cpu() - ref).abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3, (float(diff.max()), float(diff.mean()))
    assert (lse.cpu() - lref).abs().max() <= 1e-2


def bf16_case(seed, b, t, h, d, rq, rk, causal, kernel="auto", rows=None, segs=None, scale=1.0):
    q, k, v = orc.make_factors(seed, b, t, t, rq, rk, h, d, d)
    tq, tk, tv = dev(q * scale, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    ids = None if segs is None else dev(orc.segment_ids(b, t, segs))
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, ids, ids, d**-0.5, causal, kernel=kernel)
    ref, lref = orc.tpa_reference_torch(tq.float().cpu(), tk.float().cpu(), tv.float().cpu(), h,
                                        None if ids is None else ids.cpu(), None if ids is None else ids.cpu(),
                                        sm_scale=d**-0.5, causal=causal, rows=rows, return_lse=True)
    o = o.float().cpu()
    lse = lse.cpu()
    if rows is not None:
        o, lse = o[:, rows], lse[:, rows]
    diff = (o - ref).abs()
    return float(diff.max()), float(diff.mean()), float((lse - lref).abs().max()), float(ref.abs().max())


@pytest.mark.parametrize("kernel", ["simt", "sm100_fused", "auto"])
def test_bf16_config1_shape_reduced_batch(kernel):
    """Configuration 1 (bf16 causal T=4096 h=32 d=128 R 6/2/2) at batch 1, sampled rows."""
    rows = torch.cat([torch.arange(0, 4), torch.arange(4092, 4096), torch.randperm(4096, generator=torch.Generator().manual_seed(0))[:120]])
    mx, mean, lerr, _ = bf16_case(1, 1, 4096, 32, 128, 6, 2, True, kernel, rows=rows)
    assert mx <= 2e-2 and mean <= 5e-3 and lerr <= 1e-2, (mx, mean, lerr)


@pytest.mark.parametrize("kernel", ["simt", "sm100_fused", "auto"])
def test_bf16_config4_noncausal_high_rank(kernel):
    """Configuration 4 (bf16 non-causal T=2048 h=16 d=64 R 8/8/8) at batch 1, with the dense
    attention cross-check: the oracle materialises Q, K, V and runs plain softmax attention."""
    mx, mean, lerr, _ = bf16_case(4, 1, 2048, 16, 64, 8, 8, False, kernel)
    assert mx <= 2e-2 and mean <= 5e-3 and lerr <= 1e-2, (mx, mean, lerr)


@pytest.mark.parametrize("kernel", ["simt", "sm100_fused", "sm100_staged"])
def test_bf16_peaky_and_segments(kernel):
    """Large logits (online-softmax rescaling really happens) and packed segments."""
    mx, mean, lerr, refmax = bf16_case(6, 2, 512, 8, 128, 4, 4, True, kernel, segs=200, scale=24.0)
    assert mx <= 2e-2 * max(1.0, refmax) and mean <= 5e-3, (mx, mean, lerr, refmax)


def _random_cases(n=14, seed=1234):
    rng = np.random.default_rng(seed)
    cases = []
    for i in range(n):
        d = int(rng.choice([64, 128]))
        cases.append(dict(
            seed=2000 + i, b=int(rng.integers(1, 3)), lq=128 * int(rng.integers(1, 9)),
            lk=128 * int(rng.integers(1, 9)), h=int(rng.choice([8, 16])), d=d,
            rq=int(rng.integers(1, 7)), rk=int(rng.integers(1, 5)), causal=bool(rng.integers(0, 2)),
            seg=int(rng.choice([0, 0, 100, 300])), q_off=128 * int(rng.integers(0, 4)),
            k_off=128 * int(rng.integers(0, 4)), scale=float(rng.choice([1.0, 1.0, 16.0]))))
    return cases


@pytest.mark.parametrize("case", _random_cases(), ids=lambda c: f"s{c['seed']}")
@pytest.mark.parametrize("kernel", ["sm100_fused", "sm100_staged"])
def test_tensor_core_variants_agree_with_generic_kernel(case, kernel):
    """Randomised shapes, ranks, offsets, segments and logit scales: each tensor-core variant
    against the fp32-math kernel on the same bf16 inputs (the latter is pinned to the oracle)."""
    c = case
    q, k, v = orc.make_factors(c["seed"], c["b"], c["lq"], c["lk"], c["rq"], c["rk"], c["h"], c["d"], c["d"])
    tq, tk, tv = dev(q * c["scale"], torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    qs = dev(orc.segment_ids(c["b"], c["lq"], c["seg"])) if c["seg"] else None
    ks = dev(orc.segment_ids(c["b"], c["lk"], c["seg"])) if c["seg"] else None
    args = dict(q_offset=c["q_off"], k_offset=c["k_off"])
    want, wl = tpa_b200.tpa.fwd_device(tq, tk, tv, c["h"], qs, ks, c["d"] ** -0.5, c["causal"], kernel="simt", **args)
    got, gl = tpa_b200.tpa.fwd_device(tq, tk, tv, c["h"], qs, ks, c["d"] ** -0.5, c["causal"], kernel=kernel, **args)
    want, got = want.float(), got.float()
    assert torch.equal(torch.isnan(want), torch.isnan(got))
    assert torch.equal(torch.isinf(wl), torch.isinf(gl))
    ok = ~torch.isnan(want)
    scale = max(1.0, float(want[ok].abs().max())) if ok.any() else 1.0
    diff = (want[ok] - got[ok]).abs()
    if diff.numel():
        assert diff.max() <= 2e-2 * scale and diff.mean() <= 5e-3 * scale, (float(diff.max()), float(diff.mean()))
    fin = ~torch.isinf(wl)
    if fin.any():
        # the tensor-core kernels round Q and K to bf16 (2^-8 relative), so a logit, and with it
        # the LSE, moves in proportion to its size
        assert ((wl[fin] - gl[fin]).abs() <= 2e-2 + 1e-2 * wl[fin].abs()).all()


@pytest.mark.parametrize("kernel", ["sm100_fused", "sm100_staged"])
@pytest.mark.parametrize("seg", [512, 300])
def test_packed_sequences_walk_only_their_own_tiles(kernel, seg):
    """Packed causal sequences: the key-tile walk starts at the block's first segment (tile
    ranges from the segment ids), results as the oracle's, and far fewer tiles are visited."""
    t, h, d = 4096, 8, 128
    q, k, v = orc.make_factors(77, 1, t, t, 3, 2, h, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    ids = dev(orc.segment_ids(1, t, seg))
    n0 = _capi.lib.tpa_launch_count()
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, ids, ids, d**-0.5, True, kernel=kernel)
    torch.cuda.synchronize()
    assert _capi.lib.tpa_launch_count() - n0 == (3 if kernel == "sm100_staged" else 2)
    ref, lref = orc.tpa_reference_torch(tq.float().cpu(), tk.float().cpu(), tv.float().cpu(), h, ids.cpu(), ids.cpu(),
                                        sm_scale=d**-0.5, causal=True, return_lse=True)
    diff = (o.float().cpu() - ref).abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3
    assert (lse.cpu() - lref).abs().max() <= 1e-2
    # timing: segments of 1024 in 16384 tokens leave 1/16 of the causal work (long enough for the
    # kernels, not the three launches, to be what is timed)
    if seg == 512 and kernel == "sm100_staged":
        t2 = 16384
        q2, k2, v2 = orc.make_factors(78, 1, t2, t2, 3, 2, h, d, d)
        uq, uk, uv = dev(q2, torch.bfloat16), dev(k2, torch.bfloat16), dev(v2, torch.bfloat16)

        def run(s):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                tpa_b200.tpa.fwd_device(uq, uk, uv, h, s, s, d**-0.5, True, kernel=kernel)
            e0.record()
            for _ in range(10):
                tpa_b200.tpa.fwd_device(uq, uk, uv, h, s, s, d**-0.5, True, kernel=kernel)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        one = dev(np.zeros((1, t2), np.int32))
        assert run(dev(orc.segment_ids(1, t2, 1024))) < 0.6 * run(one)


@pytest.mark.parametrize("d,seg,causal", [(128, 0, True), (64, 300, True), (128, 0, False)])
def test_bounded_scratch_runs_head_groups_with_the_same_result(d, seg, causal):
    """A workspace smaller than the one-pass layout: the staged kernel takes the heads in groups
    whose tiles fit and copies each group's o / lse to its place; bitwise the one-pass result."""
    b, t, h = 2, 1024, 32
    q, k, v = orc.make_factors(80, b, t, t, 3, 2, h, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    ids = dev(orc.segment_ids(b, t, seg)) if seg else None
    a = _capi.TpaFwdArgs()
    keep = tpa_b200.tpa._fill_operands(a, tq, tk, tv, h, ids, ids)
    a.o, a.sm_scale, a.flags = 4096, d**-0.5, _capi.FLAG_CAUSAL if causal else 0
    full = _capi.lib.tpa_fwd_workspace_bytes(C.byref(a))
    least = _capi.lib.tpa_fwd_workspace_bytes_min(C.byref(a))
    assert 0 < least < full, (least, full)
    del keep
    want, wl = tpa_b200.tpa.fwd_device(tq, tk, tv, h, ids, ids, d**-0.5, causal)
    for limit in (least, (least + full) // 2):
        n0 = _capi.lib.tpa_launch_count()
        got, gl = tpa_b200.tpa.fwd_device(tq, tk, tv, h, ids, ids, d**-0.5, causal, workspace_limit=limit)
        torch.cuda.synchronize()
        assert _capi.lib.tpa_launch_count() - n0 >= 4  # at least two groups of staging + attention
        assert torch.equal(torch.nan_to_num(want.float()), torch.nan_to_num(got.float())) and torch.equal(wl, gl)
    # less than the least is refused
    a2 = _capi.TpaFwdArgs()
    keep = tpa_b200.tpa._fill_operands(a2, tq, tk, tv, h, ids, ids)
    a2.o, a2.sm_scale = want.data_ptr(), d**-0.5
    small = torch.empty(least, dtype=torch.uint8, device="cuda")
    st = _capi.lib.tpa_fwd(C.byref(a2), small.data_ptr(), least - 256, None)
    assert st == _capi.TPA_ERR_WORKSPACE, (st, least, full)
    del keep


@pytest.mark.parametrize("odd_key", [None, 5, 700, 1023])
def test_uniform_ids_are_dropped_only_when_every_walked_key_agrees(odd_key):
    """All-equal ids (what a ring call passes) cost the tensor-core kernel nothing: a block whose
    rows and walked key tiles carry one id runs without id handling.  One key with another id
    anywhere in the walk must keep the element-wise test alive for the blocks that see it."""
    b, t, h, d = 1, 1024, 8, 64
    q, k, v = orc.make_factors(79, b, t, t, 2, 2, h, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    ids = np.zeros((b, t), np.int32)
    kids = ids.copy()
    if odd_key is not None:
        kids[:, odd_key] = 3
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, dev(ids), dev(kids), d**-0.5, False, kernel="sm100_staged")
    ref, lref = orc.tpa_reference_torch(tq.float().cpu(), tk.float().cpu(), tv.float().cpu(), h, torch.from_numpy(ids),
                                        torch.from_numpy(kids), sm_scale=d**-0.5, causal=False, return_lse=True)
    diff = (o.float().cpu() - ref).abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3
    assert (lse.cpu() - lref).abs().max() <= 1e-2
    if odd_key is not None:  # and the odd key really is excluded: the result differs from the id-free call
        plain, _ = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, False, kernel="sm100_staged")
        assert (plain.float() - o.float()).abs().max() > 0


@pytest.mark.parametrize("kernel", ["sm100_fused", "sm100_staged"])
@pytest.mark.parametrize("lq,lk,h,causal", [(128, 4096, 8, False), (256, 8192, 16, True), (384, 2048, 8, True)])
def test_few_queries_many_keys_split_over_ctas(kernel, lq, lk, h, causal):
    """Decode-like / cross shapes: the key tiles are split over several CTAs per row block and the
    partials merged (one more launch); with and without carried state; against the oracle."""
    d = 128
    q, k, v = orc.make_factors(91, 1, max(lq, lk), max(lq, lk), 2, 2, h, d, d)
    tq, tk, tv = dev(q[:, :lq], torch.bfloat16), dev(k[:, :lk], torch.bfloat16), dev(v[:, :lk], torch.bfloat16)
    q_off = lk - lq if causal else 0  # the queries are the last rows of the sequence
    info = tpa_b200.tpa.query_kernel(tq, tk, tv, h, kernel=kernel, causal=causal)
    assert info["grid"][1] > 1, info  # really split
    n0 = _capi.lib.tpa_launch_count()
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, causal, q_offset=q_off, kernel=kernel)
    torch.cuda.synchronize()
    assert _capi.lib.tpa_launch_count() - n0 == info["launches"]
    ref, lref = orc.tpa_reference_torch(tq.float().cpu(), tk.float().cpu(), tv.float().cpu(), h, sm_scale=d**-0.5,
                                        causal=causal, q_offset=q_off, return_lse=True)
    diff = (o.float().cpu() - ref).abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3
    assert (lse.cpu() - lref).abs().max() <= 1e-2
    # two halves of the keys chained through the carried state give the same answer
    half = lk // 2
    state = (torch.empty(1, lq, h, d, device="cuda"), torch.empty(1, lq, h, device="cuda"))
    tpa_b200.tpa.fwd_device(tq, tk[:, :half], tv[:, :half], h, None, None, d**-0.5, causal, q_offset=q_off,
                            state=state, store_state=True, kernel=kernel)
    o2, _ = tpa_b200.tpa.fwd_device(tq, tk[:, half:], tv[:, half:], h, None, None, d**-0.5, causal, q_offset=q_off,
                                    k_offset=half, state=state, load_state=True, kernel=kernel)
    d2 = (o2.float().cpu() - ref).abs()
    assert d2.max() <= 2e-2 and d2.mean() <= 5e-3


@pytest.mark.parametrize("kernel", ["sm100_fused", "sm100_staged"])
@pytest.mark.parametrize("lq,lk,seg,causal", [(1, 1000, 0, True), (100, 333, 0, False), (200, 520, 64, True),
                                              (385, 129, 0, True), (7, 4096, 0, True), (130, 8200, 300, False)])
def test_ragged_lengths_on_tensor_cores(kernel, lq, lk, seg, causal):
    """Lengths that are not multiples of the 128-row tiles (decode: a single query row): padded
    rows and keys must not leak into results; against the generic kernel and the oracle."""
    h, d = 8, 128
    q, k, v = orc.make_factors(300 + lq, 2, lq, lk, 3, 2, h, d, d)
    tq, tk, tv = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    qs = dev(orc.segment_ids(2, lq, seg)) if seg else None
    ks = dev(orc.segment_ids(2, lk, seg)) if seg else None
    q_off = max(lk - lq, 0) if causal else 0
    assert tpa_b200.tpa.query_kernel(tq, tk, tv, h, kernel=kernel, causal=causal, segments=bool(seg))["kernel"] == kernel
    # the output sits inside a larger buffer whose guard bands must stay untouched
    n = 2 * lq * h * d
    flat = torch.full((n + 8192,), 7.0, dtype=torch.bfloat16, device="cuda")
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, qs, ks, d**-0.5, causal, q_offset=q_off, kernel=kernel,
                                     out=flat[4096:4096 + n].view(2, lq, h, d))
    want, wl = tpa_b200.tpa.fwd_device(tq, tk, tv, h, qs, ks, d**-0.5, causal, q_offset=q_off, kernel="simt")
    ref = orc.tpa_reference_torch(tq.float().cpu(), tk.float().cpu(), tv.float().cpu(), h,
                                  None if qs is None else qs.cpu(), None if ks is None else ks.cpu(),
                                  sm_scale=d**-0.5, causal=causal, q_offset=q_off)
    assert bool((flat[:4096] == 7.0).all()) and bool((flat[4096 + n:] == 7.0).all())
    assert torch.equal(torch.isnan(o), torch.isnan(want))
    ok = ~torch.isnan(ref)
    diff = (o.float().cpu() - ref)[ok].abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3, (float(diff.max()), float(diff.mean()))
    fin = ~torch.isinf(wl)
    assert ((lse - wl)[fin].abs() <= 2e-2).all()


DECODE_CASES = [
    # b, lq, lk, rq, rk, h, dk, dv, seg, causal, q_off
    (2, 1, 4096, 6, 2, 32, 128, 128, 0, False, 0),
    (3, 1, 1000, 6, 2, 32, 128, 128, 0, True, 999),     # the newest token sees the whole cache
    (1, 4, 2050, 2, 4, 16, 64, 64, 0, True, 2046),      # a few speculative rows, ragged last tile
    (2, 8, 777, 3, 3, 8, 64, 128, 100, True, 700),      # rank 3 (tiles of 21 keys), packed ids, dk != dv
    (1, 2, 3000, 12, 8, 64, 128, 128, 0, True, 10),     # 64 heads, rank 8; most keys above the diagonal
    (1, 3, 512, 1, 1, 8, 16, 16, 0, False, 0),
    (2, 1, 1500, 2, 2, 48, 64, 32, 0, True, 1499),      # 48 heads: three 16-row tiles of the p * vb product
]


@pytest.mark.parametrize("case", DECODE_CASES)
def test_decode_kernel(case):
    """Few query rows against a long factor cache: the rank-space kernel (K, V never materialised)
    (the dispatcher picks it for up to six rows); against the oracle, the generic kernel, and chained through the
    carried state in two halves."""
    b, lq, lk, rq, rk, h, dk, dv, seg, causal, q_off = case
    q, k, v = orc.make_factors(33, b, lq, lk, rq, rk, h, dk, dv)
    tq, tk, tv = (dev(x, torch.bfloat16) for x in (q, k, v))
    qs = dev(orc.segment_ids(b, lq, seg) + (q_off // seg if seg else 0)) if seg else None
    ks = dev(orc.segment_ids(b, lk, seg)) if seg else None
    scale = dk**-0.5
    info = tpa_b200.tpa.query_kernel(tq, tk, tv, h, kernel="decode", causal=causal, segments=bool(seg))
    assert info["kernel"] == "decode" and info["launches"] == 2, info
    auto = tpa_b200.tpa.query_kernel(tq, tk, tv, h, causal=causal, segments=bool(seg))["kernel"]
    assert (auto == "decode") == (lq <= 6), auto  # the dispatcher takes it where it wins
    n0 = _capi.lib.tpa_launch_count()
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, qs, ks, scale, causal, q_offset=q_off, kernel="decode")
    torch.cuda.synchronize()
    assert _capi.lib.tpa_launch_count() - n0 == 2
    f = lambda t: t.float().cpu()
    ref, lref = orc.tpa_reference_torch(f(tq), f(tk), f(tv), h, None if qs is None else qs.cpu(),
                                        None if ks is None else ks.cpu(), sm_scale=scale, causal=causal,
                                        q_offset=q_off, return_lse=True)
    assert torch.equal(torch.isnan(f(o)), torch.isnan(ref))
    diff = torch.nan_to_num(f(o) - ref).abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3
    assert torch.nan_to_num(lse.cpu() - lref, nan=0.0, posinf=0.0, neginf=0.0).abs().max() <= 1e-2
    gen, _ = tpa_b200.tpa.fwd_device(tq, tk, tv, h, qs, ks, scale, causal, q_offset=q_off, kernel="simt")
    assert torch.nan_to_num(f(o) - f(gen)).abs().max() <= 2e-2
    # two halves of the cache chained through the carried state (what a ring step does)
    half = (lk // 2) // 8 * 8
    state = (torch.empty(b, lq, h, dv, device="cuda"), torch.empty(b, lq, h, device="cuda"))
    ks1, ks2 = (None, None) if ks is None else (ks[:, :half].contiguous(), ks[:, half:].contiguous())
    tpa_b200.tpa.fwd_device(tq, tk[:, :half], tv[:, :half], h, qs, ks1, scale, causal, q_offset=q_off,
                            state=state, store_state=True, kernel="decode")
    o2, _ = tpa_b200.tpa.fwd_device(tq, tk[:, half:], tv[:, half:], h, qs, ks2, scale, causal, q_offset=q_off,
                                    k_offset=half, state=state, load_state=True, kernel="decode")
    assert torch.nan_to_num(f(o2) - ref).abs().max() <= 2e-2
    with pytest.raises(ValueError):  # forced on a shape it does not take
        tpa_b200.tpa.fwd_device(tq.float(), tk.float(), tv.float(), h, kernel="decode")


@pytest.mark.parametrize("kernel,b,lq,h,d,dv,chunk", [
    ("decode", 2, 4, 48, 64, 48, 6144),       # > 32 splits: one merge CTA per (row, head), 384 of them
    ("decode", 1, 8, 32, 128, 96, 4864),      # dv = 96: 24 float4 chunks per row
    ("decode", 3, 1, 64, 128, 128, 2048),     # few splits: eight (row, head) items per merge CTA
    ("sm100_staged", 1, 200, 8, 128, 128, 4096),   # key splits of the tensor-core kernel
])
def test_middle_ring_step_loads_and_stores_the_same_state(kernel, b, lq, h, d, dv, chunk):
    """A middle ring step reads and writes ONE carried state (TPA_FLAG_STATE_LOAD and _STORE on the
    same buffers) while its key splits are merged: three key chunks chained store / load+store /
    load must equal one call over all keys.  The merge of an item's splits must see the old
    state of that item only, whichever block or wave serves it."""
    lk = 3 * chunk
    q, k, v = orc.make_factors(123, b, max(lq, lk), max(lq, lk), 3, 2, h, d, dv)
    tq, tk, tv = dev(q[:, :lq], torch.bfloat16), dev(k[:, :lk], torch.bfloat16), dev(v[:, :lk], torch.bfloat16)
    q_off = lk - lq
    args = (h, None, None, d**-0.5, True)
    info = tpa_b200.tpa.query_kernel(tq, tk[:, :chunk], tv[:, :chunk], h, kernel=kernel, causal=True)
    assert info["launches"] >= 2 and info["grid"][0 if kernel == "decode" else 1] > 1, info
    state = (torch.empty(b, lq, h, dv, device="cuda"), torch.empty(b, lq, h, device="cuda"))
    for _ in range(3):  # a race need not show on the first attempt
        for i in range(3):
            ks = slice(i * chunk, (i + 1) * chunk)
            o, lse = tpa_b200.tpa.fwd_device(tq, tk[:, ks], tv[:, ks], *args, q_offset=q_off, k_offset=i * chunk,
                                             state=state, load_state=i > 0, store_state=i < 2, kernel=kernel)
        f = lambda t: t.float().cpu()  # noqa: E731
        ref, lref = orc.tpa_reference_torch(f(tq), f(tk), f(tv), h, sm_scale=d**-0.5, causal=True, q_offset=q_off,
                                            return_lse=True)
        diff = (f(o) - ref).abs()
        assert diff.max() <= 2e-2 and diff.mean() <= 5e-3, (float(diff.max()), float(diff.mean()))
        assert (lse.cpu() - lref).abs().max() <= 1e-2


def test_bounded_wait_runs_out_and_reports():
    """A device-side wait that nothing satisfies gives up after its cycle budget: the kernel ends
    normally, the status block says where, tpa_read_status returns TPA_ERR_DEVICE_TIMEOUT, and the
    next launch on the same context works.  (One warp, a budget of about a millisecond.)"""
    import ctypes as C
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = _capi.lib.tpa_selftest_wait_timeout(ws.data_ptr(), ws.numel(), 1 << 21, stream)
    assert st == _capi.TPA_OK, _capi.status_string(st)
    detail = (C.c_uint32 * 4)()
    st = _capi.lib.tpa_read_status(ws.data_ptr(), stream, C.byref(detail))
    assert st == _capi.TPA_ERR_DEVICE_TIMEOUT
    flag, where, block, spins = list(detail)
    assert flag == 1 and where == 0x7e57 and block == 0 and spins >= 64
    assert "wait ran out" in _capi.status_string(st)
    # the context is intact
    q, k, v = orc.make_factors(1, 1, 8, 8, 1, 1, 1, 4, 6)
    o = tpa_b200.tpa.tpa(dev(q), dev(k), dev(v), num_heads=1)
    assert np.max(np.abs(o.cpu().numpy() - orc.tpa_reference(q, k, v, 1))) <= 1e-5
