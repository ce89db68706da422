"""GPU parity at the benchmark configurations' own shapes (through the C ABI).

The numbers quoted for c1, c2 and c4 come from launches that differ from the small parity cases
in more than size: 64-bit offsets, the launch order that takes (batch, head) slices in groups
that share L2, gigabytes of staged tiles.  These tests run exactly those shapes and compare with
the CPU oracle: sampled query rows where the whole tensor would take minutes (first and last rows,
both sides of a 256-row block edge and of a slice-group edge, and random rows), the whole tensor
where it takes seconds.  bf16 bounds: max-abs <= 2e-2, mean-abs <= 5e-3.
"""

import numpy as np
import pytest
import torch

from oracle import tpa_oracle as orc

import tpa_b200

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def no_device_timeout():
    yield
    st, detail = tpa_b200.tpa.device_status()
    assert st == 0, (st, [hex(x) for x in detail])


def _bf16(x):
    return torch.from_numpy(x).cuda().to(torch.bfloat16)


def _rows(t, n_random, seed, edges=()):
    fixed = [0, 1, 2, 3, t - 4, t - 3, t - 2, t - 1]
    for e in edges:
        fixed += [e - 2, e - 1, e, e + 1]
    rnd = torch.randperm(t, generator=torch.Generator().manual_seed(seed))[:n_random].tolist()
    return torch.tensor(sorted(set(r for r in fixed + rnd if 0 <= r < t)))


def _check(tq, tk, tv, h, d, causal, rows, o, lse):
    f = lambda x: x.float().cpu()  # noqa: E731
    ref, lref = orc.tpa_reference_torch(f(tq), f(tk), f(tv), h, sm_scale=d**-0.5, causal=causal, rows=rows,
                                        return_lse=True)
    got, gl = f(o), lse.cpu()
    if rows is not None:
        got, gl = got[:, rows], gl[:, rows]
    diff = (got - ref).abs()
    assert not torch.isnan(got).any()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3, (float(diff.max()), float(diff.mean()))
    assert (gl - lref).abs().max() <= 1e-2
    return float(diff.max()), float(diff.mean())


def test_config2_full_shape_sampled_rows():
    """c2: bf16 causal B=1 T=32768 h=32 d=128 R 12/4/4, the headline shape (slice groups of 4)."""
    b, t, h, d, rq, rk = 1, 32768, 32, 128, 12, 4
    q, k, v = orc.make_factors(2, b, t, t, rq, rk, h, d, d)
    tq, tk, tv = _bf16(q), _bf16(k), _bf16(v)
    info = tpa_b200.tpa.query_kernel(tq, tk, tv, h, causal=True)
    assert info["kernel"] == "sm100_staged"
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True)
    # row-block edges at 256 and in the middle; every head is checked for each row, which covers
    # every slice group of the launch order
    rows = _rows(t, 120, 2, edges=(256, 16384, 32512))
    _check(tq, tk, tv, h, d, True, rows, o, lse)


def test_config1_full_batch_sampled_rows():
    """c1: bf16 causal B=4 T=4096 h=32 d=128 R 6/2/2 at its full batch."""
    b, t, h, d, rq, rk = 4, 4096, 32, 128, 6, 2
    q, k, v = orc.make_factors(1, b, t, t, rq, rk, h, d, d)
    tq, tk, tv = _bf16(q), _bf16(k), _bf16(v)
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True)
    _check(tq, tk, tv, h, d, True, _rows(t, 100, 1, edges=(256, 2048)), o, lse)


def test_config4_full_batch_whole_tensor_and_dense_cross_check():
    """c4: bf16 non-causal B=8 T=2048 h=16 d=64 R 8/8/8, every element, against the oracle that
    materialises Q, K, V and runs plain softmax attention (tpa/mha.py:23-37) -- and, as the speed
    half of that cross-check, the same materialised Q, K, V fed back through this library as
    rank-1 factors (a dense-attention call) must give the same output."""
    b, t, h, d, r = 8, 2048, 16, 64, 8
    q, k, v = orc.make_factors(4, b, t, t, r, r, h, d, d)
    tq, tk, tv = _bf16(q), _bf16(k), _bf16(v)
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, False)
    _check(tq, tk, tv, h, d, False, None, o, lse)
    # dense arm: materialise Q, K, V (fp32 rank mean of the bf16 factors, rounded once to bf16, which
    # is what the staging kernel produces) and run them as dense attention through the library
    def dense(x, r_):
        xf = x.float()
        return (torch.einsum("blrh,blrd->blhd", xf[..., :h], xf[..., h:]) / r_).to(torch.bfloat16)

    od, lsed = tpa_b200.mha.mha(dense(tq, r), dense(tk, r), dense(tv, r), sm_scale=d**-0.5, return_lse=True)
    diff = (od.float() - o.float()).abs()
    assert diff.max() <= 2e-2 and diff.mean() <= 5e-3, (float(diff.max()), float(diff.mean()))
    assert (lsed - lse).abs().max() <= 1e-2


@pytest.mark.parametrize("which", ["fwd", "bwd"])
def test_slice_groups_smaller_than_the_launch(which):
    """B=1 T=8192 h=32 d=128: the staged K/V of all heads (128 MB) exceed the L2 budget, so the
    launch takes the heads in groups of 16 -- the remapped block order of the long benchmark
    shapes, here at a size whose sampled rows the oracle finishes in seconds.  Forward and the
    tensor-core backward."""
    b, t, h, d, rq, rk = 1, 8192, 32, 128, 3, 2
    q, k, v = orc.make_factors(88, b, t, t, rq, rk, h, d, d)
    tq, tk, tv = _bf16(q), _bf16(k), _bf16(v)
    o, lse = tpa_b200.tpa.fwd_device(tq, tk, tv, h, None, None, d**-0.5, True)
    if which == "fwd":
        _check(tq, tk, tv, h, d, True, _rows(t, 64, 3, edges=(256, 4096)), o, lse)
        return
    # backward: a cotangent that is non-zero only on sampled rows makes dq on those rows, and dk, dv
    # everywhere, computable by the oracle from those rows alone
    rows = _rows(t, 24, 4, edges=(4096,))
    w = torch.zeros(o.shape, dtype=torch.float32)
    w[:, rows] = torch.from_numpy(np.random.default_rng(9).standard_normal((b, len(rows), h, d)).astype(np.float32))
    do = w.cuda().to(torch.bfloat16)
    dq, dk, dv = tpa_b200.tpa.bwd_device(tq, tk, tv, h, None, None, d**-0.5, True, o, lse, do, grad_dtype=torch.float32)
    assert tpa_b200.tpa.device_status_bwd()[0] == 0
    # oracle by autograd of the definition, restricted to the sampled rows
    f = lambda x: x.float().cpu()  # noqa: E731
    rq_, rk_, rv_ = (f(x).requires_grad_() for x in (tq, tk, tv))
    ref = orc.tpa_reference_torch(rq_, rk_, rv_, h, sm_scale=d**-0.5, causal=True, rows=rows)
    (ref * f(do)[:, rows]).sum().backward()
    for got, want, name in ((dq, rq_.grad, "dq"), (dk, rk_.grad, "dk"), (dv, rv_.grad, "dv")):
        err = float((f(got) - want).abs().max() / want.abs().max())
        assert err <= 3e-2, (name, err)
