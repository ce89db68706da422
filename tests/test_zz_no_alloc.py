"""tpa_fwd_static_scratch: the forward pass for callers that cannot allocate a workspace.

An XLA custom-call handler (the jax.ffi binding this library is meant for) runs while XLA's
allocator owns, and has mostly pre-reserved, the GPU's memory, and only sees the buffers XLA
passes it; an embedder with a fixed memory budget is in the same position.  Neither can size
and hand over the scratch that tpa_fwd stages its Q/K/V tiles in, so this entry point keeps
that scratch in a static device array inside the library and allocates nothing.

The test calls it through the C ABI twice in a row (second call: other inputs and a smaller
shape, so stale contents of the shared array would show) and compares each result with
tpa_fwd on a caller-allocated workspace: same kernels, so the outputs must be identical.
It also checks that a problem larger than the static array is refused without a launch.
Collected last on purpose (file name), and independent of the tests before it.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import tpa_oracle as orc

import tpa_b200
from tpa_b200 import _capi
from tpa_b200.tpa import _factor

pytestmark = pytest.mark.gpu


def _args(q, k, v, heads, out, lse, sm_scale, causal):
    b, lq, rq, hd = q.shape
    lk, rk = k.shape[1], k.shape[2]
    a = _capi.TpaFwdArgs()
    a.struct_size = C.sizeof(_capi.TpaFwdArgs)
    a.dtype = _capi.DTYPE_BF16
    a.batch, a.lq, a.lk, a.rank_q, a.rank_k = b, lq, lk, rq, rk
    a.heads, a.dk, a.dv = heads, hd - heads, v.shape[-1] - heads
    a.qa, a.qb = _factor(q, 0), _factor(q, heads)
    a.ka, a.kb = _factor(k, 0), _factor(k, heads)
    a.va, a.vb = _factor(v, 0), _factor(v, heads)
    a.o, a.lse = out.data_ptr(), lse.data_ptr()
    a.sm_scale = sm_scale
    a.flags = _capi.FLAG_CAUSAL if causal else 0
    return a


def _case(seed, b, t, h, d, rq, rk):
    q, k, v = orc.make_factors(seed, b, t, t, rq, rk, h, d, d)
    return tuple(torch.from_numpy(x).cuda().to(torch.bfloat16) for x in (q, k, v))


def test_static_scratch_matches_workspace_entry_point_twice():
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    first = True
    for seed, (b, t, h, d, rq, rk), causal in [(901, (2, 1024, 8, 128, 3, 2), True),
                                               (902, (1, 512, 16, 64, 2, 4), False)]:
        q, k, v = _case(seed, b, t, h, d, rq, rk)
        n_before = _capi.lib.tpa_launch_count()
        want, want_lse = tpa_b200.tpa.fwd_device(q, k, v, h, None, None, d**-0.5, causal,
                                                 kernel="sm100_staged")
        launches = _capi.lib.tpa_launch_count() - n_before  # staging + attention (+ split merge)
        got = torch.full_like(want, float("nan"))
        got_lse = torch.full_like(want_lse, float("nan"))
        a = _args(q, k, v, h, got, got_lse, d**-0.5, causal)
        if first:
            # the first call on a device looks the array up (and lets the driver instantiate it):
            # make it before measuring free memory, as a caller would at start-up
            assert _capi.lib.tpa_fwd_static_scratch(C.byref(a), stream) == _capi.TPA_OK
            first = False
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        n0 = _capi.lib.tpa_launch_count()
        st = _capi.lib.tpa_fwd_static_scratch(C.byref(a), stream)
        assert st == _capi.TPA_OK, _capi.status_string(st)
        torch.cuda.synchronize()
        assert _capi.lib.tpa_launch_count() == n0 + launches  # the same kernels, nothing else
        # nothing was allocated on the device: free memory is what it was before the call
        assert torch.cuda.mem_get_info()[0] == free_before
        # the status block inside the static array is readable, and no bounded wait ran out
        detail = (C.c_uint32 * 4)()
        assert _capi.lib.tpa_read_status_static_scratch(stream, C.byref(detail)) == _capi.TPA_OK, list(detail)
        # tolerance of the bf16 tests; in fact bit-identical (same kernels, same inputs)
        diff = (got.float() - want.float()).abs()
        assert diff.max() <= 2e-2 and diff.mean() <= 5e-3
        assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
        # and it is the right answer, not just the same one
        ref = orc.tpa_reference_torch(q.float().cpu(), k.float().cpu(), v.float().cpu(), h,
                                      sm_scale=d**-0.5, causal=causal)
        d2 = (got.float().cpu() - ref).abs()
        assert d2.max() <= 2e-2 and d2.mean() <= 5e-3


def test_static_scratch_refuses_what_does_not_fit():
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    b, t, h, d = 1, 16384, 16, 128  # (lq + 2 lk) * b * h * d * 2 = 201 MB > 64 MiB
    q = torch.zeros(b, t, 1, h + d, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(b, t, h, d, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(b, t, h, dtype=torch.float32, device="cuda")
    a = _args(q, q, q, h, out, lse, 1.0, True)
    n0 = _capi.lib.tpa_launch_count()
    st = _capi.lib.tpa_fwd_static_scratch(C.byref(a), stream)
    assert st == _capi.TPA_ERR_STATIC_SCRATCH
    assert "TPA_STATIC_SCRATCH_BYTES" in _capi.status_string(st)
    assert _capi.lib.tpa_launch_count() == n0
    # fp32 is outside what the staged tensor-core variant takes
    qf = torch.zeros(1, 256, 1, 8 + 64, device="cuda")
    of = torch.empty(1, 256, 8, 64, device="cuda")
    lf = torch.empty(1, 256, 8, device="cuda")
    af = _args(qf, qf, qf, 8, of, lf, 1.0, False)
    af.dtype = _capi.DTYPE_F32
    assert _capi.lib.tpa_fwd_static_scratch(C.byref(af), stream) == _capi.TPA_ERR_KERNEL_FORCED
