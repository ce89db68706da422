"""No-GPU checks: the C-ABI library loads, exports what the header declares, validates
arguments, and the Python signatures mirror the reference's error behaviour."""

import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT

import tpa_b200
from tpa_b200 import _capi


def _header_functions():
    text = open(os.path.join(ROOT, "include", "tpa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(tpa_[a-z_0-9]+)\s*\(", text))


def test_library_exports_every_declared_symbol():
    declared = _header_functions()
    assert declared == set(_capi.EXPORTS), declared ^ set(_capi.EXPORTS)
    for name in declared:
        assert getattr(_capi.lib, name) is not None
    assert _capi.lib.tpa_abi_version() == 2


def _args(**over):
    a = _capi.TpaFwdArgs()
    a.struct_size = C.sizeof(_capi.TpaFwdArgs)
    a.dtype = _capi.DTYPE_F32
    a.batch, a.lq, a.lk, a.rank_q, a.rank_k, a.heads, a.dk, a.dv = 1, 64, 64, 2, 2, 4, 16, 16
    for f in ("qa", "qb", "ka", "kb", "va", "vb"):
        fac = getattr(a, f)
        fac.ptr = 4096
        fac.stride[0], fac.stride[1], fac.stride[2] = 64 * 2 * 20, 2 * 20, 20
    a.o = 4096
    for key, val in over.items():
        setattr(a, key, val)
    return a


def test_query_kernel_and_validation_without_gpu():
    info = _capi.TpaKernelInfo()
    assert _capi.lib.tpa_query_kernel(C.byref(_args()), C.byref(info)) == _capi.TPA_OK
    assert info.kernel == _capi.KERNEL_SIMT and info.launches == 1
    assert tuple(info.grid) == (2, 4, 1) and info.threads == 256
    assert _capi.lib.tpa_fwd_workspace_bytes(C.byref(_args())) == 0
    bad = [
        (_args(struct_size=8), _capi.TPA_ERR_BAD_ARG),
        (_args(lq=0), _capi.TPA_ERR_BAD_ARG),
        (_args(o=None), _capi.TPA_ERR_BAD_ARG),
        (_args(q_segment_ids=4096), _capi.TPA_ERR_BAD_ARG),  # only one side given
        (_args(flags=_capi.FLAG_STATE_LOAD), _capi.TPA_ERR_BAD_ARG),  # state missing
        (_args(dtype=7), _capi.TPA_ERR_UNSUPPORTED),
        (_args(dk=512), _capi.TPA_ERR_UNSUPPORTED),
        (_args(kernel=_capi.KERNEL_SM100), _capi.TPA_ERR_KERNEL_FORCED),  # fp32 is SIMT only
    ]
    for a, want in bad:
        assert _capi.lib.tpa_query_kernel(C.byref(a), C.byref(info)) == want
        assert _capi.lib.tpa_fwd(C.byref(a), None, 0, None) == want  # returns before any CUDA call
    for st in range(-7, 1):
        assert _capi.lib.tpa_status_string(st)
    with pytest.raises(ValueError):
        _capi.check(_capi.TPA_ERR_BAD_ARG)
    with pytest.raises(NotImplementedError):
        _capi.check(_capi.TPA_ERR_UNSUPPORTED)


def test_backward_validation_without_gpu():
    def bargs(fwd_over=None, **over):
        a = _capi.TpaBwdArgs()
        a.struct_size = C.sizeof(_capi.TpaBwdArgs)
        a.grad_dtype = _capi.DTYPE_F32
        a.fwd = _args(**{"lse": 4096, **(fwd_over or {})})
        a.d_o, a.dq, a.dk, a.dv = 4096, 4096, 4096, 4096
        for key, val in over.items():
            setattr(a, key, val)
        return a

    # fp32: delta + dense fp32 dQ, dK, dV behind the 256-byte status block, each rounded to 256 bytes
    want = 256 + 1 * 64 * 4 * 4 + 3 * (1 * 64 * 4 * 16 * 4)
    assert _capi.lib.tpa_bwd_workspace_bytes(C.byref(bargs())) == want
    bad = [
        (bargs(struct_size=8), _capi.TPA_ERR_BAD_ARG),
        (bargs(d_o=None), _capi.TPA_ERR_BAD_ARG),
        (bargs(dk=None), _capi.TPA_ERR_BAD_ARG),
        (bargs({"lse": None}), _capi.TPA_ERR_BAD_ARG),                      # the forward's LSE is an input
        (bargs({"flags": _capi.FLAG_STATE_LOAD, "state_o": 4096, "state_lse": 4096}), _capi.TPA_ERR_BAD_ARG),
        (bargs(bwd_flags=8), _capi.TPA_ERR_BAD_ARG),
        (bargs(grad_dtype=_capi.DTYPE_BF16), _capi.TPA_ERR_UNSUPPORTED),    # bf16 gradients of fp32 factors
        (bargs({"kernel": _capi.KERNEL_SM100}), _capi.TPA_ERR_KERNEL_FORCED),  # fp32 has no tensor-core passes
        (bargs({"kernel": _capi.KERNEL_SM100_FUSED}), _capi.TPA_ERR_KERNEL_FORCED),
    ]
    for a, code in bad:
        assert _capi.lib.tpa_bwd(C.byref(a), 4096, 1 << 30, None) == code  # returns before any CUDA call
        assert _capi.lib.tpa_bwd_workspace_bytes(C.byref(a)) == 0
    # a workspace that is missing, too small or misaligned is refused before anything is enqueued
    for ws, nbytes in ((None, want), (4096, want - 1), (4096 + 64, want)):
        assert _capi.lib.tpa_bwd(C.byref(bargs()), ws, nbytes, None) == _capi.TPA_ERR_WORKSPACE


def test_python_signature_errors_match_reference():
    q = torch.zeros(1, 256, 2, 4 + 8)
    k = torch.zeros(1, 256, 2, 4 + 8)
    v = torch.zeros(1, 256, 3, 4 + 8)  # rank_v != rank_k -> assertion (tpa/tpa.py:474-475)
    with pytest.raises(AssertionError):
        tpa_b200.tpa._check_shapes(q, k, v, 4)
    v = torch.zeros(1, 256, 2, 4 + 8)
    assert tpa_b200.tpa._check_shapes(q, k, v, 4) == (1, 256, 256, 2, 2, 8, 8)
    # no CPU implementation: host inputs without a CUDA device must fail loudly
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU implementation"):
            tpa_b200.tpa.tpa(q, k, v, num_heads=4)
        with pytest.raises(RuntimeError, match="no CPU implementation"):
            tpa_b200.tpa.tpa(np.zeros((1, 8, 1, 6), np.float32), np.zeros((1, 8, 1, 6), np.float32),
                         np.zeros((1, 8, 1, 6), np.float32), num_heads=2)
        with pytest.raises(RuntimeError, match="no CPU implementation"):
            tpa_b200.ring_tpa.ring_tpa(q, k, v, torch.zeros(1, 256), torch.zeros(1, 256), None, 4)
    # ring impl switch (tpa/ring_tpa.py:237-239, 273)
    with pytest.raises(NotImplementedError):
        tpa_b200.ring_tpa.ring_tpa(q, k, v, None, None, None, 4, impl="xla")
    with pytest.raises(ValueError):
        tpa_b200.ring_tpa.ring_tpa(q, k, v, None, None, None, 4, impl="nope")
    bs = tpa_b200.tpa.BlockSizes()
    assert (bs.block_q, bs.block_kv, bs.block_h) == (128, 128, 4)
