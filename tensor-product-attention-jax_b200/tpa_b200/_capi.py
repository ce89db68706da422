"""ctypes binding of libtpa_b200.so (declarations: include/tpa_b200.h).

There is no CPU or PyTorch fallback behind this module: if the shared library is
missing or a symbol cannot be resolved, importing it raises.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# TPA_B200_LIB points at another build of the same library (tuning builds); default: in-tree.
LIB_PATH = os.environ.get("TPA_B200_LIB") or os.path.join(_PKG, "libtpa_b200.so")

TPA_OK = 0
TPA_ERR_BAD_ARG = -1
TPA_ERR_UNSUPPORTED = -2
TPA_ERR_WORKSPACE = -3
TPA_ERR_CUDA = -4
TPA_ERR_KERNEL_FORCED = -5
TPA_ERR_DEVICE_TIMEOUT = -6
TPA_ERR_STATIC_SCRATCH = -7
STATIC_SCRATCH_BYTES = 64 << 20

DTYPE_F32, DTYPE_BF16 = 0, 1
KERNEL_AUTO, KERNEL_SIMT, KERNEL_SM100, KERNEL_SM100_FUSED, KERNEL_SM100_STAGED, KERNEL_DECODE = 0, 1, 2, 3, 4, 5
KERNELS = {"auto": KERNEL_AUTO, "simt": KERNEL_SIMT, "sm100": KERNEL_SM100,
           "sm100_fused": KERNEL_SM100_FUSED, "sm100_staged": KERNEL_SM100_STAGED, "decode": KERNEL_DECODE}
KERNEL_NAMES = {KERNEL_SIMT: "simt", KERNEL_SM100_FUSED: "sm100_fused", KERNEL_SM100_STAGED: "sm100_staged",
                KERNEL_DECODE: "decode"}
FLAG_CAUSAL, FLAG_STATE_LOAD, FLAG_STATE_STORE, FLAG_REUSE_STAGED_Q, FLAG_CAUSAL_PER_PART = 1, 2, 4, 8, 16
FLAG_REUSE_STAGED_KV = 32
BWD_ACCUMULATE_DQ, BWD_ACCUMULATE_DKV = 1, 2

# Every symbol include/tpa_b200.h declares.
EXPORTS = (
    "tpa_fwd",
    "tpa_fwd_static_scratch",
    "tpa_read_status_static_scratch",
    "tpa_fwd_workspace_bytes",
    "tpa_fwd_workspace_bytes_min",
    "tpa_bwd",
    "tpa_bwd_workspace_bytes",
    "tpa_query_kernel",
    "tpa_read_status",
    "tpa_selftest_wait_timeout",
    "tpa_status_string",
    "tpa_last_cuda_error",
    "tpa_launch_count",
    "tpa_abi_version",
)


class TpaFactor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * 3)]


class TpaFwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("batch", C.c_int32),
        ("lq", C.c_int32),
        ("lk", C.c_int32),
        ("rank_q", C.c_int32),
        ("rank_k", C.c_int32),
        ("heads", C.c_int32),
        ("dk", C.c_int32),
        ("dv", C.c_int32),
        ("qa", TpaFactor),
        ("qb", TpaFactor),
        ("ka", TpaFactor),
        ("kb", TpaFactor),
        ("va", TpaFactor),
        ("vb", TpaFactor),
        ("q_segment_ids", C.c_void_p),
        ("kv_segment_ids", C.c_void_p),
        ("q_segment_batch_stride", C.c_int64),
        ("kv_segment_batch_stride", C.c_int64),
        ("o", C.c_void_p),
        ("lse", C.c_void_p),
        ("state_o", C.c_void_p),
        ("state_lse", C.c_void_p),
        ("sm_scale", C.c_float),
        ("flags", C.c_uint32),
        ("q_offset", C.c_int64),
        ("k_offset", C.c_int64),
        ("kernel", C.c_int32),
        ("reserved", C.c_int32),
        ("kv_parts", C.c_int32),
        ("window", C.c_int32),
        ("dilation", C.c_int32),
        ("rope_len", C.c_int32),
        ("k_part_stride", C.c_int64),
        ("v_part_stride", C.c_int64),
        ("kv_segment_part_stride", C.c_int64),
        ("rope_cos", C.c_void_p),
        ("rope_sin", C.c_void_p),
        ("rope_q_offset", C.c_int64),
        ("rope_k_offset", C.c_int64),
    ]


class TpaBwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("grad_dtype", C.c_int32),
        ("fwd", TpaFwdArgs),
        ("d_o", C.c_void_p),
        ("dq", C.c_void_p),
        ("dk", C.c_void_p),
        ("dv", C.c_void_p),
        ("bwd_flags", C.c_uint32),
        ("reserved", C.c_int32),
    ]


class TpaKernelInfo(C.Structure):
    _fields_ = [
        ("kernel", C.c_int32),
        ("block_q", C.c_int32),
        ("block_kv", C.c_int32),
        ("threads", C.c_int32),
        ("grid", C.c_int32 * 3),
        ("smem_bytes", C.c_int32),
        ("launches", C.c_int32),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tpa_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        getattr(lib, name)  # AttributeError if the library does not export it
    lib.tpa_fwd.argtypes = [C.POINTER(TpaFwdArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.tpa_fwd.restype = C.c_int
    lib.tpa_fwd_static_scratch.argtypes = [C.POINTER(TpaFwdArgs), C.c_void_p]
    lib.tpa_fwd_static_scratch.restype = C.c_int
    lib.tpa_read_status_static_scratch.argtypes = [C.c_void_p, C.POINTER(C.c_uint32 * 4)]
    lib.tpa_read_status_static_scratch.restype = C.c_int
    lib.tpa_fwd_workspace_bytes.argtypes = [C.POINTER(TpaFwdArgs)]
    lib.tpa_fwd_workspace_bytes.restype = C.c_size_t
    lib.tpa_fwd_workspace_bytes_min.argtypes = [C.POINTER(TpaFwdArgs)]
    lib.tpa_fwd_workspace_bytes_min.restype = C.c_size_t
    lib.tpa_bwd.argtypes = [C.POINTER(TpaBwdArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.tpa_bwd.restype = C.c_int
    lib.tpa_bwd_workspace_bytes.argtypes = [C.POINTER(TpaBwdArgs)]
    lib.tpa_bwd_workspace_bytes.restype = C.c_size_t
    lib.tpa_query_kernel.argtypes = [C.POINTER(TpaFwdArgs), C.POINTER(TpaKernelInfo)]
    lib.tpa_query_kernel.restype = C.c_int
    lib.tpa_read_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32 * 4)]
    lib.tpa_read_status.restype = C.c_int
    lib.tpa_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_size_t, C.c_int64, C.c_void_p]
    lib.tpa_selftest_wait_timeout.restype = C.c_int
    lib.tpa_status_string.argtypes = [C.c_int]
    lib.tpa_status_string.restype = C.c_char_p
    lib.tpa_last_cuda_error.argtypes = []
    lib.tpa_last_cuda_error.restype = C.c_char_p
    lib.tpa_launch_count.argtypes = []
    lib.tpa_launch_count.restype = C.c_uint64
    lib.tpa_abi_version.argtypes = []
    lib.tpa_abi_version.restype = C.c_int
    return lib


lib = _load()


def status_string(status: int) -> str:
    s = lib.tpa_status_string(status).decode()
    if status == TPA_ERR_CUDA:
        s += ": " + lib.tpa_last_cuda_error().decode()
    return s


def check(status: int):
    """Raise the Python exception that corresponds to a negative status."""
    if status == TPA_OK:
        return
    msg = f"libtpa_b200: {status_string(status)} (status {status})"
    if status in (TPA_ERR_BAD_ARG, TPA_ERR_KERNEL_FORCED):
        raise ValueError(msg)
    if status == TPA_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)
