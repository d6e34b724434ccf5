"""ctypes binding of ``libmdy_kernels.so`` (declared in ``include/mdy_kernels.h``).

There is no CPU fallback and no alternative backend: if the shared library is missing or a call
returns a non-zero status, a ``RuntimeError`` is raised.  Importing this module does not load the
library; the first call to :func:`lib` does.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libmdy_kernels.so"

MDY_F32, MDY_F16, MDY_BF16 = 0, 1, 2
DTYPE_CODE = {torch.float32: MDY_F32, torch.float16: MDY_F16, torch.bfloat16: MDY_BF16}

TUNE_CE_THREADS = 0
TUNE_CE_FUSED_CTAS_PER_SM = 1
TUNE_NORM_CTAS_PER_SM = 2
TUNE_SWIGLU_UNROLL = 3
TUNE_CE_FUSED_IMPL = 4
TUNE_ROPE_THREADS = 5
TUNE_CE_CLUSTER_SLICE_KB = 6
TUNE_CE_CLUSTER_THREADS = 7
TUNE_CE_CLUSTER_VPC = 8
TUNE_CE_WAIT_TEST = 9
TUNE_ROPE_HEADS_PER_THREAD = 10
TUNE_ROPE_GRID_PER_SM = 11
TUNE_NORM_BWD_THREADS = 12
TUNE_NORM_FWD_VPT = 13
TUNE_NORM_BWD_VPT = 14
TUNE_CE_CLUSTER_MINB = 15
TUNE_NORM_POW2_GROUPS = 16
TUNE_NORM_FWD_GROUP = 17
TUNE_NORM_BWD_GROUP = 18
TUNE_NORM_FWD_THREADS = 19
TUNE_NORM_IMPL = 20
TUNE_CE_VP_CTAS_PER_SM = 21
TUNE_CE_VP_SLOTS = 22
TUNE_CE_VP_SLICE_KB = 23
TUNE_NORM_TEAM = 24

_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float

# name -> (restype, argtypes); mirrors include/mdy_kernels.h one to one.
SIGNATURES = {
    "mdy_version": (_I, []),
    "mdy_num_sms": (_I, []),
    "mdy_launch_count": (_L, []),
    "mdy_status_string": (c_char_p, [_I]),
    "mdy_set_tunable": (_I, [_I, _I]),
    "mdy_get_tunable": (_I, [_I]),
    "mdy_last_device_error": (_I, [_I]),
    "mdy_device_error_of": (_I, [_I, _I]),
    "mdy_ce_last_geometry": (_I, [_P, _P, _P, _P]),
    "mdy_rowwise_extreme": (_I, [_P, _P, _P, _L, _L, _L, _I, _I, _P]),
    "mdy_rmsnorm_bwd_partial_rows": (_L, [_L, _L, _I]),
    "mdy_rmsnorm_fwd": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _F, _I, _I, _P]),
    "mdy_rmsnorm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _I, _I, _P]),
    "mdy_rmsnorm_bwd_noalloc": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _I, _I, _P]),
    "mdy_add_rmsnorm_fwd": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _F, _I, _I, _P]),
    "mdy_add_rmsnorm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _I, _P]),
    "mdy_rope": (_I, [_P, _P, _P, _P, _P, _P] + [_L] * 6 + [_L] * 12 + [_I, _I, _P]),
    "mdy_swiglu_fwd": (_I, [_P, _P, _P, _L, _L, _L, _L, _L, _I, _P]),
    "mdy_swiglu_bwd": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _I, _P]),
    "mdy_ce_fwd": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "mdy_ce_bwd": (_I, [_P, _L, _I, _P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "mdy_ce_fused": (_I, [_P, _P, _P, _P, _P, _P, _F, _L, _L, _L, _I, _P]),
    "mdy_scale_inplace": (_I, [_P, _L, _P, _I, _P]),
    "mdy_ce_vp_combine": (_I, [_P, _P, _P, _P, _L, _L, _P]),
    "mdy_ce_vp_fused": (_I, [_P, _P, _P, _P, _P, _P, _P, _F, _L, _L, _L, _I, _I, _I, _L, ctypes.c_uint32, _I, _P]),
    "mdy_ce_vp_exchange_bytes": (_L, [_L, _L, _I, _I]),
    "mdy_ce_vp_geometry": (_I, [_L, _I, _I, _P]),
    "mdy_peer_buffer_create": (_I, [_L, _P, _P]),
    "mdy_peer_buffer_open": (_I, [_P, _P]),
    "mdy_peer_buffer_close": (_I, [_P]),
    "mdy_peer_buffer_destroy": (_I, [_P]),
}

_lib = None
_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """Load (once) and return the shared library with argument types set."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m mdy_triton_b200.build` "
                    "(there is no fallback implementation)")
            handle = ctypes.CDLL(str(LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(handle, name)  # AttributeError here = header/library mismatch
                fn.restype = res
                fn.argtypes = args
            _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().mdy_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}: {status_string(status)}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, float16 or bfloat16") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors must live on one CUDA device; returns it."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("mdy_triton kernels run on CUDA tensors only (no CPU fallback); "
                               f"got a tensor on {t.device}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_ptr(dev: torch.device):
    return torch.cuda.current_stream(dev).cuda_stream


def launch_count() -> int:
    return int(lib().mdy_launch_count())


def set_tunable(tid: int, value: int) -> None:
    check(lib().mdy_set_tunable(tid, value), "mdy_set_tunable")
