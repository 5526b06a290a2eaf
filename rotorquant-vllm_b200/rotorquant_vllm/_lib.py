"""ctypes binding of librq_b200.so, the C-ABI CUDA library (see include/rq_b200.h).

The library is the only implementation of the hot path: there is no Triton
dispatch and no CPU fallback.  ``lib()`` raises if the shared object has not
been built (``python rotorquant-vllm_b200/csrc/build.py``).
"""

from __future__ import annotations

import ctypes as C
import os

import torch

# RQ_B200_LIBRARY: path of another build of the library (A/B comparisons of kernel variants).
_PATH = os.environ.get("RQ_B200_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "librq_b200.so")
_LIB = None

RQ_OK = 0
RQ_ERR_INVALID_ARG, RQ_ERR_UNSUPPORTED, RQ_ERR_ALIGNMENT, RQ_ERR_WORKSPACE, RQ_ERR_CUDA = (
    -1, -2, -3, -4, -5)

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

_P, _I, _L, _F, _Z = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

_SIGNATURES = {
    "rq_version": (C.c_char_p, []),
    "rq_last_error": (C.c_char_p, []),
    "rq_compress_store": (_I, [_P, _P, _I, _L, _I, _I, _L, _L, _L, _L, _P, _L, _I, _P, _P, _P, _I,
                               _P, _I, _I, _P]),
    "rq_compress": (_I, [_P, _I, _L, _I, _L, _P, _P, _I, _P, _P, _P]),
    "rq_decompress": (_I, [_P, _P, _L, _I, _P, _I, _P, _I, _P]),
    "rq_decompress_blocks": (_I, [_P, _L, _I, _I, _I, _I, _P, _L, _P, _I, _P, _I, _P, _P, _I, _P]),
    "rq_decode_workspace_bytes": (_Z, [_I, _I, _I, _I, _I, _I]),
    "rq_decode": (_I, [_P, _P, _I, _L, _L, _L, _L, _I, _I, _I, _I, _P, _L, _I, _I, _P, _L, _P, _P,
                       _I, _P, _I, _P, _F, _I, _P, _Z, _I, _P]),
    "rq_decode_sharded": (_I, [_P, _I, _L, _L, _L, _L, _I, _I, _I, _I, _P, _L, _I, _I, _P, _L, _P, _P,
                               _I, _P, _I, _P, _F, _I, _P, _Z, _I, C.POINTER(C.c_void_p), _I, _P]),
    "rq_peer_barrier": (_I, [C.POINTER(C.c_void_p), _I, _I, _P, C.c_longlong, _P]),
    "rq_decode_static_scratch": (_I, [_P, _P, _I, _L, _L, _L, _L, _I, _I, _I, _I, _P, _L, _I, _I, _P, _L, _P,
                                      _P, _I, _P, _I, _P, _F, _I, _I, _P]),
    "rq_prefill_int8": (_I, [_P, _P, _I, _L, _L, _L, _L, _P, _I, _I, _I, _I, _I, _I, _P, _L, _I, _I, _P,
                             _L, _P, _P, _I, _P, _I, _P, _F, _P, _P]),
    "rq_probe_mma_peak": (_I, [_I, _I, C.POINTER(C.c_double), _P, _P]),
    "rq_selftest_bounded_wait": (_I, [C.c_longlong, _P, _P]),
    "rq_prefill_workspace_bytes": (_Z, [_I, _I, _I]),
    "rq_prefill_int8_staged": (_I, [_P, _P, _I, _L, _L, _L, _L, _P, _I, _I, _I, _I, _I, _I, _P, _L, _I, _I, _P,
                                    _L, _P, _P, _I, _P, _I, _P, _F, _P, _I, _P, _Z, _P]),
}

_OPTIONAL: dict = {}


def library_path() -> str:
    return _PATH


def lib() -> C.CDLL:
    """The loaded library; raises ``RuntimeError`` when it is missing."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(_PATH):
            raise RuntimeError(
                f"{_PATH} is missing: build it with `python rotorquant-vllm_b200/csrc/build.py` "
                "(nvcc, sm_100a).  There is no Triton or CPU fallback for this path.")
        handle = C.CDLL(_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        for name, (res, args) in _OPTIONAL.items():
            if hasattr(handle, name):
                fn = getattr(handle, name)
                fn.restype, fn.argtypes = res, args
        _LIB = handle
    return _LIB


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def check(status: int) -> None:
    """Turn a negative rq_status into the exception the reference's launchers raise for it."""
    if status == RQ_OK:
        return
    msg = lib().rq_last_error().decode("utf-8", "replace")
    if status == RQ_ERR_CUDA:
        raise RuntimeError(msg)
    raise ValueError(msg)


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors on one CUDA device (the CPU fallbacks of the reference were removed)."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "rotorquant_vllm: this build runs on CUDA tensors only; the CPU fallbacks of the "
                "reference implementation were removed")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}") from None
