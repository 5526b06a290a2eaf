"""The C-ABI library: it loads, exports every function the header declares, and rejects bad
arguments with the documented status before touching a GPU.  Runs without a GPU."""

import ctypes
import os
import re

import pytest

from rotorquant_vllm import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "rq_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert {"rq_compress_store", "rq_decode", "rq_compress", "rq_decompress"} <= set(names)
    handle = ctypes.CDLL(_lib.library_path())
    for n in names:
        assert hasattr(handle, n), f"{n} declared in rq_b200.h but not exported"


def test_python_binding_covers_the_header():
    bound = set(_lib._SIGNATURES) | set(_lib._OPTIONAL)
    assert set(declared_functions()) <= bound


def test_version_string():
    assert b"sm_100a" in _lib.lib().rq_version()


def test_bad_arguments_are_rejected_without_a_device():
    L = _lib.lib()
    # head_dim 64 is not built
    st = L.rq_compress(1, 2, 4, 64, 64, 1, 1, 7, 1, 1, None)
    assert st == _lib.RQ_ERR_UNSUPPORTED and b"head_dim" in L.rq_last_error()
    # 5 boundaries is neither 3-bit nor 4-bit
    st = L.rq_compress(1, 2, 4, 128, 128, 1, 1, 5, 1, 1, None)
    assert st == _lib.RQ_ERR_UNSUPPORTED
    # total_bytes must be heads * 256
    st = L.rq_compress_store(16, 16, 2, 4, 8, 128, 1024, 128, 1024, 128, 16, 64, 1000, 16, 16, 16, 7,
                             16, 7, 1, None)
    assert st == _lib.RQ_ERR_INVALID_ARG
    # misaligned key pointer
    st = L.rq_compress_store(4, 16, 2, 4, 8, 128, 1024, 128, 1024, 128, 16, 64, 2048, 16, 16, 16, 7,
                             16, 7, 1, None)
    assert st == _lib.RQ_ERR_ALIGNMENT
    # decode: query dtype fp32 unsupported, workspace too small
    st = L.rq_decode(16, 16, 0, 4096, 128, 4096, 128, 4, 32, 8, 128, 16, 8, 16, 2048, 16, 8, 16, 16, 8,
                     16, 8, 16, 0.088, 128, 16, 0, 0, None)
    assert st == _lib.RQ_ERR_UNSUPPORTED
    st = L.rq_decode(16, 16, 2, 4096, 128, 4096, 128, 4, 32, 8, 128, 16, 8, 16, 2048, 16, 8, 16, 16, 8,
                     16, 8, 16, 0.088, 128, 16, 8, 0, None)
    assert st == _lib.RQ_ERR_WORKSPACE and b"workspace" in L.rq_last_error()
    with pytest.raises(ValueError):
        _lib.check(st)
    # fewer query heads than KV heads: no size, and an argument error from both decode entry points
    # (never a division by zero in the host-side planning)
    assert L.rq_decode_workspace_bytes(4, 4, 8, 128, 2048, 0) == 0
    assert L.rq_decode_workspace_bytes(4, 12, 8, 128, 2048, 0) == 0
    st = L.rq_decode(16, 16, 2, 4096, 128, 4096, 128, 4, 4, 8, 128, 16, 8, 16, 2048, 16, 8, 16, 16, 8,
                     16, 8, 16, 0.088, 128, 16, 1 << 20, 0, None)
    assert st == _lib.RQ_ERR_INVALID_ARG
    st = L.rq_decode_static_scratch(16, 16, 2, 4096, 128, 4096, 128, 4, 4, 8, 128, 16, 8, 16, 2048, 16, 8,
                                    16, 16, 8, 16, 8, 16, 0.088, 128, 0, None)
    assert st == _lib.RQ_ERR_INVALID_ARG and b"query heads" in L.rq_last_error()
    # paged decompress: slot size must match the head count; the self tests check their arguments
    st = L.rq_decompress_blocks(16, 4, 16, 1000, 8, 128, None, 2, 16, 8, 16, 8, 16, 16, 2, None)
    assert st == _lib.RQ_ERR_INVALID_ARG
    assert L.rq_selftest_bounded_wait(0, None, None) == _lib.RQ_ERR_INVALID_ARG
    assert L.rq_probe_mma_peak(2, 16, None, None, None) == _lib.RQ_ERR_INVALID_ARG
    # zero work is fine
    assert L.rq_compress(None, 2, 0, 128, 128, None, None, 7, None, None, None) == 0
    # forced: one piece per sequence -> 4 groups; rows = groups + sequences (one item), 8 KV heads x 8 slots each
    assert L.rq_decode_workspace_bytes(4, 32, 8, 128, 2048, 1) == 256 + (4 + 4) * 8 * 8 * 130 * 4


def test_launchers_refuse_cpu_tensors():
    """The CPU fallbacks of the reference are gone: CPU tensors are an error, not a slow path."""
    import torch

    from rotorquant_vllm.cuda import fused_paged_rq_decode, iso_compress

    x = torch.randn(2, 8, 128, dtype=torch.float16)
    r = torch.eye(128)
    with pytest.raises(RuntimeError, match="CUDA"):
        iso_compress(x, r[:, 0::2].contiguous(), r[:, 1::2].contiguous(), torch.linspace(-1, 1, 7))
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_paged_rq_decode(torch.zeros(1, 8, 128, dtype=torch.bfloat16),
                              torch.zeros(4, 16, 2048, dtype=torch.uint8),
                              torch.zeros(1, 4, dtype=torch.int32), torch.ones(1, dtype=torch.int32),
                              torch.zeros(8), torch.zeros(8), r, 8, 128, 16)
