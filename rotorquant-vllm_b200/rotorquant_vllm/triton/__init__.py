"""Compatibility alias: the reference exposes its launchers as ``rotorquant_vllm.triton``
(triton/__init__.py:1-15).  This build has no Triton code; the same names resolve to the CUDA
launchers in ``rotorquant_vllm.cuda``."""

from rotorquant_vllm.cuda import (
    fused_paged_rq_decode,
    iso_compress,
    iso_decompress,
    planar_compress,
    planar_decompress,
)

try:  # present once the INT8 prefill kernel is built into the library
    from rotorquant_vllm.cuda.prefill import fused_paged_rq_int8_prefill
except ImportError:  # pragma: no cover
    fused_paged_rq_int8_prefill = None

__all__ = [
    "iso_compress",
    "iso_decompress",
    "planar_compress",
    "planar_decompress",
    "fused_paged_rq_int8_prefill",
    "fused_paged_rq_decode",
]
