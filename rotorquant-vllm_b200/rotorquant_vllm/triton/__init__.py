"""Compatibility alias: the reference exposes its launchers as ``rotorquant_vllm.triton``
(triton/__init__.py:1-15).  This build has no Triton code; the same names resolve to the CUDA
launchers in ``rotorquant_vllm.cuda``."""

from rotorquant_vllm.cuda import (
    fused_paged_rq_decode,
    fused_paged_rq_int8_prefill,
    iso_compress,
    iso_decompress,
    planar_compress,
    planar_decompress,
)

__all__ = [
    "iso_compress",
    "iso_decompress",
    "planar_compress",
    "planar_decompress",
    "fused_paged_rq_int8_prefill",
    "fused_paged_rq_decode",
]
