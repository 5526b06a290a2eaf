"""Kernel launchers of the B200 build: the host-side mirror of the reference's
``rotorquant_vllm.triton`` package, calling librq_b200.so through its C ABI."""

from .compress import compress_and_store, iso_compress, planar_compress
from .decode import decode_workspace_bytes, fused_paged_rq_decode, reserve_decode_workspace
from .decompress import decompress_blocks, decompress_cache_paged, iso_decompress, planar_decompress
from .prefill import fused_paged_rq_int8_prefill, reserve_prefill_scratch
from .rotation import validate_rotation

__all__ = [
    "iso_compress",
    "planar_compress",
    "iso_decompress",
    "planar_decompress",
    "decompress_blocks",
    "decompress_cache_paged",
    "compress_and_store",
    "fused_paged_rq_decode",
    "fused_paged_rq_int8_prefill",
    "decode_workspace_bytes",
    "reserve_decode_workspace",
    "reserve_prefill_scratch",
    "validate_rotation",
]
