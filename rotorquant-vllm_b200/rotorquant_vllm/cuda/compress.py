"""Compress launchers: ``iso_compress`` / ``planar_compress`` and the fused compress-and-store.

Mirror of triton/isoquant_compress.py:104-158 and triton/planarquant_compress.py:100-154 of the
reference (same names, arguments and results) plus the cache write of
``RQAttentionImpl._compress_and_store`` (vllm/rq_backend.py:585-657) as one kernel launch.
IsoQuant and PlanarQuant share one kernel: both rotations are block diagonal.
"""

from __future__ import annotations

import torch

from .. import _lib
from .rotation import validate_rotation

# (id(even), id(odd), versions) -> (even, odd, R).  The inputs are kept alive by the entry, so
# neither their ids nor their storage can be reused by another tensor while it is cached.
_DENSE_R: dict[tuple, tuple] = {}


def _dense_rotation(rot_T_even: torch.Tensor, rot_T_odd: torch.Tensor) -> torch.Tensor:
    """``R`` from the even / odd column halves of ``R^T`` the reference API passes around."""
    key = (id(rot_T_even), id(rot_T_odd), rot_T_even._version, rot_T_odd._version)
    hit = _DENSE_R.get(key)
    if hit is not None:
        return hit[2]
    d = rot_T_even.shape[0]
    rot_t = torch.empty(d, d, dtype=torch.float32, device=rot_T_even.device)
    rot_t[:, 0::2] = rot_T_even
    rot_t[:, 1::2] = rot_T_odd
    r = rot_t.T.contiguous()
    validate_rotation(r)
    if len(_DENSE_R) >= 8:
        _DENSE_R.pop(next(iter(_DENSE_R)))
    _DENSE_R[key] = (rot_T_even, rot_T_odd, r)
    return r


def _rows_16b_aligned(x: torch.Tensor) -> bool:
    es = x.element_size()
    return (x.stride(-1) == 1 and x.data_ptr() % 16 == 0
            and all((s * es) % 16 == 0 for s in x.stride()[:-1]))


def _compress(x: torch.Tensor, rot_T_even: torch.Tensor, rot_T_odd: torch.Tensor,
              boundaries: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    n, h, d = x.shape
    dev = _lib.require_cuda(x, rot_T_even, rot_T_odd, boundaries)
    rotation = _dense_rotation(rot_T_even, rot_T_odd)
    flat = x.reshape(n * h, d)
    if not _rows_16b_aligned(flat):
        flat = flat.contiguous()
    bounds = boundaries.to(torch.float32).contiguous()
    packed = torch.empty(n * h, d // 2, dtype=torch.uint8, device=dev)
    norms = torch.empty(n * h, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().rq_compress(
            flat.data_ptr(), _lib.dtype_code(flat.dtype), n * h, d, flat.stride(0),
            rotation.data_ptr(), bounds.data_ptr(), bounds.numel(), packed.data_ptr(),
            norms.data_ptr(), _lib.stream_ptr(dev)))
    return packed.reshape(n, h, d // 2), norms.reshape(n, h, 1)


def iso_compress(x: torch.Tensor, rot_T_even: torch.Tensor, rot_T_odd: torch.Tensor,
                 boundaries: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(N, H, D)`` -> nibble-packed ``(N, H, D/2)`` uint8 and fp32 norms ``(N, H, 1)``.

    Same contract as the reference ``iso_compress``; ``x`` may be fp16, bf16 or fp32.
    """
    return _compress(x, rot_T_even, rot_T_odd, boundaries)


def planar_compress(x: torch.Tensor, rot_T_even: torch.Tensor, rot_T_odd: torch.Tensor,
                    boundaries: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """PlanarQuant flavour of :func:`iso_compress` (identical arithmetic, 2x2 blocks)."""
    return _compress(x, rot_T_even, rot_T_odd, boundaries)


def compress_and_store(key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                       slot_mapping: torch.Tensor, rotation: torch.Tensor,
                       k_boundaries: torch.Tensor, v_boundaries: torch.Tensor,
                       write_padding: bool = True) -> None:
    """Compress ``N`` new K/V tokens ``(N, H, D)`` and write their cache slots in one launch.

    ``slot_mapping`` (int64) may be shorter than ``N`` (only the first ``len(slot_mapping)``
    tokens are written, as in the reference) and negative entries are skipped.
    """
    dev = _lib.require_cuda(key, value, kv_cache, slot_mapping, rotation, k_boundaries, v_boundaries)
    validate_rotation(rotation)
    if key.shape != value.shape or key.dim() != 3:
        raise ValueError(f"key/value must both be (N, H, D); got {tuple(key.shape)} and {tuple(value.shape)}")
    if key.dtype != value.dtype:
        raise ValueError("key and value must have the same dtype")
    if kv_cache.dtype != torch.uint8 or kv_cache.dim() != 3 or not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be a contiguous uint8 (num_blocks, block_size, total_bytes) tensor")
    if slot_mapping.dtype != torch.int64:
        raise ValueError("slot_mapping must be int64")
    n, h, d = key.shape
    n = min(n, slot_mapping.shape[0])
    if n == 0:
        return
    if not _rows_16b_aligned(key):
        key = key.contiguous()
    if not _rows_16b_aligned(value):
        value = value.contiguous()
    slot_mapping = slot_mapping.contiguous()
    kb = k_boundaries.to(torch.float32).contiguous()
    vb = v_boundaries.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().rq_compress_store(
            key.data_ptr(), value.data_ptr(), _lib.dtype_code(key.dtype), n, h, d,
            key.stride(0), key.stride(1), value.stride(0), value.stride(1),
            kv_cache.data_ptr(), kv_cache.shape[0] * kv_cache.shape[1], kv_cache.shape[2],
            slot_mapping.data_ptr(), rotation.data_ptr(), kb.data_ptr(), kb.numel(),
            vb.data_ptr(), vb.numel(), 1 if write_padding else 0, _lib.stream_ptr(dev)))
