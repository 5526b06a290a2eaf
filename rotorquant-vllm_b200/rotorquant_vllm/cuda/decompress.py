"""Decompress launchers, mirror of triton/isoquant_decompress.py:63-100 and
triton/planarquant_decompress.py:63-101 of the reference."""

from __future__ import annotations

import torch

from .. import _lib


def _decompress(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor,
                dtype: torch.dtype) -> torch.Tensor:
    n, h, half = packed.shape
    dev = _lib.require_cuda(packed, norms, centroids)
    if packed.dtype != torch.uint8:
        raise ValueError("packed must be uint8")
    p = packed.reshape(n * h, half).contiguous()
    nr = norms.reshape(n * h).to(torch.float32).contiguous()
    c = centroids.to(torch.float32).contiguous()
    out = torch.empty(n * h, half * 2, dtype=dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().rq_decompress(
            p.data_ptr(), nr.data_ptr(), n * h, half * 2, c.data_ptr(), c.numel(),
            out.data_ptr(), _lib.dtype_code(dtype), _lib.stream_ptr(dev)))
    return out.reshape(n, h, half * 2)


def iso_decompress(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor,
                   dtype: torch.dtype) -> torch.Tensor:
    """Nibble-packed ``(N, H, D/2)`` + norms ``(N, H, 1)`` -> ``(N, H, D)`` in ``dtype`` (rotated space)."""
    return _decompress(packed, norms, centroids, dtype)


def planar_decompress(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor,
                      dtype: torch.dtype, d_padded: int | None = None) -> torch.Tensor:
    """PlanarQuant flavour; ``d_padded`` is accepted (the reference's backend passes it,
    vllm/rq_backend.py:704-707) and must equal the head size if given."""
    if d_padded is not None and d_padded != packed.shape[-1] * 2:
        raise ValueError(f"d_padded={d_padded} does not match head size {packed.shape[-1] * 2}")
    return _decompress(packed, norms, centroids, dtype)


def decompress_blocks(kv_cache: torch.Tensor, blocks: torch.Tensor | None, num_kv_heads: int,
                      centroids_k: torch.Tensor, centroids_v: torch.Tensor,
                      dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """Decompressed K and V ``(n, block_size, H, 128)`` of the cache blocks listed in ``blocks``
    (int32, on the device; ``None`` = every block), in one launch straight from the slot layout."""
    dev = _lib.require_cuda(kv_cache, blocks, centroids_k, centroids_v)
    if kv_cache.dtype != torch.uint8 or kv_cache.dim() != 3 or not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be a contiguous uint8 (num_blocks, block_size, total_bytes) tensor")
    nb, bs, total = kv_cache.shape
    if blocks is not None:
        if blocks.dtype != torch.int32:
            raise ValueError("blocks must be int32")
        blocks = blocks.contiguous()
    n = nb if blocks is None else blocks.numel()
    ck = centroids_k.to(torch.float32).contiguous()
    cv = centroids_v.to(torch.float32).contiguous()
    out_k = torch.empty(n, bs, num_kv_heads, 128, dtype=dtype, device=dev)
    out_v = torch.empty_like(out_k)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().rq_decompress_blocks(
            kv_cache.data_ptr(), nb, bs, total, num_kv_heads, 128,
            blocks.data_ptr() if blocks is not None else None, n, ck.data_ptr(), ck.numel(),
            cv.data_ptr(), cv.numel(), out_k.data_ptr(), out_v.data_ptr(), _lib.dtype_code(dtype),
            _lib.stream_ptr(dev)))
    return out_k, out_v


def decompress_cache_paged(kv_cache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                           num_kv_heads: int, centroids_k: torch.Tensor, centroids_v: torch.Tensor,
                           dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Mirror of ``RQAttentionImpl._decompress_cache_paged`` (vllm/rq_backend.py:737-852 of the
    reference): decompress only the physical blocks the batch references and return
    ``(key_cache, value_cache, remapped_block_table)`` with K/V ``(num_unique, block_size, H, 128)``
    and the table renumbered into that compact block space.  ``torch.unique`` sizes its result on
    the host, as upstream; the gather, the per-head split and both decompressions are one launch."""
    nb, bs, _ = kv_cache.shape
    need = (seq_lens.to(torch.int64) + bs - 1) // bs
    cols = torch.arange(block_table.shape[1], device=block_table.device).unsqueeze(0)
    unique_blocks = torch.unique(block_table[cols < need.unsqueeze(1)], sorted=True).to(torch.int32)
    k, v = decompress_blocks(kv_cache, unique_blocks, num_kv_heads, centroids_k, centroids_v, dtype)
    remap = torch.zeros(nb, dtype=block_table.dtype, device=block_table.device)
    remap[unique_blocks.long()] = torch.arange(unique_blocks.numel(), dtype=block_table.dtype,
                                               device=block_table.device)
    return k, v, remap[block_table.long()]
