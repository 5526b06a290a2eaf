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
