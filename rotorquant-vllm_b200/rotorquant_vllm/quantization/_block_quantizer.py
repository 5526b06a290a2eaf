"""Shared skeleton of the block-rotation quantisers (IsoQuant: 4-wide blocks,
PlanarQuant: 2-wide blocks): split norm and direction, rotate each block,
Lloyd-Max per coordinate, and the inverse.

These ``quantize`` / ``dequantize`` methods are the *reference quantiser* of the
upstream project (quantization/isoquant.py:156-202, planarquant.py:130-176);
they are used for quality checks only.  The serving path goes through the
CUDA compress kernel, which buckets with the codebook boundaries.

Parameters are always drawn on the CPU generator and then moved to ``device``,
so the rotation does not depend on which device the layer lives on.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .lloyd_max import LloydMaxCodebook


class BlockRotationQuantizer(nn.Module):
    """Base class: subclasses set ``block`` and implement ``_rotate`` / ``_unrotate``."""

    block: int = 1

    def __init__(self, d: int, bits: int, device="cpu"):
        super().__init__()
        self.d = d
        self.bits = bits
        self.n_groups = (d + self.block - 1) // self.block
        self.d_padded = self.n_groups * self.block
        book = LloydMaxCodebook(d, bits)
        self.register_buffer("centroids", book.centroids.to(device))
        self.register_buffer("boundaries", book.boundaries.to(device))

    # -- blocks ---------------------------------------------------------
    def _embed(self, x: torch.Tensor) -> torch.Tensor:
        """``(..., d)`` -> ``(..., n_groups, block)`` with zero padding."""
        if self.d_padded > self.d:
            x = torch.nn.functional.pad(x, (0, self.d_padded - self.d))
        return x.reshape(*x.shape[:-1], self.n_groups, self.block)

    def _extract(self, v: torch.Tensor) -> torch.Tensor:
        """``(..., n_groups, block)`` -> ``(..., d)``."""
        return v.reshape(*v.shape[:-2], -1)[..., :self.d]

    def _rotate(self, v: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def _unrotate(self, v: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    # -- quantiser ------------------------------------------------------
    def _quantize_scalar(self, x: torch.Tensor):
        idx = (x.unsqueeze(-1) - self.centroids).abs().argmin(dim=-1)
        return self.centroids[idx], idx

    def quantize(self, x: torch.Tensor):
        """``(..., d)`` -> (rotated quantised blocks, ``{'indices', '_norms'}``)."""
        norms = torch.norm(x, dim=-1, keepdim=True).clamp(min=1e-8)
        rotated = self._rotate(self._embed(x / norms))
        flat = rotated.reshape(*rotated.shape[:-2], -1)
        values, idx = self._quantize_scalar(flat)
        return values.reshape_as(rotated), {"indices": idx, "_norms": norms.squeeze(-1)}

    def dequantize(self, indices_dict: dict) -> torch.Tensor:
        """Indices (and norms, if present) -> reconstructed ``(..., d)`` vectors."""
        values = self.centroids[indices_dict["indices"]]
        blocks = values.reshape(*values.shape[:-1], self.n_groups, self.block)
        x_hat = self._extract(self._unrotate(blocks))
        norms = indices_dict.get("_norms")
        if norms is not None:
            if norms.dim() < x_hat.dim():
                norms = norms.unsqueeze(-1)
            x_hat = x_hat * norms
        return x_hat

    def forward(self, x: torch.Tensor):
        """Quantise then reconstruct."""
        _, indices = self.quantize(x)
        return self.dequantize(indices), indices
