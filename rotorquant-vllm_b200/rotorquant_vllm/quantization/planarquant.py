"""PlanarQuant: one Givens angle per pair of coordinates.

Follows src/rotorquant_vllm/quantization/planarquant.py of the reference
(``make_random_rotations`` :26-37, ``PlanarQuantMSE`` :68-182): angles are
``rand(n_groups) * 2 pi`` from seed ``seed``; the parameters are stored as
``(cos, sin)`` rows.
"""

from __future__ import annotations

import math

import torch

from ._block_quantizer import BlockRotationQuantizer


def make_random_rotations(n_groups: int, device="cpu", seed=None) -> torch.Tensor:
    """``(n_groups, 2)`` rows of ``[cos t, sin t]``, drawn on the CPU generator."""
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(seed)
    angles = torch.rand(n_groups, generator=gen) * (2 * math.pi)
    return torch.stack([angles.cos(), angles.sin()], dim=-1).to(device)


def rot2_apply(cs: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Rotate ``(..., 2)`` pairs by the angle whose ``[cos, sin]`` is ``cs``."""
    c, s = cs[..., 0], cs[..., 1]
    a, b = v[..., 0], v[..., 1]
    return torch.stack([c * a - s * b, s * a + c * b], dim=-1)


def rot2_inverse(cs: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Rotate ``(..., 2)`` pairs by minus that angle."""
    c, s = cs[..., 0], cs[..., 1]
    a, b = v[..., 0], v[..., 1]
    return torch.stack([c * a + s * b, c * b - s * a], dim=-1)


class PlanarQuantMSE(BlockRotationQuantizer):
    """Givens block rotation + Lloyd-Max codebook."""

    block = 2

    def __init__(self, d: int, bits: int, seed: int = 42, device="cpu"):
        super().__init__(d, bits, device)
        self.register_buffer("rot2", make_random_rotations(self.n_groups, device, seed))

    def _rotate(self, v: torch.Tensor) -> torch.Tensor:
        return rot2_apply(self.rot2, v)

    def _unrotate(self, v: torch.Tensor) -> torch.Tensor:
        return rot2_inverse(self.rot2, v)
