"""IsoQuant: one unit quaternion pair per 4-wide block.

``SO(4) ~ SU(2) x SU(2)``: ``T(v) = q_L v conj(q_R)`` ("full", 6 degrees of freedom
per block) or ``T(v) = q_L v`` ("fast", 3).  Follows
src/rotorquant_vllm/quantization/isoquant.py of the reference
(``make_random_unit_quaternion`` :46-55, ``IsoQuantMSE`` :60-208): ``q_L`` comes
from seed ``seed`` and ``q_R`` from ``seed + 10000`` as ``randn(n_groups, 4)``
rows normalised to unit length.
"""

from __future__ import annotations

import torch

from ._block_quantizer import BlockRotationQuantizer

_CONJ = (1.0, -1.0, -1.0, -1.0)


def quat_conjugate(q: torch.Tensor) -> torch.Tensor:
    """``(w, x, y, z) -> (w, -x, -y, -z)``."""
    return q * torch.tensor(_CONJ, dtype=q.dtype, device=q.device)


def quat_multiply(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Hamilton product of ``(..., 4)`` quaternions stored as ``[w, x, y, z]``."""
    aw, ax, ay, az = a.unbind(-1)
    bw, bx, by, bz = b.unbind(-1)
    return torch.stack([
        aw * bw - ax * bx - ay * by - az * bz,
        aw * bx + ax * bw + ay * bz - az * by,
        aw * by - ax * bz + ay * bw + az * bx,
        aw * bz + ax * by - ay * bx + az * bw,
    ], dim=-1)


def make_random_unit_quaternion(shape, device="cpu", seed=None) -> torch.Tensor:
    """Normalised Gaussian quaternions of shape ``(*shape, 4)``, drawn on the CPU generator."""
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(seed)
    q = torch.randn(*shape, 4, generator=gen)
    q = q / q.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    return q.to(device)


class IsoQuantMSE(BlockRotationQuantizer):
    """Quaternion block rotation + Lloyd-Max codebook."""

    block = 4

    def __init__(self, d: int, bits: int, seed: int = 42, mode: str = "fast", device="cpu"):
        if mode not in ("fast", "full"):
            raise ValueError(f"mode must be 'fast' or 'full', got '{mode}'")
        super().__init__(d, bits, device)
        self.mode = mode
        self.register_buffer("q_L", make_random_unit_quaternion((self.n_groups,), device, seed))
        if mode == "full":
            self.register_buffer(
                "q_R", make_random_unit_quaternion((self.n_groups,), device, seed + 10000))

    def _rotate(self, v: torch.Tensor) -> torch.Tensor:
        left = quat_multiply(self.q_L, v)
        return quat_multiply(left, quat_conjugate(self.q_R)) if self.mode == "full" else left

    def _unrotate(self, v: torch.Tensor) -> torch.Tensor:
        left = quat_multiply(quat_conjugate(self.q_L), v)
        return quat_multiply(left, self.q_R) if self.mode == "full" else left
