"""Dense block-diagonal rotation matrices from the quantiser parameters (host side).

``R`` maps original space to rotated space: queries are pre-rotated by ``R^T`` (``q @ R.T``) and
attention outputs post-rotated by ``R``.  Mirrors ``_build_iso_R`` / ``_build_planar_R`` /
``_build_rotation_matrix`` of the reference (vllm/rq_backend.py:194-264), including the fact that
IsoQuant "fast" mode in the serving path is the sandwich ``q_L v conj(q_L)`` (:226-234), not the
one-sided product of ``IsoQuantMSE._rotate``.  This module does not import vLLM.
"""

from __future__ import annotations

import torch


def _left_matrices(q: torch.Tensor) -> torch.Tensor:
    """``(n, 4, 4)`` matrices of ``v -> q v`` for quaternions ``q = [w, x, y, z]``."""
    w, x, y, z = q.unbind(-1)
    return torch.stack([
        torch.stack([w, -x, -y, -z], -1),
        torch.stack([x, w, -z, y], -1),
        torch.stack([y, z, w, -x], -1),
        torch.stack([z, -y, x, w], -1),
    ], dim=-2)


def _right_conj_matrices(q: torch.Tensor) -> torch.Tensor:
    """``(n, 4, 4)`` matrices of ``v -> v conj(q)``."""
    w, x, y, z = q.unbind(-1)
    return torch.stack([
        torch.stack([w, x, y, z], -1),
        torch.stack([-x, w, -z, y], -1),
        torch.stack([-y, z, w, -x], -1),
        torch.stack([-z, -y, x, w], -1),
    ], dim=-2)


def build_iso_R(quantizer, d: int, device, mode: str = "fast") -> torch.Tensor:
    """``(d, d)`` fp32 rotation of an ``IsoQuantMSE``: 4x4 diagonal blocks ``L(q_L) @ Rc(q)`` with
    ``q = q_R`` in full mode and ``q = q_L`` in fast mode."""
    q_l = quantizer.q_L.detach().to("cpu", torch.float32)
    q_r = quantizer.q_R.detach().to("cpu", torch.float32) if mode == "full" else q_l
    left, right = _left_matrices(q_l), _right_conj_matrices(q_r)
    rot = torch.eye(quantizer.d_padded, dtype=torch.float32)
    for g in range(quantizer.n_groups):
        rot[4 * g:4 * g + 4, 4 * g:4 * g + 4] = left[g] @ right[g]
    return rot[:d, :d].contiguous().to(device)


def build_planar_R(quantizer, d: int, device) -> torch.Tensor:
    """``(d, d)`` fp32 rotation of a ``PlanarQuantMSE``: 2x2 diagonal blocks ``[[c, -s], [s, c]]``."""
    rot2 = quantizer.rot2.detach().to("cpu", torch.float32)
    rot = torch.eye(quantizer.d_padded, dtype=torch.float32)
    idx = torch.arange(quantizer.n_groups) * 2
    c, s = rot2[:, 0], rot2[:, 1]
    rot[idx, idx] = c
    rot[idx, idx + 1] = -s
    rot[idx + 1, idx] = s
    rot[idx + 1, idx + 1] = c
    return rot[:d, :d].contiguous().to(device)


def build_rotation_matrix(quantizer, d: int, device) -> torch.Tensor:
    """Rotation matrix of either quantiser kind."""
    if hasattr(quantizer, "q_L"):
        return build_iso_R(quantizer, d, device, getattr(quantizer, "mode", "fast"))
    return build_planar_R(quantizer, d, device)
