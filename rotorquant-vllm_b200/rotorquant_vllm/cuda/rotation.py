"""Host-side check that a rotation matrix has the structure the kernels rely on."""

from __future__ import annotations

import torch

# id(tensor) -> (tensor, version).  The tensor is kept alive by the entry so that its id cannot be
# reused by a different matrix while it is cached.
_VALIDATED: dict[int, tuple] = {}


def validate_rotation(rotation: torch.Tensor) -> None:
    """Raise ``ValueError`` unless ``rotation`` is a contiguous fp32 ``(128, 128)`` matrix whose
    non-zero entries all lie in its 4x4 diagonal blocks (IsoQuant) -- 2x2 Givens blocks
    (PlanarQuant) are a special case.  The kernels read only those blocks.

    The check copies the matrix to the host once per tensor object (and again after an in-place
    modification), so the first call with a new matrix must not happen inside a CUDA graph
    capture.
    """
    hit = _VALIDATED.get(id(rotation))
    if hit is not None and hit[0] is rotation and hit[1] == rotation._version:
        return
    if rotation.dtype != torch.float32 or tuple(rotation.shape) != (128, 128):
        raise ValueError(f"rotation must be fp32 (128, 128), got {rotation.dtype} {tuple(rotation.shape)}")
    if not rotation.is_contiguous():
        raise ValueError("rotation must be contiguous")
    r = rotation.detach().to("cpu")
    blocks = torch.block_diag(*[torch.ones(4, 4) for _ in range(32)]).bool()
    if bool((r[~blocks] != 0).any()):
        raise ValueError("rotation has non-zero entries outside its 4x4 diagonal blocks")
    if len(_VALIDATED) >= 16:
        _VALIDATED.pop(next(iter(_VALIDATED)))
    _VALIDATED[id(rotation)] = (rotation, rotation._version)
