"""Host-side check that a rotation matrix has the structure the kernels rely on."""

from __future__ import annotations

import weakref

import torch

# id(tensor) -> (weak reference, version at validation time).  The table has no size limit: a
# model builds one matrix per attention layer and every layer must stay validated.  An entry
# disappears with its tensor (the weak reference's callback), so an id that Python hands to a new
# tensor afterwards cannot match an old entry.
_VALIDATED: dict[int, tuple] = {}

# Number of full validations performed (a host copy each); tests read it.
validations = 0


def validate_rotation(rotation: torch.Tensor) -> None:
    """Raise ``ValueError`` unless ``rotation`` is a contiguous fp32 ``(128, 128)`` matrix whose
    non-zero entries all lie in its 4x4 diagonal blocks (IsoQuant) -- 2x2 Givens blocks
    (PlanarQuant) are a special case.  The kernels read only those blocks.

    The check copies the matrix to the host once per tensor object (and again after an in-place
    modification), which synchronises with the device: validate a matrix where it is built, not
    on the request path.  Later calls with the same object cost one dictionary lookup and never
    touch the device, so they are legal inside a CUDA graph capture.
    """
    global validations
    key = id(rotation)
    hit = _VALIDATED.get(key)
    if hit is not None and hit[0]() is rotation and hit[1] == rotation._version:
        return
    if rotation.dtype != torch.float32 or tuple(rotation.shape) != (128, 128):
        raise ValueError(f"rotation must be fp32 (128, 128), got {rotation.dtype} {tuple(rotation.shape)}")
    if not rotation.is_contiguous():
        raise ValueError("rotation must be contiguous")
    validations += 1
    r = rotation.detach().to("cpu")
    blocks = torch.block_diag(*[torch.ones(4, 4) for _ in range(32)]).bool()
    if bool((r[~blocks] != 0).any()):
        raise ValueError("rotation has non-zero entries outside its 4x4 diagonal blocks")

    def _forget(_ref, key=key):
        entry = _VALIDATED.get(key)
        if entry is not None and entry[0] is _ref:
            del _VALIDATED[key]

    _VALIDATED[key] = (weakref.ref(rotation, _forget), rotation._version)
