"""Host-side parameters are pinned bit for bit to the reference's own.

``tests/golden/params.npz`` holds the codebooks, quaternions / Givens pairs and rotation matrices
the reference produced (quantization/lloyd_max.py:32-86, isoquant.py:46-55 and :72-102,
planarquant.py:26-37, vllm/rq_backend.py:194-264).  The product's ``rotorquant_vllm.quantization``
and ``rotorquant_vllm.vllm.rotation`` must reproduce every one of them exactly: the compress
kernel is bit-exact only if the boundaries and the rotation are.
"""

import pytest
import torch

import helpers
from rotorquant_vllm.cuda import rotation as rot_check
from rotorquant_vllm.quantization import IsoQuantMSE, PlanarQuantMSE
from rotorquant_vllm.vllm.rotation import build_rotation_matrix

CONFIGS = [("iso_fast", "iso", "fast"), ("iso_full", "iso", "full"), ("planar", "planar", "fast")]


def _quantizer(mode, iso_mode, bits):
    if mode == "iso":
        return IsoQuantMSE(128, bits, seed=42, mode=iso_mode, device="cpu")
    return PlanarQuantMSE(128, bits, seed=42, device="cpu")


def _same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.contiguous().float(), b.contiguous().float()
    return a.shape == b.shape and torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("tag,mode,iso_mode", CONFIGS)
def test_codebooks_match_the_reference_bit_for_bit(tag, mode, iso_mode):
    p = helpers.load_params()
    for bits in (3, 4):
        qz = _quantizer(mode, iso_mode, bits)
        assert _same_bits(qz.centroids, p[f"{tag}_b{bits}_centroids"]), f"{tag} {bits}-bit centroids"
        assert _same_bits(qz.boundaries, p[f"{tag}_b{bits}_boundaries"]), f"{tag} {bits}-bit boundaries"


@pytest.mark.parametrize("tag,mode,iso_mode", CONFIGS)
def test_rotation_parameters_and_matrix_match_the_reference_bit_for_bit(tag, mode, iso_mode):
    p = helpers.load_params()
    qz = _quantizer(mode, iso_mode, 3)
    if mode == "iso":
        assert _same_bits(qz.q_L, p[f"{tag}_q_L"].reshape(32, 4))
        if iso_mode == "full":
            assert _same_bits(qz.q_R, p[f"{tag}_q_R"].reshape(32, 4))
    else:
        assert _same_bits(qz.rot2, p[f"{tag}_rot2"].reshape(64, 2))
    R = build_rotation_matrix(qz, 128, "cpu")
    assert _same_bits(R, p[f"{tag}_R"].reshape(128, 128))
    # K and V quantisers of different widths share the seed, hence the matrix
    assert _same_bits(build_rotation_matrix(_quantizer(mode, iso_mode, 4), 128, "cpu"), R)


def test_rotation_validation_is_remembered_for_every_layer():
    """A model has one rotation tensor per attention layer (32 for an 8B Llama).  Each must be
    validated once, with its host copy, and never again: a second pass over all layers must not
    touch the tensors, otherwise the request path synchronises and cannot be graph-captured."""
    base = build_rotation_matrix(_quantizer("iso", "fast", 3), 128, "cpu")
    layers = [base.clone() for _ in range(40)]
    before = rot_check.validations
    for r in layers:
        rot_check.validate_rotation(r)
    assert rot_check.validations == before + 40
    for _ in range(3):
        for r in layers:
            rot_check.validate_rotation(r)
    assert rot_check.validations == before + 40
    # an in-place change is noticed
    layers[7][0, 100] = 0.5
    with pytest.raises(ValueError, match="diagonal"):
        rot_check.validate_rotation(layers[7])
    # entries vanish with their tensors, so a recycled id cannot pass for a validated matrix
    n = len(rot_check._VALIDATED)
    del layers
    import gc

    gc.collect()
    assert len(rot_check._VALIDATED) <= n - 39
