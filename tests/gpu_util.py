"""Helpers shared by the GPU parity tests."""

from __future__ import annotations

import torch

import helpers

DEV = "cuda:0"


def on_gpu(case: dict) -> dict:
    """Copy every tensor of a golden case to the GPU."""
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}


def params(tag: str, k_bits: int, v_bits: int) -> dict:
    """Reference-generated codebooks and rotation for one configuration, on the CPU."""
    p = helpers.load_params()
    return {
        "R": p[f"{tag}_R"].reshape(128, 128).contiguous(),
        "k_centroids": p[f"{tag}_b{k_bits}_centroids"], "v_centroids": p[f"{tag}_b{v_bits}_centroids"],
        "k_boundaries": p[f"{tag}_b{k_bits}_boundaries"], "v_boundaries": p[f"{tag}_b{v_bits}_boundaries"],
    }


def attention_tolerance(ref_rot: torch.Tensor, ref_out: torch.Tensor, dtype: torch.dtype,
                        floor: float = 2e-3) -> torch.Tensor:
    """Element-wise bound on |out - reference|: 2e-3, or, where the reference output itself is
    coarser than that, one unit in the last place of the largest rotated element of the 4-block
    (a legal rounding flip of one rotated element moves the four outputs of its block by that
    much) plus one unit in the last place of the output."""
    scale = 1.0 if dtype == torch.bfloat16 else 8.0
    blk = ref_rot.abs().reshape(*ref_rot.shape[:-1], 32, 4).amax(-1, keepdim=True)
    blk = blk.expand(*ref_rot.shape[:-1], 32, 4).reshape(ref_rot.shape)
    unit = (helpers.ulp_bf16(blk) + helpers.ulp_bf16(ref_out.float())) / scale
    return torch.clamp(unit, min=floor)
