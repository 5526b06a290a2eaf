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


from oracle.tolerance import attention_tolerance  # noqa: E402,F401  (shared with smoke and bench)
