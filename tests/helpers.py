"""Shared helpers for the tests: golden-vector loading and bit casts."""

from __future__ import annotations

import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def from_bits(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Inverse of the generator's ``bits_of``: raw unsigned storage -> tensor of ``dtype``."""
    if dtype in (torch.bfloat16, torch.float16):
        return torch.from_numpy(arr.view(np.int16).copy()).view(dtype)
    if dtype == torch.float32:
        return torch.from_numpy(arr.view(np.int32).copy()).view(torch.float32)
    return torch.from_numpy(arr.copy())


def load_params() -> dict:
    """Reference-generated codebooks and rotation matrices: ``{name: fp32 tensor}``."""
    z = np.load(os.path.join(GOLDEN, "params.npz"))
    return {k: from_bits(z[k], torch.float32) for k in z.files}


def case_names(prefix: str = "case_") -> list[str]:
    files = sorted(glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))
    return [os.path.basename(f)[:-4] for f in files]


def decode_case_names() -> list[str]:
    return [n for n in case_names() if "prefill" not in n and "digest" not in n]


def prefill_case_names() -> list[str]:
    return [n for n in case_names() if "prefill" in n]


def load_case(name: str) -> dict:
    """One golden case with tensors restored to their dtypes, plus its codebooks and R."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    c = {k: z[k] for k in z.files}
    out = {}
    for k in ("tag", "in_dtype", "q_dtype"):
        if k in c:
            out[k] = str(c[k])
    for k in ("k_bits", "v_bits", "num_kv_heads", "num_q_heads"):
        out[k] = int(c[k])
    out["sm_scale"] = float(c["sm_scale"])
    qdt = _DT[out["q_dtype"]]
    if "key" in c:
        idt = _DT[out["in_dtype"]]
        out["key"] = from_bits(c["key"], idt)
        out["value"] = from_bits(c["value"], idt)
        out["slot_mapping"] = torch.from_numpy(c["slot_mapping"].copy())
    out["block_table"] = torch.from_numpy(c["block_table"].copy())
    out["seq_lens"] = torch.from_numpy(c["seq_lens"].copy())
    out["kv_cache"] = torch.from_numpy(c["kv_cache"].copy())
    out["q"] = from_bits(c["q"], qdt)
    out["out"] = from_bits(c["out"], qdt)
    out["o_rot"] = torch.from_numpy(c["o_rot"].copy())
    p = load_params()
    tag = out["tag"]
    out["R"] = p[f"{tag}_R"].reshape(128, 128)
    out["k_centroids"] = p[f"{tag}_b{out['k_bits']}_centroids"]
    out["v_centroids"] = p[f"{tag}_b{out['v_bits']}_centroids"]
    out["k_boundaries"] = p[f"{tag}_b{out['k_bits']}_boundaries"]
    out["v_boundaries"] = p[f"{tag}_b{out['v_bits']}_boundaries"]
    return out


from oracle.tolerance import ulp_bf16  # noqa: E402,F401
