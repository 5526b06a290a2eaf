"""Element-wise acceptance bound for attention outputs.  TEST INFRASTRUCTURE ONLY.

The bar for attention over the compressed cache is 2e-3 max-abs against "reference decompress plus
SDPA" (vllm/rq_backend.py:938-948, :1033-1034 of the reference: the rotated output is rounded to
the query dtype and then multiplied by R).  Where the reference's own output grid is coarser than
2e-3 -- one bf16 unit in the last place is 3.9e-3 for |o| >= 0.5 -- a result that differs by one
legal rounding flip cannot be told from the reference, and the bound widens to exactly that flip.
Used by the GPU tests, ``__graft_entry__.smoke()`` and the parity check of ``bench.py``.
"""

from __future__ import annotations

import torch


def ulp_bf16(x: torch.Tensor) -> torch.Tensor:
    """Size of one bf16 unit in the last place at |x| (fp32 tensor)."""
    e = torch.floor(torch.log2(x.abs().float().clamp_min(1e-30)))
    return torch.pow(2.0, e - 7)


def attention_tolerance(ref_rot: torch.Tensor, ref_out: torch.Tensor, dtype: torch.dtype,
                        floor: float = 2e-3) -> torch.Tensor:
    """Bound on |out - reference| per element: ``floor``, or, where the reference output itself is
    coarser than that, one unit in the last place of the largest rotated element of the 4-block
    (a rounding flip of one rotated element moves the four outputs of its block by that much)
    plus one unit in the last place of the output.  fp16 units are an eighth of bf16 units."""
    scale = 1.0 if dtype == torch.bfloat16 else 8.0
    blk = ref_rot.abs().reshape(*ref_rot.shape[:-1], 32, 4).amax(-1, keepdim=True)
    blk = blk.expand(*ref_rot.shape[:-1], 32, 4).reshape(ref_rot.shape)
    unit = (ulp_bf16(blk) + ulp_bf16(ref_out.float())) / scale
    return torch.clamp(unit, min=floor)


def excess(out: torch.Tensor, ref_rot: torch.Tensor, ref_out: torch.Tensor, dtype: torch.dtype,
           floor: float = 2e-3) -> tuple[float, int]:
    """``(max |out - ref|, number of elements over the bound)``; NaNs count as over."""
    diff = (out.float() - ref_out.float()).abs()
    bad = (diff > attention_tolerance(ref_rot, ref_out, dtype, floor)) | torch.isnan(out.float())
    return float(diff.nan_to_num(nan=float("inf")).max()), int(bad.sum())
