"""Fused INT8 prefill launcher, mirror of ``fused_paged_rq_int8_prefill``
(triton/fused_paged_rq_int8_prefill.py:247-363 of the reference): same positional arguments and
result for one sequence; ``cu_seqlens_q`` adds several sequences and cached prefixes."""

from __future__ import annotations

import math

import torch

from .. import _lib
from .rotation import validate_rotation


def fused_paged_rq_int8_prefill(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    block_size: int,
    sm_scale: float | None = None,
    out: torch.Tensor | None = None,
    *,
    cu_seqlens_q: torch.Tensor | None = None,
    max_q_len: int | None = None,
    error_flag: torch.Tensor | None = None,
) -> torch.Tensor:
    """Causal attention of ``q (num_tokens, H_Q, D)`` over the compressed paged cache.

    Without ``cu_seqlens_q`` this is the reference contract: one sequence, ``seq_lens`` has one
    entry (``ValueError`` otherwise, as upstream :305-309).  With ``cu_seqlens_q`` (int32,
    ``num_seqs + 1`` entries) sequence ``s`` owns rows ``cu[s]:cu[s+1]``; in both cases the query
    rows of a sequence are the last rows of its ``seq_lens[s]`` cached tokens.
    """
    num_tokens, hq, d = q.shape
    assert d == head_dim
    assert hq % num_kv_heads == 0
    assert kv_cache.dtype == torch.uint8
    assert block_table.dtype == torch.int32
    assert seq_lens.dtype == torch.int32
    if cu_seqlens_q is None and seq_lens.numel() != 1:
        raise ValueError(
            "fused_paged_rq_int8_prefill supports only a single sequence without cu_seqlens_q, "
            f"but got seq_lens.numel() == {seq_lens.numel()}.")
    dev = _lib.require_cuda(q, kv_cache, block_table, seq_lens, k_centroids, v_centroids, rotation,
                            out, cu_seqlens_q, error_flag)
    validate_rotation(rotation)
    num_seqs = seq_lens.numel()
    if kv_cache.dim() != 3 or kv_cache.shape[1] != block_size or not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be contiguous (num_blocks, block_size, total_bytes)")
    if block_table.dim() == 1:
        block_table = block_table.unsqueeze(0)
    if block_table.shape[0] != num_seqs or block_table.stride(1) != 1:
        raise ValueError("block_table must be (num_seqs, max_blocks) with a contiguous last dim")
    if cu_seqlens_q is not None:
        if cu_seqlens_q.numel() != num_seqs + 1:
            raise ValueError(f"cu_seqlens_q needs {num_seqs + 1} entries, got {cu_seqlens_q.numel()}")
        cu_seqlens_q = cu_seqlens_q.to(torch.int32).contiguous()
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if q.stride(2) != 1:
        q = q.contiguous()
    result = out if out is not None else torch.empty_like(q)
    if result.shape != q.shape or result.dtype != q.dtype or result.stride(2) != 1:
        raise ValueError("out must match q in shape and dtype with a contiguous last dim")
    if num_tokens == 0:
        return result
    ck = k_centroids.to(torch.float32).contiguous()
    cv = v_centroids.to(torch.float32).contiguous()
    seq_lens = seq_lens.contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().rq_prefill_int8(
            q.data_ptr(), result.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
            result.stride(0), result.stride(1),
            cu_seqlens_q.data_ptr() if cu_seqlens_q is not None else None,
            num_tokens, num_seqs, int(max_q_len or 0), hq, num_kv_heads, head_dim,
            kv_cache.data_ptr(), kv_cache.shape[0], block_size, kv_cache.shape[2],
            block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
            ck.data_ptr(), ck.numel(), cv.data_ptr(), cv.numel(), rotation.data_ptr(),
            float(sm_scale), error_flag.data_ptr() if error_flag is not None else None,
            _lib.stream_ptr(dev)))
    return result
