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
    max_seq_len: int | None = None,
    workspace: torch.Tensor | None = None,
    staged: bool | None = None,
) -> torch.Tensor:
    """Causal attention of ``q (num_tokens, H_Q, D)`` over the compressed paged cache.

    Without ``cu_seqlens_q`` this is the reference contract: one sequence, ``seq_lens`` has one
    entry (``ValueError`` otherwise, as upstream :305-309).  With ``cu_seqlens_q`` (int32,
    ``num_seqs + 1`` entries) sequence ``s`` owns rows ``cu[s]:cu[s+1]``; in both cases the query
    rows of a sequence are the last rows of its ``seq_lens[s]`` cached tokens.

    Two implementations give the same result: the fused kernel rebuilds the K/V tiles for every
    block of query rows; the staged one (``rq_prefill_int8_staged``) decompresses every tile once
    into scratch memory first.  The scratch is ``num_seqs * ceil(bound / 128) * H * 49664`` bytes
    with ``bound`` = ``max_seq_len``, else the width of the block table.  ``staged=None`` picks the
    staged path when the caller lends a ``workspace`` (uint8), or when the scratch fits the buffer
    kept per device -- reserved up front by :func:`reserve_prefill_scratch`, grown on demand up to
    ``SCRATCH_CAP`` bytes but never while a CUDA graph is being captured -- and the fused kernel
    otherwise, so that no call allocates beyond the cap.
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
    lib = _lib.lib()
    bound = int(max_seq_len) if max_seq_len else block_table.shape[1] * block_size
    need = lib.rq_prefill_workspace_bytes(num_seqs, num_kv_heads, bound)
    if staged is None:
        staged = workspace is not None or _scratch_available(dev, need)
    common = (
        q.data_ptr(), result.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
        result.stride(0), result.stride(1),
        cu_seqlens_q.data_ptr() if cu_seqlens_q is not None else None,
        num_tokens, num_seqs, int(max_q_len or 0), hq, num_kv_heads, head_dim,
        kv_cache.data_ptr(), kv_cache.shape[0], block_size, kv_cache.shape[2],
        block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
        ck.data_ptr(), ck.numel(), cv.data_ptr(), cv.numel(), rotation.data_ptr(),
        float(sm_scale), error_flag.data_ptr() if error_flag is not None else None)
    with torch.cuda.device(dev):
        if staged:
            if workspace is None:
                workspace = _scratch(dev, need)
            else:
                _lib.require_cuda(workspace)
                if workspace.dtype != torch.uint8 or not workspace.is_contiguous():
                    raise ValueError("workspace must be a contiguous uint8 tensor")
            _lib.check(lib.rq_prefill_int8_staged(*common, bound, workspace.data_ptr(), workspace.numel(),
                                                   _lib.stream_ptr(dev)))
        else:
            _lib.check(lib.rq_prefill_int8(*common, _lib.stream_ptr(dev)))
    return result


_SCRATCH: dict = {}
SCRATCH_CAP = 1 << 30          # the per-device buffer never grows beyond this many bytes


def reserve_prefill_scratch(dev: torch.device, nbytes: int) -> None:
    """Allocate the per-device scratch of the staged path now (at most ``SCRATCH_CAP`` bytes), so
    that later calls inside the serving loop find it in place."""
    _scratch(torch.device(dev), min(int(nbytes), SCRATCH_CAP))


def _scratch_available(dev: torch.device, nbytes: int) -> bool:
    """True when ``nbytes`` of scratch are in place, or may be put in place now (under the cap and
    not inside a graph capture, where allocating is an error)."""
    buf = _SCRATCH.get(dev)
    if buf is not None and buf.numel() >= nbytes:
        return True
    return nbytes <= SCRATCH_CAP and not torch.cuda.is_current_stream_capturing()


def _scratch(dev: torch.device, nbytes: int) -> torch.Tensor:
    """One scratch buffer per device for the staged path, grown when a call needs more."""
    buf = _SCRATCH.get(dev)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        _SCRATCH[dev] = buf
    return buf
