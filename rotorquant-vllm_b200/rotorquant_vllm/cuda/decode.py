"""Fused paged decode launcher, mirror of ``fused_paged_rq_decode``
(triton/fused_paged_rq_decode.py:214-312 of the reference): same positional arguments, same
result, plus keyword-only knobs for callers that manage scratch memory themselves."""

from __future__ import annotations

import math

import torch

from .. import _lib
from .rotation import validate_rotation

_WORKSPACE: dict[torch.device, torch.Tensor] = {}


def decode_workspace_bytes(num_seqs: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
                           max_seq_len: int, num_splits: int = 0) -> int:
    """Scratch bytes one decode call needs (partial results of the context splits)."""
    return int(_lib.lib().rq_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim,
                                                     max_seq_len, num_splits))


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Per-device scratch buffer, grown on demand.  Calls on one stream reuse it safely; callers
    that run decode on several streams at once must pass their own ``workspace``.  Growing it
    while a CUDA graph is being captured is refused: the allocation would be an error, and graphs
    captured earlier would keep pointing at the buffer that is dropped -- reserve the largest batch
    first (:func:`reserve_decode_workspace`)."""
    buf = _WORKSPACE.get(dev)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                f"rotorquant_vllm: decode needs {nbytes} bytes of scratch during a CUDA graph capture but only "
                f"{0 if buf is None else buf.numel()} are reserved; call reserve_decode_workspace() for the largest "
                "batch before capturing")
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _WORKSPACE[dev] = buf
    return buf


def reserve_decode_workspace(dev: torch.device, num_seqs: int, num_q_heads: int, num_kv_heads: int,
                             head_dim: int, max_seq_len: int) -> int:
    """Put the scratch of the largest decode batch in place now; returns its size in bytes."""
    need = decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim, max_seq_len)
    _workspace(torch.device(dev), need)
    return need


def fused_paged_rq_decode(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    centroids_k: torch.Tensor,
    centroids_v: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    block_size: int,
    sm_scale: float | None = None,
    out: torch.Tensor | None = None,
    *,
    max_seq_len: int | None = None,
    workspace: torch.Tensor | None = None,
    num_splits: int = 0,
    peer_out_ptrs: list[int] | None = None,
) -> torch.Tensor:
    """Decode attention of one query token per sequence over the compressed paged cache.

    Args as in the reference: ``q (num_seqs, H_Q, D)`` fp16/bf16, ``kv_cache`` uint8
    ``(num_blocks, block_size, total_bytes)``, ``block_table`` int32 ``(num_seqs, max_blocks)``,
    ``seq_lens`` int32, fp32 codebooks, fp32 ``rotation (D, D)``.  Returns the attention output
    in original space, written into ``out`` when given.

    ``max_seq_len`` (host integer bounding ``seq_lens``; default: table width x block size) only
    sizes the launch; nothing is read back from the device, so the call can be graph-captured.

    ``peer_out_ptrs`` (head-sharded decode): device addresses, one per GPU of the tensor-parallel
    group, of the place of THIS GPU's heads inside each GPU's gathered output buffer, laid out like
    ``out`` (which must be this GPU's own entry).  The merge kernel then stores every output row into
    all of them; see :class:`rotorquant_vllm.parallel.PeerHeadGather`.
    """
    num_seqs, hq, d = q.shape
    assert d == head_dim, f"D={d} != head_dim={head_dim}"
    assert hq % num_kv_heads == 0
    assert kv_cache.dtype == torch.uint8
    assert block_table.dtype == torch.int32
    assert seq_lens.dtype == torch.int32
    dev = _lib.require_cuda(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation, out)
    validate_rotation(rotation)
    if kv_cache.dim() != 3 or kv_cache.shape[1] != block_size or not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be contiguous (num_blocks, block_size, total_bytes)")
    if block_table.dim() != 2 or block_table.shape[0] != num_seqs or block_table.stride(1) != 1:
        raise ValueError("block_table must be (num_seqs, max_blocks) with a contiguous last dim")
    if seq_lens.numel() != num_seqs:
        raise ValueError(f"seq_lens has {seq_lens.numel()} entries for {num_seqs} sequences")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if q.stride(2) != 1:
        q = q.contiguous()
    result = out if out is not None else torch.empty_like(q)
    if result.shape != q.shape or result.dtype != q.dtype or result.stride(2) != 1:
        raise ValueError("out must match q in shape and dtype with a contiguous last dim")
    if num_seqs == 0:
        return result
    if max_seq_len is None:
        max_seq_len = block_table.shape[1] * block_size
    ck = centroids_k.to(torch.float32).contiguous()
    cv = centroids_v.to(torch.float32).contiguous()
    seq_lens = seq_lens.contiguous()
    need = decode_workspace_bytes(num_seqs, hq, num_kv_heads, head_dim, max_seq_len, num_splits)
    ws = workspace if workspace is not None else _workspace(dev, need)
    if peer_out_ptrs:
        if out is None or int(out.data_ptr()) not in [int(p) for p in peer_out_ptrs]:
            raise ValueError("peer_out_ptrs needs `out`, and out's own address among the pointers")
        import ctypes

        ptrs = (ctypes.c_void_p * len(peer_out_ptrs))(*[int(p) for p in peer_out_ptrs])
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().rq_decode_sharded(
                q.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
                result.stride(0), result.stride(1), num_seqs, hq, num_kv_heads, head_dim,
                kv_cache.data_ptr(), kv_cache.shape[0], block_size, kv_cache.shape[2],
                block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
                ck.data_ptr(), ck.numel(), cv.data_ptr(), cv.numel(), rotation.data_ptr(),
                float(sm_scale), int(max_seq_len), ws.data_ptr(), ws.numel() * ws.element_size(),
                int(num_splits), ptrs, len(peer_out_ptrs), _lib.stream_ptr(dev)))
        return result
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().rq_decode(
            q.data_ptr(), result.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
            result.stride(0), result.stride(1), num_seqs, hq, num_kv_heads, head_dim,
            kv_cache.data_ptr(), kv_cache.shape[0], block_size, kv_cache.shape[2],
            block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
            ck.data_ptr(), ck.numel(), cv.data_ptr(), cv.numel(), rotation.data_ptr(),
            float(sm_scale), int(max_seq_len), ws.data_ptr(), ws.numel() * ws.element_size(),
            int(num_splits), _lib.stream_ptr(dev)))
    return result
