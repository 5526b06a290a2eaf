"""Sharding of the attention hot path over the GPUs of one node.

Attention over the compressed cache needs nothing across KV heads or across sequences, so the
path partitions without any collective inside a kernel:

* by KV head -- rank ``r`` owns KV heads ``[r*H/n, (r+1)*H/n)`` and their query heads, with its own
  cache in the ``H/n``-head slot layout.  This is what vLLM tensor parallelism hands the layer (the
  reference sizes everything from the rank-local ``num_kv_heads``, vllm/rq_backend.py:399-400,
  :486-490).  When one request spans GPUs its head outputs are re-assembled with ONE all-gather.
* by sequence -- independent replicas, no communication.

The reference has no distributed code; these helpers are the only communication this build adds.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_heads(num_q_heads: int, num_kv_heads: int, rank: int, world: int) -> tuple[int, int, int, int]:
    """``(kv_lo, kv_hi, q_lo, q_hi)`` of rank ``rank``; KV heads must divide evenly."""
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not split evenly over {world} ranks")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"{num_q_heads} query heads are not a multiple of {num_kv_heads} KV heads")
    per = num_kv_heads // world
    g = num_q_heads // num_kv_heads
    return rank * per, (rank + 1) * per, rank * per * g, (rank + 1) * per * g


def shard_sequences(num_seqs: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous ``[lo, hi)`` share of ``num_seqs`` sequences, sizes differing by at most one."""
    base, extra = divmod(num_seqs, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def slice_cache_heads(kv_cache: torch.Tensor, num_kv_heads: int, kv_lo: int, kv_hi: int) -> torch.Tensor:
    """The cache of KV heads ``[kv_lo, kv_hi)`` in the slot layout for that many heads.

    ``kv_cache`` is ``(num_blocks, block_size, H*256)`` uint8 with regions
    ``[K idx | K norms | V idx | V norms | padding]`` (head size 128).
    """
    h, n = num_kv_heads, kv_hi - kv_lo
    nb, bs, total = kv_cache.shape
    if total != h * 256:
        raise ValueError(f"cache slot of {total} bytes does not match {h} KV heads")
    out = torch.zeros(nb, bs, n * 256, dtype=torch.uint8, device=kv_cache.device)
    out[..., 0:n * 64] = kv_cache[..., kv_lo * 64:kv_hi * 64]
    out[..., n * 64:n * 68] = kv_cache[..., h * 64 + kv_lo * 4:h * 64 + kv_hi * 4]
    out[..., n * 68:n * 132] = kv_cache[..., h * 68 + kv_lo * 64:h * 68 + kv_hi * 64]
    out[..., n * 132:n * 136] = kv_cache[..., h * 132 + kv_lo * 4:h * 132 + kv_hi * 4]
    return out


def gather_head_outputs(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather rank-local head outputs ``(num_seqs, H_Q/n, D)`` into ``(num_seqs, H_Q, D)``.

    Ranks hold consecutive head ranges (see :func:`shard_heads`).  One collective, issued on the
    current stream by the backend of ``group`` (NCCL over NVLink on GPUs, gloo on CPU).
    """
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    local_out = local_out.contiguous()
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out, group=group)
    return torch.cat(parts, dim=1)
