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


class HeadGather:
    """Buffers of the one collective of the head-sharded path, allocated once.

    ``buffer`` is ``(world, num_seqs, H_Q/world, D)``; rank ``r`` lets its decode write straight into
    ``local`` (= ``buffer[r]``, contiguous), then :meth:`gather` runs ONE in-place
    ``all_gather_into_tensor`` on the current stream -- no list of tensors, no concatenation, no
    allocation, so the call can sit inside a captured CUDA graph.  ``result`` is the gathered output
    as a view ``(num_seqs, world, H_Q/world, D)``: the query-head axis split into (owner rank, head
    on that rank), heads in their global order; ``result.reshape(num_seqs, H_Q, D)`` gives the dense
    tensor where one is wanted (that copies).
    """

    def __init__(self, num_seqs: int, heads_per_rank: int, head_dim: int, dtype: torch.dtype, device,
                 group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.buffer = torch.zeros(self.world, num_seqs, heads_per_rank, head_dim, dtype=dtype, device=device)
        self.local = self.buffer[self.rank]
        self.result = self.buffer.permute(1, 0, 2, 3)

    def gather(self) -> torch.Tensor:
        if self.world > 1:
            dist.all_gather_into_tensor(self.buffer.view(-1, *self.local.shape[1:]), self.local, group=self.group)
        return self.result


def gather_head_outputs(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather rank-local head outputs ``(num_seqs, H_Q/n, D)`` into a dense ``(num_seqs, H_Q, D)``.

    Ranks hold consecutive head ranges (see :func:`shard_heads`).  One collective, issued on the
    current stream by the backend of ``group`` (NCCL over NVLink on GPUs, gloo on CPU).  Convenience
    form that allocates its result; a serving loop keeps a :class:`HeadGather` instead.
    """
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    local_out = local_out.contiguous()
    gathered = torch.empty(world, *local_out.shape, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered.view(-1, *local_out.shape[1:]), local_out, group=group)
    return gathered.permute(1, 0, 2, 3).reshape(local_out.shape[0], world * local_out.shape[1], local_out.shape[2])
