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


class PeerHeadGather:
    """The head-sharded path without a collective launch: the decode's merge kernel stores every output
    row into ALL GPUs' gathered buffers (plain stores into peer memory over NVLink), and one small
    arrive-and-wait kernel tells each GPU that its peers' rows have landed.

    The gathered buffers live in symmetric memory (``torch.distributed._symmetric_memory``), which maps
    every rank's allocation into every process.  ``buffer`` is ``(2, world, num_seqs, H_Q/world, D)``:
    two gathered outputs that alternate from step to step, because a GPU that has passed the wait of
    step ``i`` may already store step ``i + 1`` into a peer that still reads step ``i``.  Per step:

        g = gather.begin()                                   # picks the buffer of this step
        fused_paged_rq_decode(..., out=g.local, peer_out_ptrs=g.peer_ptrs)
        result = gather.finish()                             # rq_peer_barrier; (num_seqs, world, H_Q/world, D)

    All of it runs on the current stream; nothing allocates or synchronises with the host, and both
    calls can sit in a captured CUDA graph (one graph per parity).  The wait is bounded (about a second
    of SM clocks); :meth:`wait_expired` reads back whether one ever ran out.
    """

    class _Step:
        __slots__ = ("local", "peer_ptrs", "result")

    def __init__(self, num_seqs: int, heads_per_rank: int, head_dim: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        self._lib = _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        shape = (2, self.world, num_seqs, heads_per_rank, head_dim)
        self.buffer = symm.empty(shape, dtype=dtype, device=self.device)
        self.buffer.zero_()
        self._buf_handle = symm.rendezvous(self.buffer, self.group)
        self.flags = symm.empty((16,), dtype=torch.int64, device=self.device)
        self.flags.zero_()
        self._flag_handle = symm.rendezvous(self.flags, self.group)
        self.state = torch.zeros(2, dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)                                   # every rank's flags are zero before anyone arrives
        esz = self.buffer.element_size()
        slice_elems = num_seqs * heads_per_rank * head_dim
        self._steps = []
        for parity in range(2):
            st = PeerHeadGather._Step()
            st.local = self.buffer[parity, self.rank]
            offset = ((parity * self.world + self.rank) * slice_elems) * esz
            st.peer_ptrs = [int(base) + offset for base in self._buf_handle.buffer_ptrs]
            st.result = self.buffer[parity].permute(1, 0, 2, 3)
            self._steps.append(st)
        assert st.peer_ptrs[self.rank] == st.local.data_ptr()
        import ctypes

        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self._flag_handle.buffer_ptrs])
        self.parity = 0

    def begin(self, parity: int | None = None) -> "PeerHeadGather._Step":
        if parity is not None:
            self.parity = parity & 1
        return self._steps[self.parity]

    def finish(self, limit_cycles: int = 0) -> torch.Tensor:
        step = self._steps[self.parity]
        with torch.cuda.device(self.device):
            self._lib.check(self._lib.lib().rq_peer_barrier(
                self._flag_ptrs, self.world, self.rank, self.state.data_ptr(), int(limit_cycles),
                self._lib.stream_ptr(self.device)))
        self.parity ^= 1
        return step.result

    def wait_expired(self) -> bool:
        """Host read-back (synchronises): True when a bounded wait of this GPU has ever run out."""
        return bool(int(self.state[1].item()))
