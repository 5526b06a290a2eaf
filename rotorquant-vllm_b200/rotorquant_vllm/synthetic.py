"""Seeded synthetic workloads for the RotorQuant KV-cache path.

The reference ships no dataset: its benchmarks draw ``torch.randn`` tensors
(experiments/bench_compress.py:23-36, experiments/bench_decompress.py:13-29).
These helpers produce inputs of the same kind with the shapes and value
distributions the benchmark configurations name: N(0,1) queries, keys and
values, with 1 % of the head-dim channels (at least one, drawn from the seed)
multiplied by 10 in K and V, and paged block tables that are random
permutations of the physical blocks.

Everything is generated on the CPU generator so that the same seed gives the
same bytes on every machine; move the tensors to the device afterwards.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    """One named attention-layer configuration."""

    name: str
    rq_mode: str          # "iso" | "planar"
    iso_mode: str         # "fast" | "full"
    k_bits: int
    v_bits: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    block_size: int
    batch: int
    ctx_min: int
    ctx_max: int          # uniform context when ctx_min == ctx_max
    dtype: torch.dtype


# The benchmark configurations.  "decode_llama8b" is the one the headline
# throughput is quoted on.
WORKLOADS = {
    "cpu_roundtrip": Workload("cpu_roundtrip", "iso", "fast", 3, 3, 32, 8, 128, 16, 4, 2048, 2048,
                              torch.float32),
    "decode_llama8b": Workload("decode_llama8b", "iso", "fast", 3, 3, 32, 8, 128, 16, 64, 4096, 4096,
                               torch.bfloat16),
    "decode_qwen7b_planar": Workload("decode_qwen7b_planar", "planar", "fast", 4, 3, 28, 4, 128, 16,
                                     256, 512, 8192, torch.bfloat16),
    "prefill_int8": Workload("prefill_int8", "iso", "fast", 3, 3, 32, 8, 128, 16, 8, 2048, 2048,
                             torch.bfloat16),
    "decode_70b_long": Workload("decode_70b_long", "iso", "full", 3, 3, 64, 8, 128, 16, 8, 131072,
                                131072, torch.bfloat16),
}


def outlier_channels(head_dim: int, gen: torch.Generator, frac: float = 0.01) -> torch.Tensor:
    """Indices of the channels that get the x10 scale (at least one)."""
    n = max(1, round(frac * head_dim))
    return torch.randperm(head_dim, generator=gen)[:n]


def make_kv(num_tokens: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype, seed: int,
            outlier_scale: float = 10.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Keys and values ``(num_tokens, H, D)``: N(0,1) with x10 outlier channels, cast to ``dtype``."""
    gen = torch.Generator().manual_seed(seed)
    ch = outlier_channels(head_dim, gen)
    k = torch.randn(num_tokens, num_kv_heads, head_dim, generator=gen)
    v = torch.randn(num_tokens, num_kv_heads, head_dim, generator=gen)
    k[..., ch] *= outlier_scale
    v[..., ch] *= outlier_scale
    return k.to(dtype), v.to(dtype)


def make_queries(num_rows: int, num_q_heads: int, head_dim: int, dtype: torch.dtype,
                 seed: int) -> torch.Tensor:
    """Queries ``(num_rows, H_Q, D)`` ~ N(0,1), cast to ``dtype``."""
    gen = torch.Generator().manual_seed(seed + 7919)
    return torch.randn(num_rows, num_q_heads, head_dim, generator=gen).to(dtype)


def make_seq_lens(batch: int, ctx_min: int, ctx_max: int, seed: int) -> torch.Tensor:
    """int32 context lengths, uniform in ``[ctx_min, ctx_max]``."""
    if ctx_min == ctx_max:
        return torch.full((batch,), ctx_max, dtype=torch.int32)
    gen = torch.Generator().manual_seed(seed + 104729)
    return torch.randint(ctx_min, ctx_max + 1, (batch,), generator=gen, dtype=torch.int32)


def make_block_table(seq_lens: torch.Tensor, block_size: int, seed: int,
                     spare_blocks: int = 2) -> tuple[torch.Tensor, int]:
    """Disjoint paged layout: a random permutation of the physical blocks dealt to the sequences.

    Returns ``(block_table[int32, batch x max_blocks], num_blocks)``; unused
    table entries are 0 and ``spare_blocks`` physical blocks stay unreferenced.
    """
    gen = torch.Generator().manual_seed(seed + 15485863)
    need = (seq_lens.to(torch.int64) + block_size - 1) // block_size
    total = int(need.sum())
    num_blocks = total + spare_blocks
    perm = torch.randperm(num_blocks, generator=gen)[:total].to(torch.int32)
    max_blocks = max(1, int(need.max())) if len(need) else 1
    table = torch.zeros(len(seq_lens), max_blocks, dtype=torch.int32)
    pos = 0
    for s, nb in enumerate(need.tolist()):
        table[s, :nb] = perm[pos:pos + nb]
        pos += nb
    return table, num_blocks


def slot_mapping_for(block_table: torch.Tensor, seq_lens: torch.Tensor,
                     block_size: int) -> torch.Tensor:
    """int64 flat slot of every cached token, sequence after sequence, position ascending."""
    out = []
    for s in range(block_table.shape[0]):
        n = int(seq_lens[s])
        pos = torch.arange(n, dtype=torch.int64)
        blk = block_table[s].to(torch.int64)[pos // block_size]
        out.append(blk * block_size + pos % block_size)
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.int64)
