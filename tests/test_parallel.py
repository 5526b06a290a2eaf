"""Multi-rank host logic on CPU: two gloo ranks shard a decode by KV head (each rank computes its
heads with the CPU oracle on its slice of the cache), all-gather the head outputs and must
reproduce the unsharded result; sequence sharding covers every sequence exactly once."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers
from oracle import rq_oracle
from rotorquant_vllm import parallel


def test_shard_arithmetic():
    assert parallel.shard_heads(64, 8, 3, 8) == (3, 4, 24, 32)
    assert parallel.shard_heads(32, 8, 1, 2) == (4, 8, 16, 32)
    with pytest.raises(ValueError):
        parallel.shard_heads(28, 4, 0, 3)
    covered = []
    for r in range(4):
        lo, hi = parallel.shard_sequences(10, r, 4)
        covered += list(range(lo, hi))
    assert covered == list(range(10))
    assert parallel.shard_sequences(3, 3, 4) == (3, 3)


def test_slice_cache_heads_matches_recompression():
    c = helpers.load_case("case_iso_fast_k3v3_h8_bf16")
    sub = parallel.slice_cache_heads(c["kv_cache"], 8, 2, 4)
    want = torch.zeros_like(sub)
    rq_oracle.compress_and_store(c["key"][:, 2:4], c["value"][:, 2:4], want, c["slot_mapping"], c["R"],
                                 c["k_boundaries"], c["v_boundaries"])
    written = torch.zeros(sub.shape[0] * sub.shape[1], dtype=torch.bool)
    written[c["slot_mapping"]] = True
    flat_sub, flat_want = sub.reshape(-1, sub.shape[-1]), want.reshape(-1, want.shape[-1])
    assert torch.equal(flat_sub[written][:, :2 * 136], flat_want[written][:, :2 * 136])


def _rank_main(rank: int, world: int, port: int, result_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = helpers.load_case("case_iso_fast_k3v3_h8_bf16")
        H, HQ = c["num_kv_heads"], c["num_q_heads"]
        kv_lo, kv_hi, q_lo, q_hi = parallel.shard_heads(HQ, H, rank, world)
        local_cache = parallel.slice_cache_heads(c["kv_cache"], H, kv_lo, kv_hi)
        local = rq_oracle.decode(c["q"][:, q_lo:q_hi].contiguous(), local_cache, c["block_table"],
                                 c["seq_lens"], c["k_centroids"], c["v_centroids"], c["R"],
                                 kv_hi - kv_lo, 128, 16, sm_scale=c["sm_scale"])
        full = parallel.gather_head_outputs(local)
        # the allocation-free form: the rank's heads are written into its slice, one in-place collective
        hg = parallel.HeadGather(local.shape[0], local.shape[1], 128, local.dtype, "cpu")
        hg.local.copy_(local)
        again = hg.gather()
        assert again.shape == (local.shape[0], world, local.shape[1], 128)
        assert torch.equal(again.reshape(full.shape), full)
        if rank == 0:
            torch.save(full, result_path)
    finally:
        dist.destroy_process_group()


def test_kv_head_sharding_with_all_gather_on_two_gloo_ranks(tmp_path):
    path = str(tmp_path / "gathered.pt")
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(2, port, path), nprocs=2, join=True)
    got = torch.load(path)
    c = helpers.load_case("case_iso_fast_k3v3_h8_bf16")
    want = rq_oracle.decode(c["q"], c["kv_cache"], c["block_table"], c["seq_lens"], c["k_centroids"],
                            c["v_centroids"], c["R"], c["num_kv_heads"], 128, 16, sm_scale=c["sm_scale"])
    assert got.shape == want.shape
    assert torch.equal(got, want)
