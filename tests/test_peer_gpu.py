"""The head-sharded decode's exchange step on ONE GPU: peer stores into several buffers and the
arrive-and-wait kernel, with local memory standing in for the peers' (the real two-GPU run is part of
``bench.py --gpus 2``, which compares the gathered buffers with an NCCL all-gather on every rank).

The wait that runs out is made on the host side of the protocol: a flag slot that nothing ever sets.
The kernel must record that in its state word and return; nothing traps and the context stays usable.
"""

import ctypes

import pytest
import torch

import gpu_util
from gpu_util import DEV
from oracle import rq_oracle
from rotorquant_vllm import _lib
from rotorquant_vllm import cuda as rq
from rotorquant_vllm import synthetic as syn

pytestmark = pytest.mark.gpu


def _case(lens, H=4, HQ=16, seed=5):
    p = gpu_util.params("iso_fast", 3, 3)
    bs = 16
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, bs, seed)
    slots = syn.slot_mapping_for(bt, seq_lens, bs)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, torch.bfloat16, seed)
    cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    q = syn.make_queries(len(lens), HQ, 128, torch.bfloat16, seed)
    dev = {k: v.to(DEV) for k, v in dict(q=q, cache=cache, bt=bt, sl=seq_lens, ck=p["k_centroids"],
                                         cv=p["v_centroids"], R=p["R"]).items()}
    return dev, H, bs


def test_merge_stores_every_row_into_all_listed_buffers():
    torch.cuda.set_device(DEV)
    c, H, bs = _case([700, 33, 1, 260])
    want = rq.fused_paged_rq_decode(c["q"], c["cache"], c["bt"], c["sl"], c["ck"], c["cv"], c["R"], H, 128, bs)
    # three "GPUs": slices of one gathered buffer laid out (world, num_seqs, heads, 128); this GPU is number 1
    world, rank = 3, 1
    gathered = [torch.full((world, *c["q"].shape), 7.0, dtype=c["q"].dtype, device=DEV) for _ in range(world)]
    ptrs = [g[rank].data_ptr() for g in gathered]
    got = rq.fused_paged_rq_decode(c["q"], c["cache"], c["bt"], c["sl"], c["ck"], c["cv"], c["R"], H, 128, bs,
                                   out=gathered[rank][rank], peer_out_ptrs=ptrs)
    torch.cuda.synchronize()
    assert got.data_ptr() == gathered[rank][rank].data_ptr()
    for g in gathered:
        assert torch.equal(g[rank], want)                       # the same bits everywhere
        assert bool((g[0] == 7.0).all()) and bool((g[2] == 7.0).all())   # other GPUs' places untouched


def test_sharded_decode_checks_its_arguments():
    torch.cuda.set_device(DEV)
    c, H, bs = _case([64])
    out = torch.empty_like(c["q"])
    with pytest.raises(ValueError, match="own address"):
        rq.fused_paged_rq_decode(c["q"], c["cache"], c["bt"], c["sl"], c["ck"], c["cv"], c["R"], H, 128, bs,
                                 out=out, peer_out_ptrs=[out.data_ptr() + 4096])
    too_many = [out.data_ptr()] * 9
    with pytest.raises(ValueError, match="peer outputs"):
        rq.fused_paged_rq_decode(c["q"], c["cache"], c["bt"], c["sl"], c["ck"], c["cv"], c["R"], H, 128, bs,
                                 out=out, peer_out_ptrs=too_many)


def _barrier(flag_arrays, rank, state, limit):
    L = _lib.lib()
    ptrs = (ctypes.c_void_p * len(flag_arrays))(*[f.data_ptr() for f in flag_arrays])
    status = L.rq_peer_barrier(ptrs, len(flag_arrays), rank, state.data_ptr(), limit,
                               torch.cuda.current_stream().cuda_stream)
    assert status == 0, L.rq_last_error()


def test_arrive_and_wait_counts_steps_and_reports_a_wait_that_runs_out():
    torch.cuda.set_device(DEV)
    # a group of one: every step completes at once
    mine = torch.zeros(8, dtype=torch.int64, device=DEV)
    state = torch.zeros(2, dtype=torch.int64, device=DEV)
    for _ in range(3):
        _barrier([mine], 0, state, 0)
    torch.cuda.synchronize()
    assert state.tolist() == [3, 0] and int(mine[0]) == 3

    # two GPUs emulated by two arrays in this GPU's memory, both "ranks" launched in stream order: rank 0
    # arrives first and finds rank 1's slot behind -- the wait runs out after `limit` clocks and says so
    a, b = torch.zeros(8, dtype=torch.int64, device=DEV), torch.zeros(8, dtype=torch.int64, device=DEV)
    sa, sb = torch.zeros(2, dtype=torch.int64, device=DEV), torch.zeros(2, dtype=torch.int64, device=DEV)
    _barrier([a, b], 0, sa, 200_000)          # ~0.1 ms
    torch.cuda.synchronize()
    assert sa.tolist() == [1, 1]                                 # step counted, expiry recorded
    assert a.tolist()[:2] == [1, 0] and b.tolist()[:2] == [1, 0]   # its arrival reached both arrays
    # rank 1 arrives second: rank 0's arrival is already there, nothing to wait for
    _barrier([a, b], 1, sb, 200_000)
    torch.cuda.synchronize()
    assert sb.tolist() == [1, 0]
    assert a.tolist()[:2] == [1, 1] and b.tolist()[:2] == [1, 1]
    # the context is still usable
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


def test_peer_barrier_rejects_bad_groups():
    L = _lib.lib()
    ptrs = (ctypes.c_void_p * 1)(0)
    assert L.rq_peer_barrier(ptrs, 0, 0, None, 0, None) == _lib.RQ_ERR_INVALID_ARG
    assert L.rq_peer_barrier(ptrs, 9, 0, None, 0, None) == _lib.RQ_ERR_INVALID_ARG
    assert L.rq_peer_barrier(ptrs, 1, 0, None, 0, None) == _lib.RQ_ERR_INVALID_ARG
