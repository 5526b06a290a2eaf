"""GPU tests through the plugin surface: ``RQAttentionImpl.forward`` (compress-on-write, batched
decode, a mixed prefill batch), the paged decompress, and the bounded-wait self test.

The layer is built with ``__new__`` as the reference's own integration tests do
(tests/test_vllm_integration.py:111-121 upstream): no vLLM engine is needed to drive ``forward``.
"""

from types import SimpleNamespace

import pytest
import torch

import gpu_util
from gpu_util import DEV
from oracle import rq_oracle, tolerance
from rotorquant_vllm import _lib
from rotorquant_vllm import synthetic as syn

pytestmark = pytest.mark.gpu

vllm = pytest.importorskip("vllm")


def _impl(tag, kb, vb, H, HQ):
    from vllm.v1.attention.backend import AttentionType

    from rotorquant_vllm.vllm import rq_backend as backend

    p = gpu_util.params(tag, kb, vb)
    impl = backend.RQAttentionImpl.__new__(backend.RQAttentionImpl)
    impl.attn_type = AttentionType.DECODER
    impl._cg_buffers_ready = True
    impl._fused_paged_available = True
    impl._fused_prefill_available = True
    impl.num_kv_heads, impl.num_heads, impl.head_size = H, HQ, 128
    impl.scale = 1.0 / 128 ** 0.5
    impl._k_quantizer = SimpleNamespace(centroids=p["k_centroids"].to(DEV), boundaries=p["k_boundaries"].to(DEV))
    impl._v_quantizer = SimpleNamespace(centroids=p["v_centroids"].to(DEV), boundaries=p["v_boundaries"].to(DEV))
    impl._rq_rot = p["R"].to(DEV)
    return impl, p


def _oracle_args(p, cache, bt, lens, H):
    return (cache.cpu(), bt.cpu(), lens.cpu(), p["k_centroids"], p["v_centroids"], p["R"], H, 128, cache.shape[1])


@pytest.mark.parametrize("tag,kb,vb,H,HQ", [("iso_fast", 3, 3, 8, 32), ("planar", 4, 3, 4, 28)])
def test_forward_prefill_batch_then_batched_decode(tag, kb, vb, H, HQ):
    """A mixed prefill batch (one sequence from scratch, one with a cached prefix, one single new
    token) and then a uniform single-token decode batch, all through ``forward``: the cache bytes
    equal the oracle's compress, the outputs match the oracle's attention."""
    impl, p = _impl(tag, kb, vb, H, HQ)
    bs, dtype = 16, torch.bfloat16
    ctx = [300, 260, 70]                      # cached tokens after the prefill step
    new = [300, 100, 1]                       # query tokens of the prefill step
    seq_lens = torch.tensor(ctx, dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens + 1, bs, 17)        # room for the decode step's token
    key, value = syn.make_kv(sum(ctx) + 3, H, 128, dtype, 17)
    q_all = syn.make_queries(sum(new) + 3, HQ, 128, dtype, 17)
    cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8, device=DEV)
    want_cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)

    # tokens cached before the step (prefixes), written by an earlier forward-less compress
    starts = [0, ctx[0], ctx[0] + ctx[1]]
    slots_all = syn.slot_mapping_for(bt, seq_lens, bs)
    prefix_rows = torch.cat([torch.arange(starts[s], starts[s] + ctx[s] - new[s]) for s in range(3)])
    new_rows = torch.cat([torch.arange(starts[s] + ctx[s] - new[s], starts[s] + ctx[s]) for s in range(3)])
    impl._compress_and_store(key[prefix_rows].to(DEV), value[prefix_rows].to(DEV), cache, slots_all[prefix_rows].to(DEV))
    rq_oracle.compress_and_store(key[prefix_rows], value[prefix_rows], want_cache, slots_all[prefix_rows], p["R"],
                                 p["k_boundaries"], p["v_boundaries"])

    # ---- prefill step through forward ----
    n = sum(new)
    cu = torch.tensor([0, 300, 400, 401], dtype=torch.int32)
    md = SimpleNamespace(num_actual_tokens=n, max_query_len=max(new), max_seq_len=max(ctx), use_cascade=False,
                         query_start_loc=cu.to(DEV), slot_mapping=slots_all[new_rows].to(DEV),
                         block_table=bt.to(DEV), seq_lens=seq_lens.to(DEV))
    q = q_all[:n].to(DEV)
    out = torch.zeros_like(q)
    res = impl.forward(None, q, key[new_rows].to(DEV), value[new_rows].to(DEV), cache, md, output=out)
    assert res is out
    rq_oracle.compress_and_store(key[new_rows], value[new_rows], want_cache, slots_all[new_rows], p["R"],
                                 p["k_boundaries"], p["v_boundaries"])
    assert torch.equal(cache.cpu(), want_cache), "compress-on-write through forward differs from the oracle"
    exact = rq_oracle.prefill(q_all[:n], *_oracle_args(p, cache, bt, seq_lens, H), sm_scale=impl.scale, cu_seqlens_q=cu)
    err = (out.cpu().float() - exact.float()).abs()
    bound = 0.05 * max(1.0, exact.float().abs().max().item())      # INT8 scores: see test_prefill_gpu.py
    assert err.max().item() <= bound and err.mean().item() <= 6e-3, (err.max().item(), err.mean().item())

    # ---- decode step through forward: one new token per sequence ----
    lens2 = seq_lens + 1
    dec_rows = torch.arange(sum(ctx), sum(ctx) + 3)
    pos = lens2.long() - 1
    dec_slots = bt.long()[torch.arange(3), pos // bs] * bs + pos % bs
    md2 = SimpleNamespace(num_actual_tokens=3, max_query_len=1, slot_mapping=dec_slots.to(DEV),
                          block_table=bt.to(DEV), seq_lens=lens2.to(DEV))
    qd = torch.zeros(4, HQ, 128, dtype=dtype, device=DEV)          # padded to 4 rows as a graph batch would be
    qd[:3] = q_all[n:n + 3].to(DEV)
    kd = torch.zeros(4, H, 128, dtype=dtype, device=DEV)
    vd = torch.zeros_like(kd)
    kd[:3], vd[:3] = key[dec_rows].to(DEV), value[dec_rows].to(DEV)
    out2 = torch.full_like(qd, 5.0)
    impl.forward(None, qd, kd, vd, cache, md2, output=out2)
    rq_oracle.compress_and_store(key[dec_rows], value[dec_rows], want_cache, dec_slots, p["R"],
                                 p["k_boundaries"], p["v_boundaries"])
    assert torch.equal(cache.cpu(), want_cache)
    args = (q_all[n:n + 3], *_oracle_args(p, cache, bt, lens2, H))
    ref = rq_oracle.decode(*args, sm_scale=impl.scale)
    rot = rq_oracle.decode(*args, sm_scale=impl.scale, return_rotated_fp32=True)
    worst, over = tolerance.excess(out2[:3].cpu(), rot, ref, dtype)
    assert over == 0, f"decode through forward: max {worst:.3e}, {over} over tolerance"
    assert torch.all(out2[3] == 5.0), "rows beyond num_actual_tokens are not touched"


@pytest.mark.parametrize("tag,kb,vb,H,dtype", [
    ("iso_fast", 3, 3, 8, torch.bfloat16), ("planar", 4, 3, 4, torch.float16), ("iso_full", 3, 4, 1, torch.float32),
    ("iso_fast", 4, 4, 2, torch.bfloat16),
])
def test_paged_decompress_matches_the_oracle_bit_for_bit(tag, kb, vb, H, dtype):
    """The CUDA counterpart of ``_decompress_cache_paged``: only referenced blocks are decompressed,
    the table is renumbered, and every K/V row equals the oracle's gather + decompress exactly."""
    impl, p = _impl(tag, kb, vb, H, H)
    bs = 16
    seq_lens = torch.tensor([77, 16, 130, 1], dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, bs, 3, spare_blocks=5)
    slots = syn.slot_mapping_for(bt, seq_lens, bs)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, torch.bfloat16, 3)
    cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    k, v, remapped = impl._decompress_cache_paged(cache.to(DEV), bt.to(DEV), seq_lens.to(DEV), dtype)
    need = int(((seq_lens + bs - 1) // bs).sum())
    assert k.shape == (need, bs, H, 128) and v.shape == k.shape and remapped.shape == bt.shape
    for s, n in enumerate(seq_lens.tolist()):
        want_k, want_v = rq_oracle.gather_sequence(cache, bt[s], n, 128, H, p["k_centroids"], p["v_centroids"], dtype)
        blocks = remapped[s, :(n + bs - 1) // bs].long().cpu()
        got_k = k.cpu()[blocks].reshape(-1, H, 128)[:n]
        got_v = v.cpu()[blocks].reshape(-1, H, 128)[:n]
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v), f"sequence {s}"
    # the whole cache in one go, and the pre-allocated output buffers of the reference signature
    k_all, v_all = impl._decompress_cache(cache.to(DEV), dtype)
    assert k_all.shape == (nb, bs, H, 128)
    want_k, _ = rq_oracle.gather_sequence(cache, bt[2], 130, 128, H, p["k_centroids"], p["v_centroids"], dtype)
    assert torch.equal(k_all.cpu()[bt[2, :9].long()].reshape(-1, H, 128)[:130], want_k)
    out_k = torch.zeros(need * bs, H, 128, dtype=dtype, device=DEV)
    out_v = torch.zeros_like(out_k)
    k2, v2, _ = impl._decompress_cache_paged(cache.to(DEV), bt.to(DEV), seq_lens.to(DEV), dtype, out_k, out_v)
    assert k2.data_ptr() == out_k.data_ptr() and torch.equal(k2, k) and torch.equal(v2, v)


def test_a_bounded_wait_that_runs_out_reports_it_and_the_context_survives():
    """Every device-side wait of the library is an mbarrier wait with a clock limit.  Here one such
    wait, on a barrier nobody ever arrives on and with a limit of about a millisecond, must give up
    and say so; afterwards the GPU context still runs kernels."""
    L = _lib.lib()
    status = torch.full((2,), -1, dtype=torch.int32, device=DEV)
    limit = 2_000_000                                   # ~1 ms of SM clocks
    with torch.cuda.device(DEV):
        assert L.rq_selftest_bounded_wait(limit, status.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    gave_up, kilo_clocks = status.tolist()
    assert gave_up == 1, "the wait claimed that the barrier completed"
    assert limit // 1024 <= kilo_clocks <= 50 * limit // 1024, kilo_clocks
    assert L.rq_selftest_bounded_wait(0, status.data_ptr(), None) == _lib.RQ_ERR_INVALID_ARG
    x = torch.arange(8, device=DEV)
    assert int((x * 2).sum()) == 56
