"""GPU parity of the fused INT8 prefill kernel (tcgen05), through the C-ABI library.

Two bars.  (1) Tight: the kernel against the CPU restatement of its own INT8 arithmetic
(oracle/rq_int8_oracle.py), same tolerance rule as decode with a 1e-3 floor.  (2) Loose: against
"reference decompress + causal SDPA"; INT8 scores with per-row / per-key scales cannot meet 2e-3
there (the reference's own INT8 kernel is off by up to 7e-2 max / 6e-3 mean on a 40-token case),
so the test bounds the error at 5 % of the largest output magnitude and 6e-3 on average.
"""

import math

import pytest
import torch

import gpu_util
import helpers
from gpu_util import DEV
from oracle import rq_int8_oracle, rq_oracle
from rotorquant_vllm import synthetic as syn

pytestmark = pytest.mark.gpu


def _prefill(*a, **k):
    from rotorquant_vllm.cuda import fused_paged_rq_int8_prefill

    return fused_paged_rq_int8_prefill(*a, **k)


def _run(c, cu=None, staged=None):
    """staged: False = fused kernel, True = decompress-once scratch + attention kernel, None = launcher's choice."""
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = _prefill(c["q"].to(DEV), c["kv_cache"].to(DEV), c["block_table"].to(DEV), c["seq_lens"].to(DEV),
                   c["k_centroids"].to(DEV), c["v_centroids"].to(DEV), c["R"].to(DEV), c["num_kv_heads"],
                   128, c["kv_cache"].shape[1], sm_scale=c["sm_scale"],
                   cu_seqlens_q=None if cu is None else cu.to(DEV), error_flag=flag, staged=staged).cpu()
    assert int(flag.item()) == 0, "a bounded device-side wait expired"
    return out


def _args(c):
    return (c["q"], c["kv_cache"], c["block_table"], c["seq_lens"], c["k_centroids"], c["v_centroids"],
            c["R"], c["num_kv_heads"], 128, c["kv_cache"].shape[1])


def _check(out, c, cu):
    dtype = c["q"].dtype
    tight = rq_int8_oracle.prefill_int8(*_args(c), sm_scale=c["sm_scale"], cu_seqlens_q=cu)
    tight_rot = rq_int8_oracle.prefill_int8(*_args(c), sm_scale=c["sm_scale"], cu_seqlens_q=cu,
                                            return_rotated_fp32=True)
    tol = gpu_util.attention_tolerance(tight_rot, tight, dtype, floor=1e-3)
    diff = (out.float() - tight.float()).abs()
    assert not bool(torch.isnan(out.float()).any())
    assert not bool((diff > tol).any()), f"vs INT8 oracle: max {diff.max().item():.3e}"
    exact = rq_oracle.prefill(*_args(c), sm_scale=c["sm_scale"], cu_seqlens_q=cu)
    err = (out.float() - exact.float()).abs()
    bound = 0.05 * max(1.0, exact.float().abs().max().item())
    assert err.max().item() <= bound and err.mean().item() <= 6e-3, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("staged", [False, True])
@pytest.mark.parametrize("name", helpers.prefill_case_names())
def test_prefill_golden_cases(name, staged):
    c = helpers.load_case(name)
    t = c["q"].shape[0]
    cu = None if t == int(c["seq_lens"][0]) else torch.tensor([0, t], dtype=torch.int32)
    _check(_run(c, cu, staged), c, cu)


def _fresh(tag, kb, vb, H, HQ, ctx_lens, q_lens, bs, dtype, seed):
    p = gpu_util.params(tag, kb, vb)
    seq_lens = torch.tensor(ctx_lens, dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, bs, seed)
    slots = syn.slot_mapping_for(bt, seq_lens, bs)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, dtype, seed)
    cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    q = syn.make_queries(sum(q_lens), HQ, 128, dtype, seed)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    c = dict(p)
    c.update(q=q, kv_cache=cache, block_table=bt, seq_lens=seq_lens, num_kv_heads=H,
             sm_scale=1.0 / math.sqrt(128))
    return c, cu


@pytest.mark.parametrize("tag,kb,vb,H,HQ,ctx,ql,bs,dtype", [
    ("iso_fast", 3, 3, 8, 32, [300], [300], 16, torch.bfloat16),                # one sequence, G = 4
    ("iso_fast", 3, 3, 2, 8, [129, 128, 127, 40], [129, 128, 127, 40], 16, torch.bfloat16),
    ("planar", 4, 3, 4, 28, [260, 70], [100, 70], 16, torch.bfloat16),         # G = 7, cached prefix
    ("iso_full", 3, 3, 1, 8, [200, 33], [1, 33], 16, torch.bfloat16),          # H = 1, a decode row
    ("iso_fast", 4, 4, 2, 2, [150], [150], 32, torch.float16),                 # G = 1, fp16, block 32
    ("iso_fast", 3, 4, 1, 16, [90, 0, 17], [90, 0, 17], 8, torch.bfloat16),    # G = 16, empty sequence
])
@pytest.mark.parametrize("staged", [False, True])
def test_prefill_fresh_cases(tag, kb, vb, H, HQ, ctx, ql, bs, dtype, staged):
    c, cu = _fresh(tag, kb, vb, H, HQ, ctx, ql, bs, dtype, seed=H + len(ctx))
    _check(_run(c, cu, staged), c, cu)


def test_staged_and_fused_prefill_agree_and_workspace_is_checked():
    c, cu = _fresh("iso_fast", 3, 3, 4, 16, [700, 130], [300, 130], 16, torch.bfloat16, seed=9)
    a, b = _run(c, cu, False), _run(c, cu, True)
    assert torch.equal(a, b), (a.float() - b.float()).abs().max().item()
    g = gpu_util.on_gpu(c)
    small = torch.empty(1024, dtype=torch.uint8, device=DEV)
    with pytest.raises(ValueError, match="workspace"):
        _prefill(g["q"], g["kv_cache"], g["block_table"], g["seq_lens"], g["k_centroids"], g["v_centroids"],
                 g["R"], 4, 128, 16, cu_seqlens_q=cu.to(DEV), max_seq_len=700, workspace=small)


def test_single_sequence_contract():
    """Without cu_seqlens_q the launcher keeps the reference's single-sequence contract."""
    c, cu = _fresh("iso_fast", 3, 3, 2, 8, [20, 30], [20, 30], 16, torch.bfloat16, seed=1)
    g = gpu_util.on_gpu(c)
    with pytest.raises(ValueError, match="single sequence"):
        _prefill(g["q"], g["kv_cache"], g["block_table"], g["seq_lens"], g["k_centroids"],
                 g["v_centroids"], g["R"], 2, 128, 16)
    out_buf = torch.zeros_like(g["q"])
    res = _prefill(g["q"], g["kv_cache"], g["block_table"], g["seq_lens"], g["k_centroids"],
                   g["v_centroids"], g["R"], 2, 128, 16, cu_seqlens_q=cu.to(DEV), out=out_buf)
    assert res is out_buf


def test_prefill_configuration_shape_sample():
    """The benchmark shape (32 query / 8 KV heads, 2048 new tokens) on one sequence."""
    c, cu = _fresh("iso_fast", 3, 3, 8, 32, [2048], [2048], 16, torch.bfloat16, seed=4)
    out = _run(c, None)
    tight = rq_int8_oracle.prefill_int8(*_args(c), sm_scale=c["sm_scale"])
    diff = (out.float() - tight.float()).abs()
    assert diff.max().item() <= 4e-2 and diff.mean().item() <= 2e-4, (diff.max().item(), diff.mean().item())


@pytest.mark.parametrize("tag,kb,vb,H,HQ,T,dtype,seed", [
    ("iso_fast", 3, 3, 8, 32, 300, torch.bfloat16, 1),
    ("iso_fast", 3, 3, 8, 32, 2048, torch.bfloat16, 4),          # one sequence of the benchmark configuration
    ("iso_fast", 3, 3, 2, 8, 700, torch.float16, 2),
    ("planar", 4, 3, 4, 28, 512, torch.bfloat16, 3),
])
def test_int8_error_is_not_worse_than_the_reference_kernel(tag, kb, vb, H, HQ, T, dtype, seed):
    """INT8 scores cannot meet the 2e-3 bar against exact attention, so the bar for this kernel is
    the reference's own fused INT8 prefill kernel (triton/fused_paged_rq_int8_prefill.py:247-363,
    the unmodified copy under baseline/_ref, compiled by Triton for this GPU): on the same seeded
    single-sequence inputs, the error of the new kernel against "reference decompress + causal
    SDPA" must not exceed the reference kernel's, neither at the worst element nor on average."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from baseline import ref_kernels

    if not ref_kernels.available():
        pytest.skip("baseline/_ref is not installed (see baseline/ref_kernels.py)")
    c, _ = _fresh(tag, kb, vb, H, HQ, [T], [T], 16, dtype, seed)
    exact = rq_oracle.prefill(*_args(c), sm_scale=c["sm_scale"]).float()
    new = _run(c, None).float()
    g = gpu_util.on_gpu(c)
    try:
        ref = ref_kernels.load("fused_paged_rq_int8_prefill")(
            g["q"], g["kv_cache"], g["block_table"], g["seq_lens"], g["k_centroids"], g["v_centroids"], g["R"],
            H, 128, 16, sm_scale=c["sm_scale"]).cpu().float()
    except Exception as exc:                      # Triton could not build or launch the reference kernel here
        pytest.skip(f"reference Triton kernel unavailable: {type(exc).__name__}: {str(exc)[:200]}")
    err_new, err_ref = (new - exact).abs(), (ref - exact).abs()
    assert err_new.max().item() <= err_ref.max().item(), (err_new.max().item(), err_ref.max().item())
    assert err_new.mean().item() <= err_ref.mean().item(), (err_new.mean().item(), err_ref.mean().item())
