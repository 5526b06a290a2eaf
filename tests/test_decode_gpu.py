"""GPU parity of the fused paged decode kernel, through the C-ABI library.

Bars (north star: within 2e-3 max-abs of "reference decompress + SDPA"):
* golden cases produced by the reference itself, and fresh seeded cases against the oracle;
* rotated-space check: with R = I and pre-rotated queries the kernel returns round_T(o_rot),
  which must sit within 2e-3 of the oracle's fp32 o_rot;
* where one bf16 unit of the output exceeds 2e-3 the bound is one rounding flip (see
  gpu_util.attention_tolerance).
"""

import math

import pytest
import torch

import gpu_util
import helpers
from gpu_util import DEV
from oracle import rq_oracle
from rotorquant_vllm import synthetic as syn

pytestmark = pytest.mark.gpu


def _decode(*a, **k):
    from rotorquant_vllm.cuda import fused_paged_rq_decode

    return fused_paged_rq_decode(*a, **k)


def _run_case(c, **kw):
    return _decode(c["q"].to(DEV), c["kv_cache"].to(DEV), c["block_table"].to(DEV),
                   c["seq_lens"].to(DEV), c["k_centroids"].to(DEV), c["v_centroids"].to(DEV),
                   c["R"].to(DEV), c["num_kv_heads"], 128, c["kv_cache"].shape[1],
                   sm_scale=c["sm_scale"], **kw).cpu()


def _assert_close(out, ref_out, ref_rot, dtype, what=""):
    tol = gpu_util.attention_tolerance(ref_rot, ref_out, dtype)
    diff = (out.float() - ref_out.float()).abs()
    bad = diff > tol
    assert not bool(bad.any()), f"{what}: max diff {diff.max().item():.3e}, {int(bad.sum())} over tolerance"
    assert not bool(torch.isnan(out.float()).any())


@pytest.mark.parametrize("name", helpers.decode_case_names())
def test_decode_matches_reference_golden(name):
    c = helpers.load_case(name)
    out = _run_case(c)
    _assert_close(out, c["out"], c["o_rot"], c["q"].dtype, name)
    for s, n in enumerate(c["seq_lens"].tolist()):
        if n == 0:
            assert torch.all(out[s] == 0), "an empty sequence gives zeros"


@pytest.mark.parametrize("name", helpers.decode_case_names()[:3])
@pytest.mark.parametrize("splits", [1, 2, 3, 5])
def test_forced_split_counts_agree(name, splits):
    c = helpers.load_case(name)
    out = _run_case(c, num_splits=splits)
    _assert_close(out, c["out"], c["o_rot"], c["q"].dtype, f"{name} splits={splits}")


def _fresh_case(tag, kb, vb, H, HQ, lens, block_size, dtype, seed, aliased=False):
    p = gpu_util.params(tag, kb, vb)
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, block_size, seed)
    slots = syn.slot_mapping_for(bt, seq_lens, block_size)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, dtype, seed)
    cache = torch.zeros(nb, block_size, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    q = syn.make_queries(len(lens), HQ, 128, dtype, seed)
    c = dict(p)
    c.update(q=q, kv_cache=cache, block_table=bt, seq_lens=seq_lens, num_kv_heads=H,
             sm_scale=1.0 / math.sqrt(128))
    return c


def _oracle(c, rotated=False):
    return rq_oracle.decode(c["q"], c["kv_cache"], c["block_table"], c["seq_lens"], c["k_centroids"],
                            c["v_centroids"], c["R"], c["num_kv_heads"], 128, c["kv_cache"].shape[1],
                            sm_scale=c["sm_scale"], return_rotated_fp32=rotated)


@pytest.mark.parametrize("tag,kb,vb,H,HQ,lens,bs", [
    ("iso_fast", 3, 3, 8, 32, [700, 1, 16, 15, 17, 333], 16),      # llama-8B grouping
    ("planar", 4, 3, 4, 28, [512, 129, 1000], 16),                # qwen grouping, G = 7
    ("iso_full", 3, 3, 1, 8, [2100, 64], 16),                     # one KV head per GPU
    ("iso_fast", 4, 4, 2, 32, [300, 77], 16),                     # G = 16: two head groups
    ("iso_fast", 3, 4, 8, 8, [90, 40], 32),                       # block_size 32, G = 1
    ("planar", 3, 3, 4, 16, [100, 37, 64], 8),                    # block_size 8: tile spans blocks
    ("iso_fast", 3, 3, 2, 8, [45, 3], 1),                         # block_size 1
])
def test_decode_matches_oracle_on_fresh_cases(tag, kb, vb, H, HQ, lens, bs):
    c = _fresh_case(tag, kb, vb, H, HQ, lens, bs, torch.bfloat16, seed=len(lens) + H)
    out = _run_case(c)
    _assert_close(out, _oracle(c), _oracle(c, rotated=True), torch.bfloat16, f"{tag} H={H}")


@pytest.mark.parametrize("tag,kb,vb,H,HQ,lens,dtype", [
    ("iso_fast", 3, 3, 8, 32, [4096, 512, 64, 2048], torch.bfloat16),     # llama-8B grouping
    ("iso_fast", 3, 3, 8, 32, [4096, 512, 64, 2048], torch.float16),
    ("planar", 4, 3, 4, 28, [3000, 129, 700], torch.bfloat16),            # 4-bit K tables, G = 7
    ("iso_full", 3, 3, 1, 8, [5000, 300], torch.bfloat16),                # one KV head per GPU, G = 8
    ("iso_fast", 4, 4, 2, 32, [1500, 77], torch.bfloat16),                # 4-bit K and V, G = 16
    ("iso_full", 3, 4, 4, 16, [900, 2048], torch.float16),                # 4-bit V tables, fp16
])
def test_rotated_space_output_within_2e3(tag, kb, vb, H, HQ, lens, dtype):
    """R = I with pre-rotated queries exposes round_T(o_rot): it must be within 2e-4 (plus half a
    unit in the last place of the rounding itself) of the oracle's fp32 rotated output -- ten times
    tighter than the 2e-3 bar, in every table / grouping variant the kernel is instantiated for."""
    c = _fresh_case(tag, kb, vb, H, HQ, lens, 16, dtype, seed=5)
    ref_rot = _oracle(c, rotated=True)
    q_rot = (c["q"].float() @ c["R"].T).to(dtype)
    c2 = dict(c)
    c2["q"] = q_rot
    c2["R"] = torch.eye(128)
    got = _run_case(c2).float()
    half_ulp = helpers.ulp_bf16(ref_rot) / (2.0 if dtype == torch.bfloat16 else 16.0)
    err = (got - ref_rot).abs() - half_ulp
    assert err.max().item() <= 2e-4, err.max().item()


def test_scores_that_keep_growing_move_the_reference_maximum():
    """Keys whose norms grow along the sequence make later tiles outgrow the softmax reference of
    the first tile again and again: the rare path that hands a tile back, moves the maxima and
    rescales the accumulated output."""
    p = gpu_util.params("iso_fast", 3, 3)
    H, HQ, bs, n = 8, 32, 16, 1500
    seq_lens = torch.tensor([n, 700], dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, bs, 3)
    slots = syn.slot_mapping_for(bt, seq_lens, bs)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, torch.bfloat16, 3)
    q = syn.make_queries(2, HQ, 128, torch.bfloat16, 3)
    # every key points along its sequence's first query head, with a length that grows 30-fold
    ramp = torch.cat([torch.linspace(0.2, 6.0, n), torch.linspace(6.0, 0.2, 700)])
    q_rot = q.float() @ p["R"].T
    direction = torch.cat([q_rot[0, 0].expand(n, 128), q_rot[1, 0].expand(700, 128)]) @ p["R"]
    key = (key.float() * 0.3 + direction[:, None, :] * ramp[:, None, None]).to(torch.bfloat16)
    cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    c = dict(p)
    c.update(q=q, kv_cache=cache, block_table=bt, seq_lens=seq_lens, num_kv_heads=H,
             sm_scale=1.0 / math.sqrt(128))
    for splits in (0, 1):
        out = _run_case(c, num_splits=splits)
        _assert_close(out, _oracle(c), _oracle(c, rotated=True), torch.bfloat16, f"growing scores splits={splits}")


def test_llama8b_shape_small_batch_and_output_buffer():
    """32 query / 8 KV heads, context 4096: the benchmark shape at batch 3, writing into `out`."""
    c = _fresh_case("iso_fast", 3, 3, 8, 32, [4096, 4096, 4095], 16, torch.bfloat16, seed=0)
    out_buf = torch.full((3, 32, 128), 7.0, dtype=torch.bfloat16, device=DEV)
    res = _decode(c["q"].to(DEV), c["kv_cache"].to(DEV), c["block_table"].to(DEV),
                  c["seq_lens"].to(DEV), c["k_centroids"].to(DEV), c["v_centroids"].to(DEV),
                  c["R"].to(DEV), 8, 128, 16, out=out_buf)
    assert res is out_buf
    ref, rot = _oracle(c), _oracle(c, rotated=True)
    diff = (out_buf.cpu().float() - ref.float()).abs().max().item()
    assert diff <= 2e-3, diff
    _assert_close(out_buf.cpu(), ref, rot, torch.bfloat16)


def test_argument_checks_mirror_the_reference():
    c = _fresh_case("iso_fast", 3, 3, 8, 32, [20], 16, torch.bfloat16, seed=1)
    g = gpu_util.on_gpu(c)
    with pytest.raises(AssertionError):
        _decode(g["q"], g["kv_cache"], g["block_table"].long(), g["seq_lens"], g["k_centroids"],
                g["v_centroids"], g["R"], 8, 128, 16)
    with pytest.raises(AssertionError):
        _decode(g["q"], g["kv_cache"], g["block_table"], g["seq_lens"], g["k_centroids"],
                g["v_centroids"], g["R"], 8, 64, 16)
    bad_R = g["R"].clone()
    bad_R[0, 100] = 0.5
    with pytest.raises(ValueError, match="diagonal"):
        _decode(g["q"], g["kv_cache"], g["block_table"], g["seq_lens"], g["k_centroids"],
                g["v_centroids"], bad_R, 8, 128, 16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bytes_past_the_end_of_a_sequence_are_ignored(dtype):
    """Slots of the last block beyond seq_len may hold anything (a recycled or never written
    block): fill them with 0xFF bytes, which are neither index nibbles nor finite norms."""
    c = _fresh_case("iso_fast", 3, 3, 4, 16, [130, 17, 200, 1], 16, dtype, seed=11)
    cache = c["kv_cache"].clone()
    bs = cache.shape[1]
    for s, n in enumerate(c["seq_lens"].tolist()):
        nblk = (n + bs - 1) // bs
        last = int(c["block_table"][s, nblk - 1])
        used = n - (nblk - 1) * bs
        cache[last, used:] = 0xFF
    c2 = dict(c)
    c2["kv_cache"] = cache
    out = _run_case(c2)
    _assert_close(out, _oracle(c), _oracle(c, rotated=True), dtype, "garbage tail")


def test_row_copy_staging_in_a_subprocess():
    """RQ_DECODE_NO_TMA=1 (read once per process) makes every thread load its own index rows instead
    of staging them by TMA boxes, the path every unusual block size takes; RQ_DECODE_NO_PDL=1
    launches the merge without programmatic dependent launch and RQ_DECODE_EQUAL_PIECES=1 cuts the
    tile line into equal pieces.  Run the golden and edge cases under them in a child process."""
    import os
    import subprocess
    import sys

    if os.environ.get("RQ_DECODE_NO_TMA"):
        pytest.skip("already running with row copies")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, RQ_DECODE_NO_TMA="1", RQ_DECODE_NO_PDL="1", RQ_DECODE_EQUAL_PIECES="1")
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_decode_gpu.py"), "-x", "-q",
                          "-m", "gpu", "-k", "golden or past_the_end or fresh or growing"],
                         env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


def test_many_sequences_use_the_plan_launch():
    """More sequences than an attention CTA scans by itself (256): the tile prefix sums come from
    the separate plan launch.  300 short ragged sequences, a few of them empty."""
    gen = torch.Generator().manual_seed(77)
    lens = torch.randint(1, 200, (300,), generator=gen).tolist()
    lens[5] = 0
    lens[299] = 0
    c = _fresh_case("iso_fast", 3, 3, 4, 16, lens, 16, torch.bfloat16, seed=8)
    out = _run_case(c)
    _assert_close(out, _oracle(c), _oracle(c, rotated=True), torch.bfloat16, "300 sequences")
    assert torch.all(out[5] == 0) and torch.all(out[299] == 0)
