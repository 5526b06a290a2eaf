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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rotated_space_output_within_2e3(dtype):
    """R = I with pre-rotated queries exposes round_T(o_rot): it must be within 2e-3 (plus half a
    unit in the last place of the rounding itself) of the oracle's fp32 rotated output."""
    c = _fresh_case("iso_fast", 3, 3, 8, 32, [4096, 512, 64, 2048], 16, dtype, seed=5)
    ref_rot = _oracle(c, rotated=True)
    q_rot = (c["q"].float() @ c["R"].T).to(dtype)
    c2 = dict(c)
    c2["q"] = q_rot
    c2["R"] = torch.eye(128)
    got = _run_case(c2).float()
    half_ulp = helpers.ulp_bf16(ref_rot) / (2.0 if dtype == torch.bfloat16 else 16.0)
    err = (got - ref_rot).abs() - half_ulp
    assert err.max().item() <= 2e-4, err.max().item()


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


def test_streaming_kernels_in_a_subprocess():
    """RQ_DECODE_PATH=stream selects the warp-streaming kernel (read once per process), with and
    without its TMA ring: run the golden and edge cases under it in child processes."""
    import os
    import subprocess
    import sys

    if os.environ.get("RQ_DECODE_PATH") == "stream":
        pytest.skip("already running under the streaming kernel")
    here = os.path.dirname(os.path.abspath(__file__))
    for extra in ({"RQ_DECODE_PATH": "stream"}, {"RQ_DECODE_PATH": "stream", "RQ_DECODE_NO_TMA": "1"}):
        env = dict(os.environ, **extra)
        res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_decode_gpu.py"), "-x", "-q",
                              "-m", "gpu", "-k", "golden or past_the_end or fresh or rotated_space"],
                             env=env, capture_output=True, text=True, timeout=900)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
