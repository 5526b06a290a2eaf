"""Pin the CPU oracle to the golden vectors produced by the reference itself.

Runs without a GPU.  Bars: cache bytes and norms bit-exact; decode / prefill
outputs equal to the reference's within one bf16/fp16 unit in the last place
(both sides compute the same fp32 attention with different BLAS call shapes),
and the fp32 rotated-space output within 2e-5.
"""

import hashlib

import numpy as np
import pytest
import torch

import helpers
from oracle import rq_exact, rq_oracle

DECODE_CASES = helpers.decode_case_names()
PREFILL_CASES = helpers.prefill_case_names()


def test_golden_files_present():
    assert len(DECODE_CASES) >= 6 and len(PREFILL_CASES) >= 2


def test_layout_integers():
    """Known answers from the reference's tests (tests/test_vllm_integration.py:44-62)."""
    lay = rq_oracle.slot_layout(128, 8)
    assert lay["payload_end"] == 1088 and lay["total_bytes"] == 2048
    assert rq_oracle.slot_layout(128, 4)["total_bytes"] == 1024
    assert rq_oracle.slot_layout(128, 1)["total_bytes"] == 256
    assert (lay["k_norm"], lay["v_idx"], lay["v_norm"]) == (512, 544, 1056)


@pytest.mark.parametrize("name", DECODE_CASES)
def test_compress_store_matches_reference_bytes(name):
    c = helpers.load_case(name)
    cache = torch.full_like(c["kv_cache"], 0xAB)
    rq_oracle.compress_and_store(c["key"], c["value"], cache, c["slot_mapping"], c["R"],
                                 c["k_boundaries"], c["v_boundaries"])
    assert torch.equal(cache, c["kv_cache"])


@pytest.mark.parametrize("name", DECODE_CASES)
def test_exact_recipe_matches_reference_bytes(name):
    c = helpers.load_case(name)
    slots = rq_exact.build_slots(c["key"].float().numpy(), c["value"].float().numpy(),
                                 c["R"].numpy(), c["k_boundaries"].numpy(),
                                 c["v_boundaries"].numpy())
    flat = c["kv_cache"].reshape(-1, c["kv_cache"].shape[-1]).numpy()
    got = flat[c["slot_mapping"].numpy()]
    assert np.array_equal(got, slots)
    # slots nobody wrote keep the fill byte
    untouched = np.ones(flat.shape[0], dtype=bool)
    untouched[c["slot_mapping"].numpy()] = False
    assert np.all(flat[untouched] == 0xAB)


def test_known_answer_zero_row():
    """An all-zero row packs to 0x44 (3-bit: the middle boundary is a tiny negative
    number) and 0x77 (4-bit: it is exactly zero), with a zero norm."""
    p = helpers.load_params()
    x = np.zeros((2, 128), dtype=np.float32)
    packed3, norms, _ = rq_exact.compress_rows(x, p["iso_fast_R"].reshape(128, 128).numpy(),
                                               p["iso_fast_b3_boundaries"].numpy())
    packed4, _, _ = rq_exact.compress_rows(x, p["iso_fast_R"].reshape(128, 128).numpy(),
                                           p["iso_fast_b4_boundaries"].numpy())
    assert np.all(packed3 == 0x44) and np.all(packed4 == 0x77) and np.all(norms == 0)


@pytest.mark.parametrize("tag,bits,dtype", [
    ("iso_fast", 3, torch.float32), ("iso_fast", 4, torch.bfloat16),
    ("iso_full", 3, torch.bfloat16), ("planar", 4, torch.float16), ("planar", 3, torch.float32),
])
def test_exact_recipe_equals_library_path_on_fresh_rows(tag, bits, dtype):
    """The operation-level recipe reproduces torch.norm / sgemm / bucketize bit for bit."""
    p = helpers.load_params()
    R = p[f"{tag}_R"].reshape(128, 128)
    b = p[f"{tag}_b{bits}_boundaries"]
    gen = torch.Generator().manual_seed(99)
    x = torch.randn(4096, 4, 128, generator=gen)
    x[..., 17] *= 10
    x[5] = 0
    x[6] *= 100.0
    x[7] *= 1e-6
    x = x.to(dtype)
    packed, norms = rq_oracle.compress_rows(x, R, b)
    e_packed, e_norms, _ = rq_exact.compress_rows(x.float().reshape(-1, 128).numpy(), R.numpy(),
                                                  b.numpy())
    assert np.array_equal(packed.reshape(-1, 64).numpy(), e_packed)
    assert np.array_equal(norms.reshape(-1).numpy().view(np.uint32), e_norms.view(np.uint32))


def test_exact_rotations_equal_library_matmul():
    """q @ R.T and o @ R (fused_paged_rq_decode.py:271,:308) are the same ascending FMA chain."""
    p = helpers.load_params()
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(64, 32, 128, generator=gen).to(torch.bfloat16)
    for tag in ("iso_fast", "iso_full", "planar"):
        R = p[f"{tag}_R"].reshape(128, 128)
        blocks = rq_exact.rotation_blocks(R.numpy())
        ref_t = (q.float() @ R.T).reshape(-1, 128).numpy()
        ref_n = (q.float() @ R).reshape(-1, 128).numpy()
        x = q.float().reshape(-1, 128).numpy()
        assert np.array_equal(rq_exact.rotate_rows(x, blocks, True).view(np.uint32), ref_t.view(np.uint32))
        assert np.array_equal(rq_exact.rotate_rows(x, blocks, False).view(np.uint32), ref_n.view(np.uint32))


def _check_attention(got_out, got_rot, c):
    """fp32 rotated-space outputs agree to 2e-5.  The final output is that value rounded to the
    query dtype and multiplied by R, so a rounding flip of one rotated element (legal when the
    fp32 values differ in the last bits) moves the four outputs of its block by up to one unit
    in the last place of the block's largest rotated element."""
    ref_rot = c["o_rot"]
    assert (got_rot - ref_rot).abs().max().item() <= 2e-5
    diff = (got_out.float() - c["out"].float()).abs()
    scale = 1.0 if c["q_dtype"] == "bfloat16" else 8.0
    blk = ref_rot.abs().reshape(*ref_rot.shape[:-1], 32, 4).amax(-1, keepdim=True)
    blk = blk.expand(*ref_rot.shape[:-1], 32, 4).reshape(ref_rot.shape)
    unit = (helpers.ulp_bf16(blk) + helpers.ulp_bf16(c["out"].float())) / scale
    assert torch.all(diff <= unit + 1e-12), diff.max().item()
    assert (diff == 0).float().mean().item() > 0.995


@pytest.mark.parametrize("name", DECODE_CASES)
def test_decode_matches_reference(name):
    c = helpers.load_case(name)
    args = (c["q"], c["kv_cache"], c["block_table"], c["seq_lens"], c["k_centroids"],
            c["v_centroids"], c["R"], c["num_kv_heads"], 128, 16)
    out = rq_oracle.decode(*args, sm_scale=c["sm_scale"])
    rot = rq_oracle.decode(*args, sm_scale=c["sm_scale"], return_rotated_fp32=True)
    _check_attention(out, rot, c)
    for s, n in enumerate(c["seq_lens"].tolist()):
        if n == 0:
            assert torch.all(out[s] == 0)


@pytest.mark.parametrize("name", PREFILL_CASES)
def test_prefill_matches_reference(name):
    c = helpers.load_case(name)
    t = c["q"].shape[0]
    cu = None if t == int(c["seq_lens"][0]) else torch.tensor([0, t])
    args = (c["q"], c["kv_cache"], c["block_table"], c["seq_lens"], c["k_centroids"],
            c["v_centroids"], c["R"], c["num_kv_heads"], 128, 16)
    out = rq_oracle.prefill(*args, sm_scale=c["sm_scale"], cu_seqlens_q=cu)
    rot = rq_oracle.prefill(*args, sm_scale=c["sm_scale"], cu_seqlens_q=cu, return_rotated_fp32=True)
    _check_attention(out, rot, c)


def test_cpu_roundtrip_configuration_digest():
    """The CPU-runnable benchmark configuration (2048 tokens, 8 KV heads, iso-fast 3-bit, batch-4
    decode): inputs regenerate from the seed, cache bytes hash to the reference's digest."""
    from rotorquant_vllm import synthetic as syn

    z = np.load(helpers.GOLDEN + "/case_cpu_roundtrip_digest.npz")
    p = helpers.load_params()
    w = syn.WORKLOADS["cpu_roundtrip"]
    key, value = syn.make_kv(w.ctx_max, w.num_kv_heads, 128, w.dtype, 0)

    def sha(t):
        return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()

    if sha(key) != str(z["key_sha"]):
        pytest.skip("torch CPU generator stream differs from the one the digest was made with")
    R = p["iso_fast_R"].reshape(128, 128)
    cache = torch.zeros(w.ctx_max // 16, 16, 2048, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, torch.arange(w.ctx_max), R,
                                 p["iso_fast_b3_boundaries"], p["iso_fast_b3_boundaries"])
    assert sha(cache) == str(z["cache_sha"])
    slots = rq_exact.build_slots(key.numpy(), value.numpy(), R.numpy(),
                                 p["iso_fast_b3_boundaries"].numpy(), p["iso_fast_b3_boundaries"].numpy())
    assert np.array_equal(slots, cache.reshape(-1, 2048).numpy())
    q = syn.make_queries(w.batch, w.num_q_heads, 128, torch.bfloat16, 0)
    bt = torch.from_numpy(z["block_table"].copy())
    sl = torch.full((w.batch,), w.ctx_max, dtype=torch.int32)
    rot = rq_oracle.decode(q, cache, bt, sl, p["iso_fast_b3_centroids"], p["iso_fast_b3_centroids"],
                           R, 8, 128, 16, return_rotated_fp32=True)
    assert (rot - torch.from_numpy(z["o_rot"])).abs().max().item() <= 2e-5
