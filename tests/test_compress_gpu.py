"""GPU parity of the compress-on-write kernel: bytes bit-exact against the reference's golden
vectors and against the exact-arithmetic oracle, through the C-ABI library."""

import hashlib

import numpy as np
import pytest
import torch

import gpu_util
import helpers
from gpu_util import DEV
from oracle import rq_exact, rq_oracle

pytestmark = pytest.mark.gpu


def _cuda():
    from rotorquant_vllm import cuda as rq

    return rq


@pytest.mark.parametrize("name", helpers.decode_case_names())
def test_compress_store_matches_reference_cache_bytes(name):
    c = helpers.load_case(name)
    cache = torch.full_like(c["kv_cache"], 0xAB).to(DEV)
    _cuda().compress_and_store(c["key"].to(DEV), c["value"].to(DEV), cache, c["slot_mapping"].to(DEV),
                               c["R"].to(DEV), c["k_boundaries"].to(DEV), c["v_boundaries"].to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(cache.cpu(), c["kv_cache"]), "cache bytes (payload, padding, untouched slots)"


@pytest.mark.parametrize("tag,bits,dtype,heads", [
    ("iso_fast", 3, torch.bfloat16, 8), ("iso_fast", 4, torch.float32, 8),
    ("iso_full", 3, torch.float16, 2), ("planar", 4, torch.bfloat16, 4),
    ("planar", 3, torch.float32, 1), ("iso_full", 4, torch.bfloat16, 3),
])
def test_compress_rows_bit_exact_on_fresh_inputs(tag, bits, dtype, heads):
    p = gpu_util.params(tag, bits, bits)
    gen = torch.Generator().manual_seed(1234 + bits)
    n = 3000
    x = torch.randn(n, heads, 128, generator=gen)
    x[..., 5] *= 10
    x[7] = 0
    x[8] *= 50.0
    x[9] *= 1e-5
    x = x.to(dtype)
    R = p["R"]
    rt = R.T.contiguous()
    fn = _cuda().planar_compress if tag == "planar" else _cuda().iso_compress
    packed, norms = fn(x.to(DEV), rt[:, 0::2].contiguous().to(DEV), rt[:, 1::2].contiguous().to(DEV),
                       p["k_boundaries"].to(DEV))
    assert packed.shape == (n, heads, 64) and packed.dtype == torch.uint8
    assert norms.shape == (n, heads, 1) and norms.dtype == torch.float32
    e_packed, e_norms, _ = rq_exact.compress_rows(x.float().reshape(-1, 128).numpy(), R.numpy(),
                                                  p["k_boundaries"].numpy())
    assert np.array_equal(packed.cpu().reshape(-1, 64).numpy(), e_packed)
    assert np.array_equal(norms.cpu().reshape(-1).numpy().view(np.uint32), e_norms.view(np.uint32))
    # the library-call restatement of the reference CPU path agrees on this host as well
    o_packed, o_norms = rq_oracle.compress_rows(x, R, p["k_boundaries"])
    assert torch.equal(o_packed, packed.cpu()) and torch.equal(o_norms, norms.cpu())


def test_decompress_bit_exact():
    p = gpu_util.params("iso_fast", 4, 4)
    gen = torch.Generator().manual_seed(3)
    packed = torch.randint(0, 256, (500, 8, 64), generator=gen, dtype=torch.uint8)
    norms = torch.rand(500, 8, 1, generator=gen) * 20
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        got = _cuda().iso_decompress(packed.to(DEV), norms.to(DEV), p["k_centroids"].to(DEV), dtype)
        want = rq_oracle.decompress_rows(packed, norms, p["k_centroids"], dtype)
        assert torch.equal(got.cpu(), want)
    got = _cuda().planar_decompress(packed.to(DEV), norms.to(DEV), p["k_centroids"].to(DEV),
                                    torch.bfloat16, d_padded=128)
    assert torch.equal(got.cpu(), rq_oracle.decompress_rows(packed, norms, p["k_centroids"], torch.bfloat16))


def test_negative_and_short_slot_mapping_and_strided_inputs():
    """Padding slots (-1) are skipped, only len(slot_mapping) tokens are written, and K/V may be
    views into a fused qkv buffer."""
    p = gpu_util.params("iso_fast", 3, 3)
    H, N = 8, 21
    gen = torch.Generator().manual_seed(11)
    qkv = torch.randn(N, (32 + 2 * H) * 128, generator=gen).to(torch.bfloat16)
    key = qkv[:, 32 * 128:(32 + H) * 128].view(N, H, 128)
    value = qkv[:, (32 + H) * 128:].view(N, H, 128)
    slots = torch.randperm(64, generator=gen)[:N - 2].to(torch.int64)
    slots[4] = -1
    cache = torch.full((4, 16, 2048), 0x5C, dtype=torch.uint8, device=DEV)
    qkv_d = qkv.to(DEV)
    key_d = qkv_d[:, 32 * 128:(32 + H) * 128].view(N, H, 128)
    value_d = qkv_d[:, (32 + H) * 128:].view(N, H, 128)
    _cuda().compress_and_store(key_d, value_d, cache, slots.to(DEV), p["R"].to(DEV),
                               p["k_boundaries"].to(DEV), p["v_boundaries"].to(DEV))
    want = torch.full((64, 2048), 0x5C, dtype=torch.uint8)
    rows = rq_exact.build_slots(key.float().numpy(), value.float().numpy(), p["R"].numpy(),
                                p["k_boundaries"].numpy(), p["v_boundaries"].numpy())
    for i, s in enumerate(slots.tolist()):
        if s >= 0:
            want[s] = torch.from_numpy(rows[i])
    assert torch.equal(cache.cpu().reshape(64, 2048), want)


def test_single_token_and_no_padding_mode():
    p = gpu_util.params("planar", 4, 3)
    gen = torch.Generator().manual_seed(2)
    key = torch.randn(1, 4, 128, generator=gen).to(torch.bfloat16)
    value = torch.randn(1, 4, 128, generator=gen).to(torch.bfloat16)
    cache = torch.full((1, 16, 1024), 0xEE, dtype=torch.uint8, device=DEV)
    _cuda().compress_and_store(key.to(DEV), value.to(DEV), cache, torch.tensor([9], device=DEV),
                               p["R"].to(DEV), p["k_boundaries"].to(DEV), p["v_boundaries"].to(DEV),
                               write_padding=False)
    rows = rq_exact.build_slots(key.float().numpy(), value.float().numpy(), p["R"].numpy(),
                                p["k_boundaries"].numpy(), p["v_boundaries"].numpy())
    got = cache.cpu().reshape(16, 1024)
    assert np.array_equal(got[9, :544].numpy(), rows[0, :544])
    assert torch.all(got[9, 544:] == 0xEE) and torch.all(got[:9] == 0xEE) and torch.all(got[10:] == 0xEE)


def test_cpu_roundtrip_configuration_digest():
    """2048 tokens x 8 KV heads, iso-fast 3-bit, fp32 inputs: the cache hashes to the reference's."""
    from rotorquant_vllm import synthetic as syn

    z = np.load(helpers.GOLDEN + "/case_cpu_roundtrip_digest.npz")
    p = gpu_util.params("iso_fast", 3, 3)
    w = syn.WORKLOADS["cpu_roundtrip"]
    key, value = syn.make_kv(w.ctx_max, w.num_kv_heads, 128, w.dtype, 0)
    cache = torch.zeros(w.ctx_max // 16, 16, 2048, dtype=torch.uint8, device=DEV)
    _cuda().compress_and_store(key.to(DEV), value.to(DEV), cache,
                               torch.arange(w.ctx_max, device=DEV), p["R"].to(DEV),
                               p["k_boundaries"].to(DEV), p["v_boundaries"].to(DEV))
    rows = rq_exact.build_slots(key.numpy(), value.numpy(), p["R"].numpy(),
                                p["k_boundaries"].numpy(), p["v_boundaries"].numpy())
    assert np.array_equal(cache.cpu().reshape(-1, 2048).numpy(), rows)
    sha_in = hashlib.sha256(key.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()
    if sha_in == str(z["key_sha"]):
        sha = hashlib.sha256(cache.cpu().numpy().tobytes()).hexdigest()
        assert sha == str(z["cache_sha"])


def test_full_size_prefill_compress_properties():
    """16384 tokens x 8 heads (the prefill configuration): scaling the input by a power of two
    leaves every index byte unchanged and scales the norms exactly; a sample of rows equals the
    exact oracle; a second run is byte-identical."""
    p = gpu_util.params("iso_fast", 3, 3)
    gen = torch.Generator(device=DEV).manual_seed(0)
    N, H = 16384, 8
    key = torch.randn(N, H, 128, generator=gen, device=DEV).to(torch.bfloat16)
    value = torch.randn(N, H, 128, generator=gen, device=DEV).to(torch.bfloat16)
    key[..., 77] *= 10
    value[..., 77] *= 10
    slots = torch.randperm(N, device=DEV)
    args = (p["R"].to(DEV), p["k_boundaries"].to(DEV), p["v_boundaries"].to(DEV))
    c1 = torch.zeros(N // 16, 16, 2048, dtype=torch.uint8, device=DEV)
    c2 = torch.zeros_like(c1)
    c3 = torch.zeros_like(c1)
    _cuda().compress_and_store(key, value, c1, slots, *args)
    _cuda().compress_and_store(key, value, c2, slots, *args)
    _cuda().compress_and_store(key * 4, value * 0.5, c3, slots, *args)
    assert torch.equal(c1, c2)
    f1, f3 = c1.reshape(N, 2048), c3.reshape(N, 2048)
    assert torch.equal(f1[:, :512], f3[:, :512]) and torch.equal(f1[:, 544:1056], f3[:, 544:1056])
    kn1 = f1[:, 512:544].contiguous().view(torch.float32)
    kn3 = f3[:, 512:544].contiguous().view(torch.float32)
    vn1 = f1[:, 1056:1088].contiguous().view(torch.float32)
    vn3 = f3[:, 1056:1088].contiguous().view(torch.float32)
    assert torch.equal(kn1 * 4, kn3) and torch.equal(vn1 * 0.5, vn3)
    assert torch.all(f1[:, 1088:] == 0)
    sample = torch.arange(0, N, 97, device=DEV)
    rows = rq_exact.build_slots(key[sample].float().cpu().numpy(), value[sample].float().cpu().numpy(),
                                p["R"].numpy(), p["k_boundaries"].numpy(), p["v_boundaries"].numpy())
    assert np.array_equal(f1[slots[sample]].cpu().numpy(), rows)


def test_large_launch_divisions_equal_the_ieee_quotients_on_extreme_rows():
    """The large-launch mapping forms x / (norm + 1e-10) through double precision where the quotient is a
    normal number and with the division instruction next to the subnormal range.  Rows built to hit both
    sides: one huge element beside tiny ones (quotients of 1e-38 .. 1e-45 and exact zeros), whole rows of
    tiny or huge magnitude, all-zero rows (denominator 1e-10), and ordinary rows; every byte and norm must equal
    the exact-arithmetic oracle on a sample, and the small-launch kernel (other mapping, plain divisions)
    must give the same bytes for the same tokens."""
    p = gpu_util.params("iso_fast", 3, 3)
    gen = torch.Generator(device=DEV).manual_seed(7)
    N, H = 4096, 8                                    # 32768 rows per kind: the large-launch mapping
    key = torch.randn(N, H, 128, generator=gen, device=DEV)
    value = torch.randn(N, H, 128, generator=gen, device=DEV)
    key[0::8] *= 1e-30
    key[0::8, :, 5] = 3e8                             # quotients around 1e-38: the subnormal border
    key[1::8] *= 1e-37
    key[1::8, :, 9] = 2.5                             # quotients around 1e-37 .. 1e-45
    key[2::8] *= 1e-35                                # tiny rows, ordinary quotients
    key[3::8] *= 1e30                                 # huge rows
    key[4::8] = 0.0                                   # norm 0: denominator 1e-10
    value[0::8, :, 100] = 1e38
    value[1::8] *= 1e-38
    key, value = key.to(torch.bfloat16), value.to(torch.bfloat16)
    slots = torch.randperm(N, device=DEV)
    args = (p["R"].to(DEV), p["k_boundaries"].to(DEV), p["v_boundaries"].to(DEV))
    big = torch.zeros(N // 16, 16, 2048, dtype=torch.uint8, device=DEV)
    _cuda().compress_and_store(key, value, big, slots, *args)
    flat = big.reshape(N, 2048)
    sample = torch.arange(0, N, 61, device=DEV)
    sample = torch.unique(torch.cat([sample, torch.arange(0, 64, device=DEV)]))
    rows = rq_exact.build_slots(key[sample].float().cpu().numpy(), value[sample].float().cpu().numpy(),
                                p["R"].numpy(), p["k_boundaries"].numpy(), p["v_boundaries"].numpy())
    assert np.array_equal(flat[slots[sample]].cpu().numpy(), rows)
    # the same tokens in launches of 256 tokens (2048 rows per kind: the small-launch mapping)
    small = torch.zeros_like(big)
    for lo in range(0, N, 256):
        _cuda().compress_and_store(key[lo:lo + 256], value[lo:lo + 256], small, slots[lo:lo + 256], *args)
    assert torch.equal(big, small)
