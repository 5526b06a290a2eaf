"""Generate the golden vectors under ``tests/golden/`` by RUNNING THE REFERENCE.

Usage (only where the reference source tree is available; it is not needed to
run the tests, which read the committed ``.npz`` files)::

    python tests/golden/make_golden.py /path/to/rotorquant-vllm

The reference is imported from ``<path>/src`` and driven through its own
functions:

* host parameters   ``IsoQuantMSE`` / ``PlanarQuantMSE`` (quantization/isoquant.py:72-102,
                    planarquant.py:80-103), ``_build_rotation_matrix`` (vllm/rq_backend.py:256-264)
* compress + store  ``RQAttentionImpl._compress_and_store`` (vllm/rq_backend.py:585-657) on its
                    CPU fallbacks (triton/isoquant_compress.py:161-190)
* decompress        ``iso_decompress`` / ``planar_decompress`` CPU fallbacks
                    (triton/isoquant_decompress.py:103-133)
* attention         "reference decompress plus SDPA": ``q @ R.T`` in fp32 rounded to the query
                    dtype (rq_backend.py:938-941), torch ``scaled_dot_product_attention`` in fp32
                    over the decompressed K/V, output rounded to the query dtype, ``o @ R``
                    (rq_backend.py:1033-1034)

Nothing from this repository's product or oracle is used to produce the
numbers; ``synthetic.py`` (the seeded input generator) is loaded by file path
because the product package shares the reference's import name.
"""

from __future__ import annotations

import hashlib
import importlib.util
import math
import os
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))


def _load_synthetic():
    path = os.path.join(REPO, "rotorquant-vllm_b200", "rotorquant_vllm", "synthetic.py")
    spec = importlib.util.spec_from_file_location("rq_synthetic", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["rq_synthetic"] = mod
    spec.loader.exec_module(mod)
    return mod


def bits_of(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as an unsigned-integer numpy array (exact round trip)."""
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(bits_of(t).tobytes()).hexdigest()


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    syn = _load_synthetic()

    import rotorquant_vllm.vllm.rq_backend as rb
    from rotorquant_vllm.quantization import IsoQuantMSE, PlanarQuantMSE
    from rotorquant_vllm.triton import iso_decompress, planar_decompress

    assert os.path.realpath(rb.__file__).startswith(os.path.realpath(ref_root)), rb.__file__
    torch.set_num_threads(8)

    # ------------------------------------------------------------------ params
    def quantizer(mode, iso_mode, bits):
        if mode == "iso":
            return IsoQuantMSE(128, bits, seed=rb.RQ_SEED, mode=iso_mode, device="cpu")
        return PlanarQuantMSE(128, bits, seed=rb.RQ_SEED, device="cpu")

    params = {}
    quants = {}
    for tag, mode, iso_mode in (("iso_fast", "iso", "fast"), ("iso_full", "iso", "full"),
                                ("planar", "planar", "fast")):
        for bits in (3, 4):
            qz = quantizer(mode, iso_mode, bits)
            quants[(tag, bits)] = qz
            params[f"{tag}_b{bits}_centroids"] = bits_of(qz.centroids)
            params[f"{tag}_b{bits}_boundaries"] = bits_of(qz.boundaries)
        qz = quants[(tag, 3)]
        R = rb._build_rotation_matrix(qz, 128, "cpu")
        params[f"{tag}_R"] = bits_of(R)
        if mode == "iso":
            params[f"{tag}_q_L"] = bits_of(qz.q_L)
            if iso_mode == "full":
                params[f"{tag}_q_R"] = bits_of(qz.q_R)
        else:
            params[f"{tag}_rot2"] = bits_of(qz.rot2)
    np.savez_compressed(os.path.join(HERE, "params.npz"), **params)

    # ------------------------------------------------------------ impl factory
    def make_impl(tag, k_bits, v_bits, num_kv_heads):
        mode = "planar" if tag == "planar" else "iso"
        impl = rb.RQAttentionImpl.__new__(rb.RQAttentionImpl)
        impl.num_kv_heads = num_kv_heads
        impl.head_size = 128
        impl._rq_mode = mode
        impl._k_quantizer = quants[(tag, k_bits)]
        impl._v_quantizer = quants[(tag, v_bits)]
        R = rb._build_rotation_matrix(impl._k_quantizer, 128, "cpu")
        impl._rq_rot = R
        impl._rq_rot_T = R.T.contiguous()
        impl._rq_rot_T_even = impl._rq_rot_T[:, 0::2].contiguous()
        impl._rq_rot_T_odd = impl._rq_rot_T[:, 1::2].contiguous()
        impl._half_d = 64
        impl._k_idx_end = num_kv_heads * 64
        impl._k_norm_end = impl._k_idx_end + num_kv_heads * 4
        impl._v_idx_end = impl._k_norm_end + num_kv_heads * 64
        impl._v_norm_end = impl._v_idx_end + num_kv_heads * 4
        impl._total_bytes = rb._rq_total_bytes(128, num_kv_heads)
        return impl

    def ref_decompress_sequence(impl, kv_cache, block_row, n, dtype):
        """Reference decompress of one sequence's first n tokens -> (n,H,D) K and V."""
        bs = kv_cache.shape[1]
        nblk = (n + bs - 1) // bs
        H = impl.num_kv_heads
        flat = kv_cache[block_row[:nblk].long()].reshape(nblk * bs, -1)[:n]
        kp = flat[:, :impl._k_idx_end].reshape(n, H, 64)
        kn = flat[:, impl._k_idx_end:impl._k_norm_end].contiguous().view(torch.float32).reshape(n, H, 1)
        vp = flat[:, impl._k_norm_end:impl._v_idx_end].reshape(n, H, 64)
        vn = flat[:, impl._v_idx_end:impl._v_norm_end].contiguous().view(torch.float32).reshape(n, H, 1)
        dec = iso_decompress if impl._rq_mode == "iso" else planar_decompress
        k = dec(kp, kn, impl._k_quantizer.centroids, dtype)
        v = dec(vp, vn, impl._v_quantizer.centroids, dtype)
        return k, v

    def ref_attention(impl, q, kv_cache, block_table, seq_lens, sm_scale, causal_new_tokens):
        """q (T,HQ,D).  causal_new_tokens=None: decode (row s <-> sequence s);
        else one sequence whose last T tokens are the query rows."""
        R = impl._rq_rot
        q_rot = (q.float() @ R.T).to(q.dtype)
        T, HQ, D = q.shape
        o_rot = torch.zeros(T, HQ, D, dtype=torch.float32)
        if causal_new_tokens is None:
            for s in range(T):
                n = int(seq_lens[s])
                if n == 0:
                    continue
                k, v = ref_decompress_sequence(impl, kv_cache, block_table[s], n, q.dtype)
                o = torch.nn.functional.scaled_dot_product_attention(
                    q_rot[s].float().unsqueeze(1),               # (HQ,1,D)
                    k.float().permute(1, 0, 2), v.float().permute(1, 0, 2),
                    scale=sm_scale, enable_gqa=True)
                o_rot[s] = o[:, 0]
        else:
            n = int(seq_lens[0])
            k, v = ref_decompress_sequence(impl, kv_cache, block_table[0], n, q.dtype)
            mask = torch.ones(T, n, dtype=torch.bool).tril(diagonal=n - T)
            o = torch.nn.functional.scaled_dot_product_attention(
                q_rot.float().permute(1, 0, 2), k.float().permute(1, 0, 2),
                v.float().permute(1, 0, 2), attn_mask=mask, scale=sm_scale, enable_gqa=True)
            o_rot = o.permute(1, 0, 2).contiguous()
        out = (o_rot.to(q.dtype).float() @ R).to(q.dtype)
        return out, o_rot

    # ------------------------------------------------------- compress + decode
    cases = [
        # name, tag, kbits, vbits, H, HQ, dtype, seq_lens, seed
        ("iso_fast_k3v3_h8_f32", "iso_fast", 3, 3, 8, 32, torch.float32, [0, 1, 17, 48], 0),
        ("iso_fast_k3v3_h8_bf16", "iso_fast", 3, 3, 8, 32, torch.bfloat16, [16, 15, 33, 64, 5], 1),
        ("planar_k4v3_h4_bf16", "planar", 4, 3, 4, 28, torch.bfloat16, [31, 2, 50], 2),
        ("iso_full_k3v3_h1_bf16", "iso_full", 3, 3, 1, 8, torch.bfloat16, [40, 23], 3),
        ("iso_full_k4v4_h2_f16", "iso_full", 4, 4, 2, 8, torch.float16, [19, 32, 7], 4),
        ("planar_k3v4_h8_bf16", "planar", 3, 4, 8, 8, torch.bfloat16, [9, 26], 5),
    ]
    for name, tag, kb, vb, H, HQ, dtype, lens, seed in cases:
        impl = make_impl(tag, kb, vb, H)
        seq_lens = torch.tensor(lens, dtype=torch.int32)
        block_table, num_blocks = syn.make_block_table(seq_lens, 16, seed)
        slots = syn.slot_mapping_for(block_table, seq_lens, 16)
        n = int(seq_lens.sum())
        key, value = syn.make_kv(n, H, 128, dtype, seed)
        # edge rows: an all-zero token and a huge token
        key[3] = 0
        value[3] = 0
        key[5] *= 1000.0
        value[6] *= 1e-3
        kv_cache = torch.full((num_blocks, 16, impl._total_bytes), 0xAB, dtype=torch.uint8)
        impl._compress_and_store(key, value, kv_cache, slots)
        q = syn.make_queries(len(lens), HQ, 128, torch.bfloat16 if dtype == torch.float32 else dtype, seed)
        sm_scale = 1.0 / math.sqrt(128)
        out, o_rot = ref_attention(impl, q, kv_cache, block_table, seq_lens, sm_scale, None)
        np.savez_compressed(
            os.path.join(HERE, f"case_{name}.npz"),
            tag=tag, k_bits=kb, v_bits=vb, num_kv_heads=H, num_q_heads=HQ,
            in_dtype=str(dtype).replace("torch.", ""), q_dtype=str(q.dtype).replace("torch.", ""),
            key=bits_of(key), value=bits_of(value), slot_mapping=slots.numpy(),
            block_table=block_table.numpy(), seq_lens=seq_lens.numpy(),
            kv_cache=kv_cache.numpy(), q=bits_of(q), out=bits_of(out), o_rot=o_rot.numpy(),
            sm_scale=np.float32(sm_scale))
        print("wrote", name, "tokens", n, "blocks", num_blocks)

    # -------------------------------------------------------- prefill (causal)
    pcases = [
        ("prefill_iso_fast_k3v3_h2", "iso_fast", 3, 3, 2, 8, torch.bfloat16, 50, 50, 10),
        ("prefill_planar_k4v3_h1_prefix", "planar", 4, 3, 1, 7, torch.bfloat16, 70, 30, 11),
    ]
    for name, tag, kb, vb, H, HQ, dtype, ctx, t_new, seed in pcases:
        impl = make_impl(tag, kb, vb, H)
        seq_lens = torch.tensor([ctx], dtype=torch.int32)
        block_table, num_blocks = syn.make_block_table(seq_lens, 16, seed)
        slots = syn.slot_mapping_for(block_table, seq_lens, 16)
        key, value = syn.make_kv(ctx, H, 128, dtype, seed)
        kv_cache = torch.zeros(num_blocks, 16, impl._total_bytes, dtype=torch.uint8)
        impl._compress_and_store(key, value, kv_cache, slots)
        q = syn.make_queries(t_new, HQ, 128, dtype, seed)
        sm_scale = 1.0 / math.sqrt(128)
        out, o_rot = ref_attention(impl, q, kv_cache, block_table, seq_lens, sm_scale, t_new)
        np.savez_compressed(
            os.path.join(HERE, f"case_{name}.npz"),
            tag=tag, k_bits=kb, v_bits=vb, num_kv_heads=H, num_q_heads=HQ,
            q_dtype=str(dtype).replace("torch.", ""), block_table=block_table.numpy(),
            seq_lens=seq_lens.numpy(), kv_cache=kv_cache.numpy(), q=bits_of(q),
            out=bits_of(out), o_rot=o_rot.numpy(), sm_scale=np.float32(sm_scale))
        print("wrote", name)

    # ---------------------------- the CPU-runnable benchmark configuration, as digests
    w = syn.WORKLOADS["cpu_roundtrip"]
    impl = make_impl("iso_fast", 3, 3, w.num_kv_heads)
    key, value = syn.make_kv(w.ctx_max, w.num_kv_heads, 128, w.dtype, 0)
    nblk = w.ctx_max // 16
    kv_cache = torch.zeros(nblk, 16, impl._total_bytes, dtype=torch.uint8)
    impl._compress_and_store(key, value, kv_cache, torch.arange(w.ctx_max, dtype=torch.int64))
    gen = torch.Generator().manual_seed(12345)
    block_table = torch.stack([torch.randperm(nblk, generator=gen) for _ in range(w.batch)]).to(torch.int32)
    seq_lens = torch.full((w.batch,), w.ctx_max, dtype=torch.int32)
    q = syn.make_queries(w.batch, w.num_q_heads, 128, torch.bfloat16, 0)
    out, o_rot = ref_attention(impl, q, kv_cache, block_table, seq_lens, 1.0 / math.sqrt(128), None)
    np.savez_compressed(
        os.path.join(HERE, "case_cpu_roundtrip_digest.npz"),
        key_sha=sha(key), value_sha=sha(value), cache_sha=sha(kv_cache),
        block_table=block_table.numpy(), q_sha=sha(q), out=bits_of(out), o_rot=o_rot.numpy())
    print("wrote cpu_roundtrip digest")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of a checkout of the reference>")
    main(sys.argv[1])
