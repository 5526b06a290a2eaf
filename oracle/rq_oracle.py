"""CPU oracle for the RotorQuant KV-cache path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain PyTorch CPU ops, what the reference
(tpurtell/rotorquant-vllm) computes on its own CPU path for

* compress-on-write        (triton/isoquant_compress.py:161-190  `_iso_compress_cpu`,
                            triton/planarquant_compress.py:157-186 `_planar_compress_cpu`)
* the cache slot layout    (vllm/rq_backend.py:155-188, :484-490, :585-657 `_compress_and_store`)
* decompress               (triton/isoquant_decompress.py:103-133 `_iso_decompress_cpu`)
* attention over the compressed cache = "reference decompress plus SDPA"
                           (vllm/rq_backend.py:737-852 gather, :938-948 q rotation,
                            :1033-1034 output rotation)

Nothing in the product imports it.  Only the tests, ``__graft_entry__.smoke()``
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may call
it, and only as the checker or as the timed CPU baseline.

Parity status: pinned.  ``tests/golden/make_golden.py`` runs the reference's
own code (imported from its source tree) on seeded inputs and commits the
results under ``tests/golden/``; ``tests/test_oracle.py`` checks every function
here against those vectors (cache bytes bit-exact, norms bit-exact, attention
outputs to the stated tolerance).  The bit-exact arithmetic recipe of the
compress path lives in ``oracle/rq_exact.py`` and is pinned the same way.
"""

from __future__ import annotations

import math

import torch

NORM_BYTES = 4  # fp32 norm per (token, head, K|V)  -- rq_backend.py:54


# ---------------------------------------------------------------------------
# Slot layout (rq_backend.py:155-188, :484-490)
# ---------------------------------------------------------------------------

def _next_pow2(n: int) -> int:
    return 1 << (n - 1).bit_length() if n > 1 else 1


def slot_layout(head_dim: int, num_kv_heads: int) -> dict:
    """Byte offsets of the four regions of one token slot.

    ``[K idx | K norms | V idx | V norms | zero padding]`` with region-major,
    head-minor ordering; the slot is padded per head to a power of two.
    """
    half = head_dim // 2
    k_idx_end = num_kv_heads * half
    k_norm_end = k_idx_end + num_kv_heads * NORM_BYTES
    v_idx_end = k_norm_end + num_kv_heads * half
    v_norm_end = v_idx_end + num_kv_heads * NORM_BYTES
    per_head_raw = 2 * (half + NORM_BYTES)
    total = num_kv_heads * _next_pow2(per_head_raw)
    return {
        "half": half,
        "k_idx": 0,
        "k_norm": k_idx_end,
        "v_idx": k_norm_end,
        "v_norm": v_idx_end,
        "payload_end": v_norm_end,
        "total_bytes": total,
    }


# ---------------------------------------------------------------------------
# Compress (isoquant_compress.py:161-190)
# ---------------------------------------------------------------------------

def compress_rows(x: torch.Tensor, rotation: torch.Tensor,
                  boundaries: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(N, H, D)`` float -> nibble-packed ``(N, H, D/2)`` uint8 + raw fp32 norms ``(N, H, 1)``.

    Steps and their order follow the reference CPU path: fp32 upcast,
    ``torch.norm`` per row, divide by ``norm + 1e-10``, dense product with
    ``R^T``, ``torch.bucketize`` (strict ``boundary < value`` count), clamp to a
    nibble, pack ``even << 4 | odd``.  The *raw* norm is what gets stored.
    """
    n, h, d = x.shape
    rows = x.reshape(n * h, d).to(torch.float32)
    norms = torch.norm(rows, dim=-1, keepdim=True)
    unit = rows / (norms + 1e-10)
    rot_t = rotation.to(torch.float32).T.contiguous()
    rotated = unit @ rot_t
    idx = torch.bucketize(rotated, boundaries.to(torch.float32)).clamp_(0, 15).to(torch.uint8)
    packed = (idx[:, 0::2] << 4) | idx[:, 1::2]
    return packed.reshape(n, h, d // 2), norms.reshape(n, h, 1)


def compress_and_store(key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                       slot_mapping: torch.Tensor, rotation: torch.Tensor,
                       k_boundaries: torch.Tensor, v_boundaries: torch.Tensor) -> None:
    """Write compressed K and V of ``N`` new tokens into their cache slots.

    Mirrors ``RQAttentionImpl._compress_and_store`` (rq_backend.py:585-657):
    payload regions are filled, the padding up to ``total_bytes`` is zeroed,
    and whole slots are scattered by ``slot_mapping[:num_actual]``.
    """
    n, h, d = key.shape
    lay = slot_layout(d, h)
    total = lay["total_bytes"]
    assert kv_cache.dtype == torch.uint8 and kv_cache.shape[-1] == total
    kp, kn = compress_rows(key, rotation, k_boundaries)
    vp, vn = compress_rows(value, rotation, v_boundaries)
    row = torch.zeros(n, total, dtype=torch.uint8)
    row[:, lay["k_idx"]:lay["k_norm"]] = kp.reshape(n, -1)
    row[:, lay["k_norm"]:lay["v_idx"]] = kn.reshape(n, h).contiguous().view(torch.uint8)
    row[:, lay["v_idx"]:lay["v_norm"]] = vp.reshape(n, -1)
    row[:, lay["v_norm"]:lay["payload_end"]] = vn.reshape(n, h).contiguous().view(torch.uint8)
    num_actual = slot_mapping.shape[0]
    flat = kv_cache.view(-1, total)
    flat[slot_mapping[:num_actual].long()] = row[:num_actual]


# ---------------------------------------------------------------------------
# Decompress (isoquant_decompress.py:103-133) and paged gather
# ---------------------------------------------------------------------------

def decompress_rows(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor,
                    dtype: torch.dtype) -> torch.Tensor:
    """``(N, H, D/2)`` uint8 + ``(N, H, 1)`` fp32 -> ``(N, H, D)`` in ``dtype``.

    ``centroid[idx] * norm`` in fp32, one rounding to ``dtype``; the result stays
    in rotated space (there is no inverse rotation on this path).
    """
    n, h, half = packed.shape
    p = packed.reshape(n * h, half)
    c = centroids.to(torch.float32)
    hi = c[((p >> 4) & 0x0F).long()]
    lo = c[(p & 0x0F).long()]
    nr = norms.reshape(n * h, 1).to(torch.float32)
    out = torch.empty(n * h, half * 2, dtype=torch.float32)
    out[:, 0::2] = hi * nr
    out[:, 1::2] = lo * nr
    return out.reshape(n, h, half * 2).to(dtype)


def split_slots(slots: torch.Tensor, head_dim: int, num_kv_heads: int):
    """``(T, total_bytes)`` uint8 slots -> (k_packed, k_norms, v_packed, v_norms)."""
    lay = slot_layout(head_dim, num_kv_heads)
    t = slots.shape[0]
    h, half = num_kv_heads, lay["half"]
    kp = slots[:, lay["k_idx"]:lay["k_norm"]].reshape(t, h, half)
    kn = slots[:, lay["k_norm"]:lay["v_idx"]].contiguous().view(torch.float32).reshape(t, h, 1)
    vp = slots[:, lay["v_idx"]:lay["v_norm"]].reshape(t, h, half)
    vn = slots[:, lay["v_norm"]:lay["payload_end"]].contiguous().view(torch.float32).reshape(t, h, 1)
    return kp, kn, vp, vn


def gather_sequence(kv_cache: torch.Tensor, block_row: torch.Tensor, seq_len: int,
                    head_dim: int, num_kv_heads: int, centroids_k: torch.Tensor,
                    centroids_v: torch.Tensor, dtype: torch.dtype):
    """Decompressed ``(seq_len, H, D)`` K and V of one sequence, read through its block table."""
    nb, bs, total = kv_cache.shape
    n_blocks = (seq_len + bs - 1) // bs
    blocks = block_row[:n_blocks].long()
    slots = kv_cache[blocks].reshape(n_blocks * bs, total)[:seq_len]
    kp, kn, vp, vn = split_slots(slots, head_dim, num_kv_heads)
    k = decompress_rows(kp, kn, centroids_k, dtype)
    v = decompress_rows(vp, vn, centroids_v, dtype)
    return k, v


# ---------------------------------------------------------------------------
# Attention over the compressed cache ("reference decompress plus SDPA")
# ---------------------------------------------------------------------------

def _attend(q_rot: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: float,
            causal_offset: int | None) -> torch.Tensor:
    """fp32 softmax attention. q_rot ``(T, H_Q, D)``, k/v ``(S, H, D)`` -> ``(T, H_Q, D)`` fp32.

    ``causal_offset`` = absolute position of query row 0 (``None`` = no mask).
    """
    t, hq, d = q_rot.shape
    s, h, _ = k.shape
    g = hq // h
    qf = q_rot.to(torch.float32).reshape(t, h, g, d).permute(1, 2, 0, 3)      # (H, G, T, D)
    kf = k.to(torch.float32).permute(1, 0, 2)                                  # (H, S, D)
    vf = v.to(torch.float32).permute(1, 0, 2)
    scores = torch.matmul(qf, kf.transpose(-1, -2).unsqueeze(1)) * sm_scale    # (H, G, T, S)
    if causal_offset is not None:
        qpos = torch.arange(t).unsqueeze(1) + causal_offset
        kpos = torch.arange(s).unsqueeze(0)
        scores = scores.masked_fill(kpos > qpos, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = torch.matmul(p, vf.unsqueeze(1))                                        # (H, G, T, D)
    return o.permute(2, 0, 1, 3).reshape(t, hq, d)


def decode(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
           seq_lens: torch.Tensor, centroids_k: torch.Tensor, centroids_v: torch.Tensor,
           rotation: torch.Tensor, num_kv_heads: int, head_dim: int, block_size: int,
           sm_scale: float | None = None, return_rotated_fp32: bool = False) -> torch.Tensor:
    """Single-token decode for ``num_seqs`` sequences: same signature as the
    reference launcher (fused_paged_rq_decode.py:214-227).

    ``q_rot = (q.float() @ R.T).to(dtype)``; K, V = decompress to ``dtype``;
    fp32 softmax attention; ``out = (o_rot.to(dtype).float() @ R).to(dtype)``.
    Empty sequences give zeros (fused_paged_rq_decode.py:93-96, :201-202).
    """
    num_seqs, hq, d = q.shape
    assert d == head_dim and kv_cache.shape[1] == block_size
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    rot = rotation.to(torch.float32)
    q_rot = (q.to(torch.float32) @ rot.T).to(q.dtype)
    o_rot = torch.zeros(num_seqs, hq, d, dtype=torch.float32)
    for s in range(num_seqs):
        n = int(seq_lens[s])
        if n == 0:
            continue
        k, v = gather_sequence(kv_cache, block_table[s], n, head_dim, num_kv_heads,
                               centroids_k, centroids_v, q.dtype)
        o_rot[s] = _attend(q_rot[s:s + 1], k, v, sm_scale, None)[0]
    if return_rotated_fp32:
        return o_rot
    return (o_rot.to(q.dtype).to(torch.float32) @ rot).to(q.dtype)


def prefill(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
            seq_lens: torch.Tensor, centroids_k: torch.Tensor, centroids_v: torch.Tensor,
            rotation: torch.Tensor, num_kv_heads: int, head_dim: int, block_size: int,
            sm_scale: float | None = None, cu_seqlens_q: torch.Tensor | None = None,
            return_rotated_fp32: bool = False) -> torch.Tensor:
    """Causal attention of new query tokens over the compressed cache.

    One sequence when ``cu_seqlens_q`` is None (the reference launcher's
    contract, fused_paged_rq_int8_prefill.py:247-309, where query row ``i`` sits
    at absolute position ``i``); otherwise sequence ``s`` owns query rows
    ``cu_seqlens_q[s]:cu_seqlens_q[s+1]`` and those rows are the *last* rows of
    its ``seq_lens[s]`` cached tokens.
    """
    t, hq, d = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if cu_seqlens_q is None:
        cu = [0, t]
    else:
        cu = [int(x) for x in cu_seqlens_q]
    rot = rotation.to(torch.float32)
    q_rot = (q.to(torch.float32) @ rot.T).to(q.dtype)
    o_rot = torch.zeros(t, hq, d, dtype=torch.float32)
    for s in range(len(cu) - 1):
        lo, hi = cu[s], cu[s + 1]
        n = int(seq_lens[s])
        if hi == lo or n == 0:
            continue
        k, v = gather_sequence(kv_cache, block_table[s], n, head_dim, num_kv_heads,
                               centroids_k, centroids_v, q.dtype)
        o_rot[lo:hi] = _attend(q_rot[lo:hi], k, v, sm_scale, n - (hi - lo))
    if return_rotated_fp32:
        return o_rot
    return (o_rot.to(q.dtype).to(torch.float32) @ rot).to(q.dtype)
