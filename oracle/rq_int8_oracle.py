"""CPU restatement of the INT8 prefill arithmetic of librq_b200.  TEST INFRASTRUCTURE ONLY.

The reference's fused INT8 prefill (triton/fused_paged_rq_int8_prefill.py:43-239) has no CPU
implementation and its numerics depend on an autotuned tile size, so it cannot serve as a tight
oracle: against exact attention it is off by up to 7e-2 on short rows.  The B200 kernel uses a
different, finer INT8 scheme (one scale per query row and per key instead of one per tile).  This
module states that scheme operation by operation so that the kernel can be checked tightly, while
``rq_oracle.prefill`` ("reference decompress plus SDPA") measures how far INT8 moves the result.

Parity status: unpinned against the reference (nothing in the reference computes this scheme);
pinned to the kernel's documented arithmetic only.

Scheme, per (sequence, KV head), queries and keys in rotated space:
  q_rot       = round_T(q @ R^T)
  q_i8[m]     = rint(q_rot[m] * (127 / max|q_rot[m]|)),       q_scale[m] = max|q_rot[m]| / 127
  table[t][i] = round_T(centroid_k[i] * norm_k[t]);  code[t][i] = rint(table * (127 / max_i|table|))
  k_i8[t][d]  = code[t][idx[t][d]],                           k_scale[t] = max_i|table[t][i]| / 127
  s[m][t]     = (float(q_i8[m] . k_i8[t]) * k_scale[t]) * (q_scale[m] * sm_scale*log2 e)
  online softmax over 128-key tiles in base 2 against a lazy reference maximum (it moves to the tile
  maximum only when that exceeds it by more than 8); P is rounded to T before it multiplies V, the row
  sum adds the unrounded values; V = round_T(centroid_v[idx] * norm_v) exactly as decompressed;
  out         = round_T(round_T(O / l) @ R)
"""

from __future__ import annotations

import math

import torch

from . import rq_oracle

TILE = 128


def _f32(x):
    return torch.as_tensor(x, dtype=torch.float32)


def prefill_int8(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation,
                 num_kv_heads, head_dim, block_size, sm_scale=None, cu_seqlens_q=None,
                 return_rotated_fp32=False):
    t_all, hq, d = q.shape
    g = hq // num_kv_heads
    dtype = q.dtype
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    qk_scale = _f32(sm_scale) * _f32(1.4426950408889634)
    cu = [0, t_all] if cu_seqlens_q is None else [int(x) for x in cu_seqlens_q]
    rot = rotation.to(torch.float32)
    q_rot = (q.to(torch.float32) @ rot.T).to(dtype).to(torch.float32)
    o_rot = torch.zeros(t_all, hq, d, dtype=torch.float32)
    ck = centroids_k.to(torch.float32)
    c127 = _f32(127.0)

    for s in range(len(cu) - 1):
        lo, hi = cu[s], cu[s + 1]
        n = int(seq_lens[s])
        tq = hi - lo
        if tq == 0 or n == 0:
            continue
        nblk = (n + block_size - 1) // block_size
        slots = kv_cache[block_table[s, :nblk].long()].reshape(nblk * block_size, -1)[:n]
        kp, kn, vp, vn = rq_oracle.split_slots(slots, head_dim, num_kv_heads)
        v_all = rq_oracle.decompress_rows(vp, vn, centroids_v, dtype).to(torch.float32)   # (n, H, D)
        # K: per-key code tables
        table = (ck.view(1, 1, -1) * kn.to(torch.float32)).to(dtype).to(torch.float32)    # (n, H, NK)
        tmax = table.abs().amax(-1, keepdim=True)
        ok = tmax > 0
        inv = torch.where(ok, c127 / tmax, torch.zeros_like(tmax))
        k_scale = torch.where(ok, tmax / c127, torch.zeros_like(tmax)).squeeze(-1)         # (n, H)
        code = torch.round(table * inv)                                                     # (n, H, NK)
        idx = torch.empty(n, num_kv_heads, d, dtype=torch.long)
        idx[..., 0::2] = ((kp >> 4) & 0xF).long()
        idx[..., 1::2] = (kp & 0xF).long()
        k_i8 = torch.gather(code, 2, idx)                                                   # (n, H, D)

        pos = torch.arange(tq) + (n - tq)                                                   # absolute positions
        for h in range(num_kv_heads):
            qh = q_rot[lo:hi, h * g:(h + 1) * g]                                            # (tq, G, D)
            qmax = qh.abs().amax(-1, keepdim=True)
            okq = qmax > 0
            qinv = torch.where(okq, c127 / qmax, torch.zeros_like(qmax))
            q_scale = torch.where(okq, qmax / c127, torch.zeros_like(qmax)).squeeze(-1)     # (tq, G)
            q_i8 = torch.round(qh * qinv)
            row_factor = q_scale * qk_scale                                                 # (tq, G)
            m_run = torch.full((tq, g), float("-inf"))
            l_run = torch.zeros(tq, g)
            acc = torch.zeros(tq, g, d)
            for j in range((n + TILE - 1) // TILE):
                k0, k1 = j * TILE, min(n, (j + 1) * TILE)
                dots = torch.einsum("tgd,kd->tgk", q_i8, k_i8[k0:k1, h])                    # exact integers
                sk = dots * k_scale[k0:k1, h].view(1, 1, -1)                               # scaled by the key
                allowed = (torch.arange(k0, k1).view(1, 1, -1) <= pos.view(-1, 1, 1))
                sk_max = torch.where(allowed, sk, torch.full_like(sk, float("-inf"))).amax(-1)
                sc = torch.where(allowed, sk * row_factor.unsqueeze(-1), torch.full_like(sk, float("-inf")))
                # lazy reference: it moves only when the tile maximum exceeds it by more than 2^8
                m_tile = sk_max * row_factor
                grew = m_tile > m_run + 8.0
                m_new = torch.where(grew, m_tile, m_run)
                m_use = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                alpha = torch.where(grew, torch.where(torch.isinf(m_run), torch.zeros_like(m_new),
                                                      torch.exp2(m_run - m_use)), torch.ones_like(m_new))
                p = torch.where(allowed, torch.exp2(sc - m_use.unsqueeze(-1)), torch.zeros_like(sc))
                l_run = l_run * alpha + p.sum(-1)                                          # unrounded sum
                p = p.to(dtype).to(torch.float32)
                acc = acc * alpha.unsqueeze(-1) + torch.einsum("tgk,kd->tgd", p, v_all[k0:k1, h])
                m_run = m_new
            inv_l = torch.where(l_run > 0, 1.0 / l_run, torch.zeros_like(l_run))
            o_rot[lo:hi, h * g:(h + 1) * g] = acc * inv_l.unsqueeze(-1)
    if return_rotated_fp32:
        return o_rot
    return (o_rot.to(dtype).to(torch.float32) @ rot).to(dtype)
