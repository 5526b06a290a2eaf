"""Exact-arithmetic restatement (numpy) of the RotorQuant compress and rotation
steps.  TEST INFRASTRUCTURE ONLY -- nothing in the product imports this file.

``oracle/rq_oracle.py`` restates the reference CPU path with the same library
calls the reference makes (``torch.norm``, MKL ``sgemm``, ``torch.bucketize``).
This file states *which IEEE-754 operations, in which order,* those calls
perform for the shapes on this path, so that a CUDA kernel can reproduce the
bytes without a BLAS:

* reference norm      triton/isoquant_compress.py:174  ``torch.norm(flat, dim=-1)``
* reference divide    triton/isoquant_compress.py:175  ``flat / (raw_norms + 1e-10)``
* reference rotate    triton/isoquant_compress.py:182  ``normalized @ rotation_T``
* reference bucketize triton/isoquant_compress.py:184-185
* reference pack      triton/isoquant_compress.py:187-188
* decode rotations    triton/fused_paged_rq_decode.py:271, :308

Parity status: pinned -- ``tests/test_oracle.py`` checks ``compress_rows`` here
against the cache bytes and norms the reference produced (``tests/golden/``) and
against ``rq_oracle.compress_rows`` on fresh seeded inputs, bit for bit.

The rotation matrix ``R`` is block diagonal with 4x4 blocks (IsoQuant) or 2x2
blocks (PlanarQuant, which is a special case of 4x4 with zeros); products with
the zero entries add nothing, so only the four in-block terms are evaluated.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
F64 = np.float64


def fma32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """Correctly rounded fp32 ``a*b + c`` (what ``fmaf`` returns).

    The product of two fp32 numbers is exact in fp64.  The sum is formed in
    fp64 with round-to-odd (TwoSum gives the exact residual), which makes the
    final rounding to fp32 immune to double rounding.
    """
    p = a.astype(F64) * b.astype(F64)
    c64 = c.astype(F64)
    s = p + c64
    t = s - p
    err = (p - (s - t)) + (c64 - t)
    inexact = err != 0
    if np.any(inexact):
        lower = np.where(err > 0, s, np.nextafter(s, -np.inf))
        upper = np.nextafter(lower, np.inf)
        lower_is_odd = (lower.view(np.int64) & 1) == 1
        s = np.where(inexact, np.where(lower_is_odd, lower, upper), s)
    return s.astype(F32)


def rotation_blocks(rotation: np.ndarray) -> np.ndarray:
    """Dense ``(D, D)`` block-diagonal R -> ``(D/4, 4, 4)`` diagonal blocks.

    Raises if anything outside the 4x4 diagonal blocks is non-zero.
    """
    r = np.asarray(rotation, dtype=F32)
    d = r.shape[0]
    assert r.shape == (d, d) and d % 4 == 0
    blocks = np.stack([r[4 * g:4 * g + 4, 4 * g:4 * g + 4] for g in range(d // 4)])
    off = r.copy()
    for g in range(d // 4):
        off[4 * g:4 * g + 4, 4 * g:4 * g + 4] = 0
    if np.any(off != 0):
        raise ValueError("rotation has non-zero entries outside its 4x4 diagonal blocks")
    return blocks


def row_norms(x: np.ndarray) -> np.ndarray:
    """fp32 L2 norm per row of ``(M, 128)`` exactly as ``torch.norm`` forms it
    on the reference's CPU build: eight running sums ``s_l`` over
    ``x[8c + l]**2`` (c ascending, multiply and add rounded separately), the
    eight combined left to right, one correctly rounded square root."""
    x = np.ascontiguousarray(x, dtype=F32)
    m, d = x.shape
    assert d % 8 == 0
    sq = x * x
    lanes = sq[:, 0:8].copy()
    for c in range(1, d // 8):
        lanes = lanes + sq[:, 8 * c:8 * c + 8]
    s = lanes[:, 0]
    for l in range(1, 8):
        s = s + lanes[:, l]
    return np.sqrt(s)


def rotate_rows(x: np.ndarray, blocks: np.ndarray, transpose: bool) -> np.ndarray:
    """``x @ R.T`` (transpose=True) or ``x @ R`` (transpose=False) for ``(M, D)`` fp32 ``x``.

    Output ``j`` of block ``g`` is the fused-multiply-add chain over the block's
    four inputs in ascending order: ``fma(x3,w3, fma(x2,w2, fma(x1,w1, x0*w0)))``.
    """
    x = np.ascontiguousarray(x, dtype=F32)
    m, d = x.shape
    ng = d // 4
    xb = x.reshape(m, ng, 4)
    out = np.empty((m, ng, 4), dtype=F32)
    for j in range(4):
        # (x @ R.T)[j] = sum_k x[k] R[j][k];  (x @ R)[j] = sum_k x[k] R[k][j]
        w = blocks[:, j, :] if transpose else blocks[:, :, j]          # (ng, 4) over k
        acc = xb[:, :, 0] * w[None, :, 0]
        for k in range(1, 4):
            acc = fma32(xb[:, :, k], np.broadcast_to(w[None, :, k], acc.shape), acc)
        out[:, :, j] = acc
    return out.reshape(m, d)


def bucketize(v: np.ndarray, boundaries: np.ndarray) -> np.ndarray:
    """Number of boundaries strictly below each value, clamped to a nibble."""
    b = np.asarray(boundaries, dtype=F32)
    idx = np.zeros(v.shape, dtype=np.int32)
    for t in b:
        idx += (t < v)
    return np.clip(idx, 0, 15).astype(np.uint8)


def compress_rows(x: np.ndarray, rotation: np.ndarray, boundaries: np.ndarray):
    """``(M, 128)`` fp32 rows -> (packed ``(M, 64)`` uint8, norms ``(M,)`` fp32, rotated ``(M,128)``)."""
    x = np.ascontiguousarray(x, dtype=F32)
    blocks = rotation_blocks(rotation)
    norms = row_norms(x)
    denom = norms + F32(1e-10)
    unit = x / denom[:, None]
    rotated = rotate_rows(unit, blocks, transpose=True)
    idx = bucketize(rotated, boundaries)
    packed = (idx[:, 0::2] << 4) | idx[:, 1::2]
    return packed.astype(np.uint8), norms, rotated


def build_slots(key: np.ndarray, value: np.ndarray, rotation: np.ndarray,
                k_boundaries: np.ndarray, v_boundaries: np.ndarray) -> np.ndarray:
    """``(N, H, 128)`` K and V -> ``(N, H*256)`` uint8 cache slots (payload + zero padding)."""
    n, h, d = key.shape
    assert d == 128
    kp, kn, _ = compress_rows(key.reshape(n * h, d), rotation, k_boundaries)
    vp, vn, _ = compress_rows(value.reshape(n * h, d), rotation, v_boundaries)
    total = h * 256
    row = np.zeros((n, total), dtype=np.uint8)
    row[:, 0:h * 64] = kp.reshape(n, h * 64)
    row[:, h * 64:h * 68] = kn.reshape(n, h).view(np.uint8)
    row[:, h * 68:h * 132] = vp.reshape(n, h * 64)
    row[:, h * 132:h * 136] = vn.reshape(n, h).view(np.uint8)
    return row


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bf16, returned as fp32."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(F32)
