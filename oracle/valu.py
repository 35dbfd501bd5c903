"""CPU restatement of the element-wise / attention steps that sit between the waves of a decoder layer.

TEST INFRASTRUCTURE ONLY — imported by tests/ and by nothing in the product. Written from the semantics of the
reference kernels (not their code), in numpy float64 on the FP16 values of the canvas, with one FP16 rounding where
the reference stores FP16:

* RMSNorm over the channels of every column   kernels/common/kernel44_valu_pack.cuh:104-134
* SwiGLU product (SiLU already applied)        kernels/common/kernel44_valu_pack.cuh:135-143
* rotary embedding, half-split pairing         kernels/common/kernel44_valu_pack.cuh:65-70, 144-158
* causal grouped-query attention per sequence  kernels/common/kernel44_valu_pack.cuh:159-248
* decode attention over a key / value cache    (no counterpart: the reference reserves the cache,
                                                wavec/k44_wave_compiler.hpp:564-585, but never reads it)

PARITY UNPINNED: the reference has no fixtures for these steps either; its own example compares against the same
formulas in numpy (wavec/examples/example_llm.py:23-63) with max-abs 2e-2 / cosine 0.9999.

All tensors are channel-major: channel c of a tensor at element offset `off` occupies canvas[off + c*pitch : ... + pitch].
"""
from __future__ import annotations

import numpy as np


def _rows(canvas: np.ndarray, off: int, rows: int, pitch: int) -> np.ndarray:
    return canvas[off: off + rows * pitch].view(np.float16).reshape(rows, pitch)


def _store(canvas: np.ndarray, off: int, val: np.ndarray, pitch: int) -> None:
    rows = val.shape[0]
    canvas[off: off + rows * pitch] = val.astype(np.float16).reshape(-1).view(np.uint16)


def rmsnorm(canvas, src_off, dst_off, dim, pitch, eps, gamma_bits=None):
    x = _rows(canvas, src_off, dim, pitch).astype(np.float64)
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=0, keepdims=True) + eps)
    y = x * inv
    if gamma_bits is not None:
        y = y * np.asarray(gamma_bits, dtype=np.uint16).view(np.float16).astype(np.float64)[:, None]
    _store(canvas, dst_off, y, pitch)


def swiglu(canvas, gate_off, up_off, dst_off, rows, pitch):
    g = _rows(canvas, gate_off, rows, pitch).astype(np.float64)
    u = _rows(canvas, up_off, rows, pitch).astype(np.float64)
    _store(canvas, dst_off, g * u, pitch)


def rope_inv_freq(head_dim: int, theta: float, llama3: bool) -> np.ndarray:
    p = np.arange(head_dim // 2, dtype=np.float64)
    f = np.exp(2.0 * p * (-np.log(theta) / head_dim))
    if llama3:      # Llama-3 frequency scaling: factor 32 (1/0.03125), low / high frequency factors 1 and 4, 8192 original positions
        ratio = 1303.7972938088068 * f
        smooth = np.clip((ratio - 1.0) / 3.0, 0.0, 1.0)
        f = (1.0 - smooth) * (f * 0.03125) + smooth * f
    return f


def rope(canvas, off, heads, head_dim, pitch, seq_len, theta=10000.0, llama3=False, positions=None):
    """In place. Column t is at position t % seq_len unless `positions` ([pitch]) is given."""
    x = _rows(canvas, off, heads * head_dim, pitch).astype(np.float64)
    pos = (np.arange(pitch) % seq_len).astype(np.float64) if positions is None else np.asarray(positions, dtype=np.float64)
    ang = rope_inv_freq(head_dim, theta, llama3)[:, None] * pos[None, :]
    c, s = np.cos(ang), np.sin(ang)
    half = head_dim // 2
    y = x.copy()
    for h in range(heads):
        a, b = x[h * head_dim: h * head_dim + half], x[h * head_dim + half: (h + 1) * head_dim]
        y[h * head_dim: h * head_dim + half] = a * c - b * s
        y[h * head_dim + half: (h + 1) * head_dim] = a * s + b * c
    _store(canvas, off, y, pitch)


def causal_attention(canvas, q_off, k_off, v_off, out_off, h_q, h_kv, head_dim, pitch, seq_len, columns=None):
    """Every column attends to the columns of its own sequence (blocks of seq_len columns) up to itself."""
    cols = pitch if columns is None else columns
    q = _rows(canvas, q_off, h_q * head_dim, pitch).astype(np.float64)
    k = _rows(canvas, k_off, h_kv * head_dim, pitch).astype(np.float64)
    v = _rows(canvas, v_off, h_kv * head_dim, pitch).astype(np.float64)
    out = np.zeros((h_q * head_dim, pitch))
    grp = h_q // h_kv
    scale = 1.0 / np.sqrt(head_dim)
    for s0 in range(0, cols, seq_len):
        s1 = min(cols, s0 + seq_len)
        n = s1 - s0
        mask = np.triu(np.full((n, n), -np.inf), k=1)
        for h in range(h_q):
            kv = h // grp
            qh = q[h * head_dim:(h + 1) * head_dim, s0:s1].T
            kh = k[kv * head_dim:(kv + 1) * head_dim, s0:s1].T
            vh = v[kv * head_dim:(kv + 1) * head_dim, s0:s1].T
            sc = qh @ kh.T * scale + mask
            sc -= sc.max(axis=-1, keepdims=True)
            p = np.exp(sc)
            p /= p.sum(axis=-1, keepdims=True)
            out[h * head_dim:(h + 1) * head_dim, s0:s1] = (p @ vh).T
    _store(canvas, out_off, out, pitch)


def decode_attention(canvas, q_off, k_off, v_off, out_off, kc_off, vc_off, h_q, h_kv, head_dim, pitch, max_seq, pos,
                     theta=10000.0, llama3=False):
    """One new token per column at position `pos`: rotary on q and k at that position, k and v appended to the
    caches ([h_kv][max_seq][pitch][head_dim]: one head, position and column is one contiguous row), attention over
    cache positions 0..pos."""
    rope(canvas, q_off, h_q, head_dim, pitch, 1, theta, llama3, positions=np.full(pitch, pos))
    rope(canvas, k_off, h_kv, head_dim, pitch, 1, theta, llama3, positions=np.full(pitch, pos))
    ckv = h_kv * head_dim
    n = h_kv * max_seq * pitch * head_dim
    kc = canvas[kc_off: kc_off + n].reshape(h_kv, max_seq, pitch, head_dim)
    vc = canvas[vc_off: vc_off + n].reshape(h_kv, max_seq, pitch, head_dim)
    kc[:, pos] = canvas[k_off: k_off + ckv * pitch].reshape(h_kv, head_dim, pitch).transpose(0, 2, 1)
    vc[:, pos] = canvas[v_off: v_off + ckv * pitch].reshape(h_kv, head_dim, pitch).transpose(0, 2, 1)
    q = _rows(canvas, q_off, h_q * head_dim, pitch).astype(np.float64)
    # [h_kv, positions, pitch, hd] -> [h_kv*hd, positions, pitch]
    K = kc[:, :pos + 1].view(np.float16).astype(np.float64).transpose(0, 3, 1, 2).reshape(ckv, pos + 1, pitch)
    V = vc[:, :pos + 1].view(np.float16).astype(np.float64).transpose(0, 3, 1, 2).reshape(ckv, pos + 1, pitch)
    out = np.zeros((h_q * head_dim, pitch))
    grp = h_q // h_kv
    scale = 1.0 / np.sqrt(head_dim)
    for h in range(h_q):
        kv = h // grp
        qh = q[h * head_dim:(h + 1) * head_dim]                            # [hd, pitch]
        sc = np.einsum("db,dpb->pb", qh, K[kv * head_dim:(kv + 1) * head_dim]) * scale
        sc -= sc.max(axis=0, keepdims=True)
        p = np.exp(sc)
        p /= p.sum(axis=0, keepdims=True)
        out[h * head_dim:(h + 1) * head_dim] = np.einsum("pb,dpb->db", p, V[kv * head_dim:(kv + 1) * head_dim])
    _store(canvas, out_off, out, pitch)
